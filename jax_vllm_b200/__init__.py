"""Importable name of the package in the folder `jax-vllm_b200/` (whose name, with its
hyphen, cannot be written in an import statement): `import jax_vllm_b200` runs that
folder's `__init__.py` as this package."""

import pathlib as _pathlib

_real = _pathlib.Path(__file__).resolve().parent.parent / "jax-vllm_b200"
__path__ = [str(_real)]
__file__ = str(_real / "__init__.py")
exec(compile((_real / "__init__.py").read_text(), __file__, "exec"))
