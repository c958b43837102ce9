"""Random weights for a model, by tensor name.

Each tensor is drawn from its own generator, seeded from (seed, name), so the values do
not depend on the order in which tensors are made or on how parts pack them.  Matrices
and tables of floats are N(0, 0.02); norm weights are 1 + N(0, 0.1).  `write_model_folder`
makes a folder (config.json, model.safetensors) that loads like any other.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

MATRIX_STD = 0.02
NORM_STD = 0.1


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(seed, name))
    if spec.kind == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    z = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    if spec.init == "ones_normal":
        z = 1.0 + NORM_STD * z
    else:
        z = MATRIX_STD * z
    return z.to(dtype)


def random_tensors(specs: dict, seed: int, dtype: torch.dtype, device="cpu") -> dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, dtype, device) for name, spec in specs.items()}


def write_model_folder(folder, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors for `config` (an architecture's
    configuration object) with random weights stored as `dtype`."""
    from safetensors.torch import save_file

    from ..parts import BuildContext, Model

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    model = Model(config.to_spec(), BuildContext(dtype=dtype, device=torch.device("cpu")))
    tensors = random_tensors(model.tensor_specs(), seed, dtype, "cpu")
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
