"""One registry from the architecture name in config.json to its configuration class.

A configuration class has `from_dict(config_json) -> cfg`, `cfg.to_spec() -> ModelSpec`
and `cfg.to_dict() -> config_json`.  Everything downstream (weights, parts, cache,
engine) works from the `ModelSpec` alone.  The lookup follows the reference's
(jllm/model/weights.py:59-65,161-170): `architectures[0]` decides, and an unknown or
missing name is an error that lists what is known.
"""

from __future__ import annotations

import json
from pathlib import Path

ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    ARCHITECTURES[name] = config_cls


def read_architecture(config_json: dict, where: str = "config.json") -> str:
    archs = config_json.get("architectures") or []
    if not archs:
        raise ValueError(f"no 'architectures' field in {where}")
    return archs[0]


def config_from_dict(config_json: dict, where: str = "config.json"):
    arch = read_architecture(config_json, where)
    try:
        cls = ARCHITECTURES[arch]
    except KeyError:
        raise ValueError(f"unsupported architecture: {arch!r}. Supported: {', '.join(sorted(ARCHITECTURES))}") from None
    return cls.from_dict(config_json)


def config_from_path(path):
    p = Path(path)
    if p.is_dir():
        p = p / "config.json"
    if not p.is_file():
        raise FileNotFoundError(f"no config.json at {p}")
    return config_from_dict(json.loads(p.read_text()), str(p))


def _register_builtin() -> None:
    from .models.qwen3 import ARCHITECTURE, Qwen3Config

    register_architecture(ARCHITECTURE, Qwen3Config)


_register_builtin()
