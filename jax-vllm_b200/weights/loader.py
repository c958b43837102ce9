"""Weights from a model folder, bound by tensor name.

Every `*.safetensors` file of the folder is read (sorted; a later file wins on a
duplicate name, jllm/model/weights.py:21-30).  Tensors stored in 16-bit floats are kept
in bfloat16, tensors stored in 32-bit floats stay 32-bit, integer tensors become int32.
Before anything is handed to the model, the names and shapes in the folder are compared
with what the model's parts ask for, and ONE error lists every missing tensor, every
unexpected tensor and every wrong shape.
"""

from __future__ import annotations

from pathlib import Path

import torch


class WeightError(ValueError):
    """The folder's tensors do not fit the model.  `.missing`, `.unexpected` and `.wrong_shape`
    hold the details that the message lists."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_kind = list(wrong_shape), list(wrong_kind)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong type ({len(self.wrong_kind)}): " + ", ".join(
                f"{n} is {got}, expected {want}" for n, got, want in self.wrong_kind))
        super().__init__("\n".join(lines))


class DamagedFile(ValueError):
    """A file of the folder is not a whole safetensors file (cut short while it was copied, say)."""


_FLOAT16 = (torch.float16, torch.bfloat16)
_FLOAT32 = (torch.float32, torch.float64)
_INTS = (torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64, torch.bool)


def storage_dtype(stored: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor is kept in."""
    if stored in _FLOAT16:
        return torch.bfloat16
    if stored in _FLOAT32:
        return torch.float32
    if stored in _INTS:
        return torch.int32
    raise ValueError(f"tensors of type {stored} cannot be loaded")


def list_shards(folder) -> list[Path]:
    folder = Path(folder)
    shards = sorted(folder.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no safetensors in {folder}")
    return shards


def read_index(folder) -> dict[str, tuple[Path, tuple, str]]:
    """name -> (file, shape, stored dtype name) without reading any data."""
    from safetensors import safe_open

    index = {}
    for shard in list_shards(folder):
        try:
            with safe_open(str(shard), framework="pt") as f:
                for key in f.keys():
                    sl = f.get_slice(key)
                    index[key] = (shard, tuple(sl.get_shape()), sl.get_dtype())
        except Exception as exc:          # the library's own error type is not part of its documented interface
            raise DamagedFile(f"{shard} ({shard.stat().st_size} bytes) cannot be read as a safetensors file; it may "
                              f"have been cut short: {exc}") from exc
    return index


def check(folder, index, specs: dict, optional=()) -> None:
    missing = [n for n in specs if n not in index]
    unexpected = sorted(n for n in index if n not in specs and n not in optional)
    wrong_shape, wrong_kind = [], []
    for n, spec in specs.items():
        if n not in index:
            continue
        _, shape, dt = index[n]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((n, shape, spec.shape))
        is_int = dt.upper().startswith(("I", "U", "BOOL"))
        if (spec.kind == "table") != is_int:
            wrong_kind.append((n, dt, "integers" if spec.kind == "table" else "floats"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(folder, missing, unexpected, wrong_shape, wrong_kind)


def load_tensors(folder, specs: dict, device, optional=()) -> dict[str, torch.Tensor]:
    """Checks the folder against `specs` (name -> TensorSpec) and returns the named tensors on
    `device` in their storage dtype."""
    from safetensors import safe_open

    index = read_index(folder)
    check(folder, index, specs, optional)
    by_file: dict[Path, list[str]] = {}
    for n in specs:
        by_file.setdefault(index[n][0], []).append(n)
    out = {}
    for shard, names in by_file.items():
        with safe_open(str(shard), framework="pt") as f:
            for n in names:
                t = f.get_tensor(n)
                out[n] = t.to(device=device, dtype=storage_dtype(t.dtype))
    return out
