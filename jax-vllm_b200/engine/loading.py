"""From a model folder (or a configuration and a seed) to a model on the device.

`load_from_path` follows the reference's (jllm/model/weights.py:161-170): the folder's
config.json names the architecture, the registry gives its configuration class, the
model is built from the resulting spec and its tensors are bound by name.
"""

from __future__ import annotations

import torch

from .. import registry
from ..config import parse_dtype
from ..parts import BuildContext, Model
from ..weights import load_tensors, random_tensors


def _build(spec, dtype, device, decode_split_size) -> Model:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("models are loaded onto a CUDA device (the engine has no CPU path)")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; this engine runs on B200 (sm_100a) only")
    return Model(spec, BuildContext(dtype=parse_dtype(dtype), device=dev, decode_split_size=decode_split_size))


def load_from_path(path, dtype="bf16", device="cuda:0", decode_split_size: int = 256) -> Model:
    """The model of the folder `path` (config.json + *.safetensors), weights on `device`."""
    cfg = registry.config_from_path(path)
    model = _build(cfg.to_spec(), dtype, device, decode_split_size)
    model.config = cfg
    model.bind(load_tensors(path, model.tensor_specs(), model.ctx.device, model.optional_tensors()))
    return model


def random_model(config, seed: int, dtype="bf16", device="cuda:0", decode_split_size: int = 256,
                 generate_on_device: bool = True) -> Model:
    """A model of configuration `config` with random weights (see weights.random_init), drawn
    on the device unless `generate_on_device` is False (CPU draws equal those that
    `write_model_folder` stores)."""
    model = _build(config.to_spec(), dtype, device, decode_split_size)
    model.config = config
    store = torch.bfloat16 if model.ctx.dtype == torch.bfloat16 else torch.float32
    where = model.ctx.device if generate_on_device else "cpu"
    tensors = random_tensors(model.tensor_specs(), seed, store, where)
    model.bind({k: v.to(model.ctx.device) for k, v in tensors.items()})
    return model
