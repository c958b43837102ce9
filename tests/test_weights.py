"""Weight loading by name, its one clear error, and the random-weights mode (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from jax_vllm_b200 import registry
from jax_vllm_b200.parts import BuildContext, Model
from jax_vllm_b200.weights import WeightError, load_tensors, random_tensors, storage_dtype, write_model_folder
from tests.util import TINY_A, TINY_B, make_folder, tensor_shapes


def _model(c, dtype=torch.bfloat16):
    return Model(registry.config_from_dict(c).to_spec(), BuildContext(dtype=dtype, device=torch.device("cpu")))


def test_names_the_model_asks_for_are_the_checkpoint_names():
    for c in (TINY_A, TINY_B):
        m = _model(c)
        assert {k: tuple(v.shape) for k, v in m.tensor_specs().items()} == tensor_shapes(c)


def test_loads_and_keeps_dtypes(tmp_path):
    folder = make_folder(tmp_path / "m", "b", dtype=torch.bfloat16)
    w = load_file(str(folder / "model.safetensors"))
    w["model.norm.weight"] = w["model.norm.weight"].to(torch.float32)       # a tensor stored in 32-bit stays so
    w["model.layers.0.mlp.up_proj.weight"] = w["model.layers.0.mlp.up_proj.weight"].to(torch.float16)
    save_file(w, str(folder / "model.safetensors"))
    m = _model(TINY_B)
    t = load_tensors(folder, m.tensor_specs(), "cpu", m.optional_tensors())
    assert t["model.norm.weight"].dtype == torch.float32
    assert t["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert t["lm_head.weight"].dtype == torch.bfloat16 and set(t) == set(m.tensor_specs())
    assert storage_dtype(torch.int64) == torch.int32 and storage_dtype(torch.float64) == torch.float32


def test_one_error_lists_missing_unexpected_and_shapes(tmp_path):
    folder = make_folder(tmp_path / "m", "a")
    w = load_file(str(folder / "model.safetensors"))
    del w["model.layers.1.self_attn.q_norm.weight"]
    del w["model.layers.0.mlp.down_proj.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    w["model.norm.weight"] = torch.zeros(65)
    w["model.layers.1.mlp.up_proj.weight"] = torch.zeros(64, 160)
    save_file(w, str(folder / "model.safetensors"))
    m = _model(TINY_A)
    with pytest.raises(WeightError) as e:
        load_tensors(folder, m.tensor_specs(), "cpu", m.optional_tensors())
    err = e.value
    assert set(err.missing) == {"model.layers.1.self_attn.q_norm.weight", "model.layers.0.mlp.down_proj.weight"}
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.norm.weight", "model.layers.1.mlp.up_proj.weight"}
    msg = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "q_proj.bias", "[65]", "[64]", "[160, 64]"):
        assert needle in msg


def test_tied_model_ignores_stored_head_and_untied_needs_it(tmp_path):
    folder = make_folder(tmp_path / "a", "a")
    w = load_file(str(folder / "model.safetensors"))
    w["lm_head.weight"] = torch.zeros(256, 64)
    save_file(w, str(folder / "model.safetensors"))
    m = _model(TINY_A)
    t = load_tensors(folder, m.tensor_specs(), "cpu", m.optional_tensors())
    assert "lm_head.weight" not in t
    folder_b = make_folder(tmp_path / "b", "b")
    wb = load_file(str(folder_b / "model.safetensors")); del wb["lm_head.weight"]
    save_file(wb, str(folder_b / "model.safetensors"))
    mb = _model(TINY_B)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_tensors(folder_b, mb.tensor_specs(), "cpu", mb.optional_tensors())


def test_no_safetensors(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="no safetensors"):
        load_tensors(tmp_path, {}, "cpu")


def test_several_shards(tmp_path):
    folder = make_folder(tmp_path / "m", "a")
    w = load_file(str(folder / "model.safetensors"))
    names = sorted(w)
    save_file({k: w[k] for k in names[::2]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: w[k] for k in names[1::2]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    m = _model(TINY_A)
    t = load_tensors(folder, m.tensor_specs(), "cpu", m.optional_tensors())
    assert all(torch.equal(t[k], w[k]) for k in t)


def test_random_mode_writes_a_folder_that_loads(tmp_path):
    cfg = registry.config_from_dict(TINY_B)
    folder = write_model_folder(tmp_path / "r", cfg, seed=7)
    assert registry.config_from_path(folder) == cfg
    m = _model(TINY_B)
    t = load_tensors(folder, m.tensor_specs(), "cpu")
    again = random_tensors(m.tensor_specs(), 7, torch.bfloat16)
    other = random_tensors(m.tensor_specs(), 8, torch.bfloat16)
    assert all(torch.equal(t[k], again[k]) for k in t)
    assert not torch.equal(t["lm_head.weight"], other["lm_head.weight"])
    w = t["model.layers.2.mlp.gate_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = t["model.layers.0.input_layernorm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    # values of a tensor depend on its name and the seed only, not on what else the model holds
    sub = {k: v for k, v in m.tensor_specs().items() if "layers.1" in k}
    assert all(torch.equal(random_tensors(sub, 7, torch.bfloat16)[k], t[k]) for k in sub)


@pytest.mark.parametrize("keep", [5, 100, 0.5, -10])
def test_a_file_that_was_cut_short_is_named(tmp_path, keep):
    """A safetensors file cut short (inside its header, inside its data, ten bytes before its end) gives one
    error that names the file, not a stack of the reading library's own."""
    from jax_vllm_b200.weights import DamagedFile
    folder = make_folder(tmp_path / "m", "a")
    path = folder / "model.safetensors"
    data = path.read_bytes()
    n = int(len(data) * keep) if isinstance(keep, float) else (keep if keep > 0 else len(data) + keep)
    path.write_bytes(data[:n])
    m = _model(TINY_A)
    with pytest.raises(DamagedFile, match="model.safetensors .* cut short"):
        load_tensors(folder, m.tensor_specs(), "cpu", m.optional_tensors())
