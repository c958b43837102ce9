"""A request of several thousand tokens through the replay program, against the plain implementation run on the
device in float32 (TF32 off): block tables hundreds of pages wide, prompt portions of 2,048 tokens that begin after
thousands of cached keys, rotation angles at large positions, and single tokens decoded at the end of it, with the
head layout of the benchmarked model (32 query heads in 8 groups, head size 128: the tcgen05 kernels in bfloat16)."""

import json

import pytest
import torch

from tests.plain.qwen3_plain import PlainModel, read_config, read_weights
from tests.test_replay_gpu import compare
from tests.util import TINY_E, make_weights, random_tokens, write_folder

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
LENGTH, TAIL = 5000, 24
PORTIONS = (2048, 2048, LENGTH - TAIL - 4096)


@pytest.fixture(scope="module")
def long_case(tmp_path_factory):
    c = dict(TINY_E, max_position_embeddings=8192)
    folder = write_folder(tmp_path_factory.mktemp("long_context"), c, make_weights(c, seed=4))
    toks = random_tokens(LENGTH, c["vocab_size"], seed=77)
    before = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        plain = PlainModel(cfg=read_config(folder), weights={k: v.to(DEV) for k, v in read_weights(folder).items()})
        want = plain.logits(toks).float().cpu()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = before
    assert want.abs().max() > 1.0
    return folder, c, toks, want


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graph"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_five_thousand_tokens_in_portions_then_one_by_one(long_case, dtype, graphs, tmp_path):
    from jax_vllm_b200.engine.replay import Replayer
    folder, c, toks, want = long_case
    steps, fed = [], 0
    for n in PORTIONS:
        places = sorted(set(list(range(0, n, 509)) + [n - 2, n - 1]))
        steps.append({"step": len(steps), "entries": [{"id": "r", "tokens": toks[fed:fed + n], "want": places}], "end": []})
        fed += n
    while fed < LENGTH:
        steps.append({"step": len(steps), "entries": [{"id": "r", "tokens": toks[fed:fed + 1], "want": [0]}],
                      "end": ["r"] if fed == LENGTH - 1 else []})
        fed += 1
    rep = Replayer(folder, dtype, tmp_path, max_tokens=LENGTH + 64, page_size=16, cuda_graphs=graphs)
    rep.run_stream(json.dumps(s) for s in steps)
    rep.cache.check()
    assert not rep.cache.live
    got, _ = compare(steps, tmp_path, c["vocab_size"], {"r": want}, dtype,
                     case="five thousand tokens" + (", graph" if graphs else ""))
    assert len(got["r"]) == sum(len(s["entries"][0]["want"]) for s in steps)
    assert sum(1 for m in rep.records if m["replayed_graph"]) == (TAIL - 1 if graphs else 0)      # the first single-token step runs eagerly
    # the portions of 2,048 tokens went to the prompt kernel's whole tiles in bfloat16
    tiles = rep.records[1]["tiles"]
    assert sum(tiles.values()) >= 2048 // 128
