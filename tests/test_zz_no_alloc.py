"""The entry point that allocates nothing (csrc/attn_decode_static.cu), called through its
exported C symbol as a user without an allocator would call it, and compared with the
existing split decode attention on two calls in a row.  The file sorts last so that a run
which stops at the first failure has run everything else before."""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def problem(seed, hq, hkv, d, page, starts, split):
    """Single decoded tokens of several requests with their keys and values in shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    R = len(starts)
    total = [s + 1 for s in starts]
    pages_per = [-(-t // page) for t in total]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, max(pages_per)), -1, dtype=torch.int32)
    kc = torch.randn(num_pages, page, hkv, d, generator=g)
    vc = torch.randn(num_pages, page, hkv, d, generator=g)
    for e in range(R):
        for i in range(pages_per[e]):
            table[e, i] = perm.pop()
    q = torch.randn(R, hq * d, generator=g)
    t = lambda x, dt=torch.bfloat16: x.to(dt).to(DEV).contiguous()
    return dict(q=t(q), kc=t(kc), vc=t(vc), table=table.to(DEV), cu=torch.arange(R + 1, dtype=torch.int32, device=DEV),
                start=torch.tensor(starts, dtype=torch.int32, device=DEV),
                work=torch.tensor([[e, 0] for e in range(R)], dtype=torch.int32, device=DEV),
                R=R, hq=hq, hkv=hkv, d=d, page=page, num_pages=num_pages, split=split,
                n_splits=-(-max(total) // split), scale=1.0 / math.sqrt(d))


def call_static(fn, p, status):
    out = torch.zeros(p["R"], p["hq"] * p["d"], dtype=torch.bfloat16, device=DEV)
    rc = fn(p["q"].data_ptr(), p["hq"] * p["d"], out.data_ptr(), p["hq"] * p["d"], p["kc"].data_ptr(),
            p["vc"].data_ptr(), p["table"].data_ptr(), p["table"].shape[1], p["cu"].data_ptr(), p["start"].data_ptr(),
            p["work"].data_ptr(), p["R"], p["hq"], p["hkv"], p["d"], p["page"], p["num_pages"], 0, p["scale"],
            p["split"], p["n_splits"], status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def call_existing(ops, p):
    out = torch.zeros(p["R"], p["hq"] * p["d"], dtype=torch.bfloat16, device=DEV)
    ops.attn_mma(p["q"], p["hq"] * p["d"], out, p["kc"], p["vc"], p["table"], p["cu"], p["start"], p["work"], p["R"],
                 p["hq"], p["hkv"], p["d"], 0, p["scale"], split_size=p["split"], n_splits=p["n_splits"])
    return out


def test_static_scratch_entry_point_matches_the_existing_one_twice_in_a_row():
    from jax_vllm_b200 import ops
    from jax_vllm_b200.csrc import build

    lib = build.load("attn_decode_static")
    fn = lib.jv_attn_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    need = lib.jv_attn_decode_static_scratch_floats
    need.restype = ctypes.c_longlong
    need.argtypes = [c_int] * 4
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    # two calls in a row share the scratch array: the second (other sizes, fewer splits) must not
    # be disturbed by what the first left there
    first = problem(1, hq=32, hkv=8, d=128, page=16, starts=[0, 300, 1500, 63, 1023], split=256)
    second = problem(2, hq=6, hkv=2, d=64, page=8, starts=[700, 5, 129], split=128)
    for p in (first, second):
        assert need(p["R"], p["hq"], p["n_splits"], p["d"]) * 4 <= 16 << 20
        rc, got = call_static(fn, p, status)
        assert rc == 0
        want = call_existing(ops, p)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert status.item() == 0
    ops.check_status()

    # a call that needs more than the fixed array is refused and launches nothing
    big = dict(first, R=4096, n_splits=64)
    assert need(big["R"], big["hq"], big["n_splits"], big["d"]) * 4 > 16 << 20
    before = torch.full_like(got, 3.0)
    out = before.clone()
    rc = fn(first["q"].data_ptr(), 4096, out.data_ptr(), 4096, first["kc"].data_ptr(), first["vc"].data_ptr(),
            first["table"].data_ptr(), first["table"].shape[1], first["cu"].data_ptr(), first["start"].data_ptr(),
            first["work"].data_ptr(), 4096, 32, 8, 128, 16, first["num_pages"], 0, first["scale"], 256, 64,
            status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 2 and torch.equal(out, before)
