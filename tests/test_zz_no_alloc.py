"""The entry point that allocates nothing (csrc/attn_decode_static.cu), called through its
exported C symbol as a user without an allocator would call it.  Its output is compared with
the existing split decode attention and with a dense float32 attention written here, on two
calls in a row; device memory must be the same before and after; calls beyond the fixed array
or with sizes the kernel does not take are refused before anything reaches the stream.  The
file sorts last so that a run which stops at the first failure has run everything else before."""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def problem(seed, hq, hkv, d, page, starts, split, window=0):
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
                R=R, hq=hq, hkv=hkv, d=d, page=page, num_pages=num_pages, split=split, window=window,
                n_splits=-(-max(total) // split), scale=1.0 / math.sqrt(d), starts=list(starts))


def dense(p) -> torch.Tensor:
    """softmax(q k^T * scale) v over each request's own keys (the last `window` of them if there is a window),
    in float32 on the CPU from the values the kernels read."""
    q, kc, vc, table = p["q"].float().cpu(), p["kc"].float().cpu(), p["vc"].float().cpu(), p["table"].cpu()
    hq, hkv, d, page = p["hq"], p["hkv"], p["d"], p["page"]
    out = torch.zeros(p["R"], hq * d)
    for e, s in enumerate(p["starts"]):
        n = s + 1
        pages = table[e, :-(-n // page)].long()
        k = kc[pages].reshape(-1, hkv, d)[:n]
        v = vc[pages].reshape(-1, hkv, d)[:n]
        lo = max(0, n - p["window"]) if p["window"] else 0
        for h in range(hq):
            kv = h // (hq // hkv)
            scores = (k[lo:, kv] @ q[e, h * d:(h + 1) * d]) * p["scale"]
            out[e, h * d:(h + 1) * d] = torch.softmax(scores, 0) @ v[lo:, kv]
    return out


def call_static(fn, p, status, out=None, **over):
    a = dict(p, **over)
    if out is None:
        out = torch.zeros(p["R"], p["hq"] * p["d"], dtype=torch.bfloat16, device=DEV)
    rc = fn(a["q"].data_ptr(), a["hq"] * a["d"], out.data_ptr(), a["hq"] * a["d"], a["kc"].data_ptr(),
            a["vc"].data_ptr(), a["table"].data_ptr(), a["table"].shape[1], a["cu"].data_ptr(), a["start"].data_ptr(),
            a["work"].data_ptr(), a["R"], a["hq"], a["hkv"], a["d"], a["page"], a["num_pages"], a["window"], a["scale"],
            a["split"], a["n_splits"], status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def call_existing(ops, p):
    out = torch.zeros(p["R"], p["hq"] * p["d"], dtype=torch.bfloat16, device=DEV)
    ops.attn_mma(p["q"], p["hq"] * p["d"], out, p["kc"], p["vc"], p["table"], p["cu"], p["start"], p["work"], p["R"],
                 p["hq"], p["hkv"], p["d"], p["window"], p["scale"], split_size=p["split"], n_splits=p["n_splits"])
    return out


def load_entry_point():
    from jax_vllm_b200.csrc import build

    lib = build.load("attn_decode_static")
    fn = lib.jv_attn_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    need = lib.jv_attn_decode_static_scratch_floats
    need.restype = ctypes.c_longlong
    need.argtypes = [c_int] * 4
    return fn, need


def test_static_scratch_entry_point_matches_the_existing_one_twice_in_a_row():
    from jax_vllm_b200 import ops

    fn, need = load_entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # two calls in a row share the scratch array: the second (other sizes, fewer splits, a window) must not
    # be disturbed by what the first left there
    first = problem(1, hq=32, hkv=8, d=128, page=16, starts=[0, 300, 1500, 63, 1023], split=256)
    second = problem(2, hq=6, hkv=2, d=64, page=8, starts=[700, 5, 129], split=128, window=200)
    outs = [torch.zeros(p["R"], p["hq"] * p["d"], dtype=torch.bfloat16, device=DEV) for p in (first, second)]
    rc0, _ = call_static(fn, first, status, out=outs[0].clone())     # the first call on the device does the set-up
    assert rc0 == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for p, out in zip((first, second), outs):
        assert need(p["R"], p["hq"], p["n_splits"], p["d"]) * 4 <= 16 << 20
        rc, _ = call_static(fn, p, status, out=out)
        assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the entry point took or gave back device memory"
    for p, got in zip((first, second), outs):
        want = call_existing(ops, p)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(got.float().cpu(), dense(p), atol=2e-2, rtol=2e-2)
    assert status.item() == 0
    ops.check_status()


def test_static_scratch_entry_point_refuses_what_it_cannot_hold_and_launches_nothing():
    fn, need = load_entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    p = problem(1, hq=32, hkv=8, d=128, page=16, starts=[0, 300, 1500, 63, 1023], split=256)
    marked = torch.full((p["R"], p["hq"] * p["d"]), 3.0, dtype=torch.bfloat16, device=DEV)

    def refused(**over):
        out = marked.clone()
        rc, _ = call_static(fn, p, status, out=out, **over)
        torch.cuda.synchronize()
        return rc == 2 and torch.equal(out, marked)

    # more partial results than the fixed array holds
    assert need(4096, 32, 64, 128) * 4 > 16 << 20
    assert refused(R=4096, n_splits=64)
    # results that would fit, but more (token, kv head) counters than the array sets aside for them
    assert need(4096, 8, 1, 16) * 4 <= 15 << 20 and 4096 * 8 > 16384
    assert refused(R=4096, hq=8, hkv=8, d=16, n_splits=1)
    # a head size the kernel is not built for, and a query stride that breaks its 16-byte copies
    assert refused(d=48)
    out = marked.clone()
    rc = fn(p["q"].data_ptr(), 4100, out.data_ptr(), 4096, p["kc"].data_ptr(), p["vc"].data_ptr(), p["table"].data_ptr(),
            p["table"].shape[1], p["cu"].data_ptr(), p["start"].data_ptr(), p["work"].data_ptr(), p["R"], 32, 8, 128, 16,
            p["num_pages"], 0, p["scale"], 256, p["n_splits"], status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 2 and torch.equal(out, marked)
    assert status.item() == 0


def test_static_scratch_entry_point_reports_too_few_splits_in_the_status_word():
    """A launch with fewer splits than a request's length needs records it (the caller sized the launch wrongly)
    and still returns; the next, well-sized call is right again."""
    fn, _ = load_entry_point()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    p = problem(5, hq=8, hkv=2, d=64, page=16, starts=[500, 40], split=128)
    rc, _ = call_static(fn, p, status, n_splits=2)
    torch.cuda.synchronize()
    assert rc == 0 and status.item() & 4
    status.zero_()
    rc, got = call_static(fn, p, status)
    torch.cuda.synchronize()
    assert rc == 0 and status.item() == 0
    torch.testing.assert_close(got.float().cpu(), dense(p), atol=2e-2, rtol=2e-2)
