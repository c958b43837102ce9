"""Each CUDA kernel alone against a plain float32 reference, at sizes other than the
engine's (odd widths, vocabularies that are no power of two, many head groupings)."""

import math

import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def ops():
    from jax_vllm_b200 import ops as o
    return o


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(ops, dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1000, 200, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, 1000, (37,), generator=g, dtype=torch.int32).to(DEV)
    out = ops.embed_gather(table, ids)
    assert out.dtype == torch.float32 and torch.equal(out, table.float()[ids.long()])
    ops.check_status()
    bad = torch.tensor([3, 1000, -1], dtype=torch.int32, device=DEV)
    out = ops.embed_gather(table, bad)
    with pytest.raises(ops.KernelError, match="token id"):
        ops.check_status()
    assert torch.equal(out[1], torch.zeros(200, device=DEV))
    ops.check_status()                       # the word was cleared


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [200, 4096, 1000, 12288, 100])
@pytest.mark.parametrize("wdtype", DTYPES)
def test_rmsnorm_variants(ops, dtype, hidden, wdtype):
    g = torch.Generator().manual_seed(1)
    h = (3 * torch.randn(19, hidden, generator=g)).to(DEV)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(wdtype).to(DEV)
    delta = torch.randn(19, hidden, generator=g).to(dtype).to(DEV)
    eps = 1e-5
    y = ops.rmsnorm(h.clone(), w, eps, dtype)
    torch.testing.assert_close(y.float(), plain.rms_norm(h, w.float(), eps), **tol(dtype))
    h2 = h.clone()
    y = ops.rmsnorm(h2, w, eps, dtype, delta=delta)
    want_h = h + delta.float()
    torch.testing.assert_close(h2, want_h, atol=1e-6, rtol=1e-6)       # the sum is kept in float32
    torch.testing.assert_close(y.float(), plain.rms_norm(want_h, w.float(), eps), **tol(dtype))
    rows = torch.tensor([18, 0, 7, 7], dtype=torch.int32, device=DEV)
    h3 = h.clone()
    y = ops.rmsnorm(h3, w, eps, dtype, delta=delta, rows=rows)
    assert torch.equal(h3, h)                                          # gathered rows: h is left alone
    torch.testing.assert_close(y.float(), plain.rms_norm(want_h, w.float(), eps)[rows.long()], **tol(dtype))
    y = ops.rmsnorm(h3, w, eps, dtype, rows=rows)
    torch.testing.assert_close(y.float(), plain.rms_norm(h, w.float(), eps)[rows.long()], **tol(dtype))
    ops.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_add_and_swiglu(ops, dtype):
    g = torch.Generator().manual_seed(2)
    h = torch.randn(23, 72, generator=g).to(DEV)
    d = torch.randn(23, 72, generator=g).to(dtype).to(DEV)
    want = h + d.float()
    ops.residual_add(h, d)
    torch.testing.assert_close(h, want, atol=1e-6, rtol=1e-6)
    gu = (2 * torch.randn(23, 2 * 56, generator=g)).to(dtype).to(DEV)
    act = ops.swiglu(gu)
    gate, up = gu.float()[:, :56], gu.float()[:, 56:]
    torch.testing.assert_close(act.float(), torch.nn.functional.silu(gate) * up, **tol(dtype))
    # blocks of 8 gate columns, each followed by its 8 up columns
    blocked = torch.stack([gu[:, :56].reshape(23, 7, 8), gu[:, 56:].reshape(23, 7, 8)], dim=2).reshape(23, 112).contiguous()
    torch.testing.assert_close(ops.swiglu(blocked, 8).float(), act.float(), atol=0, rtol=0)
    with pytest.raises(ops.KernelError):
        ops.swiglu(gu, 5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(37, 70, 45), (1, 384, 96), (130, 129, 64), (5, 8, 300)])
def test_gemm_simt(ops, dtype, m, n, k):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(m, k, generator=g).to(dtype).to(DEV)
    w = torch.randn(n, k, generator=g).to(dtype).to(DEV)
    y = ops.gemm_simt(x, w, torch.float32)
    want = x.double() @ w.double().T
    torch.testing.assert_close(y.double(), want, atol=1e-4, rtol=1e-5)
    # a row's result does not depend on the other rows of the batch
    y1 = ops.gemm_simt(x[m // 2:m // 2 + 1], w, torch.float32)
    assert torch.equal(y1[0], y[m // 2])
    # strided input rows (a column slice of a wider tensor)
    wide = torch.randn(m, k + 24, generator=g).to(dtype).to(DEV)
    ys = ops.gemm_simt(wide[:, 8:8 + k], w, torch.float32)
    torch.testing.assert_close(ys.double(), wide[:, 8:8 + k].double() @ w.double().T, atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(70, 96), (4096, 4096), (1000, 1536), (24, 8), (151, 4104), (24576, 512), (4096, 12288), (50, 2056)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_skinny(ops, m, n, k, out_dtype):
    g = torch.Generator().manual_seed(m * 1000 + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(DEV)
    y = ops.linear_skinny(x, w, out_dtype)
    want = (x.double() @ w.double().T)
    if out_dtype == torch.float32:
        torch.testing.assert_close(y.double(), want, atol=1e-4, rtol=1e-4)
    else:
        torch.testing.assert_close(y.double(), want, atol=2e-2, rtol=2e-2)
    # a row's result does not depend on the rest of the batch (other batch sizes take other instantiations)
    for rows in ([m // 2], list(range(min(m, 5)))):
        ys = ops.linear_skinny(x[rows].contiguous(), w, out_dtype)
        assert torch.equal(ys, y[rows])
    # rows of a wider tensor
    wide = torch.randn(m, k + 16, generator=g).to(torch.bfloat16).to(DEV)
    y2 = ops.linear_skinny(wide[:, 8:8 + k], w, torch.float32)
    torch.testing.assert_close(y2.double(), wide[:, 8:8 + k].double() @ w.double().T, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("m", [1, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("n,k", [(70, 96), (4096, 4096), (1000, 1536), (24, 8), (151, 4104), (24576, 512), (4096, 12288), (50, 2056)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_linear_stream(ops, m, n, k, out_dtype):
    """The tcgen05 product for larger batches of decoded tokens: the weight is the 128-row operand."""
    g = torch.Generator().manual_seed(m * 1000 + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(DEV)
    y = ops.linear_stream(x, w, out_dtype)
    want = (x.double() @ w.double().T)
    if out_dtype == torch.float32:
        torch.testing.assert_close(y.double(), want, atol=1e-4, rtol=1e-4)
    else:
        torch.testing.assert_close(y.double(), want, atol=2e-2, rtol=2e-2)
    # a row's result does not depend on the rest of the batch
    for rows in ([m // 2], list(range(min(m, 21)))):
        ys = ops.linear_stream(x[rows].contiguous(), w, out_dtype)
        assert torch.equal(ys, y[rows])
    # rows of a wider tensor
    wide = torch.randn(m, k + 16, generator=g).to(torch.bfloat16).to(DEV)
    y2 = ops.linear_stream(wide[:, 8:8 + k], w, torch.float32)
    torch.testing.assert_close(y2.double(), wide[:, 8:8 + k].double() @ w.double().T, atol=1e-4, rtol=1e-4)
    ops.check_status()


@pytest.mark.parametrize("m,n,k", [(17, 4096, 4096), (64, 6144, 4096), (40, 4096, 12288), (128, 24576, 4096), (33, 1000, 1536)])
def test_linear_stream_parts_of_a_sum(ops, m, n, k):
    g = torch.Generator().manual_seed(m * 1000 + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(DEV)
    splits = ops.linear_stream_splits(DEV, n, k)
    y = ops.linear_stream(x, w, torch.bfloat16, parts_ok=True)
    want = x.double() @ w.double().T
    if splits > 1:
        assert isinstance(y, ops.PartialSum) and y.parts.shape == (splits, m, n) and tuple(y.shape) == (m, n)
        torch.testing.assert_close(y.parts.double().sum(0), want, atol=1e-4, rtol=1e-4)
        ys = ops.linear_stream(x[m // 2:m // 2 + 1].contiguous(), w, torch.bfloat16, parts_ok=True)
        assert torch.equal(ys.parts[:, 0], y.parts[:, m // 2])
    else:
        torch.testing.assert_close(y.double(), want, atol=2e-2, rtol=2e-2)
    assert ops.linear_stream_splits(DEV, 4096, 4096) > 1            # 32 strips for 148 multiprocessors: k is cut
    # through the dispatcher (up to 64 rows this kernel where the strips fill the device, else the mma.sync one or the library)
    got = ops.linear(x, w, torch.float32)
    torch.testing.assert_close(got.double(), want, atol=1e-4, rtol=1e-4)
    ops.check_status()


def test_dispatcher_leaves_a_few_strips_too_many_to_the_library(ops):
    """One tensor wanted, few rows: 448 strips of 16 rows for 444 resident blocks would leave all but four blocks idle
    for a second round, so the dispatcher takes the library's product there; the result is the same product."""
    assert ops.linear_skinny_evenness(DEV, 6144) == 1.0 and ops.linear_skinny_evenness(DEV, 96) == 1.0
    assert ops.linear_skinny_evenness(DEV, 7168) < ops.SKINNY_MIN_EVENNESS < ops.linear_skinny_evenness(DEV, 10240)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(8, 512, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(7168, 512, generator=g) / 512 ** 0.5).to(torch.bfloat16).to(DEV)
    before = ops.launch_count
    y = ops.linear(x, w, torch.bfloat16)
    assert ops.launch_count == before                      # not a kernel of this package
    torch.testing.assert_close(y.double(), x.double() @ w.double().T, atol=2e-2, rtol=2e-2)
    y2 = ops.linear(x, w[:6144], torch.bfloat16)
    assert ops.launch_count == before + 1
    torch.testing.assert_close(y2.double(), x.double() @ w[:6144].double().T, atol=2e-2, rtol=2e-2)


def test_linear_skinny_cuts_k_when_strips_are_few(ops):
    # few strips of a long k are cut into parts that other blocks take; many strips, or a short k, are not
    assert ops.linear_skinny_splits(DEV, 4096, 12288) > 1
    assert ops.linear_skinny_splits(DEV, 1024, 2048) > 1
    assert ops.linear_skinny_splits(DEV, 151936, 4096) == 1
    assert ops.linear_skinny_splits(DEV, 4096, 64) == 1


@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(4096, 12288), (4096, 4096), (1024, 2048), (1000, 2056), (151, 4104)])
def test_linear_skinny_parts_of_a_sum(ops, m, n, k):
    g = torch.Generator().manual_seed(m * 1000 + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(DEV)
    y = ops.linear_skinny(x, w, torch.bfloat16, parts_ok=True)
    assert isinstance(y, ops.PartialSum) and y.parts.shape == (ops.linear_skinny_splits(DEV, n, k), m, n)
    assert tuple(y.shape) == (m, n)
    want = x.double() @ w.double().T
    torch.testing.assert_close(y.tensor().double(), want, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(y.parts.double().sum(0), want, atol=1e-4, rtol=1e-4)
    # the parts of a row do not depend on the rest of the batch
    ys = ops.linear_skinny(x[m // 2:m // 2 + 1].contiguous(), w, torch.bfloat16, parts_ok=True)
    assert torch.equal(ys.parts[:, 0], y.parts[:, m // 2])
    # the dispatcher hands back parts only where it was allowed to (it takes the tcgen05 product for these rows)
    assert isinstance(ops.linear(x, w, torch.bfloat16, parts_ok=True), ops.PartialSum) == (ops.linear_stream_splits(DEV, n, k) > 1)
    assert isinstance(ops.linear(x, w, torch.bfloat16), torch.Tensor)


@pytest.mark.parametrize("n,hidden,parts", [(3, 96, 2), (8, 4096, 4), (5, 1000, 3), (2, 20000, 2)])
def test_readers_add_the_parts_of_a_sum(ops, n, hidden, parts):
    g = torch.Generator().manual_seed(parts + hidden)
    ps = torch.randn(parts, n, hidden, generator=g).to(DEV)
    whole = ps[0].clone()
    for s in range(1, parts):
        whole += ps[s]                                   # the same order of additions as the kernels
    weight = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(DEV)
    h0 = torch.randn(n, hidden, generator=g).to(DEV)
    # norm with the residual sum, in place and gathered
    h1, h2 = h0.clone(), h0.clone()
    y1 = ops.rmsnorm(h1, weight, 1e-6, torch.bfloat16, delta=ops.PartialSum(ps))
    y2 = ops.rmsnorm(h2, weight, 1e-6, torch.bfloat16, delta=whole)
    assert torch.equal(y1, y2) and torch.equal(h1, h2)
    rows = torch.tensor([n - 1, 0], dtype=torch.int32, device=DEV)
    y1 = ops.rmsnorm(h0.clone(), weight, 1e-6, torch.float32, delta=ops.PartialSum(ps), rows=rows)
    y2 = ops.rmsnorm(h0.clone(), weight, 1e-6, torch.float32, delta=whole, rows=rows)
    assert torch.equal(y1, y2)
    # the plain residual sum, and the sum alone
    assert torch.equal(ops.residual_add(h0.clone(), ops.PartialSum(ps)), ops.residual_add(h0.clone(), whole))
    assert torch.equal(ops.PartialSum(ps).tensor(), whole)
    # the gated activation (a gate|up of hidden columns, in blocks where they divide)
    if hidden % 8 == 0:
        for block in (None, hidden // 8 if hidden % 64 == 0 else None):
            a1 = ops.swiglu(ops.PartialSum(ps), block, out_dtype=torch.bfloat16)
            a2 = ops.swiglu(whole, block).to(torch.bfloat16)
            torch.testing.assert_close(a1.float(), a2.float(), atol=1e-2, rtol=1e-2)
            gate, up = (whole[:, :hidden // 2], whole[:, hidden // 2:]) if block is None else \
                (whole.view(n, -1, 2, block)[:, :, 0].reshape(n, -1), whole.view(n, -1, 2, block)[:, :, 1].reshape(n, -1))
            torch.testing.assert_close(a1.float(), torch.nn.functional.silu(gate) * up, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (130, 300, 72), (5, 256, 64),
                                   (2048, 1024, 4096), (300, 6144, 1024), (1000, 264, 4104)])
@pytest.mark.parametrize("epilogue", ["bf16", "f32"])
def test_gemm_tcgen05(ops, m, n, k, epilogue):
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16).to(DEV)
    y = ops.gemm_tcgen05(x, w, epilogue)
    ops.check_status()
    want = x.double() @ w.double().T
    if epilogue == "f32":
        assert y.dtype == torch.float32
        torch.testing.assert_close(y.double(), want, atol=2e-4, rtol=2e-4)
    else:
        torch.testing.assert_close(y.double(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("m,inter,k", [(128, 128, 64), (200, 256, 128), (2048, 1024, 512), (7, 384, 72)])
def test_gemm_tcgen05_gated_epilogue(ops, m, inter, k):
    g = torch.Generator().manual_seed(m + inter)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(inter, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    up = (torch.randn(inter, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    packed = torch.stack([gate.reshape(-1, 128, k), up.reshape(-1, 128, k)], dim=1).reshape(2 * inter, k).to(DEV)
    y = ops.gemm_tcgen05(x, packed, "swiglu")
    ops.check_status()
    xd = x.double().cpu()
    want = torch.nn.functional.silu(xd @ gate.double().T) * (xd @ up.double().T)
    torch.testing.assert_close(y.double().cpu(), want, atol=2e-2, rtol=2e-2)


def test_linear_dispatch(ops):
    x = torch.randn(4, 64).to(torch.bfloat16).to(DEV)
    w = torch.randn(32, 64).to(torch.bfloat16).to(DEV)
    before = ops.launch_count
    y = ops.linear(x, w, torch.float32)
    assert ops.launch_count == before + 1                   # this package's kernel, not the library
    torch.testing.assert_close(y.double(), x.double() @ w.double().T, atol=1e-3, rtol=1e-3)
    big = torch.randn(200, 64).to(torch.bfloat16).to(DEV)
    before = ops.launch_count
    ops.linear(big, w)
    assert ops.launch_count == before                       # prompts: the library product


def test_linear_uses_true_float32(ops):
    # operands whose product needs more than 10 mantissa bits: a reduced-precision matrix mode would show
    x = torch.full((4, 256), 1.0 + 2 ** -12, device=DEV)
    w = torch.full((8, 256), 1.0 + 2 ** -12, device=DEV)
    y = ops.linear(x, w)
    want = 256 * (1.0 + 2 ** -12) ** 2
    assert abs(y[0, 0].item() - want) < 1e-3 and abs(y[0, 0].item() - 256.0) > 0.1


# ------------------------------------------------------------------ rope + kv write
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 16, 16), (6, 1, 32, 8), (3, 3, 48, 4), (8, 2, 128, 16), (5, 5, 64, 8),
                                           (2, 1, 256, 16)])
@pytest.mark.parametrize("q_lens,starts", [([5, 1, 9], [3, 40, 0]), ([30, 1, 47], [3, 40, 0])],
                         ids=["few tokens", "many tokens (a block per token)"])
def test_rope_kv(ops, dtype, hq, hkv, d, page, q_lens, starts):
    g = torch.Generator().manual_seed(4)
    n = sum(q_lens)
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).to(dtype)
    positions = torch.cat([torch.arange(s, s + q) for s, q in zip(starts, q_lens)]).to(torch.int32)
    entry = torch.cat([torch.full((q,), e) for e, q in enumerate(q_lens)]).to(torch.int32)
    width = -(-48 // page)
    num_pages = 3 * width + 4
    perm = torch.randperm(num_pages, generator=g)
    table = perm[: 3 * width].reshape(3, width).to(torch.int32)
    theta, eps = 1e4, 1e-5
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kc = torch.full((num_pages, page, hkv, d), 7.0).to(dtype).to(DEV)
    vc = torch.full((num_pages, page, hkv, d), 7.0).to(dtype).to(DEV)
    dq = qkv.clone().to(DEV)
    ops.rope_kv(dq, positions.to(DEV), entry.to(DEV), table.to(DEV), inv_freq.to(DEV), qw.to(DEV), kw.to(DEV),
                eps, kc, vc, hq, hkv, d)
    ops.check_status()
    f = qkv.float()
    q = f[:, : hq * d].reshape(n, hq, d).transpose(0, 1)
    k = f[:, hq * d:(hq + hkv) * d].reshape(n, hkv, d).transpose(0, 1)
    v = f[:, (hq + hkv) * d:].reshape(n, hkv, d)
    cos, sin = plain.rope_cos_sin(positions, d, theta)
    q_want = plain.apply_rope(plain.rms_norm(q, qw.float(), eps), cos, sin).transpose(0, 1).reshape(n, hq * d)
    k_want = plain.apply_rope(plain.rms_norm(k, kw.float(), eps), cos, sin).transpose(0, 1)
    torch.testing.assert_close(dq[:, : hq * d].float().cpu(), q_want, **tol(dtype))
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for i in range(n):
        p, e = positions[i].item(), entry[i].item()
        pg, sl = table[e, p // page].item(), p % page
        written[pg, sl] = True
        torch.testing.assert_close(kc[pg, sl].float().cpu(), k_want[i], **tol(dtype))
        assert torch.equal(vc[pg, sl].cpu(), qkv[i, (hq + hkv) * d:].reshape(hkv, d))
    assert torch.all(kc.cpu()[~written] == 7.0) and torch.all(vc.cpu()[~written] == 7.0)   # nothing else touched


def test_rope_kv_without_norm_rotation_or_cache(ops):
    g = torch.Generator().manual_seed(5)
    hq, d, n = 2, 32, 4
    qkv = torch.randn(n, hq * d, generator=g)
    pos = torch.tensor([0, 5, 100, 3000], dtype=torch.int32)
    ent = torch.zeros(n, dtype=torch.int32)
    table = torch.zeros((1, 1), dtype=torch.int32)
    dq = qkv.clone().to(DEV)
    ops.rope_kv(dq, pos.to(DEV), ent.to(DEV), table.to(DEV), None, None, None, 0.0, None, None, hq, 1, d)
    assert torch.equal(dq.cpu(), qkv)
    # partial rotation: only the first 16 of 32 elements rotate; large positions keep 32-bit angles
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))
    ops.rope_kv(dq, pos.to(DEV), ent.to(DEV), table.to(DEV), inv_freq.to(DEV), None, None, 0.0, None, None, hq, 1, d)
    x = qkv.reshape(n, hq, d)
    cos, sin = plain.rope_cos_sin(pos, 16, 1e6)
    rot = plain.apply_rope(x[..., :16].transpose(0, 1), cos, sin).transpose(0, 1)
    want = torch.cat([rot, x[..., 16:]], dim=-1).reshape(n, hq * d)
    torch.testing.assert_close(dq.cpu(), want, atol=2e-5, rtol=2e-5)


def test_rope_kv_flags_a_missing_page(ops):
    hq = hkv = 1; d = 16
    qkv = torch.zeros(1, 3 * d, device=DEV)
    kc = torch.zeros(2, 4, 1, d, device=DEV); vc = torch.zeros_like(kc)
    args = (torch.tensor([5], dtype=torch.int32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV))
    ops.rope_kv(qkv, *args, torch.tensor([[0, -1]], dtype=torch.int32, device=DEV), None, None, None, 0.0, kc, vc,
                hq, hkv, d)
    with pytest.raises(ops.KernelError, match="page"):
        ops.check_status()


# ------------------------------------------------------------------------ attention
def dense_attention(q, k_all, v_all, q_pos, scale, window, g):
    """q: [n, hq, d]; k_all, v_all: [len, hkv, d]; one request; float32 throughout."""
    k = k_all.repeat_interleave(g, dim=1)
    v = v_all.repeat_interleave(g, dim=1)
    s = torch.einsum("nhd,lhd->hnl", q, k) * scale
    j = torch.arange(k_all.shape[0])[None, :]
    vis = j <= q_pos[:, None]
    if window:
        vis = vis & (j > q_pos[:, None] - window)
    s = torch.where(vis[None], s, torch.tensor(float("-inf")))
    return torch.einsum("hnl,lhd->nhd", torch.softmax(s, -1), v)


def run_attention(ops, dtype, hq, hkv, d, page, q_lens, starts, window=0, split=0, seed=6, boost=None, mma=False,
                  tc5=False, dec5=False, large=None):
    g = torch.Generator().manual_seed(seed)
    G = hq // hkv
    R, n = len(q_lens), sum(q_lens)
    total = [s + q for s, q in zip(starts, q_lens)]
    pages_per = [-(-t // page) for t in total]
    num_pages = sum(pages_per) + 5
    perm = torch.randperm(num_pages, generator=g).tolist()
    width = max(pages_per)
    table = torch.full((R, width), -1, dtype=torch.int32)
    kc = torch.full((num_pages, page, hkv, d), float("nan"))          # unowned slots hold NaN: reading one shows
    vc = torch.full((num_pages, page, hkv, d), float("nan"))
    ks, vs = [], []
    for e in range(R):
        k = torch.randn(total[e], hkv, d, generator=g).to(dtype).float()
        v = torch.randn(total[e], hkv, d, generator=g).to(dtype).float()
        if boost is not None and e == boost[0]:
            k[boost[1]] *= 6.0                                        # one far key that the last query must find
        if large is not None and (large[0] is None or e == large[0]):
            k[large[1]:] *= large[2]                                  # scores grow late: the running maximum must move
        ks.append(k); vs.append(v)
        for i in range(pages_per[e]):
            pg = perm.pop()
            table[e, i] = pg
            m = min(page, total[e] - i * page)
            kc[pg, :m] = k[i * page:i * page + m]
            vc[pg, :m] = v[i * page:i * page + m]
    q = torch.randn(n, hq, d, generator=g).to(dtype).float()
    if boost is not None:
        last = sum(q_lens[: boost[0] + 1]) - 1
        q[last] = ks[boost[0]][boost[1]].repeat_interleave(G, dim=0) * 1.0
    scale = 1.0 / math.sqrt(d)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    want = torch.cat([dense_attention(q[cu[e]:cu[e + 1]], ks[e], vs[e], torch.arange(starts[e], total[e]), scale,
                                      window, G) for e in range(R)])
    dq = q.reshape(n, hq * d).to(dtype).to(DEV)
    out = torch.zeros(n, hq * d, dtype=dtype, device=DEV)
    common = (kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), table.to(DEV), cu.to(DEV),
              torch.tensor(starts, dtype=torch.int32, device=DEV))
    tpt = (ops.attn_tcgen05_tokens_per_tile if tc5 else ops.attn_mma_tokens_per_tile if mma
           else ops.attn_simt_tokens_per_tile)(hq, hkv)
    attn = ops.attn_mma if mma else ops.attn_simt
    if split:
        assert all(ql == 1 for ql in q_lens)
        work = torch.tensor([[e, 0] for e in range(R)], dtype=torch.int32, device=DEV)
        if dec5:
            ops.attn_decode_tcgen05(dq, hq * d, out, *common, work, R, hq, hkv, d, scale)
        else:
            attn(dq, hq * d, out, *common, work, R, hq, hkv, d, window, scale, split_size=split,
                 n_splits=-(-max(total) // split))
    else:
        work = torch.tensor([[e, t] for e in range(R) for t in range(0, q_lens[e], tpt)], dtype=torch.int32, device=DEV)
        if tc5:
            ops.attn_tcgen05(dq, hq * d, out, *common, work, work.shape[0], hq, hkv, d, scale)
        else:
            attn(dq, hq * d, out, *common, work, work.shape[0], hq, hkv, d, window, scale)
    ops.check_status()
    got = out.float().cpu().reshape(n, hq, d)
    assert not torch.isnan(got).any()
    return got, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 16, 16), (6, 1, 32, 8), (5, 5, 48, 4), (8, 2, 128, 16),
                                           (20, 1, 64, 16), (2, 1, 256, 32)])
def test_attention_portions_with_context(ops, dtype, hq, hkv, d, page):
    got, want = run_attention(ops, dtype, hq, hkv, d, page, q_lens=[7, 1, 33, 2], starts=[0, 50, 21, 64])
    torch.testing.assert_close(got, want, **(dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page,split", [(4, 2, 16, 16, 32), (6, 1, 32, 8, 24), (8, 2, 128, 16, 256), (20, 2, 64, 4, 64)])
def test_attention_decode_splits(ops, dtype, hq, hkv, d, page, split):
    got, want = run_attention(ops, dtype, hq, hkv, d, page, q_lens=[1, 1, 1, 1], starts=[0, 31, 300, 63], split=split)
    torch.testing.assert_close(got, want, **(dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("window", [1, 5, 16, 40])
@pytest.mark.parametrize("split", [0, 16])
def test_attention_window_edges(ops, window, split):
    q_lens, starts = ([1, 1, 1], [0, 39, 77]) if split else ([9, 30, 1], [0, 35, 77])
    got, want = run_attention(ops, torch.float32, 4, 2, 32, 8, q_lens=q_lens, starts=starts, window=window, split=split)
    torch.testing.assert_close(got, want, atol=3e-5, rtol=3e-5)


@pytest.mark.parametrize("split", [0, 64])
@pytest.mark.parametrize("far", [0, 3, 130, 511])
def test_attention_finds_one_far_key_among_hundreds(ops, split, far):
    # the last query equals one key scaled up, so that key takes nearly all the weight
    q_lens = [1, 1] if split else [3, 2]
    starts = [10, 600 - q_lens[1]]
    got, want = run_attention(ops, torch.float32, 4, 2, 64, 16, q_lens=q_lens, starts=starts, split=split,
                              boost=(1, far))
    torch.testing.assert_close(got, want, atol=3e-5, rtol=3e-5)


# ---- the tensor-core kernels (bfloat16) against the same dense reference
BF16_TOL = dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 16, 16), (6, 1, 32, 8), (5, 5, 64, 4), (32, 8, 128, 16),
                                           (20, 1, 64, 16), (3, 1, 128, 32)])
def test_mma_attention_portions_with_context(ops, hq, hkv, d, page):
    got, want = run_attention(ops, torch.bfloat16, hq, hkv, d, page, q_lens=[7, 1, 133, 2, 70], starts=[0, 50, 21, 64, 190],
                              mma=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("hq,hkv,d,page,split", [(4, 2, 16, 16, 32), (6, 1, 32, 8, 24), (32, 8, 128, 16, 256),
                                                 (20, 2, 64, 4, 64), (8, 2, 128, 16, 1024)])
def test_mma_attention_decode_splits(ops, hq, hkv, d, page, split):
    got, want = run_attention(ops, torch.bfloat16, hq, hkv, d, page, q_lens=[1, 1, 1, 1, 1], starts=[0, 31, 300, 63, 1500],
                              split=split, mma=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("window", [1, 5, 16, 40, 100])
@pytest.mark.parametrize("split", [0, 16])
def test_mma_attention_window_edges(ops, window, split):
    q_lens, starts = ([1, 1, 1], [0, 39, 177]) if split else ([9, 130, 1], [0, 35, 177])
    got, want = run_attention(ops, torch.bfloat16, 4, 2, 32, 8, q_lens=q_lens, starts=starts, window=window, split=split,
                              mma=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("split", [0, 64])
@pytest.mark.parametrize("far", [0, 3, 130, 511])
def test_mma_attention_finds_one_far_key_among_hundreds(ops, split, far):
    q_lens = [1, 1] if split else [3, 2]
    starts = [10, 600 - q_lens[1]]
    got, want = run_attention(ops, torch.bfloat16, 4, 2, 64, 16, q_lens=q_lens, starts=starts, split=split,
                              boost=(1, far), mma=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


# ---- the tcgen05 kernel (bfloat16, head size 128)
@pytest.mark.parametrize("hq,hkv,page", [(4, 1, 16), (32, 8, 16), (8, 8, 8), (2, 1, 128), (16, 1, 32), (16, 2, 64),
                                         (40, 8, 16), (3, 1, 32), (12, 2, 16), (7, 1, 64), (13, 1, 16)])
def test_tcgen05_attention_portions_with_context(ops, hq, hkv, page):
    got, want = run_attention(ops, torch.bfloat16, hq, hkv, 128, page, q_lens=[7, 300, 133, 2, 70], starts=[0, 50, 21, 64, 190],
                              tc5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("far", [0, 3, 130, 511])
def test_tcgen05_attention_finds_one_far_key_among_hundreds(ops, far):
    got, want = run_attention(ops, torch.bfloat16, 4, 2, 128, 16, q_lens=[3, 2], starts=[10, 598], boost=(1, far), tc5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


def test_tcgen05_attention_long_prompt(ops):
    got, want = run_attention(ops, torch.bfloat16, 8, 2, 128, 16, q_lens=[1000], starts=[0], tc5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("far", [5, 9000, 20479])
def test_tcgen05_attention_portions_deep_in_a_long_context(ops, far):
    # portions that begin after tens of thousands of cached keys (block tables more than a thousand pages wide, more
    # than a hundred and sixty key tiles a block), one of them with a key far back that its last query must find
    got, want = run_attention(ops, torch.bfloat16, 8, 2, 128, 16, q_lens=[130, 64, 200], starts=[20400, 3, 8100],
                              boost=(0, far), tc5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


def test_tcgen05_attention_prompt_of_several_thousand_tokens(ops):
    got, want = run_attention(ops, torch.bfloat16, 4, 1, 128, 32, q_lens=[4100], starts=[0], tc5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


# ---- the tcgen05 decode kernel (bfloat16, head size 128, keys as tensor-core rows, persistent over all requests)
@pytest.mark.parametrize("hq,hkv,page", [(4, 1, 16), (32, 8, 16), (8, 8, 8), (2, 1, 128), (16, 1, 32), (6, 2, 64), (5, 1, 16),
                                         (12, 1, 16)])
def test_tcgen05_decode_attention(ops, hq, hkv, page):
    got, want = run_attention(ops, torch.bfloat16, hq, hkv, 128, page, q_lens=[1, 1, 1, 1, 1, 1],
                              starts=[0, 31, 300, 127, 1500, 1023], split=1, dec5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("starts", [[5], [127], [128], [40000], [20000, 3, 0, 129]])
def test_tcgen05_decode_attention_short_and_long(ops, starts):
    # one tile for the whole launch, one more key than a tile, and pairs that span many blocks
    got, want = run_attention(ops, torch.bfloat16, 8, 2, 128, 16, q_lens=[1] * len(starts), starts=starts, split=1, dec5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("far", [0, 3, 130, 511, 1290])
def test_tcgen05_decode_attention_finds_one_far_key(ops, far):
    got, want = run_attention(ops, torch.bfloat16, 4, 2, 128, 16, q_lens=[1, 1], starts=[10, 1299], split=1,
                              boost=(1, far), dec5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("from_key", [100, 128, 200, 700])
def test_tcgen05_decode_attention_moves_its_reference_when_scores_grow_late(ops, from_key):
    # keys from `from_key` on are four times larger, so scores there exceed the first tiles' maxima by far more
    # than the slack of the lazy rescaling: the accumulated output and the sums must be rescaled.  One kv head
    # and few requests make a block's run of tiles long enough to hold the change.
    got, want = run_attention(ops, torch.bfloat16, 8, 1, 128, 16, q_lens=[1] * 150, starts=[899] * 150, split=1,
                              large=(None, from_key, 4.0), dec5=True)
    torch.testing.assert_close(got, want, **BF16_TOL)


def test_tcgen05_decode_attention_twice_in_a_row_and_many_requests(ops):
    starts = [(37 * i) % 700 for i in range(300)]
    for seed in (1, 2):
        got, want = run_attention(ops, torch.bfloat16, 8, 2, 128, 16, q_lens=[1] * 300, starts=starts, split=1, seed=seed,
                                  dec5=True)
        torch.testing.assert_close(got, want, **BF16_TOL)


@pytest.mark.parametrize("hq,hkv,page,with_norm,with_rope", [(32, 8, 16, True, True), (4, 1, 8, True, True), (6, 2, 64, False, True),
                                                             (16, 1, 32, True, False), (5, 1, 128, False, False)])
def test_tcgen05_decode_attention_that_prepares_its_tokens(ops, hq, hkv, page, with_norm, with_rope):
    """The kernel is given q|k|v as the product leaves it: it must do what rope_kv does (per-head norm, rotation,
    write of the new key and value) and attend over the cached keys and the new one."""
    d, G = 128, hq // hkv
    g = torch.Generator().manual_seed(hq * 7 + page)
    starts = [0, 1, 31, 127, 128, 129, 300, 1023, 1500, 256]      # keys in the cache before the new token
    R = len(starts)
    pages_per = [-(-(t + 1) // page) for t in starts]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, max(pages_per)), -1, dtype=torch.int32)
    kc = torch.full((num_pages, page, hkv, d), float("nan"))
    vc = torch.full((num_pages, page, hkv, d), float("nan"))
    ks, vs, slot_of_new = [], [], []
    bf = lambda t: t.to(torch.bfloat16).float()
    for e in range(R):
        k, v = bf(torch.randn(starts[e], hkv, d, generator=g)), bf(torch.randn(starts[e], hkv, d, generator=g))
        ks.append(k); vs.append(v)
        for i in range(pages_per[e]):
            pg = perm.pop()
            table[e, i] = pg
            m = max(0, min(page, starts[e] - i * page))
            kc[pg, :m] = k[i * page:i * page + m]
            vc[pg, :m] = v[i * page:i * page + m]
        slot_of_new.append((int(table[e, starts[e] // page]), starts[e] % page))
    qkv = bf(torch.randn(R, (hq + 2 * hkv) * d, generator=g))
    qw = bf(1 + 0.1 * torch.randn(d, generator=g)) if with_norm else None
    kw = bf(1 + 0.1 * torch.randn(d, generator=g)) if with_norm else None
    theta, eps = 1e6, 1e-6
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d)) if with_rope else None
    # ---- what it should be: the plain formulas on the same values, rounded where the engine rounds
    pos = torch.tensor(starts)
    q = qkv[:, : hq * d].reshape(R, hq, d).transpose(0, 1)
    k_new = qkv[:, hq * d:(hq + hkv) * d].reshape(R, hkv, d).transpose(0, 1)
    v_new = qkv[:, (hq + hkv) * d:].reshape(R, hkv, d)
    if with_norm:
        q, k_new = plain.rms_norm(q, qw, eps), plain.rms_norm(k_new, kw, eps)
    if with_rope:
        cos, sin = plain.rope_cos_sin(pos, d, theta)
        q, k_new = plain.apply_rope(q, cos, sin), plain.apply_rope(k_new, cos, sin)
    q, k_new = bf(q).transpose(0, 1), bf(k_new).transpose(0, 1)          # [R, heads, d]
    scale = 1.0 / math.sqrt(d)
    want = torch.cat([dense_attention(q[e:e + 1], torch.cat([ks[e], k_new[e:e + 1]]), torch.cat([vs[e], v_new[e:e + 1]]),
                                      torch.tensor([starts[e]]), scale, 0, G) for e in range(R)])
    # ---- the kernel
    dq = qkv.to(torch.bfloat16).to(DEV)
    out = torch.zeros(R, hq * d, dtype=torch.bfloat16, device=DEV)
    dk, dv = kc.to(torch.bfloat16).to(DEV), vc.to(torch.bfloat16).to(DEV)
    work = torch.tensor([[e, 0] for e in range(R)], dtype=torch.int32, device=DEV)
    cu = torch.arange(R + 1, dtype=torch.int32, device=DEV)
    dev = lambda t: None if t is None else t.to(DEV)
    for w_dtype in ((torch.bfloat16, torch.float32) if with_norm else (None,)):
        cast = (lambda t: None if t is None else t.to(w_dtype).to(DEV))
        k_in, v_in = dk.clone(), dv.clone()
        ops.attn_decode_tcgen05(dq, dq.stride(0), out, k_in, v_in, table.to(DEV), cu,
                                torch.tensor(starts, dtype=torch.int32, device=DEV), work, R, hq, hkv, d, scale,
                                prepare=(dev(inv_freq), cast(qw), cast(kw), eps))
        ops.check_status()
        got = out.float().cpu().reshape(R, hq, d)
        assert not torch.isnan(got).any()
        torch.testing.assert_close(got, want, **BF16_TOL)
        # the new key and value are in the cache, and nothing else was written
        kk, vv = k_in.float().cpu(), v_in.float().cpu()
        for e, (pg, sl) in enumerate(slot_of_new):
            torch.testing.assert_close(kk[pg, sl], k_new[e], atol=2e-2, rtol=2e-2)
            assert torch.equal(vv[pg, sl], v_new[e])
            kk[pg, sl] = kc[pg, sl]; vv[pg, sl] = vc[pg, sl]
        same = lambda a, b: torch.equal(torch.nan_to_num(a, nan=123.0), torch.nan_to_num(b, nan=123.0))
        assert same(kk, bf(kc)) and same(vv, bf(vc))


def test_tcgen05_decode_support_rules(ops):
    from jax_vllm_b200.csrc import build
    lib = build.load("attn_decode_tcgen05")
    for d, hq, hkv, page, window, n in [(128, 32, 8, 16, 0, 8), (64, 32, 8, 16, 0, 8), (128, 6, 1, 16, 0, 1),
                                        (128, 32, 8, 4, 0, 8), (128, 32, 8, 16, 5, 8), (128, 16, 1, 128, 0, 512),
                                        (128, 20, 1, 16, 0, 8), (128, 32, 8, 16, 0, 513)]:
        assert bool(lib.jv_attn_decode_tcgen05_supports(d, hq, hkv, page, window, n)) == \
            ops.attn_decode_tcgen05_supports(torch.bfloat16, d, hq, hkv, page, window, n)


def test_tcgen05_support_rules(ops):
    from jax_vllm_b200.csrc import build
    lib = build.load("attn_tcgen05")
    for d, hq, hkv, page, window in [(128, 32, 8, 16, 0), (64, 32, 8, 16, 0), (128, 6, 1, 16, 0), (128, 32, 8, 4, 0),
                                     (128, 32, 8, 16, 5), (128, 16, 1, 128, 0), (128, 20, 1, 16, 0), (128, 40, 8, 16, 0),
                                     (128, 17, 1, 16, 0)]:
        assert bool(lib.jv_attn_tcgen05_supports(d, hq, hkv, page, window)) == \
            ops.attn_tcgen05_supports(torch.bfloat16, d, hq, hkv, page, window)
    assert lib.jv_attn_tcgen05_tokens_per_tile(32, 8) == ops.attn_tcgen05_tokens_per_tile(32, 8) == 32
    assert lib.jv_attn_tcgen05_tokens_per_tile(40, 8) == ops.attn_tcgen05_tokens_per_tile(40, 8) == 25


def test_mma_support_table_matches_the_library(ops):
    from jax_vllm_b200.csrc import build
    lib = build.load("attn_mma")
    for d in range(8, 300, 8):
        assert bool(lib.jv_attn_mma_supports(d)) == (d in ops.MMA_HEAD_DIMS)
    assert lib.jv_attn_mma_tokens_per_tile(32, 8) == ops.attn_mma_tokens_per_tile(32, 8) == 16
    assert not ops.attn_mma_supports(torch.float32, 128)


def test_attention_refuses_what_it_cannot_do(ops):
    z = torch.zeros(1, 512, device=DEV)
    i = torch.zeros(2, dtype=torch.int32, device=DEV)
    c = torch.zeros(1, 4, 1, 512, device=DEV)
    with pytest.raises(ops.KernelError, match="outside what the kernel handles"):
        ops.attn_simt(z, 512, z.clone(), c, c, i.view(1, 2), i, i[:1], i.view(1, 2), 1, 1, 1, 512, 0, 1.0)


# ------------------------------------------------------------------------- sampling
def test_greedy_is_argmax_with_lowest_index_on_ties(ops):
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(9, 1531, generator=g).to(DEV)
    logits[3, 700] = logits[3, 20] = 50.0
    z = torch.zeros(9, device=DEV); zi = torch.zeros(9, dtype=torch.int64, device=DEV)
    got = ops.sample(logits, z, zi, zi)
    want = logits.argmax(-1)
    want[3] = 20
    assert torch.equal(got.long(), want)


def test_temperature_draws_follow_the_host_restatement_and_the_distribution(ops):
    from jax_vllm_b200.sampling import uniform
    V = 11
    logits = torch.tensor([[0.3 * i for i in range(V)]])
    temp = 0.8
    n = 4000
    big = logits.repeat(n, 1).to(DEV)
    t = torch.full((n,), temp, device=DEV)
    seeds = torch.full((n,), 1234, dtype=torch.int64, device=DEV)
    counters = torch.arange(n, dtype=torch.int64, device=DEV)
    got = ops.sample(big, t, seeds, counters).cpu()
    # exact agreement with the host formula on the first draws
    for c in range(50):
        scores = [logits[0, v].item() / temp - math.log(-math.log(uniform(1234, c, v))) for v in range(V)]
        assert got[c].item() == max(range(V), key=lambda v: scores[v])
    # frequencies follow softmax(logits / T)
    p = torch.softmax(logits[0] / temp, -1)
    freq = torch.bincount(got.long(), minlength=V).float() / n
    assert (freq - p).abs().max().item() < 0.03
    # same (seed, counter) -> same token wherever the row stands; another seed -> another stream
    again = ops.sample(big.flip(0), t, seeds, counters.flip(0)).cpu().flip(0)
    assert torch.equal(again, got)
    other = ops.sample(big, t, seeds + 1, counters).cpu()
    assert (other != got).float().mean().item() > 0.3


def test_a_wait_that_nothing_ends_runs_out_is_reported_and_leaves_the_device_usable(ops):
    """The bounded wait of the TMA and tcgen05 kernels, alone (csrc/wait_probe.cu): with an arrival it succeeds;
    with none it gives up after its few thousand clocks, the kernel returns, the status word carries the bit and
    `check_status` raises an error that names the wait; the word and the split attention's arrival counters are
    clean afterwards and kernels run as before."""
    ok, _ = ops.wait_probe(20_000, arrive=True)
    assert ok
    ops.check_status()
    counters = ops._split_counters(DEV, 64)
    counters[:5] = 3                                   # what blocks that left early would leave behind
    ok, spent = ops.wait_probe(20_000, arrive=False)
    assert not ok and 20_000 <= spent < 20_000_000
    with pytest.raises(ops.KernelError, match="bounded wait"):
        ops.check_status()
    ops.check_status()                                 # cleared: the next step starts clean
    assert int(ops._split_counters(DEV, 64).abs().sum()) == 0
    x = torch.randn(3, 64, device=DEV)
    w = torch.ones(64, device=DEV)
    y = ops.rmsnorm(x.clone(), w, 1e-6, torch.float32)
    torch.testing.assert_close(y, x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6), atol=1e-5, rtol=1e-5)
    with pytest.raises(ops.KernelError, match="outside what the kernel handles"):
        ops.wait_probe(1 << 40, arrive=False)          # never longer than the product's own bound
