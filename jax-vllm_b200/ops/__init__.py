"""Python faces of the CUDA kernels in `csrc/`.

Every function here checks device, dtype, shape and contiguity of what it is given,
then passes raw pointers and the current CUDA stream to an `extern "C"` launcher loaded
by `csrc.build`.  There is no CPU path and no library fallback: a tensor on the CPU, a
missing compiler or a failed launch raises.  Matrix products of 16-bit operands with more
than 64 rows (prompt portions), except the one with the gate in its epilogue, go to cuBLAS
through `torch.mm` (a library product, as in the reference, whose every product is XLA's);
every other operation on the forward path, the products of decode steps among them, is a
kernel of this package.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc import build as _build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
STATUS_BITS = {1: "token id outside the embedding table", 2: "page id outside the pool or missing from the block table",
               4: "row index outside the batch", 8: "a bounded wait inside a kernel ran out"}


class KernelError(RuntimeError):
    pass


class PartialSum:
    """A result [n, width] that is given as `parts` [S, n, width] float32 and is their sum over S: what a
    product leaves whose k was cut into S parts for an even load (`linear(..., parts_ok=True)`).  `rmsnorm`
    and `residual_add` take it as `delta` and `swiglu` as its input and add the parts, in order, as they
    read them; `tensor()` adds them up for any other reader."""

    def __init__(self, parts: torch.Tensor):
        self.parts = parts

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def device(self):
        return self.parts.device

    def tensor(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        out = torch.zeros(tuple(self.shape), dtype=torch.float32, device=self.device)
        residual_add(out, self)
        return out if dtype == torch.float32 else out.to(dtype)


_fn_cache: dict[tuple[str, str], object] = {}
launch_count = 0     # kernels of this package launched so far (library products are not counted)
_status: dict[int, torch.Tensor] = {}


def _fn(lib: str, name: str, argtypes):
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(_build.load(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    return f


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle: asked for before every launch, so by the short way where torch has one."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str, launches: int = 1) -> None:
    if rc == 0:
        global launch_count
        launch_count += launches
        return
    if rc == 2:
        raise KernelError(f"{what}: these sizes are outside what the kernel handles")
    raise KernelError(f"{what}: the launch failed ({torch.cuda.get_device_name()}; "
                      f"the kernels are built for sm_100a only)")


def _cuda(t: torch.Tensor, name: str, dtype=None, contiguous=True) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _code(t: torch.Tensor, name: str) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def status_word(device=None) -> torch.Tensor:
    """The int32 word (one per device) in which kernels record indices outside their tables."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = w
    return w


_status_ptrs: dict[int, int] = {}


def _status_ptr(device: torch.device) -> int:
    """Address of the status word of a tensor's device (what every launcher is given), without building anything."""
    ptr = _status_ptrs.get(device.index)
    if ptr is None:
        ptr = _status_ptrs[device.index] = status_word(device).data_ptr()
    return ptr


def raise_on_status(value: int) -> None:
    if value:
        msgs = [m for bit, m in STATUS_BITS.items() if value & bit]
        raise KernelError("a kernel met " + "; ".join(msgs) + f" (status {value})")


def clear_status(device=None) -> None:
    """Zeroes the status word and what a kernel that gave up may have left half done: the arrival counters of
    the split decode attention (a block that leaves on a bounded wait never counts itself, so its row's
    counter would stay short of the total for every later launch)."""
    w = status_word(device)
    w.zero_()
    buf = _counters.get(w.device.index)
    if buf is not None:
        buf.zero_()


def check_status(device=None) -> None:
    """Reads the status word (a device synchronisation) and raises if a kernel set it."""
    w = status_word(device)
    v = int(w.item())
    if v:
        clear_status(device)
        raise_on_status(v)


# NVTX ranges around the parts of a step (JAX_VLLM_B200_NVTX=1): a profiler's timeline then shows which kernels belong
# to which layer and part.  Off by default: `trace_range` then returns one shared object that does nothing.
TRACE_RANGES = os.environ.get("JAX_VLLM_B200_NVTX", "0") not in ("", "0")


class _NoRange:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _NvtxRange:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


_NO_RANGE = _NoRange()


def trace_range(name: str):
    """A context manager that brackets what runs inside it with an NVTX range of that name, if ranges are on."""
    return _NvtxRange(name) if TRACE_RANGES else _NO_RANGE


def wait_probe(cycles: int, arrive: bool, device=None) -> tuple:
    """Runs the bounded wait of the TMA and tcgen05 kernels alone (csrc/wait_probe.cu): one barrier that a thread
    arrives on (`arrive`) or that nothing ever arrives on, waited for at most `cycles` clocks.  Returns
    (succeeded, clocks spent).  A wait that ran out leaves its bit in the status word, as in the product kernels:
    `check_status` raises afterwards."""
    word = status_word(device)
    outcome = torch.zeros(2, dtype=torch.int32, device=word.device)
    f = _fn("wait_probe", "jv_wait_probe", [c_longlong, c_int, c_void_p, c_void_p, c_void_p])
    with torch.cuda.device(word.device):
        _check(f(int(cycles), 1 if arrive else 0, word.data_ptr(), outcome.data_ptr(), _stream()), "wait_probe")
    done, spent = outcome.tolist()
    return done == 1, spent


# ------------------------------------------------------------------------ embedding
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[n, :] = table[ids[n], :] as float32."""
    _cuda(table, "table"); _cuda(ids, "ids", torch.int32)
    n, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _cuda(out, "out", torch.float32)
    f = _fn("embed", "jv_embed_gather", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(table.data_ptr(), _code(table, "table"), ids.data_ptr(), out.data_ptr(), n, hidden, vocab,
             _status_ptr(table.device), _stream()), "embed_gather")
    return out


# ----------------------------------------------------------------------------- norm
def rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of rows of the float32 stream `h`, after adding `delta` (if given).

    Without `rows` every row is normalised and, when `delta` is given, `h` is updated
    in place with the sum.  With `rows` (int32) only those rows are produced and `h`
    stays as it is.
    """
    _cuda(h, "h", torch.float32); _cuda(weight, "weight")
    n_total, hidden = h.shape
    if weight.shape != (hidden,):
        raise KernelError(f"norm weight has shape {tuple(weight.shape)}, rows have {hidden} elements")
    delta, n_parts, part_stride = _delta_parts(delta, h)
    if rows is not None:
        _cuda(rows, "rows", torch.int32)
    n_out = n_total if rows is None else rows.numel()
    y = torch.empty((n_out, hidden), dtype=out_dtype, device=h.device)
    f = _fn("norm", "jv_rmsnorm", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                   c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p, c_void_p])
    _check(f(h.data_ptr(), _ptr(delta), 0 if delta is None else _code(delta, "delta"), _ptr(rows),
             weight.data_ptr(), _code(weight, "weight"), y.data_ptr(), _code(y, "out"), n_out, n_total, hidden,
             float(eps), n_parts, part_stride, _status_ptr(h.device), _stream()), "rmsnorm")
    return y


def _delta_parts(delta, h: torch.Tensor):
    """(tensor, parts, elements between parts) for a `delta` that is a tensor, a PartialSum or None."""
    if delta is None:
        return None, 1, 0
    if isinstance(delta, PartialSum):
        parts = _cuda(delta.parts, "delta parts", torch.float32)
        if tuple(parts.shape[1:]) != tuple(h.shape):
            raise KernelError("delta and h differ in shape")
        return parts, parts.shape[0], parts.stride(0)
    _cuda(delta, "delta")
    if delta.shape != h.shape:
        raise KernelError("delta and h differ in shape")
    return delta, 1, 0


def residual_add(h: torch.Tensor, delta) -> torch.Tensor:
    """h += delta (a tensor or a PartialSum), the sum kept in float32."""
    _cuda(h, "h", torch.float32)
    delta, n_parts, part_stride = _delta_parts(delta, h)
    f = _fn("norm", "jv_residual_add", [c_void_p, c_void_p, c_int, c_longlong, c_int, c_longlong, c_void_p])
    _check(f(h.data_ptr(), delta.data_ptr(), _code(delta, "delta"), h.numel(), n_parts, part_stride, _stream()),
           "residual_add")
    return h


# ----------------------------------------------------------------------- activation
def swiglu(gate_up, block: int | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """silu(gate) * up for a packed [n, 2*inter] tensor: blocks of `block` gate columns, each followed
    by the up columns of the same indices (default: all gate columns first).  The input may be a
    PartialSum; the result then has `out_dtype`."""
    n_parts, part_stride = 1, 0
    if isinstance(gate_up, PartialSum):
        if out_dtype is None:
            raise KernelError("swiglu of a PartialSum needs out_dtype")
        gate_up = _cuda(gate_up.parts, "gate_up parts", torch.float32)
        n_parts, part_stride = gate_up.shape[0], gate_up.stride(0)
        n, two_i = gate_up.shape[1:]
        act_dtype = out_dtype
    else:
        _cuda(gate_up, "gate_up")
        n, two_i = gate_up.shape
        act_dtype = gate_up.dtype
    if two_i % 2:
        raise KernelError("packed gate|up needs an even number of columns")
    block = two_i // 2 if block is None else int(block)
    if block < 1 or (two_i // 2) % block:
        raise KernelError(f"gate|up block {block} does not divide {two_i // 2} columns")
    act = torch.empty((n, two_i // 2), dtype=act_dtype, device=gate_up.device)
    f = _fn("activation", "jv_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_void_p])
    _check(f(gate_up.data_ptr(), act.data_ptr(), _code(act, "act"), n, two_i // 2, block, n_parts, part_stride, _stream()),
           "swiglu")
    return act


# --------------------------------------------------------- rope + q/k norm + kv write
def rope_kv(qkv: torch.Tensor, positions: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor,
            inv_freq: torch.Tensor | None, q_norm_w, k_norm_w, eps: float, k_cache, v_cache,
            n_q_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Normalises and rotates the query and key heads of `qkv` in place and writes the new
    keys and values into the paged cache (see csrc/rope_kv.cu).  `inv_freq` None = no
    rotation.  `k_cache`/`v_cache` None = the layer writes no cache (queries only)."""
    _cuda(qkv, "qkv"); _cuda(positions, "positions", torch.int32); _cuda(token_entry, "token_entry", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    n, width = qkv.shape
    heads = n_q_heads + (2 * n_kv_heads if k_cache is not None else 0)
    if width < heads * head_dim:
        raise KernelError(f"qkv has {width} columns, {heads} heads of {head_dim} need {heads * head_dim}")
    rot_dim = 0
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        rot_dim = 2 * inv_freq.numel()
    w_code = 0
    for w, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if w is not None:
            _cuda(w, nm)
            if w.shape != (head_dim,):
                raise KernelError(f"{nm} weight has shape {tuple(w.shape)}, head size is {head_dim}")
            w_code = _code(w, nm)
    if (q_norm_w is not None and k_norm_w is not None) and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("q_norm and k_norm weights differ in dtype")
    page_size = num_pages = 1
    if k_cache is not None:
        _cuda(k_cache, "k_cache", qkv.dtype); _cuda(v_cache, "v_cache", qkv.dtype)
        if k_cache.shape != v_cache.shape or k_cache.shape[2:] != (n_kv_heads, head_dim):
            raise KernelError(f"cache shape {tuple(k_cache.shape)} does not fit {n_kv_heads} kv heads of {head_dim}")
        num_pages, page_size = k_cache.shape[0], k_cache.shape[1]
    f = _fn("rope_kv", "jv_rope_kv", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                      c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(qkv.data_ptr(), _code(qkv, "qkv"), qkv.stride(0), positions.data_ptr(), token_entry.data_ptr(),
             block_table.data_ptr(), block_table.shape[1], _ptr(inv_freq), rot_dim, _ptr(q_norm_w), _ptr(k_norm_w),
             w_code, float(eps), _ptr(k_cache), _ptr(v_cache), n, n_q_heads, n_kv_heads, head_dim, page_size,
             num_pages, _status_ptr(qkv.device), _stream()), "rope_kv")


# ------------------------------------------------------------------------ attention
def attn_simt_tokens_per_tile(n_q_heads: int, n_kv_heads: int) -> int:
    g = n_q_heads // n_kv_heads
    return 16 // min(g, 16)


def attn_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor,
              n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, scale: float,
              split_size: int = 0, n_splits: int = 0) -> None:
    """Paged causal attention on CUDA cores (csrc/attn_simt.cu).  `work` is [n_work, 2] int32
    (entry, first token of the tile); with `n_splits` > 0 the work items are single tokens
    whose keys are split into `n_splits` ranges of `split_size` positions."""
    for t, nm in ((q, "q"), (out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, q.dtype, contiguous=(nm != "q"))
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    part_o = part_ml = None
    if n_splits > 0:
        part_o = torch.empty(n_work * n_q_heads * n_splits * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_work * n_q_heads * n_splits * 2, dtype=torch.float32, device=q.device)
    f = _fn("attn_simt", "jv_attn_simt", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                          c_void_p])
    _check(f(q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), _code(q, "q"), _ptr(part_o), _ptr(part_ml),
             k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(), n_work, n_q_heads, n_kv_heads, head_dim,
             k_cache.shape[1], k_cache.shape[0], int(window), float(scale), int(split_size), int(n_splits),
             _status_ptr(q.device), _stream()), "attn_simt", launches=2 if n_splits > 0 else 1)


MMA_HEAD_DIMS = (16, 32, 64, 128)      # head sizes the tensor-core attention kernels are instantiated for


def attn_mma_supports(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in MMA_HEAD_DIMS


def attn_mma_tokens_per_tile(n_q_heads: int, n_kv_heads: int) -> int:
    g = n_q_heads // n_kv_heads
    return 64 // min(g, 16)


_counters: dict[int, torch.Tensor] = {}
_counters_outgrown: list = []     # smaller buffers that a captured graph may still point at: never freed


def _split_counters(device, n: int) -> torch.Tensor:
    """Zeroed arrival counters for the split decode attention: one buffer per device, kept for
    the life of the process (the kernel leaves the counters zero; launches on one stream follow
    one another, so they can share it)."""
    idx = torch.device(device).index
    idx = torch.cuda.current_device() if idx is None else idx
    buf = _counters.get(idx)
    if buf is None or buf.numel() < n:
        if buf is not None:
            _counters_outgrown.append(buf)
        buf = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _counters[idx] = buf
    return buf


def attn_mma(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor,
             n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, scale: float,
             split_size: int = 0, n_splits: int = 0) -> None:
    """Paged causal attention for bfloat16 on the tensor cores (csrc/attn_mma.cu); arguments as
    for `attn_simt`, with `attn_mma_tokens_per_tile` tokens per prompt tile."""
    for t, nm in ((q, "q"), (out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm != "q"))
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    part_o = part_ml = counters = None
    if n_splits > 0:
        part_o = torch.empty(n_work * n_q_heads * n_splits * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n_work * n_q_heads * n_splits * 2, dtype=torch.float32, device=q.device)
        counters = _split_counters(q.device, n_work * n_kv_heads * (-(-(n_q_heads // n_kv_heads) // 16)))
    f = _fn("attn_mma", "jv_attn_mma", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, out.data_ptr(), out.stride(0), _ptr(part_o), _ptr(part_ml), _ptr(counters),
             k_cache.data_ptr(),
             v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1], cu_seqlens.data_ptr(),
             start_pos.data_ptr(), work.data_ptr(), n_work, n_q_heads, n_kv_heads, head_dim, k_cache.shape[1],
             k_cache.shape[0], int(window), float(scale), int(split_size), int(n_splits),
             _status_ptr(q.device), _stream()), "attn_mma")


def attn_tcgen05_supports(dtype: torch.dtype, head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int,
                          window: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes the case (csrc/attn_tcgen05.cu)."""
    g = n_q_heads // max(n_kv_heads, 1)
    return (dtype == torch.bfloat16 and head_dim == 128 and not window and n_q_heads % n_kv_heads == 0
            and 1 <= g <= 16 and page_size in (8, 16, 32, 64, 128))


def attn_tcgen05_tokens_per_tile(n_q_heads: int, n_kv_heads: int) -> int:
    return 128 // (n_q_heads // n_kv_heads)


def attn_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, work: torch.Tensor,
                 n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float) -> None:
    """Paged causal attention of prompt portions on tcgen05 tensor cores with scores and output in tensor
    memory (csrc/attn_tcgen05.cu); `work` lists 128-row tiles of `attn_tcgen05_tokens_per_tile` tokens."""
    for t, nm in ((q, "q"), (out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm != "q"))
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    f = _fn("attn_tcgen05", "jv_attn_tcgen05", [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_float, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
             block_table.data_ptr(), block_table.shape[1], cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(),
             n_work, n_q_heads, n_kv_heads, head_dim, k_cache.shape[1], k_cache.shape[0], float(scale),
             _status_ptr(q.device), _stream()), "attn_tcgen05")


DECODE_TCGEN05_MAX_REQUESTS = 512


def attn_decode_tcgen05_supports(dtype: torch.dtype, head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int,
                                 window: int, n_requests: int = 1) -> bool:
    """Whether the tcgen05 decode-attention kernel takes the case (csrc/attn_decode_tcgen05.cu)."""
    return (dtype == torch.bfloat16 and head_dim == 128 and not window and n_kv_heads > 0
            and n_q_heads % n_kv_heads == 0 and n_q_heads // n_kv_heads <= 16
            and n_requests <= DECODE_TCGEN05_MAX_REQUESTS and page_size in (8, 16, 32, 64, 128))


_sm_count: dict = {}


def multiprocessors(device) -> int:
    """Multiprocessors of the device (what dispatch rules are scaled by)."""
    return _multiprocessors(device)


def _multiprocessors(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def attn_decode_tcgen05(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        block_table: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor,
                        work: torch.Tensor, n_work: int, n_q_heads: int, n_kv_heads: int, head_dim: int,
                        scale: float, prepare: tuple | None = None) -> None:
    """Decode attention (single tokens) with the keys of a tile as tensor-core rows and scores and output in
    tensor memory; one persistent launch shares the key tiles of all requests evenly among the
    multiprocessors (csrc/attn_decode_tcgen05.cu).  `work`, `cu_seqlens`, `start_pos` as for `attn_mma`.

    `prepare` = (inv_freq or None, q_norm_weight or None, k_norm_weight or None, eps): `q` is then the product
    q|k|v as it comes, and the kernel does what `rope_kv` does for these tokens itself (per-head norm,
    rotation at position start_pos, write of the new key and value into the caches)."""
    for t, nm in ((q, "q"), (out, "out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _cuda(t, nm, torch.bfloat16, contiguous=(nm != "q"))
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (work, "work")):
        _cuda(t, nm, torch.int32)
    if n_work == 0:
        return
    inv_freq = q_w = k_w = None
    eps, w_f32 = 0.0, 0
    if prepare is not None:
        inv_freq, q_w, k_w, eps = prepare
        if inv_freq is not None:
            _cuda(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() != head_dim // 2:
                raise KernelError("the kernel rotates whole heads only")
        if (q_w is None) != (k_w is None):
            raise KernelError("norm weights for queries and keys come together")
        if q_w is not None:
            _cuda(q_w, "q_norm_weight"); _cuda(k_w, "k_norm_weight")
            if q_w.dtype != k_w.dtype or q_w.numel() != head_dim or k_w.numel() != head_dim:
                raise KernelError("norm weights must have one dtype and head_dim elements")
            w_f32 = 1 if q_w.dtype == torch.float32 else 0
            _code(q_w, "q_norm_weight")
    n_blocks = _multiprocessors(q.device)
    slots = n_work * n_kv_heads + n_blocks
    g = n_q_heads // max(n_kv_heads, 1)
    part_o = torch.empty(slots * g * head_dim, dtype=torch.float32, device=q.device)
    part_ml = torch.empty(slots * g * 2, dtype=torch.float32, device=q.device)
    counters = _split_counters(q.device, n_work * n_kv_heads)
    f = _fn("attn_decode_tcgen05", "jv_attn_decode_tcgen05",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
             c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p])
    _check(f(q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), out.stride(0), part_o.data_ptr(), part_ml.data_ptr(),
             counters.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             cu_seqlens.data_ptr(), start_pos.data_ptr(), work.data_ptr(), n_work, n_q_heads, n_kv_heads, head_dim,
             k_cache.shape[1], k_cache.shape[0], float(scale), n_blocks, 0 if prepare is None else 1, _ptr(inv_freq),
             _ptr(q_w), _ptr(k_w), w_f32, float(eps), _status_ptr(q.device), _stream()),
           "attn_decode_tcgen05")


# --------------------------------------------------------------------------- linear
def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed, accumulated in float32 on CUDA cores."""
    _cuda(x, "x", contiguous=False); _cuda(weight, "weight")
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1:
        raise KernelError(f"gemm shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    f = _fn("gemm_simt", "jv_gemm_tn_simt", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                             c_int, c_int, c_int, c_void_p])
    _check(f(x.data_ptr(), _code(x, "x"), x.stride(0), weight.data_ptr(), _code(weight, "weight"), weight.stride(0),
             y.data_ptr(), _code(y, "out"), y.stride(0), m, n, k, _stream()), "gemm_simt")
    return y


SKINNY_MAX_ROWS = 16      # rows the mma.sync kernel takes (in a replayed decode step it beats the library up to there)


_skinny_plans: dict = {}      # (device, N, K) -> parts of k per strip


def linear_skinny_splits(device, n: int, k: int) -> int:
    """Into how many parts of k the kernel would best cut the strips of an [n, k] weight on this device
    (1: not at all): few strips, or strips that load the multiprocessors unevenly, are cut."""
    key = ((device.index if isinstance(device, torch.device) else torch.device(device).index) or 0, n, k)
    plan = _skinny_plans.get(key)
    if plan is None:
        f = _build.load("linear_skinny").jv_linear_skinny_plan
        f.argtypes = [c_int, c_int]
        f.restype = c_int
        with torch.cuda.device(key[0]):
            plan = _skinny_plans[key] = int(f(n, k))
    return plan


# Where the caller wants one tensor, the kernel's strips are not cut, and a number of strips just above a multiple of
# the resident blocks leaves most of them idle for a second round: below this evenness (the useful share of the busiest
# block's time, csrc/linear_skinny.cu) the library's product is taken instead.  7,168 x 5,120 (448 strips for 444
# blocks): 0.50 and 20.4 against 14.1 us; 6,144 x 4,096: 1; 10,240 x 5,120: 0.72 and 22.6 against 21.8 us alone,
# where starting under the kernel before still favours the kernel.
SKINNY_MIN_EVENNESS = 0.6
_skinny_fill: dict = {}


def linear_skinny_evenness(device, n: int) -> float:
    """How evenly the uncut 16-row strips of a weight of n rows fill the rounds of this device's resident blocks
    (1: every strip has a block of its own, or the rounds are full)."""
    key = ((device.index if isinstance(device, torch.device) else torch.device(device).index) or 0, n)
    fill = _skinny_fill.get(key)
    if fill is None:
        f = _build.load("linear_skinny").jv_linear_skinny_fill
        f.argtypes, f.restype = [c_int], c_int
        with torch.cuda.device(key[0]):
            fill = _skinny_fill[key] = f(n) / 1000.0
    return fill


def linear_skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, parts_ok: bool = False):
    """x [M <= 16, K] times weight [N, K] transposed, bfloat16 operands, 32-bit accumulation
    (csrc/linear_skinny.cu); the result is bfloat16 or float32, or with `parts_ok`, where the kernel cuts k
    for an even load, a PartialSum for a reader that adds the parts."""
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16, contiguous=False)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"linear shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    splits = linear_skinny_splits(x.device, n, k) if parts_ok else 1
    if splits > 1:
        parts = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
        y = None
    else:
        parts = None
        y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    f = _fn("linear_skinny", "jv_linear_skinny", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                  c_int, c_void_p, c_int, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(y), DTYPE_CODE[out_dtype],
             n if y is None else y.stride(0), m, n, k, _ptr(parts), splits, _stream()), "linear_skinny")
    return y if parts is None else PartialSum(parts)


STREAM_MAX_ROWS = 128
# up to this many rows the dispatcher takes the tcgen05 product of this package, beyond that the library's (which
# shares x between two multiprocessors)
STREAM_BEST_ROWS = 64
_stream_plans: dict = {}


def linear_stream_splits(device, n: int, k: int) -> int:
    """Into how many parts of k the product for 17 to 128 rows (csrc/linear_stream.cu) would best cut the
    128-row strips of an [n, k] weight on this device (1: not at all)."""
    key = ((device.index if isinstance(device, torch.device) else torch.device(device).index) or 0, n, k)
    plan = _stream_plans.get(key)
    if plan is None:
        f = _build.load("linear_stream").jv_linear_stream_plan
        f.argtypes = [c_int, c_int]
        f.restype = c_int
        with torch.cuda.device(key[0]):
            plan = _stream_plans[key] = int(f(n, k))
    return plan


def linear_stream(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, parts_ok: bool = False):
    """x [M <= 128, K] times weight [N, K] transposed on tcgen05 with the weight as the 128-row operand and the
    batch as the narrow one (csrc/linear_stream.cu): bfloat16 operands, 32-bit accumulation; the result is
    bfloat16 or float32, or with `parts_ok`, where the kernel cuts k for an even load, a PartialSum."""
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16, contiguous=False)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"linear shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    splits = linear_stream_splits(x.device, n, k) if parts_ok else 1
    if splits > 1:
        parts = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
        y = None
    else:
        parts = None
        y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    f = _fn("linear_stream", "jv_linear_stream", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                  c_int, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(y), DTYPE_CODE[out_dtype],
             n if y is None else y.stride(0), m, n, k, _ptr(parts), splits, _status_ptr(x.device), _stream()),
           "linear_stream")
    return y if parts is None else PartialSum(parts)


def _stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dim() == 2 and 0 < x.shape[0] <= STREAM_MAX_ROWS and x.stride(1) == 1 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and x.dtype == torch.bfloat16)


GEMM_EPILOGUES = {"bf16": 0, "f32": 1, "swiglu": 2}


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, epilogue: str = "bf16") -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed on tcgen05 tensor cores with the accumulator in
    tensor memory (csrc/gemm_tcgen05.cu).  epilogue "bf16" / "f32": the product in that type;
    "swiglu": silu(gate) * up as [M, N/2] bfloat16, for a weight whose every 256 rows are 128 gate rows
    followed by the 128 up rows of the same indices."""
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16, contiguous=False)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.stride(1) != 1 or weight.stride(1) != 1:
        raise KernelError(f"gemm shapes {tuple(x.shape)} x {tuple(weight.shape)}^T do not fit")
    m, k = x.shape
    n = weight.shape[0]
    code = GEMM_EPILOGUES[epilogue]
    if epilogue == "swiglu":
        y = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
    else:
        y = torch.empty((m, n), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=x.device)
    f = _fn("gemm_tcgen05", "jv_gemm_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_void_p, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), y.data_ptr(), y.stride(0), m, n, k, code,
             _status_ptr(x.device), _stream()), "gemm_tcgen05")
    return y


_sm_counts: dict = {}


_strips_fill: dict = {}


def _strips_fill_the_device(device, n: int) -> bool:
    """Whether the 128-row strips of a weight of n rows, uncut, keep the multiprocessors busy (0.85 of them over
    the rounds it takes): the tcgen05 product for larger batches takes a weight whole only then."""
    idx = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    fills = _strips_fill.get((idx, n))
    if fills is None:
        sms = _sm_counts.get(idx)
        if sms is None:
            sms = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
        strips = -(-n // 128)
        fills = _strips_fill[(idx, n)] = strips >= 0.85 * sms * -(-strips // sms)
    return fills


def _skinny_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.shape[0] <= SKINNY_MAX_ROWS and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and x.stride(1) == 1)


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None, parts_ok: bool = False):
    """y = x @ weight.T.  With `parts_ok` the result may be a PartialSum (the caller hands it to `rmsnorm`,
    `residual_add` or `swiglu`, which add its parts as they read them).

    float32 weights: the CUDA-core product of this package in true 32-bit (16-bit activations are read as they
    are and widened inside).  bfloat16 weights and activations: up to STREAM_BEST_ROWS rows (decoding) the
    weight-streaming product on tcgen05 (csrc/linear_stream.cu), which cuts the k of a weight with few strips into
    parts; where the reader wants one tensor and the strips are few, the mma.sync product (csrc/linear_skinny.cu, up
    to SKINNY_MAX_ROWS rows), whose strips are 16 rows; else (prompts) cuBLAS through torch.mm.  All
    accumulate in 32-bit and give the result in `out_dtype` (bfloat16 by default, float32 for logits)."""
    out_dtype = out_dtype or x.dtype
    if weight.dtype == torch.float32 or x.dtype == torch.float32:
        return gemm_simt(x, weight, out_dtype)
    _cuda(x, "x", torch.bfloat16, contiguous=False); _cuda(weight, "weight", torch.bfloat16)
    if _stream_ok(x, weight) and x.shape[0] <= STREAM_BEST_ROWS and out_dtype in (torch.bfloat16, torch.float32) and \
            (parts_ok or _strips_fill_the_device(x.device, weight.shape[0])):
        return linear_stream(x, weight, out_dtype, parts_ok)
    if _skinny_ok(x, weight) and (parts_ok or linear_skinny_evenness(x.device, weight.shape[0]) >= SKINNY_MIN_EVENNESS):
        return linear_skinny(x, weight, out_dtype, parts_ok)
    if out_dtype == torch.bfloat16:
        return torch.mm(x, weight.t())
    return torch.mm(x, weight.t(), out_dtype=out_dtype)


# ------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor) -> torch.Tensor:
    """One token per row of float32 logits: argmax where temperature is 0, else a draw from
    softmax(logits / temperature) that depends on (seed, counter) of the row only."""
    _cuda(logits, "logits", torch.float32); _cuda(temperature, "temperature", torch.float32)
    _cuda(seeds, "seeds", torch.int64); _cuda(counters, "counters", torch.int64)
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    chunks = min(128, max(1, -(-vocab // 2048)))
    part_v = torch.empty(rows * chunks, dtype=torch.float32, device=logits.device)
    part_i = torch.empty(rows * chunks, dtype=torch.int32, device=logits.device)
    f = _fn("sampling", "jv_sample", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p])
    _check(f(logits.data_ptr(), rows, vocab, temperature.data_ptr(), seeds.data_ptr(), counters.data_ptr(),
             part_v.data_ptr(), part_i.data_ptr(), out.data_ptr(), _stream()), "sample", launches=2)
    return out
