"""Python face of the hand-written sm_100a kernels.

Each function checks its tensors (device, type, layout, sizes), passes raw
pointers and the current CUDA stream to the C entry point of the same name and
raises :class:`KernelError` with the library's message when the entry point
refuses. There is no fallback: without a CUDA device or without the compiled
library every call raises.
"""

from __future__ import annotations

import ctypes as C
import threading

import torch

from ..errors import KernelError

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BAD_TOKEN = 1
STATUS_BAD_PAGE = 2
STATUS_NON_FINITE = 4
STATUS_WAIT_TIMEOUT = 8
STATUS_BAD_RANGE = 16

ABI_VERSION = 13


def status_names(code: int) -> list:
    """What the bits of a device status word mean."""
    return [name for bit, name in ((STATUS_BAD_TOKEN, "a token id outside the vocabulary"),
                                   (STATUS_BAD_PAGE, "a position without a cache page"),
                                   (STATUS_NON_FINITE, "non-finite logits"),
                                   (STATUS_WAIT_TIMEOUT, "a bounded wait inside a kernel ran out"),
                                   (STATUS_BAD_RANGE, "a position beyond the rotation table or the key ranges of a launch")) if code & bit]

_lib = None
_lib_lock = threading.Lock()


def library() -> C.CDLL:
    """The compiled kernel library; built at the first call if needed."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        if not torch.cuda.is_available():
            raise KernelError(
                "no CUDA device is visible: the engine runs only on the GPU (there is no CPU path)"
            )
        from ..csrc.build import library_path

        try:
            path = library_path()
        except Exception as exc:  # the build failed or nvcc is missing
            raise KernelError(f"the sm_100a kernel library could not be built: {exc}") from exc
        lib = C.CDLL(str(path))
        lib.qi_last_error.restype = C.c_char_p
        lib.qi_abi_version.restype = C.c_int
        if lib.qi_abi_version() != ABI_VERSION:
            raise KernelError(
                f"{path} has ABI version {lib.qi_abi_version()}, expected {ABI_VERSION}; rebuild it"
            )
        _lib = lib
    return _lib


def library_file() -> str:
    return library()._name


def _stream() -> C.c_void_p:
    """The current CUDA stream of the current device, as the raw handle the entry points take. (Through
    torch's C binding: `torch.cuda.current_stream()` builds a Python object and costs about as much as
    a whole launch; a step of a few hundred launches asks this a few hundred times.)"""
    return C.c_void_p(_raw_stream(_current_device()))


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream
    _current_device = torch._C._cuda_getDevice
except AttributeError:      # another torch: the public, slower way
    def _raw_stream(index):
        return torch.cuda.current_stream(index).cuda_stream

    _current_device = torch.cuda.current_device


launches = 0   # entry points called so far (each launches at least one kernel)


def _check(rc: int, name: str) -> None:
    global launches
    launches += 1
    if rc != 0:
        raise KernelError(f"{name}: {library().qi_last_error().decode()}")


knock_out = frozenset()   # kernel classes ("gemm", "attention", "norm", "rope", "scan", "other") whose launches are left out


def _call(cls, name: str, fn, *args) -> None:
    """Calls an entry point and raises with the library's message if it refuses. A class named in
    `knock_out` is not launched at all: a measurement leaves one class out at a time and times the
    rest of the step (the results of such a step mean nothing)."""
    if cls is not None and cls in knock_out:
        return
    _check(fn(*args), name)


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _req(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")


def _req_state(t: torch.Tensor, name: str, dtype) -> None:
    """State of fixed size [slots, ...]: the slots may lie apart (rows of the cache manager's state memory), what
    a slot holds must be contiguous."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != dtype or t.dim() < 2:
        raise KernelError(f"{name} must be a CUDA tensor of {dtype} with a slot dimension")
    if not t[0].is_contiguous() or t.stride(0) < t[0].numel():
        raise KernelError(f"{name}: what a slot holds must be contiguous and the slots must not overlap")


def _ptr(t) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


# --------------------------------------------------------------------------
# embedding


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = table[ids[t], :] * scale as float32. ids int32 [n]; out float32 [n, hidden]."""
    _req(table, "table", ndim=2)
    _req(ids, "ids", torch.int32, 1)
    _req(out, "out", torch.float32, 2)
    _req(status, "status", torch.int32)
    n, hidden = out.shape
    if ids.numel() != n or table.shape[1] != hidden:
        raise KernelError(f"embedding: shapes do not agree: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    _call('other', "embedding", library().qi_embedding_scaled,
          _ptr(table), _code(table), _ptr(ids), _ptr(out), n, hidden,
                                table.shape[0], C.c_float(scale), _ptr(status), _stream())


# --------------------------------------------------------------------------
# norms


def add_rmsnorm(resid: torch.Tensor, delta, gain: torch.Tensor, eps: float, out: torch.Tensor,
                rows=None, write_resid: bool = True) -> None:
    """Fused residual add and RMSNorm.

    resid float32 [n, h] (updated in place when write_resid); delta None, [n, h]
    or [splits, n, h] (partial sums added in order); gain float32 [h]; out
    [n, h], or [len(rows), h] when `rows` (int32) selects source rows.
    """
    _req(resid, "resid", torch.float32, 2)
    _req(gain, "gain", torch.float32, 1)
    _req(out, "out", ndim=2)
    n, h = resid.shape
    splits, stride = 1, 0
    if delta is not None:
        _req(delta, "delta")
        if delta.dim() == 3:
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
            if tuple(delta.shape[1:]) != (n, h):
                raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} does not match resid {tuple(resid.shape)}")
        elif tuple(delta.shape) != (n, h):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} does not match resid {tuple(resid.shape)}")
    if gain.numel() != h:
        raise KernelError(f"add_rmsnorm: gain has {gain.numel()} elements, rows have {h}")
    n_out = n
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
        n_out = rows.numel()
        write_resid = False
    if tuple(out.shape) != (n_out, h):
        raise KernelError(f"add_rmsnorm: out is {tuple(out.shape)}, expected {(n_out, h)}")
    _call('norm', "add_rmsnorm", library().qi_add_rmsnorm,
          _ptr(resid), _ptr(delta), _code(delta) if delta is not None else F32, splits,
        C.c_longlong(stride), _ptr(gain), C.c_float(eps), _ptr(out), _code(out), _ptr(rows), n_out, h,
        int(bool(write_resid)), _stream())


def add_layernorm(resid: torch.Tensor, delta, gain: torch.Tensor, bias, eps: float, out: torch.Tensor,
                  rows=None, write_resid: bool = True) -> None:
    """Fused residual add and layer norm: x = resid + delta; out = (x - mean) / sqrt(var + eps) * gain + bias, var the
    mean squared deviation. Arguments as for `add_rmsnorm`; bias float32 [h] or None; out float32 or the activation type."""
    _req(resid, "resid", torch.float32, 2)
    _req(gain, "gain", torch.float32, 1)
    _req(out, "out", ndim=2)
    n, h = resid.shape
    splits, stride = 1, 0
    if delta is not None:
        _req(delta, "delta")
        if delta.dim() == 3:
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        if tuple(delta.shape[-2:]) != (n, h):
            raise KernelError(f"add_layernorm: delta {tuple(delta.shape)} does not match resid {tuple(resid.shape)}")
    if bias is not None:
        _req(bias, "bias", torch.float32, 1)
    if gain.numel() != h or (bias is not None and bias.numel() != h):
        raise KernelError(f"add_layernorm: gain and bias must have {h} elements")
    n_out = n
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
        n_out = rows.numel()
        write_resid = False
    if tuple(out.shape) != (n_out, h):
        raise KernelError(f"add_layernorm: out is {tuple(out.shape)}, expected {(n_out, h)}")
    _call('norm', "add_layernorm", library().qi_add_layernorm,
          _ptr(resid), _ptr(delta), _code(delta) if delta is not None else F32, splits, C.c_longlong(stride), _ptr(gain),
          _ptr(bias), C.c_float(eps), _ptr(out), _code(out), _ptr(rows), n_out, h, int(bool(write_resid)), _stream())


def scale_add_rmsnorm(resid: torch.Tensor, delta, alpha: float, gain: torch.Tensor, eps: float, copy=None) -> None:
    """The norm that comes after the sum: resid = rmsnorm(alpha * resid + delta) * gain, in place and in 32-bit; `copy`
    (or None) receives the new rows in its own type. resid float32 [n, h]; delta None, [n, h] or [splits, n, h] (partial
    sums added in order); gain float32 [h]."""
    _req(resid, "resid", torch.float32, 2)
    _req(gain, "gain", torch.float32, 1)
    n, h = resid.shape
    splits, stride = 1, 0
    if delta is not None:
        _req(delta, "delta")
        if delta.dim() == 3:
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        if tuple(delta.shape[-2:]) != (n, h) or delta.dim() not in (2, 3):
            raise KernelError(f"scale_add_rmsnorm: delta {tuple(delta.shape)} does not match resid {tuple(resid.shape)}")
    if gain.numel() != h:
        raise KernelError(f"scale_add_rmsnorm: gain has {gain.numel()} elements, rows have {h}")
    if copy is not None:
        _req(copy, "copy", ndim=2)
        if tuple(copy.shape) != (n, h):
            raise KernelError(f"scale_add_rmsnorm: copy is {tuple(copy.shape)}, expected {(n, h)}")
    _call("norm", "scale_add_rmsnorm", library().qi_scale_add_rmsnorm, _ptr(resid), _ptr(delta),
          _code(delta) if delta is not None else F32, splits, C.c_longlong(stride), C.c_float(alpha), _ptr(gain), C.c_float(eps),
          _ptr(copy), _code(copy) if copy is not None else F32, n, h, _stream())


def normed_sum(a, b, gain_a, gain_b, eps: float, scale: float, out) -> None:
    """out = scale * (rmsnorm(a) * gain_a + rmsnorm(b) * gain_b), each norm over a row, 32-bit; out float32 [n, h]. a and
    b are [n, h] each, or [parts, n, h]: the partial sums of a split product, added here in order. Types may differ."""
    _req(a, "a")
    _req(b, "b")
    _req(out, "out", torch.float32, 2)
    _req(gain_a, "gain_a", torch.float32, 1)
    _req(gain_b, "gain_b", torch.float32, 1)
    n, h = out.shape
    for t in (a, b):
        if t.dim() not in (2, 3) or tuple(t.shape[-2:]) != (n, h) or not t.shape[0]:
            raise KernelError("normed_sum: shapes differ")
    if gain_a.numel() != h or gain_b.numel() != h:
        raise KernelError("normed_sum: the gains do not fit the rows")
    _call("norm", "normed_sum", library().qi_normed_sum, _ptr(a), a.shape[0] if a.dim() == 3 else 1, _code(a), _ptr(b),
          b.shape[0] if b.dim() == 3 else 1, _code(b), _ptr(gain_a), _ptr(gain_b), C.c_float(eps), C.c_float(scale), _ptr(out), n, h,
          _stream())


def convert(x, out) -> None:
    """out = x in out's type; x float32, same shape."""
    _req(x, "x", torch.float32)
    _req(out, "out")
    if out.shape != x.shape:
        raise KernelError("convert: shapes differ")
    _call("other", "convert", library().qi_convert, _ptr(x), _ptr(out), _code(out), C.c_longlong(x.numel()), _stream())


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = rmsnorm(x) * gain over the last dimension; x and out of one type."""
    _req(x, "x")
    _req(out, "out", x.dtype)
    _req(gain, "gain", torch.float32, 1)
    width = x.shape[-1]
    if gain.numel() != width or out.shape != x.shape:
        raise KernelError("rmsnorm: shapes do not agree")
    _call('norm', "rmsnorm", library().qi_rmsnorm,
          _ptr(x), _ptr(gain), C.c_float(eps), _ptr(out), _code(x),
                              x.numel() // width, width, _stream())


# --------------------------------------------------------------------------
# matrix products


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T with 32-bit products and sums (no tensor cores)."""
    _req(x, "x", ndim=2)
    _req(w, "w", ndim=2)
    _req(out, "out", ndim=2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _call('gemm', "gemm_simt", library().qi_gemm_simt,
          _ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), M, N, K,
                                C.c_longlong(K), C.c_longlong(K), C.c_longlong(N), _stream())


# --------------------------------------------------------------------------
# position encoding, q/k norm, cache write


def rope_table(inv_freq: torch.Tensor, max_positions: int):
    """cos and sin tables [max_positions, len(inv_freq)] in float32 from 32-bit angles."""
    _req(inv_freq, "inv_freq", torch.float32, 1)
    half = inv_freq.numel()
    cos = torch.empty((max_positions, half), dtype=torch.float32, device=inv_freq.device)
    sin = torch.empty_like(cos)
    _call(None, "rope_table", library().qi_rope_table,
          _ptr(inv_freq), _ptr(cos), _ptr(sin), max_positions, half, _stream())
    return cos, sin


def qk_norm_rope_kv(qkv, q_out, q_gain, k_gain, eps, cos, sin, rotary_dim, positions, token_req,
                    block_table, page_size, k_pages, v_pages, nq, nkv, d, status, interleaved: bool = False) -> None:
    """Per-head q/k RMSNorm, rotation, and the write of k and v into cache pages. Pairs of the
    rotation are (p, p + rotary_dim / 2), or (2p, 2p + 1) when `interleaved`.

    qkv [n, (nq + 2 nkv) d], or float32 [splits, n, (nq + 2 nkv) d] partial sums of a
    K-split projection (added here); q_out [n, nq d]; gains float32 [d] or None; cos/sin
    float32 [positions, rotary_dim / 2] or None; k_pages/v_pages
    [num_pages, nkv, page_size, d] or None (no write); block_table int32
    [requests, max_blocks].
    """
    _req(qkv, "qkv")
    _req(q_out, "q_out", ndim=2)
    splits = 1
    if qkv.dim() == 3:
        splits = qkv.shape[0]
        if qkv.dtype != torch.float32:
            raise KernelError("qk_norm_rope_kv: partial sums must be float32")
    elif qkv.dim() != 2 or qkv.dtype != q_out.dtype:
        raise KernelError(f"qk_norm_rope_kv: qkv {tuple(qkv.shape)} {qkv.dtype} does not fit q_out {q_out.dtype}")
    n = qkv.shape[-2]
    if qkv.shape[-1] != (nq + 2 * nkv) * d or tuple(q_out.shape) != (n, nq * d):
        raise KernelError(f"qk_norm_rope_kv: qkv {tuple(qkv.shape)} / q_out {tuple(q_out.shape)} do not match heads {nq}+2*{nkv} of {d}")
    for g, name in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _req(g, name, torch.float32, 1)
            if g.numel() != d:
                raise KernelError(f"{name} has {g.numel()} elements, head_dim is {d}")
    table_positions = 0
    if cos is not None:
        _req(cos, "cos", torch.float32, 2)
        _req(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != rotary_dim:
            raise KernelError("qk_norm_rope_kv: rotation tables do not match rotary_dim")
        table_positions = cos.shape[0]
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    num_pages, max_blocks = 0, 0
    if k_pages is not None:
        _req(k_pages, "k_pages", q_out.dtype, 4)
        _req(v_pages, "v_pages", q_out.dtype, 4)
        _req(block_table, "block_table", torch.int32, 2)
        if tuple(k_pages.shape[1:]) != (nkv, page_size, d) or k_pages.shape != v_pages.shape:
            raise KernelError(f"qk_norm_rope_kv: pages {tuple(k_pages.shape)} do not match (pages, {nkv}, {page_size}, {d})")
        num_pages, max_blocks = k_pages.shape[0], block_table.shape[1]
    _call('rope', "qk_norm_rope_kv", library().qi_qk_norm_rope_kv,
          _ptr(qkv), splits, _ptr(q_out), _code(q_out), _ptr(q_gain), _ptr(k_gain), C.c_float(eps), _ptr(cos),
        _ptr(sin), rotary_dim, int(bool(interleaved)), table_positions, _ptr(positions), _ptr(token_req), _ptr(block_table),
        max_blocks, page_size, num_pages, _ptr(k_pages), _ptr(v_pages), n, nq, nkv, d, _ptr(status),
        _stream())


# --------------------------------------------------------------------------
# attention


def attention_generic(q, out, k_pages, v_pages, block_table, positions, token_req, nq, nkv, d,
                      scale: float, window: int, status, chunk: int = 0, gate=None, softcap: float = 0.0,
                      out_scale: float = 1.0, sink=None) -> None:
    """Causal paged GQA attention, 32-bit arithmetic, any span length and page size. `sink` (float32 [nq] or None): the
    softmax's denominator of head h holds exp(sink[h]) once more, with no key and no value. Values may have another
    size than keys (v_pages [pages, nkv, page_size, dv], out [n, nq dv]); `chunk` > 0: a query sees only the keys
    of its own chunk of that many positions (counted from the sequence's start); `gate` [n, >= nq dv] (a view whose
    rows may lie further apart): the result is multiplied by sigmoid(gate). `softcap` c > 0: a score s becomes
    c tanh(s / c) before the softmax. `out_scale` multiplies the result."""
    _req(q, "q", ndim=2)
    _req(out, "out", q.dtype, 2)
    _req(k_pages, "k_pages", q.dtype, 4)
    _req(v_pages, "v_pages", q.dtype, 4)
    _req(block_table, "block_table", torch.int32, 2)
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    n = q.shape[0]
    dv = v_pages.shape[3]
    if q.shape[1] != nq * d or tuple(out.shape) != (n, nq * dv):
        raise KernelError(f"attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not match {nq} heads of {d} / {dv}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape[:3] != v_pages.shape[:3]:
        raise KernelError(f"attention: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} do not match {nkv} kv heads of {d}")
    ldg = 0
    if gate is not None:
        if not gate.is_cuda or gate.dtype != q.dtype or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != out.shape:
            raise KernelError("attention: the gate must be [n, nq dv] in q's type with contiguous rows")
        ldg = gate.stride(0)
    if sink is not None:
        _req(sink, "sink", torch.float32, 1)
        if sink.numel() != nq:
            raise KernelError("attention: one sink a query head")
    _call('attention', "attention_generic", library().qi_attention_generic_sink,
          _ptr(q), _ptr(out), _code(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        block_table.shape[1], k_pages.shape[2], k_pages.shape[0], _ptr(positions), _ptr(token_req), n,
        nq, nkv, d, dv, C.c_float(scale), C.c_float(softcap or 0.0), C.c_float(out_scale), int(window or 0), int(chunk or 0), _ptr(gate), C.c_longlong(ldg), _ptr(sink), _ptr(status), _stream())


def attention_mma_supported(nq: int, nkv: int, d: int) -> bool:
    """Whether the tensor-core attention kernels take this geometry (bfloat16 only)."""
    return bool(library().qi_attention_mma_supported(nq, nkv, d))


QUERY_TILE = 128   # query rows per entry of a batch's tile lists


def attention_tma_supported(nq: int, nkv: int, d: int, page_size: int, max_blocks: int = 1) -> bool:
    """Whether the TMA-fed attention kernels take this geometry (bfloat16 only)."""
    return bool(library().qi_attention_tma_supported(nq, nkv, d, page_size, max_blocks))


def attention_prefill_tcgen05_supported(nq: int, nkv: int, d: int, page_size: int, max_blocks: int = 1) -> bool:
    """Whether the tcgen05 prefill attention takes this geometry (bfloat16, head size 128)."""
    return bool(library().qi_attention_prefill_tcgen05_supported(nq, nkv, d, page_size, max_blocks))


def attention_prefill_ranges(n_ctas: int, max_kv_len: int) -> int:
    """Into how many key ranges the tcgen05 prefill attention cuts every query tile, given the CTAs
    it would launch uncut (heads x query tiles) and the longest context of the step. 296 CTAs are
    resident at once; cutting makes more and shorter ones, which fills the GPU when a step has few
    query tiles (a portion of 512 tokens of 32 heads is 128 CTAs: after 30,000 tokens 402 us uncut,
    268 in two ranges), and costs the partial results' trip through memory and a merge kernel, so
    it does not pay where the uncut launch already fills its rounds (2,048 tokens after 30,000:
    1,007 us uncut, 1,120 in four ranges). Estimated times, fitted to measurements at the 8B sizes
    (microseconds): rounds x keys of a CTA x 0.0154 (0.0132 while every CTA has an SM to itself),
    plus 0.0009 for every (query row, head, range) when cut."""
    best, best_time = 1, None
    for ranges in (1, 2, 3, 4, 6, 8):
        if ranges > 1 and max_kv_len < 2048 * ranges:
            break
        units = n_ctas * ranges
        rounds = -(-units // 296)
        time = rounds * (max_kv_len / ranges) * (0.0132 if units <= 148 else 0.0154)
        if ranges > 1:
            time += n_ctas * 128 * ranges * 0.0009
        if best_time is None or time < best_time * 0.97:
            best, best_time = ranges, time
    return best


def attention_prefill(q, out, k_pages, v_pages, block_table, q_start, start_pos, tile_req, tile_q0,
                      nq, nkv, d, scale: float, window: int, status, use_tma: bool | None = None,
                      impl: str | None = None, max_kv_len: int = 0, key_ranges: int | None = None, chunk: int = 0,
                      gate=None, softcap: float = 0.0, out_scale: float = 1.0, sink=None) -> None:
    """Causal paged GQA flash attention (bfloat16, head size 64 or 128) for spans of any
    length. `tile_req[i]`, `tile_q0[i]`: request index and first flat token of the i-th
    block of up to QUERY_TILE query rows.

    Three kernels: "tcgen05" (head size 128, page size a power of two >= 8: tcgen05.mma with
    accumulators in tensor memory, TMA loads), "tma" (mma.sync with TMA loads, same page
    sizes, head size 64 or 128) and "cpasync" (mma.sync, any page size). `impl` forces one;
    the default is the first that takes the geometry. `use_tma` is the older switch between
    the last two. `max_kv_len` (the longest context of the step) lets the tcgen05 kernel cut long
    contexts into key ranges over more CTAs (`key_ranges` forces a number). The tcgen05 kernel alone takes
    `chunk` (a query sees only the keys of its own chunk of that many positions, counted from the sequence's
    start), `gate` (bfloat16 [n, nq d], rows a multiple of 8 elements apart and 16-byte aligned: the output is
    multiplied with its sigmoid), `softcap` c > 0 (a score s becomes c tanh(s / c)), `out_scale` (a factor on the
    result) and `sink` (float32 [nq]: exp(sink[h]) once more in the softmax's denominator of head h)."""
    if impl is None and use_tma is not None:
        impl = "tma" if use_tma else "cpasync"
    _req(q, "q", torch.bfloat16, 2)
    _req(out, "out", torch.bfloat16, 2)
    _req(k_pages, "k_pages", torch.bfloat16, 4)
    _req(v_pages, "v_pages", torch.bfloat16, 4)
    for t, name in ((block_table, "block_table"), (q_start, "q_start"), (start_pos, "start_pos"),
                    (tile_req, "tile_req"), (tile_q0, "tile_q0")):
        _req(t, name, torch.int32)
    if q.shape[1] != nq * d or out.shape != q.shape:
        raise KernelError(f"attention_prefill: q {tuple(q.shape)} does not match {nq} heads of {d}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape != v_pages.shape:
        raise KernelError(f"attention_prefill: pages {tuple(k_pages.shape)} do not match {nkv} kv heads of {d}")
    if tile_req.numel() != tile_q0.numel():
        raise KernelError("attention_prefill: tile lists differ in length")
    if impl is None:
        if attention_prefill_tcgen05_supported(nq, nkv, d, k_pages.shape[2], block_table.shape[1]):
            impl = "tcgen05"
        elif attention_tma_supported(nq, nkv, d, k_pages.shape[2], block_table.shape[1]):
            impl = "tma"
        else:
            impl = "cpasync"
    if impl == "tcgen05":
        ranges = key_ranges or attention_prefill_ranges(nq * tile_req.numel(), max_kv_len)
        if q.shape[0] > 65535:
            ranges = 1
        ws = torch.empty(q.shape[0] * nq * ranges * (d + 2), dtype=torch.float32, device=q.device) if ranges > 1 else None
        ldg = 0
        if gate is not None:
            if not gate.is_cuda or gate.dtype != torch.bfloat16 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != out.shape:
                raise KernelError("attention_prefill: the gate must be bfloat16 [n, nq d] with contiguous rows")
            ldg = gate.stride(0)
        if sink is not None:
            _req(sink, "sink", torch.float32, 1)
        _call('attention', "attention_prefill_tcgen05", library().qi_attention_prefill_tcgen05_sink,
              _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
            k_pages.shape[2], k_pages.shape[0], _ptr(q_start), _ptr(start_pos), _ptr(tile_req), _ptr(tile_q0),
            tile_req.numel(), q.shape[0], nq, nkv, d, C.c_float(scale), int(window or 0), int(chunk or 0), _ptr(gate),
            C.c_longlong(ldg), ranges, _ptr(ws), _ptr(status), C.c_float(softcap or 0.0), C.c_float(out_scale), _ptr(sink), _stream())
        return
    if chunk or gate is not None or softcap or out_scale != 1.0 or sink is not None:
        raise KernelError(f"attention_prefill: the {impl!r} kernel takes neither a chunk bound, a gate, a soft cap, an output factor nor a sink")
    if impl not in ("tma", "cpasync"):
        raise KernelError(f"attention_prefill: unknown kernel {impl!r}")
    if impl == "tma":
        _call('attention', "attention_prefill_tma", library().qi_attention_prefill_tma,
              _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
            k_pages.shape[2], k_pages.shape[0], _ptr(q_start), _ptr(start_pos), _ptr(tile_req), _ptr(tile_q0),
            tile_req.numel(), q.shape[0], nq, nkv, d, C.c_float(scale), int(window or 0), _ptr(status), _stream())
        return
    _call('attention', "attention_prefill", library().qi_attention_prefill,
          _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
        k_pages.shape[2], k_pages.shape[0], _ptr(q_start), _ptr(start_pos), _ptr(tile_req), _ptr(tile_q0),
        tile_req.numel(), QUERY_TILE, nq, nkv, d, C.c_float(scale), int(window or 0), _ptr(status), _stream())


def attention_decode_plan(batch: int, nkv: int, max_kv_len: int):
    """(keys per CTA, number of key ranges) for a decode batch: as many CTAs as are resident
    at once (two on each of 148 SMs) and no more, so that each requests its first tiles while
    the kernel before it still runs; ranges a multiple of 64 keys, independent of the
    requests' actual lengths."""
    target = max(1, 296 // max(batch * nkv, 1))
    chunk = max(64, -(-(-(-max_kv_len // target)) // 64) * 64)
    return chunk, -(-max_kv_len // chunk)


def attention_decode(q, out, k_pages, v_pages, block_table, kv_len, q_start, nq, nkv, d, scale: float,
                     window: int, chunk: int, n_splits: int, status, workspace=None,
                     use_tma: bool | None = None) -> None:
    """Paged GQA attention for one query token per request (bfloat16, head size 64 or
    128), a request's key tiles dealt out evenly over `n_splits` ranges of at most `chunk` positions
    (`n_splits * chunk` must cover the longest request). `workspace`: float32,
    at least batch * nq * n_splits * (d + 2) elements (allocated when None)."""
    _req(q, "q", torch.bfloat16, 2)
    _req(out, "out", torch.bfloat16, 2)
    _req(k_pages, "k_pages", torch.bfloat16, 4)
    _req(v_pages, "v_pages", torch.bfloat16, 4)
    for t, name in ((block_table, "block_table"), (kv_len, "kv_len"), (q_start, "q_start")):
        _req(t, name, torch.int32)
    batch = kv_len.numel()
    if q.shape[1] != nq * d or out.shape != q.shape or q.shape[0] < batch:
        raise KernelError(f"attention_decode: q {tuple(q.shape)} does not match {batch} requests, {nq} heads of {d}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape != v_pages.shape:
        raise KernelError(f"attention_decode: pages {tuple(k_pages.shape)} do not match {nkv} kv heads of {d}")
    need = batch * nq * n_splits * (d + 2)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.float32, device=q.device)
    _req(workspace, "workspace", torch.float32, 1)
    if workspace.numel() < need:
        raise KernelError(f"attention_decode: workspace has {workspace.numel()} floats, {need} are needed")
    ws_o = workspace
    ws_ml = workspace[batch * nq * n_splits * d:]
    if use_tma is None:
        use_tma = attention_tma_supported(nq, nkv, d, k_pages.shape[2], block_table.shape[1])
    fn = library().qi_attention_decode_tma if use_tma else library().qi_attention_decode
    _call('attention', "attention_decode", fn,
          _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
        k_pages.shape[2], k_pages.shape[0], _ptr(kv_len), _ptr(q_start), batch, nq, nkv, d, C.c_float(scale),
        int(window or 0), chunk, n_splits, _ptr(ws_o), _ptr(ws_ml), _ptr(status), _stream())


def attention_decode_rope(qkv, out, q_gain, k_gain, eps, cos, sin, k_pages, v_pages, writes: bool, block_table, kv_len,
                          q_start, nq, nkv, d, scale: float, window: int, chunk: int, n_splits: int, status,
                          workspace=None) -> None:
    """`qk_norm_rope_kv` and `attention_decode` in one launch, for a decode step: qkv is the
    q/k/v projection's output, bfloat16 [tokens, (nq + 2 nkv) d], or its float32 K-split partial
    sums [splits, tokens, (nq + 2 nkv) d]. The kernel makes each request's queries from it, and
    its new key and value, which it writes to the cache at position kv_len - 1 (`writes` False:
    another layer wrote them). Rotation over the whole head or none (cos None)."""
    _req(qkv, "qkv")
    if qkv.dim() == 3:
        if qkv.dtype != torch.float32:
            raise KernelError("attention_decode_rope: partial sums must be float32")
        splits, n_tokens, width = qkv.shape
    elif qkv.dim() == 2 and qkv.dtype in (torch.bfloat16, torch.float32):
        splits, (n_tokens, width) = 1, qkv.shape
    else:
        raise KernelError(f"attention_decode_rope: qkv {tuple(qkv.shape)} {qkv.dtype} is neither an output nor partial sums")
    _req(out, "out", torch.bfloat16, 2)
    _req(k_pages, "k_pages", torch.bfloat16, 4)
    _req(v_pages, "v_pages", torch.bfloat16, 4)
    for t, name in ((block_table, "block_table"), (kv_len, "kv_len"), (q_start, "q_start")):
        _req(t, name, torch.int32)
    batch = kv_len.numel()
    if width != (nq + 2 * nkv) * d or tuple(out.shape) != (n_tokens, nq * d) or n_tokens < batch:
        raise KernelError(f"attention_decode_rope: qkv {tuple(qkv.shape)} / out {tuple(out.shape)} do not match {batch} requests, heads {nq}+2*{nkv} of {d}")
    if k_pages.shape[1] != nkv or k_pages.shape[3] != d or k_pages.shape != v_pages.shape:
        raise KernelError(f"attention_decode_rope: pages {tuple(k_pages.shape)} do not match {nkv} kv heads of {d}")
    for g, name in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _req(g, name, torch.float32, 1)
            if g.numel() != d:
                raise KernelError(f"{name} has {g.numel()} elements, head_dim is {d}")
    table_positions = 0
    if cos is not None:
        _req(cos, "cos", torch.float32, 2)
        _req(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != d:
            raise KernelError("attention_decode_rope: rotation tables must cover the whole head")
        table_positions = cos.shape[0]
    need = batch * nq * n_splits * (d + 2)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.float32, device=out.device)
    _req(workspace, "workspace", torch.float32, 1)
    if workspace.numel() < need:
        raise KernelError(f"attention_decode_rope: workspace has {workspace.numel()} floats, {need} are needed")
    _call('attention', "attention_decode_rope", library().qi_attention_decode_rope_tma,
          _ptr(qkv), _code(qkv), splits, n_tokens, _ptr(q_gain), _ptr(k_gain), C.c_float(eps), _ptr(cos), _ptr(sin),
        table_positions, int(bool(writes)), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
        block_table.shape[1], k_pages.shape[2], k_pages.shape[0], _ptr(kv_len), _ptr(q_start), batch, nq, nkv, d,
        C.c_float(scale), int(window or 0), chunk, n_splits, _ptr(workspace), _ptr(workspace[batch * nq * n_splits * d:]),
        _ptr(status), _stream())


# --------------------------------------------------------------------------
# feed-forward


ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "relu": 3, "relu2": 4, "tanh": 5}


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """`act_mul` with the activation silu."""
    act_mul(gate_up, out, "silu", interleaved)


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu", interleaved: bool = False) -> None:
    """out[t, i] = act(gate[t, i]) * up[t, i]; gate, up = gate_up[t, i], gate_up[t, I + i],
    or gate_up[t, 2i], gate_up[t, 2i + 1] when `interleaved`. `activation`: one of ACTIVATIONS."""
    if activation not in ACTIVATIONS:
        raise KernelError(f"act_mul: activation {activation!r} has no kernel (one of {sorted(ACTIVATIONS)})")
    _req(gate_up, "gate_up", ndim=2)
    _req(out, "out", gate_up.dtype, 2)
    n, two_i = gate_up.shape
    if two_i % 2 or tuple(out.shape) != (n, two_i // 2):
        raise KernelError(f"act_mul: gate_up {tuple(gate_up.shape)} / out {tuple(out.shape)} do not agree")
    _call("other", "act_mul", library().qi_act_mul,
          _ptr(gate_up), _ptr(out), _code(out), n, two_i // 2, int(bool(interleaved)), ACTIVATIONS[activation], _stream())


# --------------------------------------------------------------------------
# sampling


def sample(logits, temperature, top_k, top_p, seed, counter, out_token, status) -> None:
    """Token per row of float32 logits [rows, vocab]; temperature 0 = first maximum.

    temperature/top_p float32 [rows], top_k/counter int32 [rows], seed int64
    [rows]; any of them may be None (greedy / no truncation / seed 0 / counter 0).
    """
    _req(logits, "logits", torch.float32, 2)
    _req(out_token, "out_token", torch.int32, 1)
    rows, vocab = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (seed, "seed", torch.int64),
                        (counter, "counter", torch.int32)):
        if t is not None:
            _req(t, name, dt, 1)
            if t.numel() < rows:
                raise KernelError(f"sample: {name} has {t.numel()} entries for {rows} rows")
    if out_token.numel() < rows:
        raise KernelError("sample: out_token is too short")
    _call('other', "sample", library().qi_sample,
          _ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                             _ptr(seed), _ptr(counter), _ptr(out_token), _ptr(status), _stream())


def sample_slots(logits, logit_rows, token_req, slot_ids, slots, all_greedy: bool, out_token, status) -> None:
    """Token per row of float32 logits [rows, vocab] with the options of the row's request, read from
    the slot records `slots` (int32 [num_slots, 8], sampling/slots.py). The request of row r is the one
    in slot slot_ids[token_req[logit_rows[r]]] (the step's device arrays). The kernel adds one to the
    record's count of emitted tokens after the draw. `all_greedy`: no row draws (the host knows)."""
    _req(logits, "logits", torch.float32, 2)
    _req(out_token, "out_token", torch.int32, 1)
    _req(slots, "slots", torch.int32, 2)
    rows, vocab = logits.shape
    for t, name in ((logit_rows, "logit_rows"), (token_req, "token_req"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    if logit_rows.numel() < rows or out_token.numel() < rows:
        raise KernelError(f"sample_slots: {rows} rows of logits, {logit_rows.numel()} wanted rows, {out_token.numel()} places for tokens")
    _call("other", "sample_slots", library().qi_sample_slots,
          _ptr(logits), rows, vocab, _ptr(logit_rows), _ptr(token_req), _ptr(slot_ids), _ptr(slots), slots.shape[1],
          int(bool(all_greedy)), _ptr(out_token), _ptr(status), _stream())


def advance_decode(token_ids, positions, start_pos, kv_len, counter, sampled, history) -> None:
    """In place, for a decode batch kept on the device: token_ids = sampled, positions,
    start_pos and kv_len + 1, counter + 1 (may be None), history = sampled (may be None)."""
    for t, name in ((token_ids, "token_ids"), (positions, "positions"), (start_pos, "start_pos"),
                    (kv_len, "kv_len"), (sampled, "sampled")):
        _req(t, name, torch.int32, 1)
    b = token_ids.numel()
    _call(None, "advance_decode", library().qi_advance_decode,
          _ptr(token_ids), _ptr(positions), _ptr(start_pos), _ptr(kv_len),
                                     _ptr(counter), _ptr(sampled), _ptr(history), b, _stream())


def gemm_qkv_rope_supported(M: int, K: int, d: int, rotary_dim: int, dtype, weight_dtype) -> bool:
    """Whether `gemm_qkv_rope` takes this problem: many tokens (the operands are not swapped),
    bfloat16, heads of 128, rotation over the whole head or none."""
    return (M > 256 and K % 8 == 0 and d == 128 and rotary_dim in (0, d)
            and dtype == torch.bfloat16 and weight_dtype == torch.bfloat16)


def gemm_qkv_rope(x, w, q_out, q_gain, k_gain, eps, cos, sin, positions, token_req, block_table, page_size,
                  k_pages, v_pages, nq, nkv, status) -> None:
    """The q/k/v projection x[M, K] @ w[(nq + 2 nkv) 128, K]^T on the tcgen05 tensor cores with
    the q/k RMSNorm, the rotation and the cache write in its epilogue: what `gemm_bf16` followed
    by `qk_norm_rope_kv` computes, without the projection's output crossing memory.
    Arguments as for `qk_norm_rope_kv`."""
    d = 128
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    _req(q_out, "q_out", torch.bfloat16, 2)
    M, K = x.shape
    if tuple(w.shape) != ((nq + 2 * nkv) * d, K) or tuple(q_out.shape) != (M, nq * d):
        raise KernelError(f"gemm_qkv_rope: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)} do not match heads {nq}+2*{nkv} of {d}")
    for g, name in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _req(g, name, torch.float32, 1)
            if g.numel() != d:
                raise KernelError(f"{name} has {g.numel()} elements, head_dim is {d}")
    table_positions = 0
    if cos is not None:
        _req(cos, "cos", torch.float32, 2)
        _req(sin, "sin", torch.float32, 2)
        if cos.shape != sin.shape or cos.shape[1] * 2 != d:
            raise KernelError("gemm_qkv_rope: rotation tables must cover the whole head")
        table_positions = cos.shape[0]
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    if positions.numel() != M or token_req.numel() != M:
        raise KernelError("gemm_qkv_rope: positions and token_req must have one entry per token")
    num_pages, max_blocks = 0, 0
    if k_pages is not None:
        _req(k_pages, "k_pages", torch.bfloat16, 4)
        _req(v_pages, "v_pages", torch.bfloat16, 4)
        _req(block_table, "block_table", torch.int32, 2)
        if tuple(k_pages.shape[1:]) != (nkv, page_size, d) or k_pages.shape != v_pages.shape:
            raise KernelError(f"gemm_qkv_rope: pages {tuple(k_pages.shape)} do not match (pages, {nkv}, {page_size}, {d})")
        num_pages, max_blocks = k_pages.shape[0], block_table.shape[1]
    _call('gemm', "gemm_qkv_rope", library().qi_gemm_bf16_qkv_rope,
          _ptr(x), _ptr(w), M, K, _ptr(q_out), _ptr(q_gain), _ptr(k_gain), C.c_float(eps), _ptr(cos), _ptr(sin),
        table_positions, _ptr(positions), _ptr(token_req), _ptr(block_table), max_blocks, page_size, num_pages,
        _ptr(k_pages), _ptr(v_pages), nq, nkv, _ptr(status), _stream())


def stage_step(host_meta: torch.Tensor, meta: torch.Tensor, device_tokens=None) -> None:
    """meta[:n] = host_meta[:n] read by a kernel straight from pinned host memory (n =
    host_meta.numel()); the first device_tokens.numel() entries come from `device_tokens`
    (int32, on the device) when given."""
    if not isinstance(host_meta, torch.Tensor) or host_meta.is_cuda or not host_meta.is_pinned() or host_meta.dtype != torch.int32:
        raise KernelError("stage_step: host_meta must be a pinned int32 host tensor")
    _req(meta, "meta", torch.int32, 1)
    n = host_meta.numel()
    if meta.numel() < n:
        raise KernelError(f"stage_step: meta has {meta.numel()} entries, {n} are needed")
    n_tok = 0
    if device_tokens is not None:
        _req(device_tokens, "device_tokens", torch.int32, 1)
        n_tok = device_tokens.numel()
    _call(None, "stage_step", library().qi_stage_step,
          C.c_void_p(host_meta.data_ptr()), _ptr(meta), n, _ptr(device_tokens), n_tok, _stream())


def publish(src: torch.Tensor, host_out: torch.Tensor, n: int) -> None:
    """host_out[:n] = src[:n], written by a kernel into pinned host memory; read it after an
    event recorded behind this call."""
    _req(src, "src", torch.int32, 1)
    if host_out.is_cuda or not host_out.is_pinned() or host_out.dtype != torch.int32:
        raise KernelError("publish: host_out must be a pinned int32 host tensor")
    if n > src.numel() or n > host_out.numel():
        raise KernelError("publish: more entries than the buffers hold")
    _call(None, "publish", library().qi_publish,
          _ptr(src), C.c_void_p(host_out.data_ptr()), n, _stream())


# --------------------------------------------------------------------------
# tensor-core matrix product (bfloat16 operands, 32-bit accumulation)

_gemm_status = {}


def gemm_bf16_supported(M: int, N: int, K: int, out_dtype) -> bool:
    """Whether `gemm_bf16` takes this problem; callers use `gemm_simt` otherwise."""
    return M > 0 and K % 8 == 0 and out_dtype in (torch.bfloat16, torch.float32)


def gemm_bf16_plan(M: int, N: int, K: int, allow_split: bool = True):
    """(orientation, tile width, K splits) the library would choose; allow_split=False for a
    product whose epilogue needs the whole sum (the fused activation). Orientation 0: the tokens
    ride the 128 rows of the tensor-core tile; 1: the weights do (few tokens); 2: tokens on the rows
    of tiles of 256 x 256 computed by pairs of CTAs (many tokens)."""
    key = (M, N, K, bool(allow_split))
    plan = _plans.get(key)
    if plan is None:
        swap, bn, splits = C.c_int(), C.c_int(), C.c_int()
        library().qi_gemm_bf16_plan(M, N, K, int(allow_split), C.byref(swap), C.byref(bn), C.byref(splits))
        plan = _plans[key] = (swap.value, bn.value, splits.value)
    return plan


_plans = {}


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out, plan=None, status=None, epilogue: str | None = None,
              keep_partials: bool = False):
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores; x, w bfloat16; out
    bfloat16 or float32. `plan` = (orientation, tile width, splits) overrides the choice.

    epilogue="silu_mul": w's rows are (gate, up) pairs and out is [M, N / 2] =
    silu(gate) * up. keep_partials=True: when the plan splits K, the float32 partial sums
    [splits, M, N] are returned unreduced (and `out` is not written); else `out` is returned."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if epilogue not in (None, "silu_mul"):
        raise KernelError(f"gemm_bf16: unknown epilogue {epilogue!r}")
    swap, bn, splits = plan if plan is not None else gemm_bf16_plan(M, N, K, allow_split=epilogue is None)
    epi = 0
    if epilogue == "silu_mul":
        epi, splits = 1, 1
    n_out = N // 2 if epi else N
    partial_only = keep_partials and splits > 1
    if not partial_only:
        _req(out, "out", ndim=2)
        if w.shape[1] != K or tuple(out.shape) != (M, n_out):
            raise KernelError(f"gemm: shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    ws = torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None
    if status is None:
        status = _gemm_status.get(x.device)
        if status is None:
            status = _gemm_status[x.device] = torch.zeros(1, dtype=torch.int32, device=x.device)
    _call('gemm', "gemm_bf16", library().qi_gemm_bf16,
          _ptr(x), _ptr(w), _ptr(None if partial_only else out),
                                BF16 if partial_only else _code(out), M, N, K, int(swap), bn, splits, epi,
                                _ptr(ws), _ptr(status), _stream())
    return ws if partial_only else out


# --------------------------------------------------------------------------
# bigram embedding, short convolutions, per-head products, gates, soft cap


def embedding_bigram(table, bigram, ids, positions, token_req, q_start, slot_ids, prev_state, out, buckets: int,
                     mul_prev: int, mul_cur: int, status) -> None:
    """out[t] = table[ids[t]] + bigram[row_t] as float32: row_t = (previous id * mul_prev + ids[t] * mul_cur) mod
    buckets, or the row `buckets` for a sequence's first token. `prev_state` (int32, one word a slot) carries a
    request's last token from step to step; the launch reads and advances it."""
    _req(table, "table", ndim=2)
    _req(bigram, "bigram", table.dtype, 2)
    _req(out, "out", torch.float32, 2)
    for t, name in ((ids, "ids"), (positions, "positions"), (token_req, "token_req"), (q_start, "q_start"),
                    (slot_ids, "slot_ids")):
        _req(t, name, torch.int32)
    _req_state(prev_state, "prev_state", torch.int32)
    n, hidden = out.shape
    if ids.numel() != n or table.shape[1] != hidden or tuple(bigram.shape) != (buckets + 1, hidden):
        raise KernelError(f"embedding_bigram: shapes do not agree: table {tuple(table.shape)}, bigram {tuple(bigram.shape)} "
                          f"for {buckets} buckets, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    _call("other", "embedding_bigram", library().qi_embedding_bigram,
          _ptr(table), _ptr(bigram), _code(table), _ptr(ids), _ptr(positions), _ptr(token_req), _ptr(q_start),
          _ptr(slot_ids), _ptr(prev_state), _ptr(out), n, hidden, table.shape[0], C.c_longlong(buckets),
          C.c_longlong(mul_prev), C.c_longlong(mul_cur), C.c_longlong(prev_state.stride(0)), _ptr(status), _stream())


def short_conv(h, weights, state, outs, copy, token_req, q_start, start_pos, slot_ids, residual: bool = True,
               bias=None, act: str | None = None) -> None:
    """outs[k][t] = f((h[t] if residual) + sum_j weights[k, j] * h[t - taps + 1 + j] (+ bias[k])) per channel, over each
    request's own time axis: rows before a step's first token come from `state` (float32 [slots, taps - 1, channels],
    the request's last inputs; advanced by the launch), zeros before the sequence's start. h [n, channels], float32 or
    the outputs' type; it may be a block of columns of wider rows (a view whose rows lie `h.stride(0)` apart);
    weights float32 [filters, taps, channels] with one or two filters; bias float32 [filters, channels] or None; f is
    silu when `act` is "silu", else nothing; `copy`, if given, receives h in its type."""
    if not isinstance(h, torch.Tensor) or not h.is_cuda or h.dim() != 2 or h.stride(1) != 1 or h.stride(0) < h.shape[1]:
        raise KernelError("short_conv: h must be a CUDA tensor [n, channels] whose rows are contiguous")
    _req(weights, "weights", torch.float32, 3)
    n, ch = h.shape
    filters, taps = weights.shape[0], weights.shape[1]
    if weights.shape[2] != ch or len(outs) != filters:
        raise KernelError(f"short_conv: weights {tuple(weights.shape)} and {len(outs)} outputs do not fit h {tuple(h.shape)}")
    for o in list(outs) + ([copy] if copy is not None else []):
        _req(o, "out", outs[0].dtype, 2)
        if tuple(o.shape) != (n, ch):
            raise KernelError(f"short_conv: an output is {tuple(o.shape)}, expected {(n, ch)}")
    if bias is not None:
        _req(bias, "bias", torch.float32, 2)
        if tuple(bias.shape) != (filters, ch):
            raise KernelError(f"short_conv: bias {tuple(bias.shape)} does not fit {filters} filters of {ch} channels")
    if act not in (None, "silu"):
        raise KernelError(f"short_conv: activation {act!r} is not known (silu or None)")
    if taps > 1:
        _req_state(state, "state", torch.float32)
        if tuple(state.shape[1:]) != (taps - 1, ch):
            raise KernelError(f"short_conv: state {tuple(state.shape)} does not fit {taps} taps of {ch} channels")
    for t, name in ((token_req, "token_req"), (q_start, "q_start"), (start_pos, "start_pos"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32)
    _call("other", "short_conv", library().qi_short_conv,
          _ptr(h), _code(h), C.c_longlong(h.stride(0)), _ptr(bias), 1 if act == "silu" else 0,
          _ptr(weights), _ptr(state if taps > 1 else None), _ptr(outs[0]), _ptr(outs[1] if filters > 1 else None),
          _ptr(copy), _code(outs[0]), _ptr(token_req), _ptr(q_start), _ptr(start_pos), _ptr(slot_ids), n, ch, taps, filters,
          int(bool(residual)), C.c_longlong(state.stride(0) if taps > 1 else 0), _stream())


def head_linear(x, x_head_width: int, x_offset: int, k: int, w, out, out_head_width: int, out_offset: int) -> None:
    """Per-head projections in one launch. Heads lie side by side in the rows of x [n, >= heads * x_head_width] and
    of out [n, >= heads * out_head_width]; for head h,
        out[:, h * out_head_width + out_offset : ... + N] = x[:, h * x_head_width + x_offset : ... + k] @ w[h]^T
    with w [heads, N, k]. 32-bit products and sums; any element types."""
    _req(x, "x", ndim=2)
    _req(w, "w", ndim=3)
    _req(out, "out", ndim=2)
    n = x.shape[0]
    heads, N = w.shape[0], w.shape[1]
    if (w.shape[2] != k or out.shape[0] != n or x_offset + k > x_head_width or out_offset + N > out_head_width
            or heads * x_head_width > x.shape[1] or heads * out_head_width > out.shape[1]):
        raise KernelError(f"head_linear: x {tuple(x.shape)} (heads of {x_head_width}), w {tuple(w.shape)}, out {tuple(out.shape)} "
                          f"(heads of {out_head_width}) do not fit")
    xp = x.data_ptr() + x_offset * x.element_size()
    op = out.data_ptr() + out_offset * out.element_size()
    strides = (C.c_longlong(x.shape[1]), C.c_longlong(k), C.c_longlong(out.shape[1]))
    batch = (heads, C.c_longlong(x_head_width), C.c_longlong(N * k), C.c_longlong(out_head_width))
    lib = library()
    if (x.dtype == w.dtype == out.dtype == torch.bfloat16 and lib.qi_gemm_mma_batched_supported(
            C.c_void_p(xp), _ptr(w), C.c_void_p(op), k, *strides, *batch[1:])):
        # bfloat16 throughout and aligned for 16-byte loads: the tensor-core kernel
        _call("gemm", "head_linear", lib.qi_gemm_mma_batched, C.c_void_p(xp), _ptr(w), C.c_void_p(op), n, N, k, *strides, *batch, _stream())
        return
    _call("gemm", "head_linear", lib.qi_gemm_simt_batched, C.c_void_p(xp), _code(x), _ptr(w), _code(w), C.c_void_p(op), _code(out),
          n, N, k, *strides, *batch, _stream())


def activation(x, out, name: str) -> None:
    """out = act(x), elementwise, x and out of one type and shape."""
    if name not in ACTIVATIONS:
        raise KernelError(f"activation: {name!r} has no kernel (one of {sorted(ACTIVATIONS)})")
    _req(x, "x")
    _req(out, "out", x.dtype)
    if out.shape != x.shape:
        raise KernelError("activation: shapes differ")
    _call("other", "activation", library().qi_activation, _ptr(x), _ptr(out), _code(x), C.c_longlong(x.numel()),
          ACTIVATIONS[name], _stream())


def gated_sum(gates, b0, b1, y0, y1, out) -> None:
    """out = sigmoid(gates[:, :C] + b0) * y0 (+ sigmoid(gates[:, C:2C] + b1) * y1 when y1 is given); out float32
    [n, C], biases float32 [C], y0 and y1 of one type."""
    _req(gates, "gates", ndim=2)
    _req(out, "out", torch.float32, 2)
    _req(y0, "y0", ndim=2)
    _req(b0, "b0", torch.float32, 1)
    n, ch = out.shape
    if y1 is not None:
        _req(y1, "y1", y0.dtype, 2)
        _req(b1, "b1", torch.float32, 1)
    if (gates.shape[0] != n or gates.shape[1] < (2 if y1 is not None else 1) * ch or tuple(y0.shape) != (n, ch)
            or b0.numel() != ch or (y1 is not None and (tuple(y1.shape) != (n, ch) or b1.numel() != ch))):
        raise KernelError(f"gated_sum: gates {tuple(gates.shape)}, y {tuple(y0.shape)}, out {tuple(out.shape)} do not fit")
    _call("other", "gated_sum", library().qi_gated_sum, _ptr(gates), _code(gates), gates.shape[1], _ptr(b0), _ptr(b1),
          _ptr(y0), _ptr(y1), _code(y0), _ptr(out), n, ch, _stream())


def sigmoid_gate(x, gate) -> None:
    """x *= sigmoid(gate) in place; x [n, c] contiguous; gate [n, c], possibly a block of columns of wider rows."""
    _req(x, "x", ndim=2)
    if not gate.is_cuda or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != x.shape:
        raise KernelError("sigmoid_gate: the gate must match x, with contiguous rows")
    _call("other", "sigmoid_gate", library().qi_sigmoid_gate, _ptr(x), _code(x), _ptr(gate), _code(gate), C.c_longlong(gate.stride(0)),
          x.shape[0], x.shape[1], _stream())


def softcap(x, cap: float) -> None:
    """x = cap * tanh(x / cap) in place; x float32."""
    _req(x, "x", torch.float32)
    _call("other", "softcap", library().qi_softcap, _ptr(x), C.c_longlong(x.numel()), C.c_float(cap), _stream())


# --------------------------------------------------------------------------
# attention over a cached latent


def latent_prepare(proj, kv_offset, q_out, gain, eps: float, inv_freq, rot_dims: int, positions, token_req,
                   block_table, cache, heads: int, d: int, r: int, rank: int, status, half_split: bool = False,
                   magnitude: float = 1.0) -> None:
    """From the fused projection's rows [heads x (d + r) | latent projection (rank + r) at column kv_offset]: rotates
    every head's r-part into q_out[:, h, rank:], and, unless kv_offset is None, normalises the latent (gain float32
    [rank]), rotates the shared key part and writes [latent | key part] into `cache` [pages, page_size, rank + r] at
    each token's position. Pairs (2i, 2i + 1) of the part's first rot_dims coordinates, or (i, i + rot_dims / 2) when
    `half_split`, turn by position * inv_freq[i]; cos and sin are multiplied by `magnitude`. The rows of `proj` may be
    wider than what is read here."""
    _req(proj, "proj", ndim=2)
    _req(q_out, "q_out", ndim=3)
    n = proj.shape[0]
    if tuple(q_out.shape) != (n, heads, rank + r):
        raise KernelError(f"latent_prepare: q_out {tuple(q_out.shape)} is not {(n, heads, rank + r)}")
    if rot_dims:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() * 2 != rot_dims:
            raise KernelError("latent_prepare: inv_freq does not match rot_dims")
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    page_size = num_pages = max_blocks = 0
    if kv_offset is not None:
        _req(cache, "cache", q_out.dtype, 3)
        _req(gain, "gain", torch.float32, 1)
        _req(block_table, "block_table", torch.int32, 2)
        if cache.shape[2] != rank + r or gain.numel() != rank:
            raise KernelError(f"latent_prepare: cache {tuple(cache.shape)} / gain {gain.numel()} do not fit rank {rank} + {r}")
        num_pages, page_size, max_blocks = cache.shape[0], cache.shape[1], block_table.shape[1]
    _call("rope", "latent_prepare", library().qi_latent_prepare,
          _ptr(proj), _code(proj), C.c_longlong(proj.shape[1]), -1 if kv_offset is None else int(kv_offset), _ptr(q_out),
          _code(q_out), _ptr(gain if kv_offset is not None else None), C.c_float(eps), _ptr(inv_freq if rot_dims else None),
          rot_dims, _ptr(positions), _ptr(token_req), _ptr(block_table if kv_offset is not None else None), max_blocks,
          page_size, num_pages, _ptr(cache if kv_offset is not None else None), n, heads, d, r, rank, int(bool(half_split)),
          C.c_float(magnitude), _ptr(status), _stream())


def latent_attention_generic(q, out, cache, sink, block_table, positions, token_req, scale: float, window: int, status) -> None:
    """Causal attention of every head over one shared cached row per position: q [n, heads, W], cache [pages,
    page_size, W], out [n, heads, R] = sum_j p_j cache[j, :R]; the softmax's denominator also holds exp(sink[h])
    when `sink` (float32 [heads]) is given. 32-bit arithmetic, any sizes."""
    _req(q, "q", ndim=3)
    _req(out, "out", q.dtype, 3)
    _req(cache, "cache", q.dtype, 3)
    _req(block_table, "block_table", torch.int32, 2)
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    n, heads, W = q.shape
    R = out.shape[2]
    if out.shape[0] != n or out.shape[1] != heads or cache.shape[2] != W or R > W:
        raise KernelError(f"latent_attention: q {tuple(q.shape)}, out {tuple(out.shape)}, cache {tuple(cache.shape)} do not fit")
    if sink is not None:
        _req(sink, "sink", torch.float32, 1)
        if sink.numel() != heads:
            raise KernelError("latent_attention: one sink a head")
    _call("attention", "latent_attention_generic", library().qi_latent_attention_generic,
          _ptr(q), _ptr(out), _code(q), _ptr(cache), _ptr(sink), _ptr(block_table), block_table.shape[1], cache.shape[1],
          cache.shape[0], _ptr(positions), _ptr(token_req), n, heads, W, R, C.c_float(scale), int(window or 0), _ptr(status),
          _stream())


def latent_attention_mma_supported(W: int, R: int) -> bool:
    """Whether the tensor-core latent attention takes rows of W with a latent of R (bfloat16 only)."""
    return bool(library().qi_latent_attention_mma_supported(W, R))


def latent_attention_ranges(n_tiles: int, max_keys: int, W: int) -> int:
    """Into how many key ranges the tensor-core latent attention cuts every query tile: as many as fill the CTAs
    that are resident at once (two on each of 148 SMs), at most one per key tile."""
    key_tile = library().qi_latent_attention_mma_key_tile(W)
    return max(1, min(-(-max_keys // key_tile), 296 // max(n_tiles, 1), 128))


def latent_attention(q, out, cache, sink, block_table, q_start, start_pos, positions, token_req, scale: float, window: int,
                     status, impl: str | None = None, key_ranges: int = 1) -> None:
    """`latent_attention_generic`'s result by the kernel that fits: "mma" (bfloat16, latent widths the tensor-core
    kernel covers: flash form, one key tile for all heads) or "generic". `q_start`, `start_pos`: the step's per-entry
    arrays (the tensor-core kernel finds its query tiles from them on the device). `key_ranges` > 1 spreads every
    query tile's keys over that many CTAs and adds their partial sums in a second kernel (decode steps)."""
    n, heads, W = q.shape
    R = out.shape[2]
    if impl is None:
        impl = "mma" if q.dtype == torch.bfloat16 and latent_attention_mma_supported(W, R) else "generic"
    if impl == "generic":
        return latent_attention_generic(q, out, cache, sink, block_table, positions, token_req, scale, window, status)
    if impl != "mma":
        raise KernelError(f"latent_attention: unknown kernel {impl!r}")
    _req(q, "q", torch.bfloat16, 3)
    _req(out, "out", torch.bfloat16, 3)
    _req(cache, "cache", torch.bfloat16, 3)
    for t, name in ((block_table, "block_table"), (q_start, "q_start"), (start_pos, "start_pos")):
        _req(t, name, torch.int32)
    if out.shape[0] != n or out.shape[1] != heads or cache.shape[2] != W or q_start.numel() != start_pos.numel() + 1:
        raise KernelError(f"latent_attention: q {tuple(q.shape)}, out {tuple(out.shape)}, cache {tuple(cache.shape)} do not fit")
    if sink is not None:
        _req(sink, "sink", torch.float32, 1)
        if sink.numel() != heads:
            raise KernelError("latent_attention: one sink a head")
    ws_o = ws_ml = None
    if key_ranges > 1:
        ws_o = torch.empty((n * heads, key_ranges, R), dtype=torch.float32, device=q.device)
        ws_ml = torch.empty((n * heads, key_ranges, 2), dtype=torch.float32, device=q.device)
    _call("attention", "latent_attention_mma", library().qi_latent_attention_mma,
          _ptr(q), _ptr(out), _ptr(cache), _ptr(sink), _ptr(block_table), block_table.shape[1], cache.shape[1], cache.shape[0],
          _ptr(q_start), _ptr(start_pos), start_pos.numel(), n, heads, W, R, C.c_float(scale), int(window or 0), key_ranges,
          _ptr(ws_o), _ptr(ws_ml), _ptr(status), _stream())


# --------------------------------------------------------------------------
# dynamic tanh, biases + direct rotation, state-space recurrence, mixture of experts


def dyt(resid, y=None, y_bias=None, post=None, mult: float = 1.0, pre=None, out=None, rows=None, write_resid: bool = True) -> None:
    """The elementwise work around a sublayer of a model normalised by dynamic tanh, dyt(v) = tanh(alpha v) w + b:
    resid += mult * dyt_post(y + y_bias) (or resid += y + y_bias without `post`), then out = dyt_pre(resid).
    resid float32 [n, h]; y [n, h] (or the partial sums [splits, n, h] of a K-split product, added here) or None;
    y_bias float32 [h] or None; post, pre: (w, b, alpha) float32 [h], [h], [1]
    or None; out [n, h] (or [len(rows), h] when `rows` picks source rows; the stream is then not written)."""
    _req(resid, "resid", torch.float32, 2)
    n, h = resid.shape
    splits, stride = 1, 0
    if y is not None:
        _req(y, "y")
        if y.dim() == 3:
            splits, stride = y.shape[0], y.shape[1] * y.shape[2]
        if tuple(y.shape[-2:]) != (n, h) or y.dim() not in (2, 3):
            raise KernelError(f"dyt: y {tuple(y.shape)} does not match resid {tuple(resid.shape)}")
    for trio, name in ((post, "post"), (pre, "pre")):
        if trio is not None:
            w, b, alpha = trio
            _req(w, name + " w", torch.float32, 1)
            _req(b, name + " b", torch.float32, 1)
            _req(alpha, name + " alpha", torch.float32)
            if w.numel() != h or b.numel() != h or alpha.numel() != 1:
                raise KernelError(f"dyt: the {name}-norm's tensors do not fit rows of {h}")
    if y_bias is not None:
        _req(y_bias, "y_bias", torch.float32, 1)
        if y_bias.numel() != h:
            raise KernelError("dyt: the bias does not fit the rows")
    n_out = n
    if rows is not None:
        _req(rows, "rows", torch.int32, 1)
        n_out, write_resid = rows.numel(), False
    if (pre is None) != (out is None):
        raise KernelError("dyt: a pre-norm and an output come together")
    if out is not None:
        _req(out, "out", ndim=2)
        if tuple(out.shape) != (n_out, h):
            raise KernelError(f"dyt: out is {tuple(out.shape)}, expected {(n_out, h)}")
    pw, pb, pa = post if post is not None else (None, None, None)
    rw, rb, ra = pre if pre is not None else (None, None, None)
    _call("norm", "dyt", library().qi_dyt, _ptr(resid), _ptr(y), _code(y) if y is not None else F32, splits, C.c_longlong(stride),
          _ptr(y_bias), _ptr(pw), _ptr(pb), _ptr(pa), C.c_float(mult), _ptr(rw), _ptr(rb), _ptr(ra), _ptr(out),
          _code(out) if out is not None else F32, _ptr(rows), n_out, h, int(bool(write_resid)), _stream())


def concat_cast(a, b, out) -> None:
    """out[t] = [a[t] | b[t]]: two float32 streams [n, h] side by side in out's type [n, 2 h]."""
    _req(a, "a", torch.float32, 2)
    _req(b, "b", torch.float32, 2)
    _req(out, "out", ndim=2)
    n, h = a.shape
    if b.shape != a.shape or tuple(out.shape) != (n, 2 * h):
        raise KernelError("concat_cast: shapes do not agree")
    _call("other", "concat_cast", library().qi_concat_cast, _ptr(a), _ptr(b), _ptr(out), _code(out), n, h, _stream())


def bias_rope_kv(proj, bias, q_out, inv_freq, rot: int, interleaved: bool, positions, token_req, block_table, page_size: int,
                 k_pages, v_pages, nq: int, nkv: int, d: int, dv: int, status, q_gain=None, k_gain=None, norm_eps: float = 0.0,
                 values_from_keys: bool = False) -> None:
    """proj [n, >= (nq + nkv) d + nkv dv] holds q | k | v (more columns may follow); bias float32 over those columns or
    None; the first `rot` coordinates of each q and k head turn by position * inv_freq[pair] (computed here in 32-bit:
    no table, no limit on positions); q goes to q_out [n, nq d], k and v into the pages (None: nothing is written).
    q_gain, k_gain (float32 [nq d], [nkv d]; both or neither): all of q and all of k each pass one RMS norm with that gain
    and `norm_eps` before the rotation. values_from_keys: the rows hold no v; a position's value is its key as
    projected, before norm and rotation (dv = d)."""
    if not proj.is_cuda or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("bias_rope_kv: proj must be a CUDA tensor with contiguous rows")
    _req(q_out, "q_out", proj.dtype, 2)
    n = proj.shape[0]
    cols = (nq + nkv) * d + (0 if values_from_keys else nkv * dv)
    if (q_gain is None) != (k_gain is None) or (values_from_keys and dv != d):
        raise KernelError("bias_rope_kv: the norms of q and k come together; values that are keys have the keys' size")
    if q_gain is not None:
        _req(q_gain, "q_gain", torch.float32, 1)
        _req(k_gain, "k_gain", torch.float32, 1)
        if q_gain.numel() != nq * d or k_gain.numel() != nkv * d:
            raise KernelError("bias_rope_kv: the gains do not fit q and k")
    if proj.shape[1] < cols or tuple(q_out.shape) != (n, nq * d):
        raise KernelError(f"bias_rope_kv: proj {tuple(proj.shape)} / q_out {tuple(q_out.shape)} do not match the heads")
    if bias is not None:
        _req(bias, "bias", torch.float32, 1)
        if bias.numel() != cols:
            raise KernelError("bias_rope_kv: the bias does not fit q | k | v")
    if rot:
        _req(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() * 2 != rot:
            raise KernelError("bias_rope_kv: one inverse frequency a pair")
    _req(positions, "positions", torch.int32, 1)
    _req(token_req, "token_req", torch.int32, 1)
    num_pages = max_blocks = 0
    if k_pages is not None:
        _req(k_pages, "k_pages", proj.dtype, 4)
        _req(v_pages, "v_pages", proj.dtype, 4)
        _req(block_table, "block_table", torch.int32, 2)
        if tuple(k_pages.shape[1:]) != (nkv, page_size, d) or tuple(v_pages.shape) != (k_pages.shape[0], nkv, page_size, dv):
            raise KernelError(f"bias_rope_kv: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} do not fit")
        num_pages, max_blocks = k_pages.shape[0], block_table.shape[1]
    _call("rope", "bias_rope_kv", library().qi_norm_rope_kv, _ptr(proj), C.c_longlong(proj.stride(0)), _ptr(bias), _ptr(q_out),
          _code(proj), _ptr(inv_freq if rot else None), rot, int(bool(interleaved)), _ptr(positions), _ptr(token_req),
          _ptr(block_table), max_blocks, page_size, num_pages, _ptr(k_pages), _ptr(v_pages), n, nq, nkv, d, dv, _ptr(q_gain),
          _ptr(k_gain), C.c_float(norm_eps), int(bool(values_from_keys)), _ptr(status), _stream())


def ssm_scan(xbc, raw_dt, dt_bias, a_log, d_skip, state, y, q_start, start_pos, slot_ids, heads: int, groups: int, P: int, N: int,
             write_state: bool = True, long_entries: bool = False) -> None:
    """The recurrence S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + d_skip x_t with
    dt_t = softplus(raw_t + dt_bias), per head over each entry's tokens. xbc [n, heads P + 2 groups N] holds x | B | C;
    raw_dt [n, heads] may be a block of columns of wider rows; state float32 [slots, heads, P, N] (read at an entry's first
    token unless it starts its sequence, written after its last unless `write_state` is False); y float32 [n, heads P], or
    None for a pass that wants the end states only. `long_entries`: every entry has many tokens, so the kernel that keeps a
    channel's column of the state in one thread is worth its start (states of at most 128 rows; others run as before)."""
    for t, name in ((xbc, "xbc"), (raw_dt, "raw_dt")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"ssm_scan: {name} must be a CUDA tensor with contiguous rows")
    if raw_dt.dtype != xbc.dtype or xbc.shape[1] != heads * P + 2 * groups * N or raw_dt.shape != (xbc.shape[0], heads):
        raise KernelError("ssm_scan: the inputs do not fit the sizes")
    for t, name in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        _req(t, name, torch.float32, 1)
        if t.numel() != heads:
            raise KernelError(f"ssm_scan: {name} needs one number a head")
    _req_state(state, "state", torch.float32)
    if tuple(state.shape[1:]) != (heads, P, N):
        raise KernelError(f"ssm_scan: state {tuple(state.shape)} does not fit [slots, {heads}, {P}, {N}]")
    if y is not None:
        _req(y, "y", torch.float32, 2)
        if tuple(y.shape) != (xbc.shape[0], heads * P):
            raise KernelError("ssm_scan: y does not fit")
    for t, name in ((q_start, "q_start"), (start_pos, "start_pos"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    cols = long_entries and (y is not None or write_state) and bool(library().qi_ssm_scan_cols_supported(N))
    _call("scan", "ssm_scan", library().qi_ssm_scan_cols if cols else library().qi_ssm_scan, _ptr(xbc), C.c_longlong(xbc.stride(0)), _ptr(raw_dt),
          C.c_longlong(raw_dt.stride(0)), _code(xbc), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state),
          C.c_longlong(state.stride(0)), _ptr(y), _ptr(q_start), _ptr(start_pos), _ptr(slot_ids), start_pos.numel(), heads, groups,
          P, N, int(bool(write_state)), _stream())


def ssm_chain(seg_state, state, raw_dt, dt_bias, a_log, seg_q_start, entry_seg, start_pos, slot_ids, max_segments: int) -> None:
    """Between the two passes of a recurrence cut into segments: seg_state [segments, heads, P, N] holds each segment's
    own contribution to its end state and receives the state each segment begins with; the requests' states
    (state [slots, heads, P, N]) advance to their entries' ends. seg_q_start [segments + 1], entry_seg [entries + 1]."""
    _req(seg_state, "seg_state", torch.float32, 4)
    _req_state(state, "state", torch.float32)
    if tuple(state.shape[1:]) != tuple(seg_state.shape[1:]) or raw_dt.dim() != 2 or raw_dt.stride(1) != 1:
        raise KernelError("ssm_chain: shapes do not agree")
    for t, name in ((seg_q_start, "seg_q_start"), (entry_seg, "entry_seg"), (start_pos, "start_pos"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    if seg_q_start.numel() != seg_state.shape[0] + 1 or entry_seg.numel() != start_pos.numel() + 1:
        raise KernelError("ssm_chain: the segment lists do not fit")
    heads, P, N = seg_state.shape[1:]
    _call("scan", "ssm_chain", library().qi_ssm_chain, _ptr(seg_state), _ptr(state), C.c_longlong(state.stride(0)), _ptr(raw_dt),
          C.c_longlong(raw_dt.stride(0)), _code(raw_dt), _ptr(dt_bias), _ptr(a_log), _ptr(seg_q_start), _ptr(entry_seg),
          _ptr(start_pos), _ptr(slot_ids), start_pos.numel(), int(max_segments), heads, P, N, _stream())


GATE_MODES = {"silu_before": 0, "silu": 1, "sigmoid": 2, "plain": 3}


def gated_group_rmsnorm(y, z, gain, eps: float, out, groups: int, gate: str = "silu_before", out_scale: float = 1.0) -> None:
    """Every width / groups coordinates of a row by their own root mean square, a gain, and a gate z:
    "silu_before": rmsnorm_groups(y * silu(z)) * gain; "silu": rmsnorm_groups(y) * gain * silu(z); "sigmoid": ... * sigmoid(z);
    "plain": ... * z. `out_scale` multiplies the result.
    y float32 [n, width]; z [n, width] (may be a block of columns of wider rows); gain float32 [width]."""
    if gate not in GATE_MODES:
        raise KernelError(f"gated_group_rmsnorm: gate {gate!r} is not known (one of {sorted(GATE_MODES)})")
    _req(y, "y", torch.float32, 2)
    if not z.is_cuda or z.dim() != 2 or z.stride(1) != 1 or z.shape != y.shape:
        raise KernelError("gated_group_rmsnorm: z must match y, with contiguous rows")
    _req(gain, "gain", torch.float32, 1)
    _req(out, "out", ndim=2)
    n, width = y.shape
    if gain.numel() != width or out.shape != y.shape or groups <= 0 or width % groups:
        raise KernelError("gated_group_rmsnorm: shapes do not agree")
    _call("norm", "gated_group_rmsnorm", library().qi_group_rmsnorm_gate, _ptr(y), _ptr(z), _code(z), C.c_longlong(z.stride(0)),
          _ptr(gain), C.c_float(eps), _ptr(out), _code(out), n, width, groups, GATE_MODES[gate], C.c_float(out_scale), _stream())


# --------------------------------------------------------------------------
# recurrent mixers with a state of fixed size


def _cols(t, name: str, dtype=None) -> None:
    """A block of columns of wider rows: [n, c] with unit stride inside a row."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        raise KernelError(f"{name} must be a CUDA tensor [n, columns] whose rows are contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def mingru_scan(proj, bz, bx, state, out, q_start, start_pos, slot_ids, width: int, slices: int = 1) -> None:
    """S_t = (1 - z) S_(t-1) + z c, out_t = S_t silu(g) per channel over each entry's tokens, with z = sigmoid(pz + bz),
    u = px + bx, c = u + 1/2 where u >= 0 and sigmoid(u) below. proj [n, 3 width] holds pz | px | pg (it may be a block of
    columns of wider rows); state float32 [slots, width] (read at an entry's first token unless it starts its sequence,
    written after its last); out [n, width]. `slices`: parts an entry is cut into that run side by side (1 .. 32)."""
    _cols(proj, "proj")
    _req(bz, "bz", torch.float32, 1)
    _req(bx, "bx", torch.float32, 1)
    _req_state(state, "state", torch.float32)
    _req(out, "out", ndim=2)
    n = proj.shape[0]
    if proj.shape[1] != 3 * width or bz.numel() != width or bx.numel() != width or tuple(out.shape) != (n, width) or tuple(
            state.shape[1:]) != (width,):
        raise KernelError("mingru_scan: shapes do not agree")
    for t, name in ((q_start, "q_start"), (start_pos, "start_pos"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    _call("scan", "mingru_scan", library().qi_mingru_scan, _ptr(proj), C.c_longlong(proj.stride(0)), _code(proj), _ptr(bz), _ptr(bx),
          _ptr(state), C.c_longlong(state.stride(0)), _ptr(out), _code(out), _ptr(q_start), _ptr(start_pos), _ptr(slot_ids),
          start_pos.numel(), width, int(slices), _stream())


def token_shift(h, mu, state, out, token_req, q_start, start_pos, slot_ids) -> None:
    """out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]: every token's input mixed with its predecessor's, once per row of
    mu. h [n, C]; mu float32 [mixes, C]; state float32 [slots, C]: the last input of a request's step before (zeros at a
    sequence's start), replaced by this step's last; out [mixes, n, C] in h's type."""
    _req(h, "h", ndim=2)
    _req(mu, "mu", torch.float32, 2)
    _req_state(state, "state", torch.float32)
    _req(out, "out", h.dtype, 3)
    n, ch = h.shape
    if mu.shape[1] != ch or tuple(out.shape) != (mu.shape[0], n, ch) or tuple(state.shape[1:]) != (ch,):
        raise KernelError("token_shift: shapes do not agree")
    for t, name in ((token_req, "token_req"), (q_start, "q_start"), (start_pos, "start_pos"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    _call("other", "token_shift", library().qi_token_shift, _ptr(h), _code(h), _ptr(mu), _ptr(state), C.c_longlong(state.stride(0)),
          _ptr(out), _ptr(token_req), _ptr(q_start), _ptr(start_pos), _ptr(slot_ids), n, ch, mu.shape[0], _stream())


def matrix_state_scan(mode: str, r, k, v, state, o, q_start, start_pos, slot_ids, heads: int, dk: int, dv: int, *, log_decay=None,
                      decay_bias=None, bonus=None, head_decay=None, decay_out=None, write_state: bool = True, beta=None,
                      qk_heads: int | None = None, unit_eps: float = 1e-6, q_scale: float = 1.0, prepared: bool | None = None) -> None:
    """A recurrence over a matrix state S [dk, dv] a head that decays and receives k_t v_t^T with every token.
    mode "channel_decay": o_t = S_(t-1)^T r_t + (sum_i r_i bonus_i k_i) v_t, then S_t = diag(w_t) S_(t-1) + k_t v_t^T with
    w_t = exp(-exp(log_decay_t + decay_bias)) per head and key channel. mode "head_decay": r, k, v pass silu first,
    S_t = head_decay S_(t-1) + k_t v_t^T, o_t = S_t^T r_t. r, k, log_decay [n, heads dk], v [n, heads dv] (blocks of
    columns of wider rows are fine); decay_bias, bonus float32 [heads dk]; head_decay float32 [heads]; state float32
    [slots, heads, dv, dk]; o float32 [n, heads dv], or None: the state moves on and nothing else is written. decay_out
    (or None): float32 [entries, heads, dk], receives the product of each entry's decays per key channel. write_state
    False: the state is only read. The last three serve long entries cut into segments (`matrix_state_chain`).
    mode "delta": the gated delta rule. S' = diag(w_t) S_(t-1), u_t = beta_t (v_t - S'^T k_t), S_t = S' + k_t u_t^T,
    o_t = S_t^T r_t, with r and k [n, qk_heads dk] made unit vectors per head (x / sqrt(sum x^2 + unit_eps)), r times
    q_scale; heads / qk_heads heads share one head of r and k; beta = sigmoid of `beta` [n, heads]; w_t =
    exp(-exp(head_decay_h) softplus(log_decay_t + decay_bias)) with head_decay the logarithm of each head's rate. Entries
    run in one piece (the recurrence's factor is not diagonal), so `decay_out` is not offered; instead a column's key
    channels are spread over neighbouring lanes, so that a token costs a few multiply-adds and shuffles on the way from one
    state to the next, and a prompt of one request spreads over heads x (dv / columns a block) blocks. `prepared`: True
    runs the two-launch form (unit vectors, decays and beta once a token, then a scan fed by asynchronous copies), False
    the one-launch form; None: the two-launch form for steps of more than four tokens an entry."""
    if mode not in ("channel_decay", "head_decay", "delta"):
        raise KernelError(f"matrix_state_scan: unknown mode {mode!r}")
    for t, name in ((r, "r"), (k, "k"), (v, "v")):
        _cols(t, name, r.dtype)
    n = r.shape[0]
    delta = mode == "delta"
    qk_heads = (qk_heads or heads) if delta else heads
    if qk_heads <= 0 or heads % qk_heads or r.shape[1] != qk_heads * dk or k.shape != r.shape or tuple(v.shape) != (n, heads * dv):
        raise KernelError("matrix_state_scan: r, k, v do not fit the heads")
    channel = mode == "channel_decay"
    if delta:
        _cols(log_decay, "log_decay", r.dtype)
        _cols(beta, "beta", r.dtype)
        _req(decay_bias, "decay_bias", torch.float32)
        _req(head_decay, "head_decay", torch.float32, 1)
        if tuple(log_decay.shape) != (n, heads * dk) or tuple(beta.shape) != (n, heads) or decay_bias.numel() != heads * dk or (
                head_decay.numel() != heads) or decay_out is not None:
            raise KernelError("matrix_state_scan: the delta rule's operands do not fit the heads")
    elif channel:
        _cols(log_decay, "log_decay", r.dtype)
        _req(decay_bias, "decay_bias", torch.float32)
        _req(bonus, "bonus", torch.float32)
        if log_decay.shape != r.shape or decay_bias.numel() != heads * dk or bonus.numel() != heads * dk:
            raise KernelError("matrix_state_scan: the decay's operands do not fit the heads")
    else:
        _req(head_decay, "head_decay", torch.float32, 1)
        if head_decay.numel() != heads:
            raise KernelError("matrix_state_scan: one decay a head")
    _req_state(state, "state", torch.float32)
    if o is not None:
        _req(o, "o", torch.float32, 2)
    elif not write_state:
        raise KernelError("matrix_state_scan: neither outputs nor the state are wanted")
    if tuple(state.shape[1:]) != (heads, dv, dk) or (o is not None and tuple(o.shape) != (n, heads * dv)):
        raise KernelError(f"matrix_state_scan: state {tuple(state.shape)} / o do not fit")
    for t, name in ((q_start, "q_start"), (start_pos, "start_pos"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    if decay_out is not None:
        _req(decay_out, "decay_out", torch.float32, 3)
        if tuple(decay_out.shape) != (start_pos.numel(), heads, dk):
            raise KernelError("matrix_state_scan: decay_out must be [entries, heads, dk]")
    if delta:       # a kernel of its own: a column's key channels spread over neighbouring lanes
        # steps with prompt portions (known from the shapes alone, so that a captured step stays what it was): unit vectors,
        # decays and beta once a token by a kernel of their own, then a scan that only moves rows
        scratch = None
        if prepared if prepared is not None else n > 4 * start_pos.numel():
            lib = library()
            lib.qi_delta_rule_scratch_floats.restype = C.c_longlong
            scratch = torch.empty(lib.qi_delta_rule_scratch_floats(n, heads, qk_heads, dk), dtype=torch.float32, device=r.device)
        _call("scan", "delta_rule_scan", library().qi_delta_rule_scan, _ptr(r), C.c_longlong(r.stride(0)), _ptr(k), C.c_longlong(k.stride(0)),
              _ptr(v), C.c_longlong(v.stride(0)), _ptr(log_decay), C.c_longlong(log_decay.stride(0)), _ptr(beta), C.c_longlong(beta.stride(0)),
              _code(r), _ptr(decay_bias), _ptr(head_decay), _ptr(state), C.c_longlong(state.stride(0)), _ptr(o), int(bool(write_state)),
              _ptr(q_start), _ptr(start_pos), _ptr(slot_ids), start_pos.numel(), heads, qk_heads, dk, dv, C.c_float(unit_eps),
              C.c_float(q_scale), _ptr(scratch), n, _stream())
        return
    _call("scan", "matrix_state_scan", library().qi_matrix_state_scan, 0 if channel else 1, _ptr(r), C.c_longlong(r.stride(0)), _ptr(k),
          C.c_longlong(k.stride(0)), _ptr(v), C.c_longlong(v.stride(0)), _ptr(log_decay), C.c_longlong(log_decay.stride(0) if channel else 0),
          _code(r), _ptr(decay_bias), _ptr(bonus), _ptr(head_decay), _ptr(state), C.c_longlong(state.stride(0)), _ptr(o),
          _ptr(decay_out), int(bool(write_state)), _ptr(q_start), _ptr(start_pos), _ptr(slot_ids), start_pos.numel(), heads, dk, dv,
          _stream())


def matrix_state_chain(seg_state, seg_decay, state, entry_seg, start_pos, slot_ids) -> None:
    """Between the two passes of `matrix_state_scan` over a long entry's segments: seg_state [segments, heads, dv, dk]
    holds every segment's own contribution and receives the state each segment starts from; seg_decay [segments, heads, dk]
    the product of each segment's decays; the requests' states (state [slots, heads, dv, dk]) move to their entries'
    ends. entry_seg [entries + 1]: the first segment of every entry."""
    _req(seg_state, "seg_state", torch.float32, 4)
    _req(seg_decay, "seg_decay", torch.float32, 3)
    _req_state(state, "state", torch.float32)
    segs, heads, dv, dk = seg_state.shape
    if tuple(state.shape[1:]) != (heads, dv, dk) or tuple(seg_decay.shape) != (segs, heads, dk):
        raise KernelError("matrix_state_chain: shapes do not agree")
    for t, name in ((entry_seg, "entry_seg"), (start_pos, "start_pos"), (slot_ids, "slot_ids")):
        _req(t, name, torch.int32, 1)
    if entry_seg.numel() != start_pos.numel() + 1:
        raise KernelError("matrix_state_chain: the segment list does not fit the entries")
    _call("scan", "matrix_state_chain", library().qi_matrix_state_chain, _ptr(seg_state), _ptr(seg_decay), _ptr(state),
          C.c_longlong(state.stride(0)), _ptr(entry_seg), _ptr(start_pos), _ptr(slot_ids), start_pos.numel(), heads, dk, dv, _stream())


def scaled_sum(a, b, sa: float, sb: float, out) -> None:
    """out = sa * a + sb * b in 32-bit; out float32 [n, h]. a and b are [n, h] each, or [parts, n, h]: the partial sums of
    a product whose contraction was split, added here in their order. Their types may differ."""
    _req(a, "a")
    _req(b, "b")
    _req(out, "out", torch.float32)
    for t in (a, b):
        if t.dim() not in (out.dim(), out.dim() + 1) or tuple(t.shape[-out.dim():]) != tuple(out.shape) or not t.shape[0]:
            raise KernelError("scaled_sum: shapes differ")
    ka = a.shape[0] if a.dim() > out.dim() else 1
    kb = b.shape[0] if b.dim() > out.dim() else 1
    _call("other", "scaled_sum", library().qi_scaled_sum, _ptr(a), ka, _code(a), _ptr(b), kb, _code(b), C.c_float(sa), C.c_float(sb),
          _ptr(out), C.c_longlong(out.numel()), _stream())


MATRIX_STATE_COLUMNS = 64      # value columns a block of `matrix_state_scan` owns (kColThreads in recurrent.cu)
_SCAN_BLOCKS: dict = {}


def matrix_state_scan_blocks(mode: str, dk: int, dtype) -> int:
    """How many blocks of `matrix_state_scan` (mode, key size, operand type) the device holds at a time; 0 when that
    cannot be told. For whoever cuts long entries into segments: a launch of whole waves wastes no time on a tail."""
    key = (mode, dk, dtype)
    if key not in _SCAN_BLOCKS:
        a_sm = int(library().qi_matrix_state_scan_blocks_per_sm(0 if mode == "channel_decay" else 1, int(dk), _DTYPE_CODE[dtype]))
        _SCAN_BLOCKS[key] = max(0, a_sm) * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _SCAN_BLOCKS[key]


def glu_clamped(gate_up, out, limit: float, alpha: float, interleaved: bool = False) -> None:
    """out = g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); gate and up side by side
    or interleaved in rows of gate_up [rows, 2 I]; out [rows, I]."""
    _req(gate_up, "gate_up", ndim=2)
    _req(out, "out", gate_up.dtype, 2)
    rows, inter = out.shape
    if tuple(gate_up.shape) != (rows, 2 * inter):
        raise KernelError("glu_clamped: shapes do not agree")
    _call("other", "glu_clamped", library().qi_glu_clamped, _ptr(gate_up), _ptr(out), _code(out), C.c_longlong(rows), inter,
          int(bool(interleaved)), C.c_float(limit), C.c_float(alpha), _stream())


def moe_tile_rows() -> int:
    return int(library().qi_moe_tile_rows())


def moe_route(logits, correction, ids, weights, scale: float) -> None:
    """Per token: softmax over all experts, the `top` largest of softmax + correction, weights = the chosen experts' softmax
    over their sum, times scale. logits float32 [n, E]; ids int32 [n, top]; weights float32 [n, top]."""
    _req(logits, "logits", torch.float32, 2)
    _req(ids, "ids", torch.int32, 2)
    _req(weights, "weights", torch.float32, 2)
    n, E = logits.shape
    if ids.shape != weights.shape or ids.shape[0] != n:
        raise KernelError("moe_route: shapes do not agree")
    if correction is not None:
        _req(correction, "correction", torch.float32, 1)
        if correction.numel() != E:
            raise KernelError("moe_route: one correction an expert")
    _call("gemm", "moe_route", library().qi_moe_route, _ptr(logits), _ptr(correction), _ptr(ids), _ptr(weights), n, E,
          ids.shape[1], C.c_float(scale), _stream())


def moe_group(ids, n_experts: int, offsets, order, place, tiles) -> None:
    """Sorts the (token, choice) pairs by expert on the device: offsets int32 [E + 1], order and place int32 [pairs],
    tiles int32 [max_tiles, 3] (expert or -1, first sorted row, rows)."""
    for t, name in ((ids, "ids"), (offsets, "offsets"), (order, "order"), (place, "place"), (tiles, "tiles")):
        _req(t, name, torch.int32)
    pairs = ids.numel()
    if offsets.numel() != n_experts + 1 or order.numel() != pairs or place.numel() != pairs or tiles.dim() != 2 or tiles.shape[1] != 3:
        raise KernelError("moe_group: shapes do not agree")
    _call("gemm", "moe_group", library().qi_moe_group, _ptr(ids), pairs, n_experts, moe_tile_rows(), tiles.shape[0], _ptr(offsets),
          _ptr(order), _ptr(place), _ptr(tiles), _stream())


def moe_gemm(x, w, y, tiles, order, top: int, gather: bool) -> None:
    """y[i] = w[expert of sorted row i] . x[order[i] // top if gather else i]. x [rows, K]; w [E, N, K]; y [pairs, N]."""
    _req(x, "x", ndim=2)
    _req(w, "w", ndim=3)
    _req(y, "y", ndim=2)
    _req(tiles, "tiles", torch.int32, 2)
    _req(order, "order", torch.int32)
    N, K = w.shape[1], w.shape[2]
    if x.shape[1] != K or y.shape[1] != N:
        raise KernelError(f"moe_gemm: shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    _call("gemm", "moe_gemm", library().qi_moe_gemm, _ptr(x), _code(x), _ptr(w), _code(w), _ptr(y), _code(y), _ptr(tiles),
          tiles.shape[0], _ptr(order), top, int(bool(gather)), N, K, C.c_longlong(K), C.c_longlong(N), x.shape[0], y.shape[0],
          w.shape[0], _stream())


def moe_gather(x, order, top: int, out) -> None:
    """out[i] = x[order[i] // top]: the tokens' rows in the experts' order. x [n, K]; out [pairs, K]."""
    _req(x, "x", ndim=2)
    _req(out, "out", x.dtype, 2)
    _req(order, "order", torch.int32)
    if out.shape[1] != x.shape[1] or order.numel() != out.shape[0]:
        raise KernelError("moe_gather: shapes do not agree")
    _call("gemm", "moe_gather", library().qi_moe_gather, _ptr(x), _code(x), _ptr(order), top, _ptr(out), out.shape[0], x.shape[0],
          x.shape[1], _stream())


def moe_gemm_by_expert(x, w, y, bounds, status) -> None:
    """y[rows of expert e] = x[rows of expert e] . w[e]^T through the tcgen05 product, one launch an expert. x [pairs, K]
    in the experts' order, w [E, N, K], y [pairs, N], bfloat16; bounds: E + 1 ascending row numbers, on the HOST."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 3)
    _req(y, "y", torch.bfloat16, 2)
    E, N, K = w.shape
    if x.shape[1] != K or y.shape[1] != N or x.shape[0] != y.shape[0] or len(bounds) != E + 1 or bounds[-1] > x.shape[0]:
        raise KernelError("moe_gemm_by_expert: shapes do not agree")
    arr = (C.c_int * (E + 1))(*bounds)
    _call("gemm", "moe_gemm_by_expert", library().qi_moe_gemm_by_expert, _ptr(x), _ptr(w), _ptr(y), arr, E, N, K, _ptr(status), _stream())


def moe_combine(y, place, weights, shared, out) -> None:
    """out[t] = sum_k weights[t, k] * y[place[t, k]] (+ shared[t]). y [n top, width]; out [n, width]."""
    _req(y, "y", ndim=2)
    _req(place, "place", torch.int32)
    _req(weights, "weights", torch.float32, 2)
    _req(out, "out", ndim=2)
    n, top = weights.shape
    width = out.shape[1]
    if y.shape != (n * top, width) or out.shape[0] != n or place.numel() != n * top:
        raise KernelError("moe_combine: shapes do not agree")
    if shared is not None:
        _req(shared, "shared", y.dtype, 2)
        if shared.shape != out.shape:
            raise KernelError("moe_combine: the shared output does not fit")
    _call("gemm", "moe_combine", library().qi_moe_combine, _ptr(y), _code(y), _ptr(place), _ptr(weights), _ptr(shared), _ptr(out),
          _code(out), n, top, width, _stream())


class _LeadRows:
    """The single-token entries at the front of a mixed step, as the batch fields the attention kernels read."""

    def __init__(self, batch, lead: int):
        self.q_start, self.start_pos, self.n_requests = batch.q_start[:lead + 1], batch.start_pos[:lead], lead
        self.positions, self.token_req = batch.positions[:lead], batch.token_req[:lead]


def gated_attention_mma_supported(nq: int, nkv: int, d: int, dv: int) -> bool:
    """Whether the tensor-core kernel for separate key and value sizes takes this geometry (bfloat16 only)."""
    return bool(library().qi_gated_attention_mma_supported(nq, nkv, d, dv))


def gated_attention(q, out, k_pages, v_pages, block_table, batch, nq, nkv, d, dv, scale: float, window: int, chunk: int, gate,
                    status, impl: str | None = None, softcap: float = 0.0, out_scale: float = 1.0, sink=None,
                    key_ranges: int | None = None) -> None:
    """Attention with separate key and value sizes, an optional chunk bound and an optional output gate, by the
    kernel that fits: "mma" (bfloat16, head sizes that are multiples of 8 up to 128: flash form on the tensor
    cores, tiles found on the device from the step's arrays) or "generic" (32-bit arithmetic, any sizes). A step
    with prompt portions whose keys and values are both of size 128 goes to "tcgen05": the portions' query tiles
    to the tcgen05 flash kernel (chunk bound and gate included), the single tokens in front of them to "mma".
    `softcap` c > 0 (a score s becomes c tanh(s / c)), `out_scale` (a factor on the result) and `sink` (float32 [nq]:
    exp(sink[h]) once more in the softmax's denominator of head h) are known to all three. A step of single tokens on
    "mma" cuts every token's keys into `key_ranges` ranges over separate CTAs (None: as many as fill the device, from
    the longest context and the window, so that a captured step serves its whole context bucket) and adds the parts
    in a second kernel."""
    if impl is None and q.dtype == torch.bfloat16 and d == dv and not batch.all_decode and batch.tile_req.numel() and (
            gate is None or (gate.stride(0) % 8 == 0 and gate.data_ptr() % 16 == 0)) and attention_prefill_tcgen05_supported(
            nq, nkv, d, k_pages.shape[2], block_table.shape[1]):
        impl = "tcgen05"
    if impl == "tcgen05":
        lead = batch.n_lead_decode
        if lead:
            gated_attention(q[:lead], out[:lead], k_pages, v_pages, block_table[:lead], _LeadRows(batch, lead), nq, nkv, d, dv,
                            scale, window, chunk, gate[:lead] if gate is not None else None, status, impl="mma", softcap=softcap,
                            out_scale=out_scale, sink=sink)
        return attention_prefill(q, out, k_pages, v_pages, block_table, batch.q_start, batch.start_pos, batch.tile_req,
                                 batch.tile_q0, nq, nkv, d, scale, window, status, impl="tcgen05", max_kv_len=batch.max_kv_len,
                                 key_ranges=1 if chunk else None, chunk=chunk, gate=gate, softcap=softcap, out_scale=out_scale,
                                 sink=sink)
    if impl is None:
        impl = "mma" if q.dtype == torch.bfloat16 and gated_attention_mma_supported(nq, nkv, d, dv) and (
            gate is None or gate.stride(0) % 2 == 0) else "generic"
    if impl == "generic":
        return attention_generic(q, out, k_pages, v_pages, block_table, batch.positions, batch.token_req, nq, nkv, d, scale,
                                 window, status, chunk=chunk, gate=gate, softcap=softcap, out_scale=out_scale, sink=sink)
    if sink is not None:
        _req(sink, "sink", torch.float32, 1)
        if sink.numel() != nq:
            raise KernelError("gated_attention: one sink a query head")
    _req(q, "q", torch.bfloat16, 2)
    _req(out, "out", torch.bfloat16, 2)
    _req(k_pages, "k_pages", torch.bfloat16, 4)
    _req(v_pages, "v_pages", torch.bfloat16, 4)
    _req(block_table, "block_table", torch.int32, 2)
    n = q.shape[0]
    if q.shape[1] != nq * d or tuple(out.shape) != (n, nq * dv):
        raise KernelError(f"gated_attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not match {nq} heads of {d} / {dv}")
    if tuple(k_pages.shape[1:]) != (nkv, k_pages.shape[2], d) or tuple(v_pages.shape) != (k_pages.shape[0], nkv, k_pages.shape[2], dv):
        raise KernelError(f"gated_attention: pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} do not fit")
    ldg = 0
    if gate is not None:
        if not gate.is_cuda or gate.dtype != q.dtype or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != out.shape:
            raise KernelError("gated_attention: the gate must be [n, nq dv] in q's type with contiguous rows")
        ldg = gate.stride(0)
    ranges, ws = 1, None
    if getattr(batch, "all_decode", False) and n <= 65535:
        keys = min(window or batch.max_kv_len, chunk or batch.max_kv_len, batch.max_kv_len)
        ranges = key_ranges or max(1, min(-(-keys // 128), 296 // max(n * nq, 1), 64))
        if ranges > 1:
            ws = torch.empty(n * nq * ranges * (dv + 2), dtype=torch.float32, device=q.device)
    _call("attention", "gated_attention_mma", library().qi_gated_attention_mma_ranges, _ptr(q), _ptr(out), _ptr(k_pages), _ptr(v_pages),
          _ptr(block_table), block_table.shape[1], k_pages.shape[2], k_pages.shape[0], _ptr(batch.q_start), _ptr(batch.start_pos),
          batch.n_requests, n, nq, nkv, d, dv, C.c_float(scale), C.c_float(softcap or 0.0), C.c_float(out_scale), int(window or 0),
          int(chunk or 0), _ptr(gate), C.c_longlong(ldg), _ptr(sink), ranges, _ptr(ws),
          _ptr(status), _stream())
