"""Torch-facing operators over the C ABI: each one allocates its outputs with torch, passes raw device
pointers and torch's current CUDA stream to libpq_b200.so, and is registered as a torch custom op
(namespace ``pq_b200``) with a fake implementation for shape propagation.

CUDA tensors only: a CPU tensor raises AssertionError, as the reference's ``quant_rows`` does
(deploy/int8_exec.py:221).  There is no fallback implementation.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _lib

Tensor = torch.Tensor

_DT = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16}
# rank-32 term of the fused GEMM: tcgen05 tensor cores (True) or warp-level mma.sync in the epilogue (False)
LOWRANK_ON_TENSOR_CORES = True
# epilogue variants of pq_int8_gemm_ex
EPI_ACCUMULATE = 1      # out += y (both rounded to the output type first)
EPI_GELU_TANH = 2       # out = gelu_tanh(y rounded to the output type)
MAX_OUT_MORE = 7        # further output buffers of pq_int8_gemm_bcast
_status_words: Dict[int, Tensor] = {}


def _dt(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise TypeError(f"pq_b200 supports bfloat16 and float16, got {dtype}") from None


def _stream(t: Tensor) -> int:
    """Raw handle of torch's current stream on the tensor's device (the cheap private accessor when it exists)."""
    idx = t.device.index
    try:
        return torch._C._cuda_getCurrentRawStream(idx)
    except AttributeError:                      # pragma: no cover
        return torch.cuda.current_stream(t.device).cuda_stream


class _on_device:
    """`with torch.cuda.device(...)` only when the tensor lives on another device than the current one: the
    context manager costs several microseconds, which matters for the small 1K-stage layers."""
    __slots__ = ("ctx",)

    def __init__(self, t: Tensor):
        self.ctx = None if t.device.index == torch.cuda.current_device() else torch.cuda.device(t.device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None:
            self.ctx.__exit__(*a)


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _written_in_place(t: Tensor) -> None:
    """The library writes through raw pointers, which torch cannot see: tell it that `t` changed, so that anything
    keyed on the tensor's version counter (autograd's saved-tensor check, SharedInputGroup's cache) notices."""
    if not t.is_inference():
        torch.autograd.graph.increment_version(t)


def tensor_version(t: Tensor) -> int:
    """Version counter of `t`, or -1 for inference tensors (which do not keep one)."""
    return -1 if t.is_inference() else t._version


_lib_handle = None


def _LIB():
    global _lib_handle
    if _lib_handle is None:
        _lib_handle = _lib.load()
    return _lib_handle


def status_word(device: torch.device) -> Tensor:
    """Per-device workspace whose word 0 the GEMM kernels set when a bounded wait gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(_lib.GEMM_WORKSPACE_BYTES // 4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_device_status(device=None, clear: bool = True) -> None:
    """Synchronises and raises RuntimeError if any GEMM launched so far on `device` gave up a wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(dev)
    raw = ctypes.c_int32(0)
    with torch.cuda.device(dev):
        rc = _lib.load().pq_read_status_word(w.data_ptr(), ctypes.byref(raw), int(clear),
                                             torch.cuda.current_stream(dev).cuda_stream)
    if rc == _lib.PQ_ERR_TIMEOUT:
        raise RuntimeError(f"pq_b200: a device-side wait gave up (status word 0x{raw.value & 0xffffffff:08x})")
    _lib.check(rc, "pq_read_status_word")


def _rows_ok(x2: Tensor) -> Tensor:
    """Row-strided views are consumed in place; anything the kernels cannot address is made contiguous."""
    assert x2.dim() == 2 and x2.is_cuda
    if x2.stride(1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8 != 0) or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    return x2


# ------------------------------------------------------------------------------------------------ quantisation
def _quant_rows_impl(x2: Tensor) -> Tuple[Tensor, Tensor]:
    x2 = _rows_ok(x2)
    M, K = x2.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x2.device)
    s = torch.empty((M,), dtype=torch.float32, device=x2.device)
    ld = x2.stride(0) if M > 1 else max(K, x2.stride(0))
    with _on_device(x2):
        rc = _LIB().pq_quant_rows(x2.data_ptr(), _dt(x2.dtype), M, K, ld, q.data_ptr(), s.data_ptr(), _stream(x2))
    if rc:
        _lib.check(rc, f"pq_quant_rows(M={M}, K={K})")
    return q, s


def _quant_rows_g32_impl(x2: Tensor) -> Tuple[Tensor, Tensor]:
    x2 = _rows_ok(x2)
    M, K = x2.shape
    assert K % 32 == 0, K
    q = torch.empty((M, K), dtype=torch.int8, device=x2.device)
    s = torch.empty((M, K // 32), dtype=torch.float32, device=x2.device)
    ld = x2.stride(0) if M > 1 else max(K, x2.stride(0))
    with _on_device(x2):
        rc = _LIB().pq_quant_rows_g32(x2.data_ptr(), _dt(x2.dtype), M, K, ld, q.data_ptr(), s.data_ptr(),
                                           _stream(x2))
    _lib.check(rc, f"pq_quant_rows_g32(M={M}, K={K})")
    return q, s


def cat_sources_ok(x0: Tensor, x1: Tensor) -> bool:
    """Whether the two-source entry points take x0 / x1 as they are (the seam on a 64-element boundary, rows up to
    16384 elements, aligned row-strided views)."""
    def ok(t):
        return (t.dim() == 2 and t.is_cuda and t.stride(1) == 1 and (t.shape[0] <= 1 or t.stride(0) % 8 == 0)
                and t.data_ptr() % 16 == 0)
    return (ok(x0) and ok(x1) and x0.dtype == x1.dtype and x0.dtype in _DT and x0.shape[0] == x1.shape[0]
            and x0.device == x1.device and x0.shape[1] % 64 == 0 and x1.shape[1] % 8 == 0
            and x0.shape[1] + x1.shape[1] <= 16384)


def quant_rows_cat(x0: Tensor, x1: Tensor) -> Tuple[Tensor, Tensor]:
    """quant_rows(torch.cat([x0, x1], 1)) without the concatenated tensor (pq_quant_rows_cat)."""
    assert cat_sources_ok(x0, x1)
    M, K0 = x0.shape
    K1 = x1.shape[1]
    q = torch.empty((M, K0 + K1), dtype=torch.int8, device=x0.device)
    s = torch.empty((M,), dtype=torch.float32, device=x0.device)
    with _on_device(x0):
        rc = _LIB().pq_quant_rows_cat(x0.data_ptr(), K0, x0.stride(0) if M > 1 else max(K0, x0.stride(0)), x1.data_ptr(), K1,
                                      x1.stride(0) if M > 1 else max(K1, x1.stride(0)), _dt(x0.dtype), M, q.data_ptr(),
                                      s.data_ptr(), _stream(x0))
    if rc:
        _lib.check(rc, f"pq_quant_rows_cat(M={M}, K={K0}+{K1})")
    return q, s


def lowrank_down_cat(x0: Tensor, x1: Tensor, a_t: Tensor) -> Tensor:
    """lowrank_down(torch.cat([x0, x1], 1), a_t) without the concatenated tensor (pq_lowrank_down_cat)."""
    assert cat_sources_ok(x0, x1)
    M, K0 = x0.shape
    K1 = x1.shape[1]
    R = a_t.shape[0]
    assert R in LOWRANK_DOWN_COLS and a_t.dtype == x0.dtype and a_t.shape == (R, K0 + K1) and a_t.is_contiguous()
    t = torch.empty((M, R), dtype=x0.dtype, device=x0.device)
    ws = status_word(x0.device)
    with _on_device(x0):
        rc = _LIB().pq_lowrank_down_cat(x0.data_ptr(), K0, x0.stride(0) if M > 1 else max(K0, x0.stride(0)), x1.data_ptr(), K1,
                                        x1.stride(0) if M > 1 else max(K1, x1.stride(0)), _dt(x0.dtype), a_t.data_ptr(),
                                        K0 + K1, R, t.data_ptr(), R, M, ws.data_ptr(), ws.numel() * 4, _stream(x0))
    if rc:
        _lib.check(rc, f"pq_lowrank_down_cat(M={M}, K={K0}+{K1})")
    return t


def adaln_quant_rows(x2: Tensor, scale: Tensor, shift: Tensor, eps: float = 1e-6, rows_per_sample: int = 0,
                     want_modulated: bool = True) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """(q, s, z) with z = LayerNorm(x2) * (1 + scale) + shift and (q, s) = quant_rows(z), in one pass over x2
    (pq_adaln_quant_rows).  scale / shift: [K] or [samples, K]; row m belongs to sample m // rows_per_sample.
    z is None unless want_modulated."""
    x2 = _rows_ok(x2)
    M, K = x2.shape
    scale = scale.reshape(-1, K); shift = shift.reshape(-1, K)
    assert scale.shape == shift.shape and scale.dtype == x2.dtype and shift.dtype == x2.dtype, (scale.shape, shift.shape)
    assert scale.is_cuda and shift.is_cuda and K % 8 == 0 and K <= 16384, K
    samples = scale.shape[0]
    if samples == 1:
        rows_per_sample = 0
    else:
        assert rows_per_sample > 0 and samples * rows_per_sample >= M, (samples, rows_per_sample, M)
    scale = scale.contiguous(); shift = shift.contiguous()
    q = torch.empty((M, K), dtype=torch.int8, device=x2.device)
    s = torch.empty((M,), dtype=torch.float32, device=x2.device)
    z = torch.empty((M, K), dtype=x2.dtype, device=x2.device) if want_modulated else None
    ld = x2.stride(0) if M > 1 else max(K, x2.stride(0))
    with _on_device(x2):
        rc = _LIB().pq_adaln_quant_rows(x2.data_ptr(), _dt(x2.dtype), M, K, ld, scale.data_ptr(), shift.data_ptr(), K,
                                        int(rows_per_sample), float(eps), _ptr(z), K, q.data_ptr(), s.data_ptr(), _stream(x2))
    if rc:
        _lib.check(rc, f"pq_adaln_quant_rows(M={M}, K={K})")
    return q, s, z


def _gather_quant_rows_impl(canvas: Tensor, row_idx: Tensor) -> Tuple[Tensor, Tensor]:
    canvas = _rows_ok(canvas)
    assert row_idx.is_cuda and row_idx.dtype == torch.int32 and row_idx.dim() == 1 and row_idx.is_contiguous()
    rows, K = canvas.shape
    M = row_idx.numel()
    q = torch.empty((M, K), dtype=torch.int8, device=canvas.device)
    s = torch.empty((M,), dtype=torch.float32, device=canvas.device)
    with _on_device(canvas):
        rc = _LIB().pq_gather_quant_rows(canvas.data_ptr(), _dt(canvas.dtype), rows, K, max(K, canvas.stride(0)),
                                              row_idx.data_ptr(), M, q.data_ptr(), s.data_ptr(), _stream(canvas))
    _lib.check(rc, f"pq_gather_quant_rows(M={M}, K={K})")
    return q, s


def _gather_rows_impl(canvas: Tensor, row_idx: Tensor) -> Tensor:
    canvas = _rows_ok(canvas)
    assert row_idx.is_cuda and row_idx.dtype == torch.int32 and row_idx.dim() == 1 and row_idx.is_contiguous()
    rows, K = canvas.shape
    M = row_idx.numel()
    out = torch.empty((M, K), dtype=canvas.dtype, device=canvas.device)
    with _on_device(canvas):
        rc = _LIB().pq_gather_rows(canvas.data_ptr(), _dt(canvas.dtype), rows, K, max(K, canvas.stride(0)),
                                        row_idx.data_ptr(), M, out.data_ptr(), K, _stream(canvas))
    _lib.check(rc, f"pq_gather_rows(M={M}, K={K})")
    return out


# ------------------------------------------------------------------------------------------------ low-rank down-projection
# True: t = x @ lr_A runs on this library's streaming tcgen05 kernel; False: torch's matmul, as the reference does
LOWRANK_DOWN_NATIVE = True
# rows from which the library's own kernel is used.  Measured back to back on inputs rotating through HBM (native /
# torch's cuBLAS matmul, us): 66048 rows 308 / 349 at K = 15360 and 70 / 76 at K = 3072; 33024 rows 162 / 164 and
# 38 / 37; 16896 rows 84 / 79 and 22 / 21; 8256 rows 44 / 43 and 16 / 15; 4608 rows 34 / 32 and 16 / 15 (both at the
# launch floor).  Below 33024 rows the library call is ahead by 2-8 % (its split-K fills the SMs when there are fewer
# 64-row tiles than SMs); the path stays on this library's kernel all the same, the difference being under 1 % of a
# Linear's forward.
LOWRANK_DOWN_MIN_ROWS = 1
# output widths the kernel is built for: one rank-32 factor, or up to four side by side
LOWRANK_DOWN_COLS = (32, 64, 96, 128)


def lowrank_down(x2: Tensor, a_t: Tensor) -> Tensor:
    """t [M, R] = x2 [M, K] @ A [K, R] with A given transposed (a_t [R, K] contiguous; R in LOWRANK_DOWN_COLS), fp32
    accumulation, rounded to the activation dtype (pq_lowrank_down)."""
    assert x2.is_cuda and x2.dim() == 2 and x2.stride(1) == 1 and x2.dtype in _DT
    R = a_t.shape[0]
    assert R in LOWRANK_DOWN_COLS, f"{R} columns; supported: {LOWRANK_DOWN_COLS}"
    assert a_t.dtype == x2.dtype and a_t.shape == (R, x2.shape[1]) and a_t.is_contiguous() and a_t.device == x2.device
    M, K = x2.shape
    t = torch.empty((M, R), dtype=x2.dtype, device=x2.device)
    ws = status_word(x2.device)
    ld = x2.stride(0) if M > 1 else max(K, x2.stride(0))
    with _on_device(x2):
        rc = _LIB().pq_lowrank_down(x2.data_ptr(), _dt(x2.dtype), ld, a_t.data_ptr(), K, R, t.data_ptr(), R, M, K,
                                    ws.data_ptr(), ws.numel() * 4, _stream(x2))
    _lib.check(rc, f"pq_lowrank_down(M={M}, K={K})")
    return t


def lowrank_down_ok(x2: Tensor) -> bool:
    """Shapes pq_lowrank_down takes without a copy and is the faster choice for."""
    return (LOWRANK_DOWN_NATIVE and x2.is_cuda and x2.dtype in _DT and x2.dim() == 2 and x2.stride(1) == 1
            and x2.shape[1] % 8 == 0 and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0
            and x2.shape[0] >= LOWRANK_DOWN_MIN_ROWS)


# ------------------------------------------------------------------------------------------------ 4-bit storage
def pack_int4(codes: Tensor) -> Tensor:
    """int8 codes in [-8, 7], shape [N, K] with K even -> uint8 [N, K/2]: element 2b in the low nibble of byte b,
    element 2b+1 in the high nibble (two's complement).  Plain tensor arithmetic: done once per layer, on any device."""
    assert codes.dtype == torch.int8 and codes.dim() == 2 and codes.shape[1] % 2 == 0
    assert int(codes.min()) >= -8 and int(codes.max()) <= 7, "codes do not fit four bits"
    u = codes.to(torch.int16) & 0xF
    return (u[:, 0::2] | (u[:, 1::2] << 4)).to(torch.uint8).contiguous()


def unpack_int4(packed: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """uint8 [N, K/2] packed nibbles -> int8 [N, K] on the device (pq_unpack_int4)."""
    assert packed.is_cuda and packed.dtype == torch.uint8 and packed.dim() == 2 and packed.is_contiguous()
    N, K = packed.shape[0], packed.shape[1] * 2
    assert K % 32 == 0, f"K={K} must be a multiple of 32"
    if out is None:
        out = torch.empty((N, K), dtype=torch.int8, device=packed.device)
    assert out.shape == (N, K) and out.dtype == torch.int8 and out.is_contiguous() and out.device == packed.device
    with _on_device(packed):
        rc = _LIB().pq_unpack_int4(packed.data_ptr(), K // 2, out.data_ptr(), K, N, K, _stream(packed))
    _lib.check(rc, f"pq_unpack_int4(N={N}, K={K})")
    _written_in_place(out)
    return out


# ------------------------------------------------------------------------------------------------ GEMM
def epilogue_supported(N: int, out_stride0: int, out_ptr: int, has_lowrank: bool, rank: int = 32) -> bool:
    """Whether pq_int8_gemm_ex takes this problem (its variants live in the CTA-pair kernel's vector stores)."""
    return N % 32 == 0 and out_stride0 % 8 == 0 and out_ptr % 16 == 0 and (not has_lowrank or rank == 32)


def check_gemm_extents(M: int, N: int, K: int, s_row: Tensor, w_scale: Tensor, bias: Optional[Tensor],
                        t: Optional[Tensor], lb: Optional[Tensor], lb_t: Optional[Tensor] = None,
                        s_lo: Optional[Tensor] = None, m_hi: Optional[int] = None) -> None:
    """The C ABI receives bare pointers, so a scale, bias or low-rank tensor that is too short would be read out of
    bounds on the device.  Every operand's extent is checked here, on the host, before anything is launched
    (AssertionError, like the reference's shape asserts)."""
    assert s_row.numel() == M, f"s_row has {s_row.numel()} entries for {M} rows"
    assert w_scale.numel() == N, f"w_scale has {w_scale.numel()} entries for {N} output channels"
    assert bias is None or bias.numel() == N, f"bias has {bias.numel()} entries for {N} output channels"
    assert s_lo is None or s_lo.numel() == N, f"low-tier scale has {s_lo.numel()} entries for {N} output channels"
    assert m_hi is None or 0 <= int(m_hi) <= M, f"m_hi={m_hi} outside [0, {M}]"
    assert (t is None) == (lb is None), "t and lb go together"
    if t is not None:
        assert t.dim() == 2 and lb.dim() == 2 and t.shape[0] == M and lb.shape == (t.shape[1], N), \
            f"low-rank operands t {tuple(t.shape)} / lb {tuple(lb.shape)} do not fit [M={M}, R] / [R, N={N}]"
        assert lb_t is None or tuple(lb_t.shape) == (N, t.shape[1]), f"lb_t {tuple(lb_t.shape)} is not [N, R]"


def _gemm_impl(xq: Tensor, s_row: Tensor, w_int8: Tensor, w_scale: Tensor, bias: Optional[Tensor],
               t: Optional[Tensor], lb: Optional[Tensor], out_dtype: torch.dtype,
               dbg_acc: Optional[Tensor] = None, w_lo: Optional[Tensor] = None, s_lo: Optional[Tensor] = None,
               m_hi: Optional[int] = None, lb_t: Optional[Tensor] = None, epilogue: int = 0,
               out: Optional[Tensor] = None, out_more: Optional[Sequence[Tensor]] = None,
               gate: Optional[Tensor] = None, gate_rows: int = 0) -> Tensor:
    assert xq.is_cuda and xq.dtype == torch.int8 and xq.dim() == 2 and xq.stride(1) == 1
    assert w_int8.dtype == torch.int8 and w_int8.dim() == 2 and w_int8.stride(1) == 1
    M, K = xq.shape
    N = w_int8.shape[0]
    assert w_int8.shape[1] == K, (w_int8.shape, K)
    assert K % 16 == 0, f"K={K} must be a multiple of 16"
    assert s_row.dtype == torch.float32 and w_scale.dtype == torch.float32
    check_gemm_extents(M, N, K, s_row, w_scale, bias, t, lb, lb_t, s_lo, m_hi if w_lo is not None else None)
    s_row = s_row.contiguous(); w_scale = w_scale.contiguous()
    if bias is not None:
        assert bias.dtype == torch.float32
        bias = bias.contiguous()
    if xq.stride(0) % 16 != 0 or xq.data_ptr() % 16 != 0:
        xq = xq.contiguous()
    if w_int8.stride(0) % 16 != 0 or w_int8.data_ptr() % 16 != 0:
        w_int8 = w_int8.contiguous()
    if out is None:
        assert not (epilogue & EPI_ACCUMULATE), "accumulation needs the tensor to add onto"
        out = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1 and out.device == xq.device
    R = 0
    ldt = ldb = 0
    if t is not None:
        assert lb is not None and t.dtype == out_dtype and lb.dtype == out_dtype, (t.dtype, lb.dtype, out_dtype)
        if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
            t = t.contiguous()
        if lb.stride(1) != 1 or lb.stride(0) % 8 != 0 or lb.data_ptr() % 16 != 0:
            lb = lb.contiguous()
        R = t.shape[1]
        ldt, ldb = t.stride(0), lb.stride(0)
        if M == 1:
            ldt = max(ldt, R)
        if lb_t is None and R == 32 and LOWRANK_ON_TENSOR_CORES:
            lb_t = lb.t().contiguous()        # K-major copy for the tcgen05 low-rank path (callers may cache it)
        if lb_t is not None:
            assert lb_t.shape == (N, R) and lb_t.dtype == out_dtype and lb_t.is_contiguous()
    ws = status_word(xq.device)
    lib = _LIB()
    ldx = xq.stride(0) if M > 1 else max(K, xq.stride(0))
    ldo = out.stride(0) if M > 1 else max(N, out.stride(0))
    if out_more:
        # further destinations of the output stores (pq_int8_gemm_bcast): same extent, dtype and row stride as `out`;
        # they may live on other GPUs of the node (peer memory mapped into this process)
        assert w_lo is None and dbg_acc is None and len(out_more) <= MAX_OUT_MORE, len(out_more)
        assert epilogue_supported(N, ldo, out.data_ptr(), t is not None, R or 32), "shape needs the CTA-pair kernel"
        for o in out_more:
            assert o.shape == (M, N) and o.dtype == out_dtype and o.stride(1) == 1 and o.is_cuda, (o.shape, o.dtype)
            assert (o.stride(0) if M > 1 else ldo) == ldo and o.data_ptr() % 16 == 0, (o.stride(), ldo)
        ptrs = (ctypes.c_void_p * len(out_more))(*[o.data_ptr() for o in out_more])
        with _on_device(xq):
            rc = lib.pq_int8_gemm_bcast(xq.data_ptr(), ldx, s_row.data_ptr(), w_int8.data_ptr(), w_int8.stride(0),
                                        w_scale.data_ptr(), _ptr(bias), _ptr(t), ldt, _ptr(lb), ldb, _ptr(lb_t), R,
                                        _dt(out_dtype), out.data_ptr(), ptrs, len(out_more), _dt(out_dtype), ldo,
                                        M, N, K, int(epilogue), ws.data_ptr(), ws.numel() * 4, _stream(xq))
        if rc:
            _lib.check(rc, f"pq_int8_gemm_bcast(M={M}, N={N}, K={K}, copies={len(out_more)})")
        _written_in_place(out)
        for o in out_more:
            _written_in_place(o)
        return out
    if gate is not None:
        # out = out + gate[sample] * y (pq_int8_gemm_gated): gate [samples, N] in the output type; rows of sample b are
        # [b * gate_rows, (b + 1) * gate_rows)
        assert w_lo is None and dbg_acc is None and not out_more
        gate = gate.reshape(-1, N)
        assert gate.is_cuda and gate.dtype == out_dtype and gate.device == xq.device, (gate.dtype, out_dtype)
        assert gate.shape[0] == 1 or (gate_rows > 0 and gate.shape[0] * gate_rows >= M), (gate.shape, gate_rows, M)
        if gate.stride(1) != 1 or gate.stride(0) % 8 != 0 or gate.data_ptr() % 16 != 0:
            gate = gate.contiguous()
        assert epilogue_supported(N, ldo, out.data_ptr(), t is not None, R or 32), "shape needs the CTA-pair kernel"
        with _on_device(xq):
            rc = lib.pq_int8_gemm_gated(xq.data_ptr(), ldx, s_row.data_ptr(), w_int8.data_ptr(), w_int8.stride(0),
                                        w_scale.data_ptr(), _ptr(bias), _ptr(t), ldt, _ptr(lb), ldb, _ptr(lb_t), R,
                                        _dt(out_dtype), gate.data_ptr(), gate.stride(0) if gate.shape[0] > 1 else N,
                                        int(gate_rows) if gate.shape[0] > 1 else 0, out.data_ptr(), _dt(out_dtype), ldo,
                                        M, N, K, int(epilogue), ws.data_ptr(), ws.numel() * 4, _stream(xq))
        if rc:
            _lib.check(rc, f"pq_int8_gemm_gated(M={M}, N={N}, K={K})")
        _written_in_place(out)
        return out
    with _on_device(xq):
        if epilogue:
            assert w_lo is None and dbg_acc is None
            rc = lib.pq_int8_gemm_ex(xq.data_ptr(), ldx, s_row.data_ptr(), w_int8.data_ptr(), w_int8.stride(0),
                                     w_scale.data_ptr(), _ptr(bias), _ptr(t), ldt, _ptr(lb), ldb, _ptr(lb_t), R,
                                     _dt(out_dtype), out.data_ptr(), _dt(out_dtype), ldo,
                                     M, N, K, int(epilogue), ws.data_ptr(), ws.numel() * 4, _stream(xq))
        elif w_lo is None:
            rc = lib.pq_int8_gemm(xq.data_ptr(), ldx, s_row.data_ptr(), w_int8.data_ptr(), w_int8.stride(0),
                                  w_scale.data_ptr(), _ptr(bias), _ptr(t), ldt, _ptr(lb), ldb, _ptr(lb_t), R,
                                  _dt(out_dtype), out.data_ptr(), _dt(out_dtype), ldo, M, N, K, ws.data_ptr(), ws.numel() * 4,
                                  _ptr(dbg_acc), _stream(xq))
        else:
            assert w_lo.shape == w_int8.shape and w_lo.stride() == w_int8.stride() and s_lo is not None
            rc = lib.pq_int8_gemm_grouped(xq.data_ptr(), ldx, s_row.data_ptr(), w_int8.data_ptr(),
                                          w_scale.data_ptr(), w_lo.data_ptr(), s_lo.contiguous().data_ptr(),
                                          w_int8.stride(0), _ptr(bias), _ptr(t), ldt, _ptr(lb), ldb, _ptr(lb_t), R,
                                          _dt(out_dtype), out.data_ptr(), _dt(out_dtype), ldo, int(m_hi), M, N, K,
                                          ws.data_ptr(), ws.numel() * 4, _stream(xq))
    if rc:
        _lib.check(rc, f"pq_int8_gemm(M={M}, N={N}, K={K})")
    if epilogue & EPI_ACCUMULATE:
        _written_in_place(out)
    return out


def _gemm_g32_impl(xq: Tensor, s_a: Tensor, w_int8: Tensor, s_w_gm: Tensor, bias: Optional[Tensor],
                   out_dtype: torch.dtype) -> Tensor:
    """s_a [M, K/32]; s_w_gm [K/32, N] (group-major)."""
    assert xq.is_cuda and xq.dtype == torch.int8 and xq.dim() == 2 and w_int8.dtype == torch.int8
    M, K = xq.shape
    N = w_int8.shape[0]
    assert w_int8.shape[1] == K and K % 128 == 0, (w_int8.shape, K)
    assert s_a.shape == (M, K // 32) and s_w_gm.shape == (K // 32, N), (s_a.shape, s_w_gm.shape)
    assert bias is None or bias.numel() == N, f"bias has {bias.numel()} entries for {N} output channels"
    xq = xq.contiguous(); w_int8 = w_int8.contiguous()
    s_a = s_a.contiguous().float(); s_w_gm = s_w_gm.contiguous().float()
    if bias is not None:
        bias = bias.contiguous().float()
    out = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    ws = status_word(xq.device)
    with _on_device(xq):
        rc = _LIB().pq_int8_gemm_g32(xq.data_ptr(), K, s_a.data_ptr(), w_int8.data_ptr(), K, s_w_gm.data_ptr(),
                                          _ptr(bias), out.data_ptr(), _dt(out_dtype), N, M, N, K, ws.data_ptr(),
                                          ws.numel() * 4, _stream(xq))
    _lib.check(rc, f"pq_int8_gemm_g32(M={M}, N={N}, K={K})")
    return out


def _dequant_epilogue_impl(acc: Tensor, s_row: Tensor, s_col: Tensor, bias: Optional[Tensor],
                           out_dtype: torch.dtype) -> Tensor:
    assert acc.is_cuda and acc.dtype == torch.int32 and acc.is_contiguous()
    M, N = acc.shape
    out = torch.empty((M, N), dtype=out_dtype, device=acc.device)
    with _on_device(acc):
        rc = _LIB().pq_dequant_epilogue(acc.data_ptr(), s_row.contiguous().data_ptr(),
                                             s_col.contiguous().data_ptr(), _ptr(bias), out.data_ptr(),
                                             _dt(out_dtype), M, N, _stream(acc))
    _lib.check(rc, "pq_dequant_epilogue")
    return out


def check_scatter_extents(m_act: int, canvas_rows: int, tokens: Tensor, ptr: Tensor, src: Tensor, beta: Tensor) -> None:
    """Extents of the contributor lists (their contents are trusted: they come from routing.build_route_plan)."""
    assert tokens.dim() == 1 and ptr.dim() == 1 and src.dim() == 1 and beta.dim() == 1
    assert ptr.numel() == tokens.numel() + 1, f"ptr has {ptr.numel()} entries for {tokens.numel()} tokens"
    assert src.numel() == beta.numel(), f"{src.numel()} sources but {beta.numel()} weights"
    assert tokens.numel() <= canvas_rows, f"{tokens.numel()} touched tokens on a canvas of {canvas_rows}"
    assert src.numel() == 0 or m_act > 0, "contributors without rows to take them from"


def _scatter_rows_impl(y: Tensor, tokens: Tensor, ptr: Tensor, src: Tensor, beta: Tensor, canvas: Tensor) -> None:
    assert y.is_cuda and canvas.is_cuda and y.dtype == canvas.dtype and y.dim() == 2 and canvas.dim() == 2
    assert y.stride(1) == 1 and canvas.stride(1) == 1 and y.shape[1] == canvas.shape[1]
    for v in (tokens, ptr, src):
        assert v.is_cuda and v.dtype == torch.int32 and v.is_contiguous()
    assert beta.is_cuda and beta.dtype == torch.float32 and beta.is_contiguous()
    n_tokens = tokens.numel()
    check_scatter_extents(y.shape[0], canvas.shape[0], tokens, ptr, src, beta)
    with _on_device(canvas):
        rc = _LIB().pq_scatter_rows(y.data_ptr(), max(y.stride(0), y.shape[1]), y.shape[0], tokens.data_ptr(),
                                         ptr.data_ptr(), src.data_ptr(), beta.data_ptr(), n_tokens,
                                         canvas.data_ptr(), max(canvas.stride(0), canvas.shape[1]), canvas.shape[0],
                                         canvas.shape[1], _dt(canvas.dtype), _stream(canvas))
    _lib.check(rc, "pq_scatter_rows")


# ------------------------------------------------------------------------------------------------ custom ops
# torch.library schemas cannot carry torch.dtype arguments portably, so out_dtype travels as the dtype code.
_CODE2DT = {_lib.DTYPE_BF16: torch.bfloat16, _lib.DTYPE_FP16: torch.float16}


@torch.library.custom_op("pq_b200::quant_rows", mutates_args=(), device_types="cuda")
def quant_rows_op(x2: Tensor) -> Tuple[Tensor, Tensor]:
    return _quant_rows_impl(x2)


@quant_rows_op.register_fake
def _(x2):
    return x2.new_empty(x2.shape, dtype=torch.int8), x2.new_empty((x2.shape[0],), dtype=torch.float32)


@torch.library.custom_op("pq_b200::quant_rows_g32", mutates_args=(), device_types="cuda")
def quant_rows_g32_op(x2: Tensor) -> Tuple[Tensor, Tensor]:
    return _quant_rows_g32_impl(x2)


@quant_rows_g32_op.register_fake
def _(x2):
    return (x2.new_empty(x2.shape, dtype=torch.int8),
            x2.new_empty((x2.shape[0], x2.shape[1] // 32), dtype=torch.float32))


@torch.library.custom_op("pq_b200::gather_quant_rows", mutates_args=(), device_types="cuda")
def gather_quant_rows_op(canvas: Tensor, row_idx: Tensor) -> Tuple[Tensor, Tensor]:
    return _gather_quant_rows_impl(canvas, row_idx)


@gather_quant_rows_op.register_fake
def _(canvas, row_idx):
    M = row_idx.shape[0]
    return canvas.new_empty((M, canvas.shape[1]), dtype=torch.int8), canvas.new_empty((M,), dtype=torch.float32)


@torch.library.custom_op("pq_b200::gather_rows", mutates_args=(), device_types="cuda")
def gather_rows_op(canvas: Tensor, row_idx: Tensor) -> Tensor:
    return _gather_rows_impl(canvas, row_idx)


@gather_rows_op.register_fake
def _(canvas, row_idx):
    return canvas.new_empty((row_idx.shape[0], canvas.shape[1]))


@torch.library.custom_op("pq_b200::int8_gemm", mutates_args=(), device_types="cuda")
def int8_gemm_op(xq: Tensor, s_row: Tensor, w_int8: Tensor, w_scale: Tensor, bias: Optional[Tensor],
                 t: Optional[Tensor], lb: Optional[Tensor], out_dtype_code: int,
                 lb_t: Optional[Tensor] = None) -> Tensor:
    return _gemm_impl(xq, s_row, w_int8, w_scale, bias, t, lb, _CODE2DT[out_dtype_code], lb_t=lb_t)


@int8_gemm_op.register_fake
def _(xq, s_row, w_int8, w_scale, bias, t, lb, out_dtype_code, lb_t=None):
    return xq.new_empty((xq.shape[0], w_int8.shape[0]), dtype=_CODE2DT[out_dtype_code])


@torch.library.custom_op("pq_b200::int8_gemm_grouped", mutates_args=(), device_types="cuda")
def int8_gemm_grouped_op(xq: Tensor, s_row: Tensor, w_hi: Tensor, s_hi: Tensor, w_lo: Tensor, s_lo: Tensor,
                         bias: Optional[Tensor], t: Optional[Tensor], lb: Optional[Tensor], m_hi: int,
                         out_dtype_code: int, lb_t: Optional[Tensor] = None) -> Tensor:
    return _gemm_impl(xq, s_row, w_hi, s_hi, bias, t, lb, _CODE2DT[out_dtype_code], None, w_lo, s_lo, m_hi, lb_t)


@int8_gemm_grouped_op.register_fake
def _(xq, s_row, w_hi, s_hi, w_lo, s_lo, bias, t, lb, m_hi, out_dtype_code, lb_t=None):
    return xq.new_empty((xq.shape[0], w_hi.shape[0]), dtype=_CODE2DT[out_dtype_code])


@torch.library.custom_op("pq_b200::int8_gemm_g32", mutates_args=(), device_types="cuda")
def int8_gemm_g32_op(xq: Tensor, s_a: Tensor, w_int8: Tensor, s_w_gm: Tensor, bias: Optional[Tensor],
                     out_dtype_code: int) -> Tensor:
    return _gemm_g32_impl(xq, s_a, w_int8, s_w_gm, bias, _CODE2DT[out_dtype_code])


@int8_gemm_g32_op.register_fake
def _(xq, s_a, w_int8, s_w_gm, bias, out_dtype_code):
    return xq.new_empty((xq.shape[0], w_int8.shape[0]), dtype=_CODE2DT[out_dtype_code])


@torch.library.custom_op("pq_b200::dequant_epilogue", mutates_args=(), device_types="cuda")
def dequant_epilogue_op(acc: Tensor, s_row: Tensor, s_col: Tensor, bias: Optional[Tensor],
                        out_dtype_code: int) -> Tensor:
    return _dequant_epilogue_impl(acc, s_row, s_col, bias, _CODE2DT[out_dtype_code])


@dequant_epilogue_op.register_fake
def _(acc, s_row, s_col, bias, out_dtype_code):
    return acc.new_empty(acc.shape, dtype=_CODE2DT[out_dtype_code])


@torch.library.custom_op("pq_b200::scatter_rows_", mutates_args=("canvas",), device_types="cuda")
def scatter_rows_op(y: Tensor, tokens: Tensor, ptr: Tensor, src: Tensor, beta: Tensor, canvas: Tensor) -> None:
    _scatter_rows_impl(y, tokens, ptr, src, beta, canvas)


def dtype_code(dtype: torch.dtype) -> int:
    return _dt(dtype)


def int8_gemm_debug(xq: Tensor, s_row: Tensor, w_int8: Tensor, w_scale: Tensor, bias: Optional[Tensor],
                    t: Optional[Tensor], lb: Optional[Tensor], out_dtype: torch.dtype) -> Tuple[Tensor, Tensor]:
    """GEMM that also returns the raw int32 accumulators (parity tests)."""
    acc = torch.full((xq.shape[0], w_int8.shape[0]), -2**31, dtype=torch.int32, device=xq.device)
    out = _gemm_impl(xq, s_row, w_int8, w_scale, bias, t, lb, out_dtype, dbg_acc=acc)
    return out, acc
