"""Drop-in for PyraQuant's ``deploy/int8_exec.py``: same public names, argument meaning and error
behaviour, executed by libpq_b200.so (hand-written sm_100a CUDA) through torch custom ops.

What stays the same for a caller of the reference module
  * ``Int8Linear(lin, device=None, lowrank=None)`` with buffers ``weight_int8``, ``w_scale``, ``bias``,
    ``lr_A``, ``lr_B`` and attributes ``in_features`` / ``out_features`` (reference :345-411);
  * ``quant_rows``, ``int8_gemm_fused``, ``int8_gemm_lr``, ``int8_linear_2d``, ``dequant_epilogue``
    (reference :202-261, :327-336) -- outputs freshly allocated, inputs never modified, launched on
    torch's current stream without synchronising;
  * ``set_backend`` / ``get_backend`` / ``BACKENDS`` / ``DEFAULT_BACKEND`` / ``BACKEND`` (reference :58-74):
    both names are accepted because drivers pass them, and both select the one native backend;
  * ``convert_linears_to_int8``, ``is_bf16_whitelisted``, ``warm_kernels``, ``FLUX_TOKEN_SHAPES``,
    ``LOWRANK_A_ATTR`` / ``LOWRANK_B_ATTR``, ``selftest_and_bench`` and the module CLI (reference :415-588).
What differs: no Triton, no cuBLAS ``_int_mm`` path, no CPU path (CPU tensors raise AssertionError exactly
as the reference's ``quant_rows`` does, :221), and the shape rules are wider (K % 16 == 0, any N that is a
multiple of 8, instead of K % 64 == 0 and N % 256 == 0).

Added entry points (not in the reference module): ``quant_rows_g32``, ``gather_quant_rows``,
``int8_gemm_grouped``, ``int8_gemm_g32``, ``nested4_codes``, ``Int8LinearRouted``, ``Int8LinearG32``.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops

# --------------------------------------------------------------------------- backend names (API parity only)
BACKENDS = ("triton", "cublas")
DEFAULT_BACKEND = "triton"
BACKEND = DEFAULT_BACKEND


def set_backend(name: str) -> str:
    """Accepted for compatibility with drivers that pass ``--int8-backend``; every name maps to the
    sm_100a library.  Unknown names raise ValueError like the reference (:67-68)."""
    global BACKEND
    if name not in BACKENDS:
        raise ValueError(f"unknown INT8 backend {name!r} (expected one of {BACKENDS})")
    BACKEND = name
    return BACKEND


def get_backend() -> str:
    return BACKEND


def _m_bucket(M: int) -> int:
    """Reference autotune bucket of M (:198-199); kept because drivers import it."""
    return 0 if M < 8192 else (1 if M < 32768 else 2)


# --------------------------------------------------------------------------- operator wrappers
# Every operator exists as a torch custom op (torch.ops.pq_b200.*, with fake implementations, for tracing and
# torch.compile).  In eager mode the wrappers below call the same implementation function directly: the
# dispatcher round trip of a Python custom op costs tens of microseconds per call, more than the kernels
# themselves at the 1K stage (the reference met the same problem with Triton's launcher,
# deploy/run_sdxl_latency.py:144-147).
def _eager() -> bool:
    return not torch.compiler.is_compiling()


def quant_rows(x2: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[M,K] bf16/fp16 -> (int8 codes [M,K], fp32 scale [M]); rows may be strided (no copy)."""
    assert x2.dim() == 2 and x2.is_cuda
    if _eager():
        return ops._quant_rows_impl(x2)
    return torch.ops.pq_b200.quant_rows(x2)


def quant_rows_g32(x2: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token, per-32-channel scales: (int8 [M,K], fp32 [M, K/32])."""
    assert x2.dim() == 2 and x2.is_cuda
    if _eager():
        return ops._quant_rows_g32_impl(x2)
    return torch.ops.pq_b200.quant_rows_g32(x2)


def gather_quant_rows(canvas: torch.Tensor, row_idx: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows ``row_idx`` (int32, -1 = zero padding row) of ``canvas`` [rows,K], quantised per token."""
    assert canvas.dim() == 2 and canvas.is_cuda
    if _eager():
        return ops._gather_quant_rows_impl(canvas, row_idx)
    return torch.ops.pq_b200.gather_quant_rows(canvas, row_idx)


def int8_gemm_fused(xq: torch.Tensor, s_row: torch.Tensor, w_int8: torch.Tensor, w_scale: torch.Tensor,
                    bias: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    assert xq.is_cuda
    if _eager():
        return ops._gemm_impl(xq, s_row, w_int8, w_scale, bias, None, None, out_dtype)
    return torch.ops.pq_b200.int8_gemm(xq, s_row, w_int8, w_scale, bias, None, None, ops.dtype_code(out_dtype))


def int8_gemm_lr(xq, s_row, w_i8, w_scale, bias, t, lb, out_dtype, lb_t=None):
    """Fused GEMM with the low-rank up-projection ``t @ lb`` added before the bias (reference :303-309).
    ``lb_t`` (optional, not in the reference signature) is a cached ``lb.t().contiguous()``; without it the
    transpose is made on every call."""
    assert xq.is_cuda
    if _eager():
        return ops._gemm_impl(xq, s_row, w_i8, w_scale, bias, t, lb, out_dtype, lb_t=lb_t)
    return torch.ops.pq_b200.int8_gemm(xq, s_row, w_i8, w_scale, bias, t, lb, ops.dtype_code(out_dtype), lb_t)


def int8_gemm_grouped(xq, s_row, w_hi, s_hi, w_lo, s_lo, bias, t, lb, m_hi: int, out_dtype, lb_t=None):
    """Rows [0, m_hi) against (w_hi, s_hi), rows [m_hi, M) against (w_lo, s_lo), one launch."""
    assert xq.is_cuda
    if _eager():
        return ops._gemm_impl(xq, s_row, w_hi, s_hi, bias, t, lb, out_dtype, None, w_lo, s_lo, int(m_hi), lb_t)
    return torch.ops.pq_b200.int8_gemm_grouped(xq, s_row, w_hi, s_hi, w_lo, s_lo, bias, t, lb, int(m_hi),
                                               ops.dtype_code(out_dtype), lb_t)


def int8_gemm_g32(xq, s_a, w_int8, s_w_gm, bias, out_dtype):
    """Group-32 GEMM: s_a [M, K/32] (from ``quant_rows_g32``), s_w_gm [K/32, N] group-major weight scales."""
    assert xq.is_cuda
    if _eager():
        return ops._gemm_g32_impl(xq, s_a, w_int8, s_w_gm, bias, out_dtype)
    return torch.ops.pq_b200.int8_gemm_g32(xq, s_a, w_int8, s_w_gm, bias, ops.dtype_code(out_dtype))


def dequant_epilogue(acc: torch.Tensor, s_row: torch.Tensor, s_col: torch.Tensor,
                     bias: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    assert acc.dtype == torch.int32 and acc.is_contiguous()
    return torch.ops.pq_b200.dequant_epilogue(acc, s_row, s_col, bias, ops.dtype_code(out_dtype))


def int8_linear_2d(x2: torch.Tensor, w_int8: torch.Tensor, w_scale: torch.Tensor,
                   bias: Optional[torch.Tensor], backend: Optional[str] = None) -> torch.Tensor:
    """x2 [M,K] -> [M,N] in x2's dtype.  ``backend`` is validated and otherwise ignored."""
    if backend is not None and backend not in BACKENDS:
        raise ValueError(f"unknown INT8 backend {backend!r} (expected one of {BACKENDS})")
    xq, sx = quant_rows(x2)
    return int8_gemm_fused(xq, sx, w_int8, w_scale, bias, x2.dtype)


# --------------------------------------------------------------------------- module
LOWRANK_A_ATTR = "_lowrank_A"
LOWRANK_B_ATTR = "_lowrank_B"


def _quantize_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel symmetric absmax INT8 (reference :355-357): fp32 math, round-half-even.

    The scale is formed exactly as the reference forms it, `amax / 127.0` with a Python scalar, so that a layer
    converted on a device gets the codes and scales the reference's constructor produces on that device, bit for bit.
    (torch's CUDA kernel multiplies by fl32(1 / 127) where the CPU divides; a few per cent of the channels then differ
    by one code at rounding ties between a CPU-converted and a GPU-converted layer, in the reference as here.)"""
    wf = w.float()
    scale = wf.abs().amax(dim=1).clamp_min(1e-8) / 127.0
    codes = torch.round(wf / scale[:, None]).clamp_(-127, 127).to(torch.int8)
    return codes.contiguous(), scale.contiguous()


def nested4_codes(weight_int8: torch.Tensor, w_scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """INT8 codes re-rounded to the nested 4-bit grid (pyraquant/quantizers_weight.py:182-199):
    c = round(q8 * 7/127) in [-7, 7], dequantised as c * (127/7) * s8.  Returned as int8 codes plus the
    matching per-channel scale so that the same INT8 kernel executes the low tier."""
    c = torch.round(weight_int8.float() * (7.0 / 127.0)).clamp_(-7, 7).to(torch.int8)
    return c.contiguous(), (w_scale.float() * (127.0 / 7.0)).contiguous()


class SharedInputGroup:
    """Sibling ``Int8Linear`` layers that are called one after the other on the SAME input tensor (FLUX: to_q / to_k /
    to_v, add_*_proj, and proj_mlp next to the attention projections of a single-stream block) share one per-token
    quantisation and one down-projection ``x @ [A_1 | A_2 | ...]`` instead of one each.  The first member called on
    an input does both and keeps the results; the others recognise the input (same storage, shape, strides,
    version counter and CUDA stream) and reuse them.  Inference tensors keep no version counter, so under
    ``torch.inference_mode()`` the members run ungrouped.  The library's own in-place writes (the accumulate epilogue,
    the 4-bit expansion) bump the version of what they write, as torch's in-place operators do.  Results are bit-identical to the ungrouped layers except for the
    down-projection, whose fp32 summation order may differ with the width (same caveat as between any two GEMM
    shapes).
    The cache keeps the last input and its codes alive until the next input arrives or ``clear()`` is called."""

    def __init__(self, layers: Sequence["Int8Linear"]):
        layers = list(layers)
        assert len(layers) >= 2 and all(isinstance(m, Int8Linear) for m in layers)
        K = layers[0].in_features
        assert all(m.in_features == K for m in layers), "members must have the same in_features"
        self.layers = layers
        self._key = None
        self._val = None
        self._A_cat = None
        self._A_cat_t = None
        self._A_slots: Dict[int, int] = {}
        for m in layers:
            m.__dict__["_shared_input"] = self

    def clear(self) -> None:
        self._key = None
        self._val = None

    def _a_cat(self, dtype: torch.dtype, device: torch.device) -> Optional[torch.Tensor]:
        c = self._A_cat
        if c is None or c.dtype != dtype or c.device != device:
            mats, self._A_slots, off = [], {}, 0
            for m in self.layers:
                if m.lr_A is not None and m.lr_A.shape[1] == 32 and m.lr_A.dtype == dtype:
                    self._A_slots[id(m)] = off
                    mats.append(m.lr_A.to(device))
                    off += 32
            c = torch.cat(mats, dim=1).contiguous() if mats else torch.empty((0, 0), dtype=dtype, device=device)
            self._A_cat = c
            self._A_cat_t = c.t().contiguous() if c.numel() else None
        return c if c.numel() else None

    def prepare(self, x2: torch.Tensor):
        """(codes, row scales, T) for x2; T [M, 32 * members with a rank-32 branch] or None."""
        key = (x2.data_ptr(), tuple(x2.shape), tuple(x2.stride()), x2.dtype, x2._version, x2.device, ops._stream(x2))
        if key != self._key:
            a_cat = self._a_cat(x2.dtype, x2.device)
            if a_cat is None:
                T = None
            elif a_cat.shape[1] in ops.LOWRANK_DOWN_COLS and ops.lowrank_down_ok(x2):
                T = ops.lowrank_down(x2, self._A_cat_t)
            else:
                T = x2 @ a_cat
            xq, sx = ops._quant_rows_impl(x2)
            self._key, self._val = key, (x2, xq, sx, T)          # x2 kept so that its storage cannot be recycled
        _x, xq, sx, T = self._val
        return xq, sx, T

    def prime_adaln(self, h: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
        """Returns ``z = LayerNorm(h) * (1 + scale[:, None]) + shift[:, None]`` (the block's adaLN output,
        flux/transformer_flux.py:133, :206, :236-239) and leaves the group primed for it: normalisation, modulation and the
        members' shared quantisation are one pass over ``h`` (``ops.adaln_quant_rows``), the shared down-projection
        reads ``z``, and the members called on ``z`` afterwards go straight to their GEMMs.  h [B, T, K] with scale / shift
        [B, K], or h [M, K] with [K]; CUDA tensors of the members' activation type."""
        K = h.shape[-1]
        x2 = h.reshape(-1, K)
        xq, sx, z2 = ops.adaln_quant_rows(x2, scale, shift, eps, h.shape[-2] if h.dim() == 3 else 0, want_modulated=True)
        a_cat = self._a_cat(z2.dtype, z2.device)
        if a_cat is None:
            T = None
        elif a_cat.shape[1] in ops.LOWRANK_DOWN_COLS and ops.lowrank_down_ok(z2):
            T = ops.lowrank_down(z2, self._A_cat_t)
        else:
            T = z2 @ a_cat
        self._key = (z2.data_ptr(), tuple(z2.shape), tuple(z2.stride()), z2.dtype, z2._version, z2.device, ops._stream(z2))
        self._val = (z2, xq, sx, T)
        return z2.reshape(h.shape)

    def t_of(self, member: "Int8Linear", T: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        off = self._A_slots.get(id(member))
        if T is None or off is None:
            return None
        return T[:, off:off + 32]                                # row stride 32 * members: the kernel takes strided t


def share_input_quantisation(layers: Sequence["Int8Linear"]) -> SharedInputGroup:
    """Groups converted layers that are always called on the same input; see ``SharedInputGroup``."""
    return SharedInputGroup(layers)


# Sibling layers of the FLUX blocks that read the same tensor (flux/transformer_flux.py:135-145, 727-729, 821-823),
# as paths relative to a common parent module.
FLUX_SHARED_INPUT_GROUPS = (
    ("proj_mlp", "attn.to_q", "attn.to_k", "attn.to_v"),
    ("to_q", "to_k", "to_v"),
    ("add_q_proj", "add_k_proj", "add_v_proj"),
)


class Int8Linear(nn.Module):
    """INT8 stand-in for ``nn.Linear``: per-channel INT8 weights held as buffers, per-token dynamic INT8
    activations, optional rank-r low-rank branch executed for real (down-projection as a small GEMM,
    up-projection inside the INT8 GEMM epilogue)."""

    def __init__(self, lin: nn.Linear, device: Optional[torch.device] = None,
                 lowrank: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        super().__init__()
        w = lin.weight.detach()
        if device is not None:
            w = w.to(device, non_blocking=False)
        codes, scale = _quantize_weight(w)
        self.register_buffer("weight_int8", codes)
        self.register_buffer("w_scale", scale)
        if lin.bias is not None:
            b = lin.bias.detach().float()
            if device is not None:
                b = b.to(device)
            self.register_buffer("bias", b.contiguous())
        else:
            self.bias = None
        self.in_features = int(lin.in_features)
        self.out_features = int(lin.out_features)
        if lowrank is not None:
            A, B = lowrank
        else:
            A, B = getattr(lin, LOWRANK_A_ATTR, None), getattr(lin, LOWRANK_B_ATTR, None)
        if A is not None and B is not None:
            if device is not None:
                A, B = A.to(device), B.to(device)
            self.register_buffer("lr_A", A.contiguous())
            self.register_buffer("lr_B", B.contiguous())
        else:
            self.lr_A = None
            self.lr_B = None

    def _lr_Bt(self) -> torch.Tensor:
        """K-major copy of lr_B for the tensor-core low-rank path, made once per device/dtype (not part of the state)."""
        return self._transposed("lr_B")

    def _lr_At(self) -> torch.Tensor:
        """K-major copy of lr_A ([32, K]) for the native down-projection kernel, made once (not part of the state)."""
        return self._transposed("lr_A")

    def _transposed(self, name: str) -> torch.Tensor:
        """Contiguous transpose of a low-rank factor, remade whenever the buffer is replaced, converted (.to / .half),
        moved or written in place."""
        src = getattr(self, name)
        key = (src.data_ptr(), src.dtype, src.device, tuple(src.shape), ops.tensor_version(src))
        c = self.__dict__.get("_t_cache_" + name)
        if c is None or c[0] != key:
            c = (key, src.t().contiguous())
            self.__dict__["_t_cache_" + name] = c
        return c[1]

    def _down(self, x2: torch.Tensor) -> torch.Tensor:
        """t = x2 @ lr_A rounded to the activation dtype (reference :390): the native streaming kernel for rank 32
        on inputs it takes as they are (any row count), torch's matmul otherwise (other ranks, dtypes, unaligned rows)."""
        if self.lr_A.shape[1] == 32 and self.lr_A.dtype == x2.dtype and ops.lowrank_down_ok(x2):
            return ops.lowrank_down(x2, self._lr_At())
        return x2.to(self.lr_A.dtype) @ self.lr_A

    def _fusable_lowrank(self, x2: torch.Tensor) -> bool:
        return (self.lr_A is not None and self.lr_A.shape[1] == 32 and x2.shape[1] % 32 == 0
                and self.lr_A.dtype == x2.dtype and self.lr_B.dtype == x2.dtype and self.out_features % 8 == 0)

    def _lean_forward(self, x2: torch.Tensor):
        """Eager fast path for the common case (aligned rows, rank-32 branch or none): the two C-ABI calls are made
        straight from here with the per-layer constants cached, skipping the generic wrappers' checks.  Returns
        None when the input does not qualify."""
        M, K = x2.shape
        if (M == 0 or not x2.is_cuda or x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16 or K % 16
                or x2.device != self.weight_int8.device or x2.dtype not in ops._DT or torch.compiler.is_compiling()):
            return None
        lr = self.lr_A is not None
        if lr and not self._fusable_lowrank(x2):
            return None
        c = self.__dict__.get("_lean_cache")
        wptr = self.weight_int8.data_ptr()
        # every buffer whose address is cached takes part in the key: .to(dtype) / .half() / load_state_dict(assign=True)
        # replace the float buffers while the int8 weight stays where it is
        lbt = self._lr_Bt() if lr else None
        key = (wptr, x2.dtype, self.w_scale.data_ptr(), self.bias.data_ptr() if self.bias is not None else 0,
               self.lr_B.data_ptr() if lr else 0, lbt.data_ptr() if lr else 0)
        if c is None or c[0] != key:
            assert self.w_scale.dtype == torch.float32 and (self.bias is None or self.bias.dtype == torch.float32), \
                "w_scale and bias are fp32 buffers"
            assert self.w_scale.numel() == self.out_features and (self.bias is None or self.bias.numel() == self.out_features)
            c = (key, x2.dtype, self.weight_int8.stride(0), self.w_scale.data_ptr(),
                 self.bias.data_ptr() if self.bias is not None else None,
                 self.lr_B.data_ptr() if lr else None, self.lr_B.stride(0) if lr else 0,
                 lbt.data_ptr() if lr else None, ops._DT[x2.dtype], ops._LIB(), ops.status_word(x2.device))
            self.__dict__["_lean_cache"] = c
        _w, _dt_t, ldw, sc_ptr, b_ptr, lb_ptr, ldb, lbt_ptr, code, lib, ws = c
        N = self.out_features
        dev = x2.device
        t_ptr = None
        ldt = 0
        if lr:
            t = self._down(x2)                                  # [M, 32]
            t_ptr, ldt = t.data_ptr(), t.stride(0)
        q = torch.empty((M, K), dtype=torch.int8, device=dev)
        sx = torch.empty((M,), dtype=torch.float32, device=dev)
        out = torch.empty((M, N), dtype=x2.dtype, device=dev)
        stream = ops._stream(x2)
        with ops._on_device(x2):
            rc = lib.pq_quant_rows(x2.data_ptr(), code, M, K, x2.stride(0) if M > 1 else K, q.data_ptr(), sx.data_ptr(), stream)
            if rc == 0:
                rc = lib.pq_int8_gemm(q.data_ptr(), K, sx.data_ptr(), wptr, ldw, sc_ptr, b_ptr, t_ptr, ldt, lb_ptr, ldb,
                                      lbt_ptr, 32 if lr else 0, code, out.data_ptr(), code, N, M, N, K, ws.data_ptr(),
                                      ws.numel() * 4, None, stream)
        if rc:
            ops._lib.check(rc, f"Int8Linear(M={M}, N={N}, K={K})")
        return out

    def _shared_forward(self, x2: torch.Tensor):
        """Forward through the group's shared quantisation / down-projection; None when the input does not qualify."""
        grp = self.__dict__.get("_shared_input")
        M, K = x2.shape
        if (grp is None or M == 0 or not x2.is_cuda or x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16
                or K % 32 or x2.dtype not in ops._DT or torch.compiler.is_compiling() or x2.is_inference()):
            return None
        if self.lr_A is not None and not self._fusable_lowrank(x2):
            return None
        xq, sx, T = grp.prepare(x2)
        t = grp.t_of(self, T) if self.lr_A is not None else None
        if t is not None:
            return int8_gemm_lr(xq, sx, self.weight_int8, self.w_scale, self.bias, t, self.lr_B, x2.dtype, self._lr_Bt())
        return int8_gemm_fused(xq, sx, self.weight_int8, self.w_scale, self.bias, x2.dtype)

    def forward_ex(self, x: torch.Tensor, epilogue: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``gelu_tanh(self(x))`` (``ops.EPI_GELU_TANH``) or ``out += self(x)`` (``ops.EPI_ACCUMULATE``, in place, returns
        ``out``), with the extra step done in the GEMM epilogue when the shapes allow it and by the separate torch
        kernels the reference's callers use otherwise.  The activation sees the Linear's output rounded to the
        activation dtype, the sum is the sum of two rounded tensors: the values match the unfused sequence (the
        GELU up to the hardware tanh approximation)."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        M, K = x2.shape
        N = self.out_features
        out2 = out.reshape(-1, N) if out is not None else None
        assert not (epilogue & ops.EPI_ACCUMULATE) or (out2 is not None and out2.shape[0] == M and out2.dtype == x2.dtype)
        lr = self.lr_A is not None
        fused = (epilogue != 0 and M > 0 and x2.is_cuda and x2.dtype in ops._DT and K % 16 == 0
                 and not torch.compiler.is_compiling() and (not lr or self._fusable_lowrank(x2))
                 and (out2 is None or (out2.stride(1) == 1 and out2.data_ptr() == out.data_ptr()))
                 and ops.epilogue_supported(N, out2.stride(0) if out2 is not None else N,
                                            out2.data_ptr() if out2 is not None else 0, lr))
        if not fused:
            y = self.forward(x)
            if epilogue & ops.EPI_GELU_TANH:
                y = F.gelu(y, approximate="tanh")
            if epilogue & ops.EPI_ACCUMULATE:
                out.add_(y.reshape(out.shape))
                return out
            return y
        grp = self.__dict__.get("_shared_input")
        if (grp is not None and x2.stride(1) == 1 and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0 and K % 32 == 0
                and not x2.is_inference()):
            xq, sx, T = grp.prepare(x2)
            t = grp.t_of(self, T) if lr else None
        else:
            t = self._down(x2) if lr else None
            xq, sx = quant_rows(x2)
        y2 = ops._gemm_impl(xq, sx, self.weight_int8, self.w_scale, self.bias, t, self.lr_B if lr else None, x2.dtype,
                            lb_t=self._lr_Bt() if lr else None, epilogue=epilogue,
                            out=out2 if (epilogue & ops.EPI_ACCUMULATE) else None)
        if epilogue & ops.EPI_ACCUMULATE:
            return out
        return y2.reshape(*shape[:-1], N)

    def forward_adaln(self, h: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-6,
                      return_modulated: bool = False):
        """``self(LayerNorm(h) * (1 + scale[:, None]) + shift[:, None])``: the feed-forward's first Linear behind the
        adaLN modulation of a FLUX block (flux/transformer_flux.py:236-240; LayerNorm without affine parameters, :195).
        h [B, T, K] with scale / shift [B, K], or h [M, K] with [K].  On CUDA the normalisation, the modulation and the
        Linear's per-token quantisation are one pass over h (``ops.adaln_quant_rows``); the modulated activations are
        written out only when the layer has a low-rank branch or the caller wants them (``return_modulated``: the
        single-stream blocks feed them to the attention as well).  Values match the separate torch kernels except where
        LayerNorm's fp32 row statistics, summed in another order, move a normalised value across a rounding boundary."""
        K = h.shape[-1]
        x2 = h.reshape(-1, K)
        lr = self.lr_A is not None
        fused = (x2.shape[0] > 0 and x2.is_cuda and x2.dtype in ops._DT and K % 16 == 0 and K <= 16384
                 and scale.dtype == x2.dtype and shift.dtype == x2.dtype and not torch.compiler.is_compiling()
                 and (not lr or self._fusable_lowrank(x2)))
        if not fused:
            y = F.layer_norm(h, (K,), eps=eps)
            z = y * (1 + scale[:, None]) + shift[:, None] if h.dim() == 3 else y * (1 + scale) + shift
            out = self.forward(z)
            return (out, z) if return_modulated else out
        rows_per_sample = h.shape[-2] if h.dim() == 3 else 0
        xq, sx, z = ops.adaln_quant_rows(x2, scale, shift, eps, rows_per_sample, want_modulated=lr or return_modulated)
        t = self._down(z) if lr else None
        y2 = ops._gemm_impl(xq, sx, self.weight_int8, self.w_scale, self.bias, t, self.lr_B if lr else None, x2.dtype,
                            lb_t=self._lr_Bt() if lr else None)
        out = y2.reshape(*h.shape[:-1], self.out_features)
        return (out, z.reshape(h.shape)) if return_modulated else out

    def _prologue(self, x2: torch.Tensor, x_more: Optional[torch.Tensor] = None):
        """(codes, row scales, t or None) of the layer's input; with ``x_more`` the input is ``[x2 | x_more]`` along the
        features, read from its two sources where the kernels take them and concatenated otherwise."""
        lr = self.lr_A is not None
        if x_more is not None:
            if (ops.cat_sources_ok(x2, x_more) and not torch.compiler.is_compiling()
                    and (not lr or (self.lr_A.shape[1] == 32 and self.lr_A.dtype == x2.dtype))):
                t = ops.lowrank_down_cat(x2, x_more, self._lr_At()) if lr else None
                xq, sx = ops.quant_rows_cat(x2, x_more)
                return xq, sx, t
            x2 = torch.cat([x2, x_more], dim=1)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        t = self._down(x2) if lr else None
        xq, sx = quant_rows(x2)
        return xq, sx, t

    def forward_cat(self, x0: torch.Tensor, x1: torch.Tensor) -> torch.Tensor:
        """``self(torch.cat([x0, x1], dim=-1))`` without building the concatenated tensor: the single-stream blocks'
        ``proj_out(torch.cat([attn_output, mlp_hidden_states], dim=2))`` (flux/transformer_flux.py:143-145).  Identical
        values (one row scale over all the features, as for the concatenated tensor)."""
        K0, K1, N = x0.shape[-1], x1.shape[-1], self.out_features
        assert K0 + K1 == self.in_features and x0.shape[:-1] == x1.shape[:-1], (x0.shape, x1.shape, self.in_features)
        a, b = x0.reshape(-1, K0), x1.reshape(-1, K1)
        lr = self.lr_A is not None
        if (a.shape[0] == 0 or not a.is_cuda or a.dtype not in ops._DT or (K0 + K1) % 16 != 0
                or (lr and not (self.lr_A.shape[1] == 32 and (K0 + K1) % 32 == 0 and self.lr_A.dtype == a.dtype
                                and self.lr_B.dtype == a.dtype and N % 8 == 0))):
            return self.forward(torch.cat([x0, x1], dim=-1))
        xq, sx, t = self._prologue(a, b)
        y = ops._gemm_impl(xq, sx, self.weight_int8, self.w_scale, self.bias, t, self.lr_B if lr else None, a.dtype,
                           lb_t=self._lr_Bt() if lr else None)
        return y.reshape(*x0.shape[:-1], N)

    def forward_gated_residual(self, x: torch.Tensor, gate: torch.Tensor, residual: torch.Tensor,
                               x_more: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += gate.unsqueeze(1) * self(x)``, in place, returns ``residual``: the tail of a FLUX block
        (flux/transformer_flux.py:145-149: ``hidden_states = residual + gate.unsqueeze(1) * proj_out(...)``, fp16 clipped to
        the finite range; likewise :224-225 and :240-242 for the attention and feed-forward outputs of the double-stream
        blocks).  x [B, T, K] with gate [B, N] and residual [B, T, N], or x [M, K] with gate [N]; with ``x_more`` the layer's
        input is ``[x | x_more]`` along the features, read from the two tensors in place (``proj_out`` of the single-stream
        blocks, whose input the reference concatenates first).  On CUDA the product
        and the sum happen in the GEMM epilogue (``pq_int8_gemm_gated``), rounding where the separate torch kernels round:
        the values are identical to the unfused sequence."""
        K, N = x.shape[-1], self.out_features
        x2 = x.reshape(-1, K)
        M = x2.shape[0]
        res2 = residual.reshape(-1, N)
        lr = self.lr_A is not None
        if x_more is not None and not (x2.is_cuda and ops.cat_sources_ok(x2, x_more.reshape(-1, x_more.shape[-1]))):
            x = torch.cat([x, x_more], dim=-1)
            x_more = None
            K = x.shape[-1]
            x2 = x.reshape(-1, K)
        fused = (M > 0 and x2.is_cuda and x2.dtype in ops._DT and self.in_features % 16 == 0 and not torch.compiler.is_compiling()
                 and gate.dtype == x2.dtype and residual.dtype == x2.dtype and res2.shape[0] == M
                 and res2.stride(1) == 1 and res2.data_ptr() == residual.data_ptr()
                 and (not lr or self._fusable_lowrank(x2)) and ops.epilogue_supported(N, res2.stride(0), res2.data_ptr(), lr))
        if not fused:
            y = self.forward(x if x_more is None else torch.cat([x, x_more], dim=-1))
            residual.add_((gate.unsqueeze(1) if x.dim() == 3 else gate) * y)
            if residual.dtype == torch.float16:
                residual.clamp_(-65504, 65504)
            return residual
        xq, sx, t = self._prologue(x2, None if x_more is None else x_more.reshape(-1, x_more.shape[-1]))
        ops._gemm_impl(xq, sx, self.weight_int8, self.w_scale, self.bias, t, self.lr_B if lr else None, x2.dtype,
                       lb_t=self._lr_Bt() if lr else None, epilogue=ops.EPI_ACCUMULATE, out=res2,
                       gate=gate, gate_rows=x.shape[-2] if x.dim() == 3 else 0)
        return residual

    def forward_into(self, x2: torch.Tensor, out: torch.Tensor, out_more: Sequence[torch.Tensor] = ()) -> torch.Tensor:
        """``out[:] = self(x2)`` for 2-D ``x2``, the same values also stored to every tensor of ``out_more`` (same shape,
        dtype and row stride as ``out``; up to ``ops.MAX_OUT_MORE``).  When the shapes allow it the GEMM epilogue
        writes all destinations itself (``pq_int8_gemm_bcast``): with ``out`` / ``out_more`` being this rank's row block
        inside the full output buffers of this GPU and of its peers, the all-gather of a row-sharded layer happens
        inside the GEMM.  Otherwise the layer runs as usual and the result is copied."""
        M, K = x2.shape
        N = self.out_features
        assert out.shape == (M, N) and out.dtype == x2.dtype and out.stride(1) == 1, (out.shape, out.dtype)
        lr = self.lr_A is not None
        direct = (M > 0 and x2.is_cuda and x2.dtype in ops._DT and K % 16 == 0 and len(out_more) <= ops.MAX_OUT_MORE
                  and not torch.compiler.is_compiling() and (not lr or self._fusable_lowrank(x2))
                  and ops.epilogue_supported(N, out.stride(0), out.data_ptr(), lr)
                  and all(o.stride(0) == out.stride(0) and o.data_ptr() % 16 == 0 for o in out_more))
        if not direct:
            y = self.forward(x2)
            out.copy_(y)
            for o in out_more:
                o.copy_(y, non_blocking=True)
            return out
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        t = self._down(x2) if lr else None
        xq, sx = quant_rows(x2)
        return ops._gemm_impl(xq, sx, self.weight_int8, self.w_scale, self.bias, t, self.lr_B if lr else None, x2.dtype,
                              lb_t=self._lr_Bt() if lr else None, out=out, out_more=list(out_more))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        y = self._shared_forward(x2)
        if y is None:
            y = self._lean_forward(x2)
        if y is not None:
            return y.reshape(*shape[:-1], self.out_features)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        if self._fusable_lowrank(x2):
            t = self._down(x2)                                     # [M, r], rounded to the activation dtype
            xq, sx = quant_rows(x2)
            y = int8_gemm_lr(xq, sx, self.weight_int8, self.w_scale, self.bias, t, self.lr_B, x2.dtype, self._lr_Bt())
            return y.reshape(*shape[:-1], self.out_features)
        y = int8_linear_2d(x2, self.weight_int8, self.w_scale, self.bias)
        if self.lr_A is not None:                                  # shapes the fused epilogue does not take
            xa = x2.to(self.lr_A.dtype) @ self.lr_A
            if y.dtype == self.lr_B.dtype and y.is_contiguous():
                y.addmm_(xa, self.lr_B)
            else:
                y = torch.addmm(y, xa.to(y.dtype), self.lr_B.to(y.dtype))
        return y.reshape(*shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, int8 per-channel W / per-token A, "
                f"sm_100a tcgen05 kernel")


class SplitInInt8Linear(nn.Module):
    """A Linear split along its inputs, ``y = L0(x[..., :in0]) + L1(x[..., in0:])`` (the reference's ``SplitInLinear``,
    pyraquant/external_quant.py:174-192, after conversion of its two halves): each half keeps its own per-token
    quantisation and low-rank branch, and the second half's GEMM adds onto the first half's output in its epilogue
    instead of a separate elementwise sum."""

    def __init__(self, l0: "Int8Linear", l1: "Int8Linear", in0: Optional[int] = None):
        super().__init__()
        assert isinstance(l0, Int8Linear) and isinstance(l1, Int8Linear) and l0.out_features == l1.out_features
        self.linears = nn.ModuleList([l0, l1])
        self.in0 = int(l0.in_features if in0 is None else in0)
        assert self.in0 == l0.in_features
        self.in_features = l0.in_features + l1.in_features
        self.out_features = l0.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.linears[0](x[..., : self.in0])
        return self.linears[1].forward_ex(x[..., self.in0:], ops.EPI_ACCUMULATE, out=y)


def fuse_split_inputs(model: nn.Module) -> int:
    """Replaces every module that has the reference ``SplitInLinear`` layout (``linears`` = two converted halves and
    ``in0``) by ``SplitInInt8Linear``.  Returns the number replaced."""
    n = 0
    for name, m in list(model.named_modules()):
        halves = getattr(m, "linears", None)
        if (isinstance(m, SplitInInt8Linear) or not isinstance(halves, nn.ModuleList) or len(halves) != 2
                or not hasattr(m, "in0") or not all(isinstance(h, Int8Linear) for h in halves)):
            continue
        parent_name, _, attr = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, attr, SplitInInt8Linear(halves[0], halves[1], int(m.in0)))
        n += 1
    return n


def _quantize_weight_g32(w: torch.Tensor, group: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group-32 symmetric absmax INT8 weights: the integer grid behind ``qdq_weight(w, 8, 32)``
    (pyraquant/quantizers_weight.py:96-109).  Returns codes [N,K] and scales [N, K/32]."""
    out_f, in_f = w.shape
    wg = w.float().reshape(out_f, in_f // group, group)
    scale = wg.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8) / 127        # the reference's expression, scalar divisor
    codes = torch.round(wg / scale).clamp_(-127, 127).to(torch.int8)
    return codes.reshape(out_f, in_f).contiguous(), scale[..., 0].contiguous()


class Int8LinearG32(nn.Module):
    """W8A8 Linear with one scale per 32 input channels on both operands (the SDXL round-to-nearest arm:
    weights on the ``qdq_weight(w, 8, 32)`` grid, activations on the per-token ``dyn_group`` grid with group 32),
    executed on the integer grid.  Needs in_features % 128 == 0."""

    def __init__(self, lin: nn.Linear, device: Optional[torch.device] = None):
        super().__init__()
        w = lin.weight.detach()
        if device is not None:
            w = w.to(device)
        codes, scale = _quantize_weight_g32(w)
        self.register_buffer("weight_int8", codes)
        self.register_buffer("w_scale", scale)                               # [N, K/32]
        self.register_buffer("w_scale_gm", scale.t().contiguous(), persistent=False)   # [K/32, N] for the kernel
        if lin.bias is not None:
            b = lin.bias.detach().float()
            self.register_buffer("bias", (b.to(device) if device is not None else b).contiguous())
        else:
            self.bias = None
        self.in_features = int(lin.in_features)
        self.out_features = int(lin.out_features)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        xq, sa = quant_rows_g32(x2)
        y = int8_gemm_g32(xq, sa, self.weight_int8, self.w_scale_gm, self.bias, x2.dtype)
        return y.reshape(*shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, int8 group-32 W / per-token group-32 A"


_LO_SCRATCH: Dict[Tuple[int, int, int], torch.Tensor] = {}      # (device index, stream, bytes) -> expansion buffer


class Int8LinearRouted(Int8Linear):
    """Two-tier routed Linear: rows gathered from a token canvas, the first ``m_hi`` rows run against
    the INT8 codes, the rest against the nested 4-bit grid derived from them (``nested4_codes``).

    ``pack_lo=True`` keeps the low tier at rest as packed nibbles (``weight_lo_packed`` uint8 [N, K/2], half the
    bytes of ``weight_lo``) and expands it right before each forward (one small HBM-bound kernel) into a scratch
    buffer that all layers of the same size share: the reference's storage-only W4 tier made real.  The buffer is
    refilled by every forward and read by the GEMM that follows on the same stream, so there is one per CUDA stream:
    layers running on different streams never see each other's weights.

    A low-rank branch the fused epilogue does not take (rank other than 32, factors in another dtype than the
    activations, in_features not a multiple of 32) is added after the GEMM as ``(x @ lr_A) @ lr_B``, the way
    ``Int8Linear.forward`` does."""

    def __init__(self, lin: nn.Linear, device: Optional[torch.device] = None,
                 lowrank: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, pack_lo: bool = False):
        super().__init__(lin, device=device, lowrank=lowrank)
        c4, s4 = nested4_codes(self.weight_int8, self.w_scale)
        self.pack_lo = bool(pack_lo)
        if self.pack_lo:
            assert self.in_features % 32 == 0, "packed low tier needs in_features % 32 == 0"
            self.register_buffer("weight_lo_packed", ops.pack_int4(c4))
        else:
            self.register_buffer("weight_lo", c4)
        self.register_buffer("w_scale_lo", s4)

    def _lo_codes(self) -> torch.Tensor:
        """The low tier as int8 [N, K]: the buffer itself, or the packed nibbles expanded into this stream's scratch."""
        if not self.pack_lo:
            return self.weight_lo
        p = self.weight_lo_packed
        key = (p.device.index if p.device.index is not None else torch.cuda.current_device(), ops._stream(p), p.numel() * 2)
        buf = _LO_SCRATCH.get(key)
        if buf is None:
            buf = torch.empty(p.numel() * 2, dtype=torch.int8, device=p.device)
            _LO_SCRATCH[key] = buf
        return ops.unpack_int4(p, buf.view(self.out_features, self.in_features))

    def _two_tier(self, xq, sx, x_rows: Callable[[], torch.Tensor], m_hi: int, dtype: torch.dtype, fused: bool):
        t = lb = lbt = None
        if fused:
            t = self._down(x_rows())
            lb = self.lr_B; lbt = self._lr_Bt()
        y = int8_gemm_grouped(xq, sx, self.weight_int8, self.w_scale, self._lo_codes(), self.w_scale_lo,
                              self.bias, t, lb, m_hi, dtype, lbt)
        if self.lr_A is not None and not fused:                    # branch the fused epilogue does not take
            xa = x_rows().to(self.lr_A.dtype) @ self.lr_A
            y.addmm_(xa.to(y.dtype), self.lr_B.to(y.dtype))
        return y

    def forward_rows(self, x2: torch.Tensor, m_hi: int) -> torch.Tensor:
        """x2 [M,K] already gathered and ordered hi-tier rows first."""
        xq, sx = quant_rows(x2)
        return self._two_tier(xq, sx, lambda: x2, m_hi, x2.dtype, self._fusable_lowrank(x2))

    def forward_gathered(self, canvas: torch.Tensor, row_idx: torch.Tensor, m_hi: int) -> torch.Tensor:
        """Gather + quantise in one kernel straight from the canvas, then the two-tier GEMM."""
        xq, sx = gather_quant_rows(canvas, row_idx)
        return self._two_tier(xq, sx, lambda: (ops._gather_rows_impl(canvas, row_idx) if _eager() else
                                               torch.ops.pq_b200.gather_rows(canvas, row_idx)), m_hi, canvas.dtype,
                              self._fusable_lowrank(canvas))


# --------------------------------------------------------------------------- model conversion
def is_bf16_whitelisted(name: str) -> bool:
    """Layers that stay in 16 bit: embedders, the output projection, time/text embedding, the final norm
    and every adaLN modulation projection ``*.norm*.linear`` (reference :415-421)."""
    parts = name.split(".")
    if parts[0] in ("x_embedder", "context_embedder", "proj_out", "time_text_embed", "norm_out"):
        return True
    return len(parts) >= 2 and parts[-1] == "linear" and parts[-2].startswith("norm")


def group_shared_inputs(model: nn.Module, groups: Sequence[Sequence[str]] = FLUX_SHARED_INPUT_GROUPS) -> int:
    """For every module of ``model`` under which all relative paths of a group name converted ``Int8Linear`` layers,
    ties those layers into a ``SharedInputGroup`` (a layer joins at most one group: the first that matches, so list
    the widest group first).  Returns the number of groups made."""
    made = 0
    taken = set()
    for _name, parent in model.named_modules():
        for paths in groups:
            members = []
            for rel in paths:
                try:
                    m = parent.get_submodule(rel)
                except AttributeError:
                    m = None
                if not isinstance(m, Int8Linear) or id(m) in taken:
                    members = []
                    break
                members.append(m)
            if len(members) >= 2 and len({m.in_features for m in members}) == 1:
                SharedInputGroup(members)
                taken.update(id(m) for m in members)
                made += 1
    return made


def convert_linears_to_int8(model: nn.Module, device: Optional[str] = "cuda",
                            whitelist: Callable[[str], bool] = is_bf16_whitelisted,
                            shared_input_groups: Optional[Sequence[Sequence[str]]] = None,
                            fuse_split: bool = False) -> Dict[str, object]:
    """Swaps every non-whitelisted ``nn.Linear`` for ``Int8Linear`` in place and returns the same
    statistics dictionary as the reference (:444-445).  ``shared_input_groups`` (not in the reference; e.g.
    ``FLUX_SHARED_INPUT_GROUPS``) additionally ties sibling layers that read the same tensor into one quantisation
    and one down-projection per input; the count is reported as ``n_shared_input_groups``.  ``fuse_split`` (not in the
    reference) replaces converted ``SplitInLinear`` modules by ``SplitInInt8Linear`` (``n_split_fused``)."""
    dev = torch.device(device) if device is not None else None
    stats = {"n_int8_linear": 0, "n_bf16_linear_kept": 0, "params_int8": 0, "params_bf16_linear_kept": 0,
             "bf16_kept_names": []}
    for name, lin in [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear)]:
        if whitelist(name):
            stats["n_bf16_linear_kept"] += 1
            stats["params_bf16_linear_kept"] += lin.weight.numel()
            stats["bf16_kept_names"].append(name)
            continue
        parent_name, _, attr = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, attr, Int8Linear(lin, device=dev))
        stats["n_int8_linear"] += 1
        stats["params_int8"] += lin.weight.numel()
    if dev is not None and dev.type == "cuda":
        torch.cuda.synchronize()
    stats["int8_weight_gib"] = stats["params_int8"] / 2**30
    stats["bf16_equiv_gib"] = stats["params_int8"] * 2 / 2**30
    if shared_input_groups is not None:
        stats["n_shared_input_groups"] = group_shared_inputs(model, shared_input_groups)
    if fuse_split:
        stats["n_split_fused"] = fuse_split_inputs(model)
    return stats


FLUX_TOKEN_SHAPES = {   # (K, N): number of such token-level Linears in FLUX.1-schnell (reference :478-483)
    (3072, 3072): 19 * 8 + 38 * 3,
    (3072, 12288): 19 * 2 + 38,
    (12288, 3072): 19 * 2,
    (15360, 3072): 38,
}


def warm_kernels(Ms=(4352, 16640, 65792), device="cuda", lowrank_R=32, warm_lowrank: bool = True):
    """Nothing is compiled at run time; this loads the library, creates the per-device status word and
    runs each FLUX shape once so that first-call costs (module load, tensor-map cache) stay outside
    timed regions.  Signature as the reference (:448-474)."""
    t0 = time.perf_counter()
    for (K, N) in FLUX_TOKEN_SHAPES:
        w = torch.randint(-127, 127, (N, K), device=device, dtype=torch.int8)
        s = torch.rand(N, device=device); b = torch.rand(N, device=device)
        lb = torch.randn(lowrank_R, N, device=device, dtype=torch.bfloat16)
        x = torch.randn(min(Ms), K, device=device, dtype=torch.bfloat16)
        int8_linear_2d(x, w, s, b)
        if warm_lowrank:
            xq, sx = quant_rows(x)
            t = torch.randn(x.shape[0], lowrank_R, device=device, dtype=torch.bfloat16)
            int8_gemm_lr(xq, sx, w, s, b, t, lb, torch.bfloat16)
        del w, s, b, lb, x
    torch.cuda.synchronize(); torch.cuda.empty_cache()
    ops.check_device_status(device)
    print(f"[int8_exec] kernels warmed (backend={BACKEND} -> sm_100a native, lowrank r={lowrank_R}) "
          f"in {time.perf_counter() - t0:.1f}s", flush=True)


# --------------------------------------------------------------------------- self-test / micro-benchmark
def _bench(fn, iters=20, warm=3):
    """Mean milliseconds per call of `fn` (same signature and unit as the reference's helper, :486-492), timed on the
    device with CUDA events on the current stream."""
    for _ in range(warm):
        fn()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    stop.synchronize()
    return start.elapsed_time(stop) / iters


def _rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    return float(((a - b).norm() / b.norm()).item())


def _selftest(dev: str) -> Dict[str, object]:
    """The reference's numerical self-test (:498-536) on its input (seed 0, 4352 x 3072 -> 12288, channel 5 scaled by
    30), reported under the same keys and asserted with the same thresholds."""
    torch.manual_seed(0)
    lin = nn.Linear(3072, 12288, bias=True).to(dev, torch.bfloat16)
    x = (torch.randn(4352, 3072, device=dev) * 2).to(torch.bfloat16)
    x[:, 5] *= 30.0
    layer = Int8Linear(lin, device=torch.device(dev))

    def unfused(rows: torch.Tensor) -> torch.Tensor:
        """codes @ codes in fp32, the two scales applied one after the other, bias, rounded (:506-510)."""
        codes, scale = quant_rows(rows)
        acc = codes.float() @ layer.weight_int8.float().t()
        return ((acc * scale[:, None] * layer.w_scale[None, :] + layer.bias[None, :]).to(torch.bfloat16).float())

    y = layer(x).float()
    y_unfused = unfused(x)
    y_bf16 = F.linear(x, lin.weight, lin.bias).float()
    # torch's quantiser evaluated on the CPU, where division by a Python scalar is an IEEE division
    xf = x.float().cpu()
    scale_ref = xf.abs().amax(1, keepdim=True).clamp_min(1e-8) / 127
    codes_ref = torch.round(xf / scale_ref).clamp(-127, 127).to(torch.int8)
    codes, scale = quant_rows(x)
    plain = torch.randn(4352, 3072, device=dev).to(torch.bfloat16)
    few = x[:8]
    stacked = x[:2048].reshape(8, 256, 3072)
    rep = {
        "act_quant_mismatch_elems": int((codes.cpu() != codes_ref).sum().item()),
        "act_scale_max_rel_err": float(((scale.cpu() - scale_ref[:, 0]).abs() / scale_ref[:, 0]).max().item()),
        "fused_vs_unfused_int8_max_abs": float((y - y_unfused).abs().max().item()),
        "fused_vs_unfused_int8_rel": _rel_l2(y, y_unfused),
        "int8_vs_bf16_rel_outlier30x": _rel_l2(y, y_bf16),
        "int8_vs_bf16_rel_plain": _rel_l2(layer(plain).float(), F.linear(plain, lin.weight, lin.bias).float()),
        "smallM_fused_vs_unfused_rel": _rel_l2(layer(few).float(), unfused(few)),
        "3d_input_ok": bool(torch.equal(layer(stacked).reshape(2048, -1), layer(x[:2048]))),
    }
    rep["act_quant_mismatch_frac"] = rep["act_quant_mismatch_elems"] / x.numel()
    print("[int8_exec] selftest:", rep, flush=True)
    assert rep["act_quant_mismatch_frac"] <= 1e-4, rep
    assert rep["fused_vs_unfused_int8_rel"] < 1e-3 and rep["int8_vs_bf16_rel_plain"] < 2e-2, rep
    assert rep["smallM_fused_vs_unfused_rel"] < 1e-3 and rep["3d_input_ok"], rep
    ops.check_device_status(dev)
    return rep


def selftest_and_bench(Ms=(4352, 16640, 33744, 65792), iters=10):
    """Self-test, then the per-M micro-benchmark over the FLUX token-level shapes weighted by how often each occurs
    in the model (:541-570); result layout as the reference's (``selftest``, ``gpu``, ``per_M`` -> totals and
    ``per_shape``)."""
    dev = "cuda"
    out = {"selftest": _selftest(dev), "gpu": torch.cuda.get_device_name(), "per_M": {}}
    torch.cuda.empty_cache()
    columns = ("bf16_ms", "int8_fused_ms", "quant_ms", "gemm_fused_ms")
    for M in Ms:
        image = dict.fromkeys(columns, 0.0)
        per_shape = {}
        for (K, N), count in FLUX_TOKEN_SHAPES.items():
            lin = nn.Linear(K, N, bias=True).to(dev, torch.bfloat16)
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            layer = Int8Linear(lin, device=torch.device(dev))
            codes, scale = quant_rows(x)
            ms = dict(zip(columns, (
                _bench(lambda: F.linear(x, lin.weight, lin.bias), iters),
                _bench(lambda: layer(x), iters),
                _bench(lambda: quant_rows(x), iters),
                _bench(lambda: int8_gemm_fused(codes, scale, layer.weight_int8, layer.w_scale, layer.bias,
                                               torch.bfloat16), iters))))
            for c in columns:
                image[c] += ms[c] * count
            per_shape[f"{K}x{N}"] = {"count": count, **{c: round(v, 3) for c, v in ms.items()},
                                     "speedup": round(ms["bf16_ms"] / ms["int8_fused_ms"], 3),
                                     "gemm_tops": round(2.0 * M * N * K / (ms["gemm_fused_ms"] * 1e-3) / 1e12, 1)}
            del lin, x, layer, codes, scale
            torch.cuda.empty_cache()
        tot = {c: round(v, 2) for c, v in image.items()}
        tot["speedup_fused_vs_bf16"] = round(tot["bf16_ms"] / tot["int8_fused_ms"], 3)
        tot["per_shape"] = per_shape
        out["per_M"][str(M)] = tot
        print(f"[int8_exec] M={M}: bf16 {tot['bf16_ms']} ms | int8 {tot['int8_fused_ms']} ms "
              f"(quant {tot['quant_ms']}, gemm {tot['gemm_fused_ms']}) -> x{tot['speedup_fused_vs_bf16']}", flush=True)
    return out


if __name__ == "__main__":
    import argparse
    import json
    ap = argparse.ArgumentParser(description="INT8 kernel self-test and micro-benchmark on the FLUX token-level "
                                             "Linear shapes (needs a B200).")
    ap.add_argument("out", nargs="?", default=None, help="optional JSON path for the results")
    ap.add_argument("--int8-backend", choices=BACKENDS, default=DEFAULT_BACKEND,
                    help="accepted for compatibility; both names run the sm_100a library")
    args = ap.parse_args()
    set_backend(args.int8_backend)
    res = selftest_and_bench()
    res["int8_backend"] = BACKEND
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(res, fh, indent=1)
        print(f"[int8_exec] saved {args.out}")
