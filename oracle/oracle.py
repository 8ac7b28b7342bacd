"""CPU oracle for the INT8 deployment hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this file, and only
as the checker or the timed CPU baseline -- the product (pyraquant_b200/) never imports it and has no
CPU path.

It is a plain torch-on-CPU restatement of the reference's algorithm; each function cites the reference
lines it follows (paths inside the PyraQuant repository).  The reference's own forward needs CUDA +
Triton (deploy/int8_exec.py:221 asserts is_cuda), so the forward is restated from its kernel sources
and its self-test expressions; the pieces of the reference that do run on CPU (weight quantisation in
Int8Linear.__init__, _ActFakeQuant, qdq_weight, nested4_qdq_weight, ExtActQuant._qdq_rows,
build_patch_buckets, fuse_patch_predictions, inner_split_median) were executed in the build container
and their outputs are committed under tests/golden/ (made by tests/golden/make_golden.py); the oracle
is pinned against those fixtures by tests/test_oracle_golden.py.

Parity status: integer codes, scales and int32 accumulators are pinned by the CPU-made fixtures; the assembled
forward (quantise -> int32 GEMM -> epilogue) is pinned by tests/golden/forward_reference_gpu.npz, made by running the
reference's unmodified Int8Linear.forward on a B200 (tests/golden/make_golden_gpu.py; its "cublas" backend, because
its Triton GEMM kernels do not compile under the installed Triton), against which tests/test_reference_forward.py
checks this oracle on the CPU and the CUDA path on the GPU.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

Box = Tuple[int, int, int, int]


# ------------------------------------------------------------------------------------------------ quantisers
def quant_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token symmetric INT8.  deploy/int8_exec.py:508-509 (torch form of the kernel at :83-101);
    same math as pyraquant/quant_unet.py:52-54."""
    xf = x.float()
    sc = xf.abs().amax(1, keepdim=True).clamp_min(1e-8) / 127
    xq = torch.round(xf / sc).clamp(-127, 127).to(torch.int8)
    return xq, sc[:, 0].contiguous()


def adaln_modulate(h: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Input of the feed-forward's first Linear in a FLUX block: flux/transformer_flux.py:236-237
    `norm2(h) * (1 + scale_mlp[:, None]) + shift_mlp[:, None]` with `norm2 = nn.LayerNorm(dim, elementwise_affine=False,
    eps=1e-6)` (:195), evaluated in the tensors' own 16-bit type like the reference.  h [B, T, K]; scale, shift [B, K]."""
    y = torch.nn.functional.layer_norm(h, (h.shape[-1],), eps=eps)
    return y * (1 + scale[:, None]) + shift[:, None]


def quant_rows_g32(x: torch.Tensor, group: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token, per-group symmetric INT8 ("dyn_group", 8 bits signed => qmax 127).
    pyraquant/external_quant.py:104-109 with _qrange at :60-61."""
    xf = x.float()
    M, K = xf.shape
    xg = xf.reshape(M, K // group, group)
    s = xg.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8) / 127
    q = (xg / s).round().clamp(-127, 127)
    return q.reshape(M, K).to(torch.int8), s[..., 0].contiguous()


def over_qmax(amax: torch.Tensor, qmax: float, where: str) -> torch.Tensor:
    """`amax / qmax` with qmax a Python scalar, as torch evaluates it where the reference's constructor runs.
    On the CPU it is an IEEE division.  torch's CUDA kernel for division by a host scalar multiplies by the fp32
    reciprocal instead (amax * fl32(1 / qmax)), which differs from the quotient by one unit in the last place for some
    inputs and moves weights that sit on a rounding tie to the neighbouring code.  `where` = "cpu" | "cuda" selects
    which of the two results is restated; both are pinned by fixtures made by the reference (int8linear_ctor.npz on
    the CPU, the w_scale / code row sums of forward_reference_gpu.npz on a B200)."""
    if where == "cpu":
        return amax / qmax
    assert where == "cuda", where
    return amax * torch.tensor(float(np.float32(1.0) / np.float32(qmax)), dtype=torch.float32)


def quant_weight(w: torch.Tensor, where: str = "cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel symmetric INT8 weights.  deploy/int8_exec.py:355-357."""
    wf = w.float()
    s = over_qmax(wf.abs().amax(dim=1).clamp_min(1e-8), 127.0, where)
    q = torch.round(wf / s[:, None]).clamp_(-127, 127).to(torch.int8)
    return q.contiguous(), s.contiguous()


def quant_weight_g32(w: torch.Tensor, group: int = 32, where: str = "cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """Group-32 INT8 weight grid = the codes and scales behind qdq_weight(w, 8, 32).
    pyraquant/quantizers_weight.py:96-109 (W8_GROUPED is True, :65)."""
    out_f, in_f = w.shape
    wg = w.detach().float().reshape(out_f, in_f // group, group)
    scale = over_qmax(wg.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8), 127, where)
    q = (wg / scale).round().clamp_(-127, 127)
    return q.reshape(out_f, in_f).to(torch.int8), scale[..., 0].contiguous()


def nested4_from_int8(q8: torch.Tensor, s8: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Nested 4-bit codes derived from the INT8 codes: c = round(q8*7/127) clamp +-7, scale s8*127/7.
    pyraquant/quantizers_weight.py:196-199."""
    c = (q8.float() * (7 / 127)).round().clamp_(-7, 7)
    return c.to(torch.int8), (s8.float() * (127 / 7))


# ------------------------------------------------------------------------------------------------ GEMM
def int_mm(xq: torch.Tensor, w_int8: torch.Tensor) -> torch.Tensor:
    """Exact int32 accumulators of xq [M,K] @ w_int8[N,K]^T.  The reference's own call is
    torch._int_mm(xq, w.t()) (deploy/int8_exec.py:259); on CPU it is used when it accepts the shape,
    otherwise an int64 matmul (also exact) takes over."""
    try:
        if xq.shape[0] > 16:
            return torch._int_mm(xq.contiguous(), w_int8.t())
    except RuntimeError:
        pass
    return (xq.to(torch.int64) @ w_int8.to(torch.int64).t()).to(torch.int32)


def epilogue(acc: torch.Tensor, s_row: torch.Tensor, s_col: torch.Tensor, bias: Optional[torch.Tensor],
             t: Optional[torch.Tensor], lb: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """Kernel epilogue order of deploy/int8_exec.py:303-309 (and :176-178 without the low-rank term):
    y = float(acc) * (s_row * s_col);  y += t @ lb (16-bit inputs, fp32 accumulate);  y += bias;  cast."""
    y = acc.float() * (s_row[:, None] * s_col[None, :])
    if t is not None:
        y = y + t.float() @ lb.float()
    if bias is not None:
        y = y + bias[None, :]
    return y.to(out_dtype)


def int8_linear_forward(x: torch.Tensor, w_int8: torch.Tensor, w_scale: torch.Tensor,
                        bias: Optional[torch.Tensor], lr_A: Optional[torch.Tensor] = None,
                        lr_B: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Int8Linear.forward, fused path.  deploy/int8_exec.py:382-393: t = x @ lr_A rounded to the
    activation dtype (:390), quantise (:391), fused GEMM + low-rank + bias (:392)."""
    x2 = x.reshape(-1, x.shape[-1])
    t = lb = None
    if lr_A is not None:
        t = (x2.to(lr_A.dtype).float() @ lr_A.float()).to(lr_A.dtype)
        lb = lr_B
    xq, sx = quant_rows(x2)
    acc = int_mm(xq, w_int8)
    y = epilogue(acc, sx, w_scale, bias, t, lb, x2.dtype)
    return y.reshape(*x.shape[:-1], w_int8.shape[0])


def exact_dequant_f64(acc: torch.Tensor, s_row: torch.Tensor, s_col: torch.Tensor, bias, t, lb) -> torch.Tensor:
    """The "reference dequantised math" in fp64: the value every rounding variant approximates."""
    y = acc.double() * s_row.double()[:, None] * s_col.double()[None, :]
    if t is not None:
        y = y + t.double() @ lb.double()
    if bias is not None:
        y = y + bias.double()[None, :]
    return y


def selftest_unfused_reference(xq, sx, w_int8, w_scale, bias, out_dtype=torch.bfloat16) -> torch.Tensor:
    """The unfused expression the reference's self-test compares its kernels with
    (deploy/int8_exec.py:506,510): fp32 matmul of the codes, scales applied one after the other."""
    ref = (xq.float() @ w_int8.float().t()) * sx[:, None] * w_scale[None, :]
    if bias is not None:
        ref = ref + bias[None, :]
    return ref.to(out_dtype)


def gemm_g32(xq: torch.Tensor, s_a: torch.Tensor, wq: torch.Tensor, s_w: torch.Tensor, bias, out_dtype,
             group: int = 32) -> torch.Tensor:
    """y[m,n] = sum_g s_a[m,g] s_w[n,g] sum_{k in g} xq[m,k] wq[n,k] (+bias): exact per-group int32
    partials, fp32 combination in ascending group order with one fused multiply-add per group.  Grids: pyraquant/quantizers_weight.py:96-109
    and pyraquant/external_quant.py:104-109."""
    M, K = xq.shape
    N = wq.shape[0]
    G = K // group
    y = torch.zeros(M, N, dtype=torch.float32)
    for g in range(G):
        a = xq[:, g * group:(g + 1) * group].to(torch.int32)
        b = wq[:, g * group:(g + 1) * group].to(torch.int32)
        part = (a @ b.t()).double()                       # |part| <= 32 * 127^2: exact
        s = (s_a[:, g][:, None] * s_w[:, g][None, :])     # fp32 product of the two scales
        # fused multiply-add in fp32: the product part * s is exact in fp64 (20 + 24 bits) and the sum is rounded
        # to fp32 afterwards
        y = (y.double() + part * s.double()).float()
    if bias is not None:
        y = y + bias[None, :]
    return y.to(out_dtype)


def gemm_g32_f64(xq, s_a, wq, s_w, bias, group: int = 32) -> torch.Tensor:
    M, K = xq.shape
    G = K // group
    a = xq.double().reshape(M, G, group) * s_a.double()[..., None]
    b = wq.double().reshape(wq.shape[0], G, group) * s_w.double()[..., None]
    y = a.reshape(M, K) @ b.reshape(-1, K).t()
    if bias is not None:
        y = y + bias.double()[None, :]
    return y


# ------------------------------------------------------------------------------------------------ routing
def leaf_run_boxes(sel: np.ndarray, leaf_latent: int) -> List[Box]:
    """flux/run_flux.py:341-355: row-wise runs of selected leaves become latent boxes."""
    sm = np.asarray(sel) > 0.5
    boxes = []
    for i in range(sm.shape[0]):
        j = 0
        while j < sm.shape[1]:
            if sm[i, j]:
                j0 = j
                while j < sm.shape[1] and sm[i, j]:
                    j += 1
                boxes.append((i * leaf_latent, (i + 1) * leaf_latent, j0 * leaf_latent, j * leaf_latent))
            else:
                j += 1
    return boxes


def token_box(box: Box) -> Box:
    """flux/routing.py:226-232 with packing offset 0."""
    y0, y1, x0, x1 = (int(v) for v in box)
    return (y0 // 2, (y1 + 1) // 2, x0 // 2, (x1 + 1) // 2)


def halo_box(core: Box, halo: int, token_hw) -> Box:
    """flux/routing.py:235-244."""
    y0, y1, x0, x1 = core
    return (max(0, y0 - halo), min(int(token_hw[0]), y1 + halo), max(0, x0 - halo), min(int(token_hw[1]), x1 + halo))


def gather_buckets(grid: torch.Tensor, boxes_latent: Sequence[Box], halo: int):
    """build_patch_buckets (flux/routing.py:253-315) on a [1,H,W,C] token grid: returns
    [(patch_hw, tensor [n, ph*pw, C], [(core, outer, inner), ...])] sorted by patch shape."""
    _, H, W, C = grid.shape
    by_shape = {}
    seen = set()
    for box in boxes_latent:
        core = token_box(box)
        if core in seen:
            continue
        seen.add(core)
        outer = halo_box(core, halo, (H, W))
        oy0, oy1, ox0, ox1 = outer
        hw = (oy1 - oy0, ox1 - ox0)
        inner = (core[0] - oy0, core[1] - oy0, core[2] - ox0, core[3] - ox0)
        patch = grid[:, oy0:oy1, ox0:ox1, :].reshape(1, hw[0] * hw[1], C)
        by_shape.setdefault(hw, []).append((patch, (core, outer, inner)))
    out = []
    for hw in sorted(by_shape):
        items = by_shape[hw]
        out.append((hw, torch.cat([it[0] for it in items], dim=0), [it[1] for it in items]))
    return out


def feather_mask(hw, inner, dtype) -> torch.Tensor:
    """halo_feather_mask with the cosine ramp (flux/routing.py:34-75, _smooth_ramp :22-31)."""
    H, W = hw
    iy0, iy1, ix0, ix1 = inner
    yw = torch.ones(H, dtype=torch.float32)
    xw = torch.ones(W, dtype=torch.float32)

    def ramp(v):
        return (0.5 - 0.5 * torch.cos(torch.pi * v.clamp(0.0, 1.0))).clamp(0.0, 1.0)

    if iy0 > 0:
        yw[:iy0] = ramp(torch.linspace(0.0, 1.0, iy0))
    if iy1 < H:
        yw[iy1:] = ramp(torch.linspace(1.0, 0.0, H - iy1))
    if ix0 > 0:
        xw[:ix0] = ramp(torch.linspace(0.0, 1.0, ix0))
    if ix1 < W:
        xw[ix1:] = ramp(torch.linspace(1.0, 0.0, W - ix1))
    return torch.minimum(yw[:, None], xw[None, :]).clamp(0.0, 1.0).to(dtype)


def fuse_buckets(background: torch.Tensor, bucket_outputs, fusion_beta: float = 1.0) -> torch.Tensor:
    """fuse_patch_predictions (flux/routing.py:328-379): accumulators in the background dtype,
    patches added in bucket order, normalised blend over the background."""
    _, H, W, C = background.shape
    local = torch.zeros_like(background)
    bacc = torch.zeros((1, H, W, 1), dtype=background.dtype)
    for (hw, geoms), output in bucket_outputs:
        og = output.reshape(output.shape[0], hw[0], hw[1], C)
        for i, (_core, outer, inner) in enumerate(geoms):
            y0, y1, x0, x1 = outer
            beta = feather_mask(hw, inner, background.dtype)
            beta = (float(fusion_beta) * beta).clamp(0.0, 1.0)[None, :, :, None]
            local[:, y0:y1, x0:x1, :] += beta * og[i:i + 1]
            bacc[:, y0:y1, x0:x1, :] += beta
    bmap = bacc.clamp(0.0, 1.0)
    combined = torch.where(bacc > 0.0, local / bacc.clamp_min(1e-8), torch.zeros_like(local))
    return (1.0 - bmap) * background + bmap * combined


def inner_split_median(scores: torch.Tensor, sel: torch.Tensor, inner_thresh: float) -> torch.Tensor:
    """flux/run_flux.py:238-250."""
    cand = sel > 0.5
    v = scores[cand]
    if v.numel() == 0:
        return torch.zeros_like(scores)
    ref = float(v.median().item()) if v.numel() > 1 else float(v.max().item())
    hi = ((scores >= float(inner_thresh) * max(ref, 1e-12)) & cand).float()
    if float(hi.sum().item()) == 0:
        masked = torch.where(cand, scores, torch.full_like(scores, -1e30))
        hi = ((masked >= masked.max()) & cand).float()
    return hi


# ------------------------------------------------------------------------------------------------ workloads
def make_layer(seed: int, M: int, K: int, N: int, *, dtype=torch.bfloat16, outlier_frac: float = 0.005,
               outlier_scale: float = 20.0, lowrank: bool = True, bias: bool = True):
    """Seeded synthetic layer with the distributions the benchmark configurations state: X ~ N(0,1) with a
    fraction of channels scaled up, W ~ N(0,0.02), low-rank factors ~ N(0,0.02), bias ~ N(0,0.01).
    Generated on CPU so that CPU oracle and GPU kernels see identical bits."""
    g = torch.Generator().manual_seed(int(seed))
    x = torch.randn(M, K, generator=g)
    n_out = int(round(K * outlier_frac))
    if n_out > 0:
        ch = torch.randperm(K, generator=g)[:n_out]
        x[:, ch] *= outlier_scale
    w = torch.randn(N, K, generator=g) * 0.02
    out = {"x": x.to(dtype), "w": w.to(dtype)}
    if lowrank:
        out["lr_A"] = (torch.randn(K, 32, generator=g) * 0.02).to(dtype)
        out["lr_B"] = (torch.randn(32, N, generator=g) * 0.02).to(dtype)
    if bias:
        out["bias"] = torch.randn(N, generator=g) * 0.01
    return out
