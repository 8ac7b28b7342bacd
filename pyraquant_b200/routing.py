"""Host-side planning for the routed executor's token gather / scatter.

The reference (flux/routing.py) slices every active box out of the token grid, concatenates same-shape
patches into buckets, and later blends the per-patch outputs back with per-patch tensor arithmetic.
Here the same geometry is turned ONCE per stage into flat index lists that two CUDA kernels consume:

  gather : ``row_idx[m]`` = canvas token feeding gathered row m.  Rows are laid out exactly like the
           reference's buckets concatenated in order (buckets sorted by patch shape, patches in first-seen
           order, tokens row-major inside a patch; flux/routing.py:253-315), optionally re-ordered so
           that high-precision rows come first (two-tier routing).
  scatter: for every canvas token touched by a patch, its contributor list (gathered row, blend weight)
           in the reference's accumulation order (flux/routing.py:343-379), as CSR arrays.

Box construction from a leaf selection map follows flux/run_flux.py:341-355, the latent->token mapping
flux/routing.py:202-232, the halo expansion :235-244 and the feather weights :34-75.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops

Box = Tuple[int, int, int, int]   # y0, y1, x0, x1 (half-open)


def leaf_run_boxes(selected: np.ndarray, leaf_latent: int) -> List[Box]:
    """Row-wise runs of selected leaves -> boxes in latent coordinates (flux/run_flux.py:341-355)."""
    sel = np.asarray(selected) > 0.5
    boxes: List[Box] = []
    for i in range(sel.shape[0]):
        j = 0
        while j < sel.shape[1]:
            if not sel[i, j]:
                j += 1
                continue
            j0 = j
            while j < sel.shape[1] and sel[i, j]:
                j += 1
            boxes.append((i * leaf_latent, (i + 1) * leaf_latent, j0 * leaf_latent, j * leaf_latent))
    return boxes


def latent_box_to_token_box(box: Sequence[int], packing_offset_latent: int = 0) -> Box:
    """Token box covering a latent box under FLUX's 2x2 packing: a latent row/column v belongs to token
    (v + offset) // 2, so a half-open latent span [a, b) maps to tokens [(a + offset) // 2, (b + offset + 1) // 2)
    (the mapping of flux/routing.py:202-232).  Rejected with ValueError: an offset other than 0 or 1, negative or odd
    coordinates, spans without area."""
    off = int(packing_offset_latent)
    if off != 0 and off != 1:
        raise ValueError(f"packing_offset_latent is 0 or 1 (got {packing_offset_latent!r})")
    y0, y1, x0, x1 = (int(v) for v in box)
    problem = None
    if min(y0, y1, x0, x1) < 0:
        problem = "negative coordinate"
    elif (y0 | y1 | x0 | x1) & 1:
        problem = "coordinates must be even (2x2 packing)"
    elif y1 <= y0 or x1 <= x0:
        problem = "no area"
    if problem is not None:
        raise ValueError(f"route box {(y0, y1, x0, x1)}: {problem}")
    first = lambda v: (v + off) >> 1
    end = lambda v: (v + off + 1) >> 1
    return (first(y0), end(y1), first(x0), end(x1))


def expand_box(box: Box, halo_tokens: int, token_hw: Tuple[int, int]) -> Box:
    y0, y1, x0, x1 = box
    h = max(0, int(halo_tokens))
    return (max(0, y0 - h), min(int(token_hw[0]), y1 + h), max(0, x0 - h), min(int(token_hw[1]), x1 + h))


# Halo profiles: u runs over [0, 1] across the halo (0 at the patch border, 1 where the core begins).
_RAMP_SHAPES = {
    "cosine": lambda u: 0.5 - 0.5 * torch.cos(torch.pi * u),
    "smoothstep": lambda u: u * u * (3.0 - 2.0 * u),
    "linear": lambda u: u,
}


def _axis_profile(length: int, core_lo: int, core_hi: int, shape, power: float) -> torch.Tensor:
    """fp32 blend weights along one axis of a patch: 1 on [core_lo, core_hi), the halo profile on either side.  A halo
    of h tokens samples the profile at h evenly spaced points including both ends, so its outermost token weighs 0."""
    core_lo = min(max(core_lo, 0), length)
    core_hi = min(max(core_hi, core_lo), length)
    w = torch.ones(length, dtype=torch.float32)
    for sl, u0, u1 in ((slice(0, core_lo), 0.0, 1.0), (slice(core_hi, length), 1.0, 0.0)):
        n = sl.stop - sl.start
        if n <= 0:
            continue
        v = shape(torch.linspace(u0, u1, n).clamp_(0.0, 1.0))
        if power != 1.0:
            v = v.pow(max(power, 1e-6))
        w[sl] = v.clamp_(0.0, 1.0)
    return w


def feather_weights(patch_hw: Tuple[int, int], inner: Box, dtype: torch.dtype, fusion_beta: float = 1.0,
                    mode: str = "cosine", power: float = 1.0) -> torch.Tensor:
    """[H, W] blend weights of one patch = min(row profile, column profile), evaluated in fp32, rounded to `dtype`
    and then scaled by fusion_beta in `dtype`: the values of flux/routing.py:34-75 and :361-370 (the tests compare
    them with masks produced by the reference).  ``mode``: "cosine" (the reference's default), "smoothstep" or
    "linear"; ``power`` sharpens (> 1) or softens (< 1) the profile."""
    try:
        shape = _RAMP_SHAPES[mode]
    except KeyError:
        raise ValueError(f"feather mode {mode!r}; known: {sorted(_RAMP_SHAPES)}") from None
    rows = _axis_profile(int(patch_hw[0]), int(inner[0]), int(inner[1]), shape, float(power))
    cols = _axis_profile(int(patch_hw[1]), int(inner[2]), int(inner[3]), shape, float(power))
    mask = torch.minimum(rows[:, None], cols[None, :]).to(dtype)
    return (float(fusion_beta) * mask).clamp_(0.0, 1.0)


@dataclass
class Patch:
    core: Box
    outer: Box
    hw: Tuple[int, int]
    row0: int = 0          # first gathered row of this patch (bucket order)


@dataclass
class RoutePlan:
    """Flat gather / scatter index lists for one routed stage (host arrays; ``to(device)`` uploads them)."""
    token_hw: Tuple[int, int]
    patches: List[Patch]
    bucket_shapes: List[Tuple[int, int]]
    row_idx: np.ndarray            # int32 [M_act]   canvas token of each gathered row
    m_hi: int                      # rows [0, m_hi) are high precision (== M_act without tiers)
    tokens: np.ndarray             # int32 [n_tokens] canvas tokens with at least one contributor
    ptr: np.ndarray                # int32 [n_tokens + 1]
    src: np.ndarray                # int32 [nnz] gathered row of each contribution
    beta: np.ndarray               # fp32  [nnz] blend weight (a value of the canvas dtype)
    device_cache: Dict[str, Dict[str, torch.Tensor]] = field(default_factory=dict)

    @property
    def n_rows(self) -> int:
        return int(self.row_idx.shape[0])

    def to(self, device) -> Dict[str, torch.Tensor]:
        key = str(torch.device(device))
        if key not in self.device_cache:
            self.device_cache[key] = {
                "row_idx": torch.from_numpy(self.row_idx).to(device),
                "tokens": torch.from_numpy(self.tokens).to(device),
                "ptr": torch.from_numpy(self.ptr).to(device),
                "src": torch.from_numpy(self.src).to(device),
                "beta": torch.from_numpy(self.beta).to(device),
            }
        return self.device_cache[key]


def build_route_plan(token_hw: Tuple[int, int], route_boxes_latent: Sequence[Box], halo_tokens: int, *,
                     dtype: torch.dtype = torch.bfloat16, fusion_beta: float = 1.0,
                     packing_offset_latent: int = 0, feather_mode: str = "cosine", feather_power: float = 1.0,
                     token_tier_hi: Optional[np.ndarray] = None) -> RoutePlan:
    """Turns latent route boxes into the gather list and the scatter contributor lists.

    token_tier_hi: optional bool [H, W] map, True where a canvas token is high precision; when given the
    gathered rows are stably re-ordered so that all high-precision rows come first.
    """
    if not 0.0 <= float(fusion_beta) <= 1.0:
        raise ValueError(f"fusion_beta must be in [0,1], got {fusion_beta}")
    H, W = int(token_hw[0]), int(token_hw[1])
    seen = set()
    by_shape: Dict[Tuple[int, int], List[Patch]] = {}
    for box in route_boxes_latent:
        core = latent_box_to_token_box(tuple(box), packing_offset_latent)
        if core in seen:
            continue
        seen.add(core)
        y0, y1, x0, x1 = core
        if not (0 <= y0 < y1 <= H and 0 <= x0 < x1 <= W):
            raise ValueError(f"Route box {core} lies outside token grid {token_hw}")
        outer = expand_box(core, halo_tokens, (H, W))
        hw = (outer[1] - outer[0], outer[3] - outer[2])
        by_shape.setdefault(hw, []).append(Patch(core=core, outer=outer, hw=hw))

    patches: List[Patch] = []
    rows: List[np.ndarray] = []
    contrib_tok: List[np.ndarray] = []
    contrib_src: List[np.ndarray] = []
    contrib_beta: List[np.ndarray] = []
    cursor = 0
    shapes = sorted(by_shape)
    for hw in shapes:
        for pch in by_shape[hw]:
            oy0, oy1, ox0, ox1 = pch.outer
            ys, xs = np.meshgrid(np.arange(oy0, oy1), np.arange(ox0, ox1), indexing="ij")
            tok = (ys * W + xs).reshape(-1).astype(np.int64)
            pch.row0 = cursor
            inner = (pch.core[0] - oy0, pch.core[1] - oy0, pch.core[2] - ox0, pch.core[3] - ox0)
            b = feather_weights(hw, inner, dtype, fusion_beta, feather_mode, feather_power).float().reshape(-1).numpy()
            rows.append(tok)
            contrib_tok.append(tok)
            contrib_src.append(np.arange(cursor, cursor + tok.shape[0], dtype=np.int64))
            contrib_beta.append(b.astype(np.float32))
            cursor += tok.shape[0]
            patches.append(pch)

    if rows:
        row_idx = np.concatenate(rows)
        ctok = np.concatenate(contrib_tok); csrc = np.concatenate(contrib_src); cbeta = np.concatenate(contrib_beta)
    else:
        row_idx = np.zeros(0, np.int64); ctok = np.zeros(0, np.int64); csrc = np.zeros(0, np.int64)
        cbeta = np.zeros(0, np.float32)

    m_hi = int(row_idx.shape[0])
    if token_tier_hi is not None and row_idx.shape[0] > 0:
        tier = np.asarray(token_tier_hi, dtype=bool).reshape(-1)[row_idx]
        perm = np.argsort(~tier, kind="stable")            # high-precision rows first, order kept inside a tier
        inv = np.empty_like(perm)
        inv[perm] = np.arange(perm.shape[0])
        row_idx = row_idx[perm]
        csrc = inv[csrc]
        m_hi = int(tier.sum())

    # CSR over canvas tokens; a stable sort keeps the reference's accumulation order per token
    order = np.argsort(ctok, kind="stable")
    ctok_s, csrc_s, cbeta_s = ctok[order], csrc[order], cbeta[order]
    tokens, counts = np.unique(ctok_s, return_counts=True)
    ptr = np.zeros(tokens.shape[0] + 1, np.int64)
    np.cumsum(counts, out=ptr[1:])
    return RoutePlan(token_hw=(H, W), patches=patches, bucket_shapes=shapes,
                     row_idx=row_idx.astype(np.int32), m_hi=m_hi, tokens=tokens.astype(np.int32),
                     ptr=ptr.astype(np.int32), src=csrc_s.astype(np.int32), beta=cbeta_s.astype(np.float32))


def leaf_tier_to_token_map(leaf_hi: np.ndarray, token_hw: Tuple[int, int]) -> np.ndarray:
    """Nearest-neighbour expansion of an [n,n] leaf map to a [H,W] token map: a token takes the tier of
    the leaf that contains it (the hard-routing form of flux/run_flux.py:117-123)."""
    n0, n1 = leaf_hi.shape
    H, W = token_hw
    ly = (np.arange(H) * n0) // H
    lx = (np.arange(W) * n1) // W
    return (np.asarray(leaf_hi) > 0.5)[ly][:, lx]


def inner_split_median(scores: np.ndarray, sel: np.ndarray, inner_thresh: float) -> np.ndarray:
    """High tier = active leaves whose score >= inner_thresh * median of the active scores, at least one
    leaf stays high (flux/run_flux.py:238-250; torch.median returns the lower of the two middle values)."""
    cand = np.asarray(sel) > 0.5
    v = np.sort(np.asarray(scores, dtype=np.float32)[cand])
    if v.size == 0:
        return np.zeros_like(scores, dtype=np.float32)
    ref = float(v[(v.size - 1) // 2]) if v.size > 1 else float(v.max())
    hi = (scores >= np.float32(float(inner_thresh) * max(ref, 1e-12))) & cand
    if hi.sum() == 0:
        masked = np.where(cand, scores, -1e30)
        hi = (masked >= masked.max()) & cand
    return hi.astype(np.float32)


# ------------------------------------------------------------------------------------------------ device ops
# In eager mode the implementation functions are called directly: the dispatcher round trip of a Python custom op costs
# tens of microseconds per call, as much as these kernels run.  Under torch.compile the registered ops are used.
def _eager() -> bool:
    return not torch.compiler.is_compiling()


def gather_rows(canvas: torch.Tensor, plan: RoutePlan) -> torch.Tensor:
    """[tokens, C] canvas -> [M_act, C] gathered rows (no quantisation)."""
    idx = plan.to(canvas.device)["row_idx"]
    if _eager():
        return ops._gather_rows_impl(canvas, idx)
    return torch.ops.pq_b200.gather_rows(canvas, idx)


def gather_quant_rows(canvas: torch.Tensor, plan: RoutePlan):
    """Gather fused with per-token INT8 quantisation: (int8 [M_act, C], fp32 [M_act])."""
    idx = plan.to(canvas.device)["row_idx"]
    if _eager():
        return ops._gather_quant_rows_impl(canvas, idx)
    return torch.ops.pq_b200.gather_quant_rows(canvas, idx)


def scatter_rows_(y: torch.Tensor, plan: RoutePlan, canvas: torch.Tensor) -> torch.Tensor:
    """Blends routed rows y [M_act, C] over `canvas` [tokens, C] in place and returns it."""
    d = plan.to(canvas.device)
    if _eager():
        ops._scatter_rows_impl(y, d["tokens"], d["ptr"], d["src"], d["beta"], canvas)
        ops._written_in_place(canvas)
    else:
        torch.ops.pq_b200.scatter_rows_(y, d["tokens"], d["ptr"], d["src"], d["beta"], canvas)
    return canvas


def fuse_rows(background: torch.Tensor, y: torch.Tensor, plan: RoutePlan) -> torch.Tensor:
    """Out-of-place form with the reference's calling shape: background [1,H,W,C] -> fused [1,H,W,C]."""
    b, H, W, C = background.shape
    if int(b) != 1:
        raise ValueError("Only batch-one full-image fusion is supported")
    out = background.reshape(H * W, C).clone()
    scatter_rows_(y, plan, out)
    return out.reshape(1, H, W, C)
