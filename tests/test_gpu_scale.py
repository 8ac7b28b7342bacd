"""Parity at the sizes the benchmark configurations state (through the C ABI, on the GPU).

The CPU oracle cannot finish these shapes in seconds, so every case combines
  * the full oracle (codes, scales, int32 accumulators bit-exact; outputs within max-rel-err 1e-2 of the exact
    dequantised math) on a few hundred sampled rows spread over the first, middle and last row tiles and the
    ragged tail, and
  * exact size-independent identities over ALL rows: int64 column and row checksums of the int32 accumulators,
    and bit-equality of the production kernel's output with the accumulator-dumping instantiation's.
Configurations: FLUX 2K-stage double-block set (four layers, M = 16896), FLUX 4K-stage single-block set (two layers,
M = 66048, and its 8-GPU shard of 8256 rows), SDXL group-32 set (six shapes), routed nested-precision FLUX 4K linear
(256 x 256 token canvas, 16 x 16-token leaves active with probability 0.3, halo 2).
"""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import oracle
from pyraquant_b200 import int8_exec, ops, routing

pytestmark = pytest.mark.gpu
TOL = 1e-2


def max_rel_err(y: torch.Tensor, ref64: torch.Tensor) -> float:
    ref = ref64.double()
    denom = torch.maximum(ref.abs(), 1e-3 * ref.abs().max())
    return float(((y.double() - ref).abs() / denom).max())


@pytest.fixture(autouse=True)
def _clean(cuda_dev):
    yield
    ops.check_device_status(cuda_dev)
    torch.cuda.empty_cache()


def spread_rows(M: int, n_spread: int = 320) -> torch.Tensor:
    """First 64 rows, 64 rows around the middle, the last 64 rows (the ragged tail when M is not a tile multiple) and
    n_spread rows evenly spread over the rest."""
    parts = [np.arange(0, min(64, M)), np.arange(max(0, M // 2 - 32), min(M, M // 2 + 32)), np.arange(max(0, M - 64), M),
             np.linspace(0, M - 1, n_spread).round().astype(np.int64)]
    return torch.from_numpy(np.unique(np.concatenate(parts)).astype(np.int64))


def device_activations(dev, M, K, seed, dtype=torch.bfloat16, outliers=True):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(M, K, generator=g, device=dev)
    if outliers:
        x[:, torch.randperm(K, generator=g, device=dev)[: max(1, round(K * 0.005))]] *= 20.0
    return x.to(dtype)


def exact_matvec_i64(mat_i8: torch.Tensor, vec_i64: torch.Tensor) -> torch.Tensor:
    """mat [R, C] int8 @ vec [C] int64 on the device, exactly: every partial sum is an integer below 2^53, so the
    fp64 products and sums are exact in any order."""
    out = torch.empty(mat_i8.shape[0], dtype=torch.int64, device=mat_i8.device)
    v = vec_i64.double()
    assert float(v.abs().sum()) * 127.0 < 2.0 ** 53
    for i in range(0, mat_i8.shape[0], 8192):
        out[i:i + 8192] = (mat_i8[i:i + 8192].double() @ v).round().to(torch.int64)
    return out


def down_projection_close(t: torch.Tensor, t_o: torch.Tensor, xs: torch.Tensor, A: torch.Tensor) -> bool:
    """t = round16(x @ A) against the restatement's: the fp32 dot products differ only by summation order (error far
    below 1e-5 of the sum of the terms' magnitudes), so the rounded results agree or are neighbours."""
    d = (t.float() - t_o.float()).abs()
    scale = xs.float().abs() @ A.float().abs()
    return bool((d <= t_o.float().abs() * 2.0 ** -7 + 1e-5 * scale).all()) and float((d > 0).float().mean()) < 0.05


FLUX_CASES = [  # (config, M, K, N)
    ("2K qkv", 16896, 3072, 9216), ("2K attn-out", 16896, 3072, 3072), ("2K mlp-up", 16896, 3072, 12288),
    ("2K mlp-down", 16896, 12288, 3072),
    ("4K qkv+mlp-in", 66048, 3072, 21504), ("4K proj-out", 66048, 15360, 3072),
    ("4K qkv+mlp-in, 8-GPU shard", 8256, 3072, 21504), ("4K proj-out, 8-GPU shard", 8256, 15360, 3072),
]


@pytest.mark.parametrize("name,M,K,N", FLUX_CASES, ids=[c[0] for c in FLUX_CASES])
def test_flux_layer_at_stated_size(cuda_dev, name, M, K, N):
    d = cuda_dev
    g = torch.Generator().manual_seed(K * 7 + N)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(N, generator=g) * 0.01).to(torch.bfloat16)
    A = (torch.randn(K, 32, generator=g) * 0.02).to(torch.bfloat16)
    B = (torch.randn(32, N, generator=g) * 0.02).to(torch.bfloat16)
    lin = nn.Linear(K, N, bias=True).to(torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(w); lin.bias.copy_(bias)
    layer = int8_exec.Int8Linear(lin, device=d, lowrank=(A, B))
    wq, ws = oracle.quant_weight(w, where="cuda")
    assert torch.equal(layer.weight_int8.cpu(), wq) and torch.equal(layer.w_scale.cpu(), ws)
    b32 = bias.float()

    x = device_activations(d, M, K, seed=M + K)
    y = layer(x)                                                   # production path: down-projection, quantise, GEMM
    xq, sx = int8_exec.quant_rows(x)
    t = layer._down(x)
    y_dbg, acc = ops.int8_gemm_debug(xq, sx, layer.weight_int8, layer.w_scale, layer.bias, t, layer.lr_B, torch.bfloat16)
    assert torch.equal(y, y_dbg)

    # ---- all rows: exact checksums of the int32 accumulators
    col = acc.sum(0, dtype=torch.int64)
    row = acc.sum(1, dtype=torch.int64)
    q_colsum = xq.sum(0, dtype=torch.int64)                        # [K]
    w_colsum = layer.weight_int8.sum(0, dtype=torch.int64)         # [K]
    assert torch.equal(col, exact_matvec_i64(layer.weight_int8, q_colsum))
    assert torch.equal(row, exact_matvec_i64(xq, w_colsum))
    # ---- all rows: quantisation identities
    amax = x.float().abs().amax(1).clamp_min(1e-8)
    assert torch.equal(sx, amax / torch.full_like(amax, 127.0))
    assert int(xq.abs().amax(1).min()) == 127
    del amax, col, row

    # ---- sampled rows: the full oracle
    idx = spread_rows(M)
    xs = x[idx.to(d)].cpu()
    xq_o, sx_o = oracle.quant_rows(xs)
    assert torch.equal(xq[idx.to(d)].cpu(), xq_o) and torch.equal(sx[idx.to(d)].cpu(), sx_o)
    acc_o = oracle.int_mm(xq_o, wq)
    assert torch.equal(acc[idx.to(d)].cpu(), acc_o)
    # down-projection: the restatement's value up to the summation order of the fp32 dot product, i.e. at most one
    # unit in the last place of the 16-bit result, and that for few elements
    t_s = t[idx.to(d)].cpu()
    t_o = (xs.float() @ A.float()).to(torch.bfloat16)
    assert down_projection_close(t_s, t_o, xs, A)
    # fused GEMM on its actual inputs (the codes, scales and t it was given) against the exact dequantised math
    ref64 = oracle.exact_dequant_f64(acc_o, sx_o, ws, b32, t_s, B)
    ys = y[idx.to(d)].cpu()
    assert max_rel_err(ys, ref64) <= TOL
    y_o = oracle.epilogue(acc_o, sx_o, ws, b32, t_s, B, torch.bfloat16)
    assert float((ys.float() - y_o.float()).norm() / y_o.float().norm()) < 2e-3
    # the whole forward against the restated forward (its own down-projection): relative L2
    y_f = oracle.epilogue(acc_o, sx_o, ws, b32, t_o, B, torch.bfloat16)
    assert float((ys.float() - y_f.float()).norm() / y_f.float().norm()) < 2e-3
    assert len(idx) >= 400


G32_CASES = [(65536, 640, 640), (65536, 640, 5120), (65536, 2560, 640), (16384, 1280, 1280), (16384, 1280, 10240),
             (16384, 5120, 1280)]


@pytest.mark.parametrize("M,K,N", G32_CASES)
def test_sdxl_group32_layer_at_stated_size(cuda_dev, M, K, N):
    d = cuda_dev
    g = torch.Generator().manual_seed(K + 3 * N)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.float16)
    bias = (torch.randn(N, generator=g) * 0.01).to(torch.float16)
    lin = nn.Linear(K, N, bias=True).to(torch.float16)
    with torch.no_grad():
        lin.weight.copy_(w); lin.bias.copy_(bias)
    layer = int8_exec.Int8LinearG32(lin, device=d)
    wq, sw = oracle.quant_weight_g32(w.float(), where="cuda")
    assert torch.equal(layer.weight_int8.cpu(), wq) and torch.equal(layer.w_scale.cpu(), sw)
    x = device_activations(d, M, K, seed=M + N, dtype=torch.float16, outliers=False)
    y = layer(x)
    xq, sa = int8_exec.quant_rows_g32(x)
    idx = spread_rows(M, 128)
    xs = x[idx.to(d)].cpu()
    xq_o, sa_o = oracle.quant_rows_g32(xs)
    assert torch.equal(xq[idx.to(d)].cpu(), xq_o) and torch.equal(sa[idx.to(d)].cpu(), sa_o)
    want = oracle.gemm_g32(xq_o, sa_o, wq, sw, bias.float(), torch.float16)
    assert torch.equal(y[idx.to(d)].cpu(), want)
    # all rows: per-group identities of the codes
    amax = x.float().reshape(M, K // 32, 32).abs().amax(-1).clamp_min(1e-8)
    assert torch.equal(sa, amax / torch.full_like(amax, 127.0))
    assert int(xq.reshape(M, K // 32, 32).abs().amax(-1).min()) == 127


def test_routed_flux4k_at_stated_size(cuda_dev):
    """256 x 256 token canvas, 16 x 16-token leaves active with probability 0.3, halo 2, C = 3072 -> 12288 -> 3072 with
    per-leaf high / nested-4-bit weights: gather + quantise and the feathered scatter bit-exact over every row, the
    routed Linears within tolerance on sampled rows of both tiers."""
    d = cuda_dev
    H = W = 256
    C, F = 3072, 12288
    rng = np.random.default_rng(4)
    sel = (rng.random((16, 16)) < 0.3).astype(np.float32)
    hi = routing.inner_split_median(rng.random((16, 16)).astype(np.float32), sel, 1.0)
    boxes = routing.leaf_run_boxes(sel, 32)                        # 32 latent = 16 tokens per leaf
    plan = routing.build_route_plan((H, W), boxes, 2, token_tier_hi=routing.leaf_tier_to_token_map(hi, (H, W)))
    plain = routing.build_route_plan((H, W), boxes, 2)              # bucket order, as the reference lays rows out
    M, mh = plan.n_rows, plan.m_hi
    assert 15000 < M < 40000 and 0 < mh < M
    canvas = device_activations(d, H * W, C, seed=44)
    canvas_cpu = canvas.cpu()

    # ---- gather (+ quantise): every row, both orders
    buckets = oracle.gather_buckets(canvas_cpu.reshape(1, H, W, C), boxes, 2)
    rows_ref = torch.cat([t.reshape(-1, C) for _hw, t, _g in buckets])
    assert torch.equal(routing.gather_rows(canvas, plain).cpu(), rows_ref)
    gq, gs = routing.gather_quant_rows(canvas, plain)
    q_ref, s_ref = oracle.quant_rows(rows_ref)
    assert torch.equal(gq.cpu(), q_ref) and torch.equal(gs.cpu(), s_ref)
    rows_tier = canvas_cpu[torch.from_numpy(plan.row_idx).long()]
    tq, ts = routing.gather_quant_rows(canvas, plan)
    tq_ref, ts_ref = oracle.quant_rows(rows_tier)
    assert torch.equal(tq.cpu(), tq_ref) and torch.equal(ts.cpu(), ts_ref)
    del gq, gs, q_ref, s_ref

    # ---- scatter: every canvas token against the restated fuse_patch_predictions
    go = torch.Generator().manual_seed(45)
    outs = [((hw, geoms), (torch.randn(t.shape, generator=go) * 1.5).to(torch.bfloat16)) for hw, t, geoms in buckets]
    bg = (torch.randn(1, H, W, C, generator=go)).to(torch.bfloat16)
    want = oracle.fuse_buckets(bg, outs, 1.0)
    y_rows = torch.cat([o.reshape(-1, C) for _m, o in outs]).to(d)
    got = routing.fuse_rows(bg.to(d), y_rows, plain)
    assert torch.equal(got.cpu(), want)
    del want, got, outs, bg, y_rows, buckets

    # ---- routed Linears, sampled rows of both tiers
    g = torch.Generator().manual_seed(46)

    def routed(K, N):
        lin = nn.Linear(K, N, bias=True).to(torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(N, K, generator=g) * 0.02); lin.bias.copy_(torch.randn(N, generator=g) * 0.01)
        A = (torch.randn(K, 32, generator=g) * 0.02).to(torch.bfloat16)
        B = (torch.randn(32, N, generator=g) * 0.02).to(torch.bfloat16)
        return lin, A, B, int8_exec.Int8LinearRouted(lin, device=d, lowrank=(A, B))

    def check(layer_in_cpu, y_dev, lin, A, B, t_dev):
        idx = torch.from_numpy(np.unique(np.concatenate([np.linspace(0, mh - 1, 96).round(), np.arange(max(0, mh - 32), mh),
                                                          np.arange(mh, min(M, mh + 32)),
                                                          np.linspace(mh, M - 1, 96).round()]).astype(np.int64)))
        xs = layer_in_cpu[idx]
        w8, s8 = oracle.quant_weight(lin.weight.detach(), where="cuda")
        w4, s4 = oracle.nested4_from_int8(w8, s8)
        xq, sx = oracle.quant_rows(xs)
        t_o = (xs.float() @ A.float()).to(torch.bfloat16)
        t = t_dev[idx.to(d)].cpu()                               # the GEMM's actual low-rank input
        assert down_projection_close(t, t_o, xs, A)
        b32 = lin.bias.detach().float()
        is_hi = idx < mh
        ref = torch.empty(len(idx), lin.out_features, dtype=torch.float64)
        ref[is_hi] = oracle.exact_dequant_f64(oracle.int_mm(xq[is_hi], w8), sx[is_hi], s8, b32, t[is_hi], B)
        ref[~is_hi] = oracle.exact_dequant_f64(oracle.int_mm(xq[~is_hi], w4), sx[~is_hi], s4, b32, t[~is_hi], B)
        assert int(is_hi.sum()) > 64 and int((~is_hi).sum()) > 64
        assert max_rel_err(y_dev[idx.to(d)].cpu(), ref) <= TOL

    lin_u, A_u, B_u, up = routed(C, F)
    h = up.forward_gathered(canvas, plan.to(d)["row_idx"], mh)
    check(rows_tier, h, lin_u, A_u, B_u, up._down(routing.gather_rows(canvas, plan)))
    lin_d, A_d, B_d, down = routed(F, C)
    y = down.forward_rows(h, mh)
    check(h.cpu(), y, lin_d, A_d, B_d, down._down(h))
