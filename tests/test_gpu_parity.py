"""Parity of the CUDA path (through the C ABI) with the CPU oracle on identical seeded inputs.

Bars: int8 codes, fp32 scales, int32 accumulators and all index work bit-exact; 16-bit outputs within
max-rel-err 1e-2 of the exact dequantised math (fp64), where
    rel = |y - ref| / max(|ref|, 1e-3 * max|ref|).
"""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from conftest import from_bf16_bits
from oracle import oracle
from pyraquant_b200 import _lib, int8_exec, ops, routing

pytestmark = pytest.mark.gpu
TOL = 1e-2


def max_rel_err(y: torch.Tensor, ref64: torch.Tensor) -> float:
    ref = ref64.double()
    denom = torch.maximum(ref.abs(), 1e-3 * ref.abs().max())
    return float(((y.double() - ref).abs() / denom).max())


@pytest.fixture(autouse=True)
def _status_clean(cuda_dev):
    yield
    ops.check_device_status(cuda_dev)


def rand_act(M, K, dtype, seed, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    if outliers and K >= 16:
        x[:, torch.randperm(K, generator=g)[: max(1, K // 200)]] *= 20.0
    return x.to(dtype)


# ------------------------------------------------------------------------------------------------ quantisation
@pytest.mark.parametrize("M,K", [(1, 64), (8, 64), (17, 640), (154, 1280), (513, 2048), (4350, 3072),
                                 (300, 5120), (200, 10240), (130, 12288), (96, 15360), (5, 20480), (33, 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quant_rows_bit_exact(cuda_dev, M, K, dtype):
    x = rand_act(M, K, dtype, 100 + M + K)
    if M > 3:
        x[2].zero_()                          # all-zero token -> 1e-8 floor
        x[3] = x[3].abs().max()               # constant row: every code is 127
    q, s = int8_exec.quant_rows(x.to(cuda_dev))
    qo, so = oracle.quant_rows(x)
    assert q.dtype == torch.int8 and s.dtype == torch.float32 and q.shape == (M, K) and s.shape == (M,)
    assert torch.equal(s.cpu(), so)
    assert torch.equal(q.cpu(), qo)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quant_scales_for_every_absmax(cuda_dev, dtype):
    """Every positive finite value of the activation type as a row's absmax: the scale equals the IEEE quotient
    absmax / 127 bit for bit (the kernel computes it with a multiply-and-correct sequence), and so do the group scales."""
    top = 0x7F80 if dtype == torch.bfloat16 else 0x7C00
    bits = torch.arange(1, top, dtype=torch.int32).to(torch.int16)
    vals = bits.view(dtype)
    M = vals.numel()
    x = torch.zeros(M, 32, dtype=dtype)
    x[:, 5] = vals
    x[::2, 17] = -vals[::2]
    _q, s = int8_exec.quant_rows(x.to(cuda_dev))
    want = vals.float().clamp_min(1e-8) / torch.full((M,), 127.0)
    assert torch.equal(s.cpu(), want)
    _q, sg = int8_exec.quant_rows_g32(x.to(cuda_dev))
    assert torch.equal(sg.cpu()[:, 0], want)


def test_quant_rows_cfg0_full(cuda_dev):
    L = oracle.make_layer(0, 4608, 3072, 8, lowrank=False, bias=False)
    q, s = int8_exec.quant_rows(L["x"].to(cuda_dev))
    qo, so = oracle.quant_rows(L["x"])
    assert torch.equal(s.cpu(), so) and torch.equal(q.cpu(), qo)


def test_quant_rows_strided_rows_and_views(cuda_dev):
    x = rand_act(64, 3072 + 1024, torch.bfloat16, 7).to(cuda_dev)
    view = x[:, 1024:]                                    # row stride 4096, offset 2048 bytes
    q, s = int8_exec.quant_rows(view)
    qo, so = oracle.quant_rows(view.cpu())
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    odd = x[:, 3:3 + 64]                                  # misaligned start: falls back to a copy, same result
    q2, s2 = int8_exec.quant_rows(odd)
    qo2, so2 = oracle.quant_rows(odd.cpu())
    assert torch.equal(q2.cpu(), qo2) and torch.equal(s2.cpu(), so2)
    tr = x[:32, :32].t()                                  # last dim not contiguous
    q3, _ = int8_exec.quant_rows(tr)
    assert torch.equal(q3.cpu(), oracle.quant_rows(tr.cpu())[0])


def test_quant_rows_empty(cuda_dev):
    q, s = int8_exec.quant_rows(torch.empty(0, 64, dtype=torch.bfloat16, device=cuda_dev))
    assert q.shape == (0, 64) and s.shape == (0,)


def test_quant_rows_ties_exact(cuda_dev):
    # rows built so that many quotients land exactly on or next to .5: amax = 127 * 2^e makes scale a power of two
    base = torch.arange(-254, 255, dtype=torch.float32) * 0.5            # includes every k + 0.5
    rows = []
    for e in (-3, 0, 2):
        r = base * 2.0 ** e
        r = torch.cat([r, torch.tensor([127.0 * 2.0 ** e])])
        rows.append(torch.nn.functional.pad(r, (0, 512 - r.numel())))
    x = torch.stack(rows).to(torch.bfloat16)
    q, s = int8_exec.quant_rows(x.to(cuda_dev))
    qo, so = oracle.quant_rows(x)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)


@pytest.mark.parametrize("M,K", [(9, 64), (300, 640), (257, 1280), (64, 5120), (31, 2560)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quant_rows_g32_bit_exact(cuda_dev, M, K, dtype):
    x = rand_act(M, K, dtype, 200 + M + K)
    x[0, :32] = 0
    q, s = int8_exec.quant_rows_g32(x.to(cuda_dev))
    qo, so = oracle.quant_rows_g32(x)
    assert s.shape == (M, K // 32)
    assert torch.equal(s.cpu(), so) and torch.equal(q.cpu(), qo)


def test_gather_quant_rows_bit_exact(cuda_dev):
    canvas = rand_act(1024, 3072, torch.bfloat16, 11)
    g = torch.Generator().manual_seed(5)
    idx = torch.randint(0, 1024, (777,), generator=g, dtype=torch.int32)
    idx[5] = -1; idx[100] = -1; idx[776] = 1023; idx[0] = 0
    q, s = int8_exec.gather_quant_rows(canvas.to(cuda_dev), idx.to(cuda_dev))
    src = canvas[idx.clamp_min(0).long()].clone()
    src[idx < 0] = 0
    qo, so = oracle.quant_rows(src)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    plain = torch.ops.pq_b200.gather_rows(canvas.to(cuda_dev), idx.to(cuda_dev))
    assert torch.equal(plain.cpu(), src)


# ------------------------------------------------------------------------------------------------ GEMM
def run_gemm_case(dev, M, N, K, *, lowrank, bias, dtype=torch.bfloat16, seed=0, extreme=False):
    g = torch.Generator().manual_seed(seed)
    if extreme:
        xq = torch.full((M, K), 127, dtype=torch.int8); xq[::2] = -127
        wq = torch.full((N, K), 127, dtype=torch.int8); wq[1::3] = -127
    else:
        xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
        wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    sr = torch.rand(M, generator=g) * 0.05 + 0.001
    sc = torch.rand(N, generator=g) * 0.002 + 0.0001
    b = torch.randn(N, generator=g) * 0.01 if bias else None
    t = lb = None
    if lowrank:
        t = (torch.randn(M, 32, generator=g) * 1.0).to(dtype)
        lb = (torch.randn(32, N, generator=g) * 0.02).to(dtype)
    to = lambda v: None if v is None else v.to(dev)
    out, acc = ops.int8_gemm_debug(to(xq), to(sr), to(wq), to(sc), to(b), to(t), to(lb), dtype)
    torch.cuda.synchronize()
    acc_ref = oracle.int_mm(xq, wq)
    assert torch.equal(acc.cpu(), acc_ref), f"int32 accumulators differ at {(acc.cpu() != acc_ref).sum().item()} places"
    ref64 = oracle.exact_dequant_f64(acc_ref, sr, sc, b, t, lb)
    err = max_rel_err(out.cpu(), ref64)
    assert err <= TOL, err
    # against the fp32 restatement of the kernel's epilogue: identical bits without the low-rank term (same
    # operations in the same order), summation-order noise of the rank-32 dot product with it
    y32 = oracle.epilogue(acc_ref, sr, sc, b, t, lb, dtype)
    if not lowrank:
        assert torch.equal(out.cpu(), y32)
    else:
        assert max_rel_err(out.cpu(), y32.double()) <= 8e-3
    return out


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (1, 256, 64), (8, 128, 64), (17, 384, 192), (154, 640, 640),
                                   (300, 512, 1280), (1000, 3072, 512), (257, 1280, 2560), (129, 264, 80),
                                   (4350, 1288, 144)])
def test_gemm_small_shapes(cuda_dev, M, N, K):
    run_gemm_case(cuda_dev, M, N, K, lowrank=True, bias=True, seed=M + N + K)        # low-rank term on tcgen05
    run_gemm_case(cuda_dev, M, N, K, lowrank=False, bias=False, seed=M + N + K + 1)
    ops.LOWRANK_ON_TENSOR_CORES = False                                             # low-rank term by mma.sync
    try:
        run_gemm_case(cuda_dev, M, N, K, lowrank=True, bias=True, seed=M + N + K)
    finally:
        ops.LOWRANK_ON_TENSOR_CORES = True


def test_gemm_extreme_accumulators_exact(cuda_dev):
    # |acc| = K * 127^2 = 2.0e8 > 2^24: only true int32 accumulation gets this right
    run_gemm_case(cuda_dev, 256, 512, 12288, lowrank=False, bias=True, extreme=True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("lowrank,bias", [(True, True), (True, False), (False, True)])
def test_gemm_dtypes_and_options(cuda_dev, dtype, lowrank, bias):
    run_gemm_case(cuda_dev, 777, 768, 1024, lowrank=lowrank, bias=bias, dtype=dtype, seed=3)


@pytest.mark.parametrize("bn,stages", [(128, 2), (128, 4), (128, 6), (256, 2), (256, 3), (256, 4)])
def test_gemm_tile_variants(cuda_dev, bn, stages):
    _lib.set_option("gemm_block_n", bn); _lib.set_option("gemm_stages", stages)
    try:
        run_gemm_case(cuda_dev, 1500, 1024, 768, lowrank=True, bias=True, seed=bn + stages)
    finally:
        _lib.set_option("gemm_block_n", 0); _lib.set_option("gemm_stages", 0)


def test_gemm_persistent_many_tiles_per_cta(cuda_dev):
    # few CTAs, many tiles each: exercises the accumulator double buffer and barrier phases
    _lib.set_option("gemm_max_ctas", 3)
    try:
        run_gemm_case(cuda_dev, 2000, 2048, 384, lowrank=True, bias=True, seed=9)
    finally:
        _lib.set_option("gemm_max_ctas", 0)


@pytest.mark.parametrize("pm,pn", [(1, 1), (2, 3), (5, 2), (16, 8)])
def test_gemm_schedule_grids(cuda_dev, pm, pn):
    # ragged CTA grids over the tile matrix: idle steps, column tile changes, both accumulator buffers
    _lib.set_option("gemm_pn", pn); _lib.set_option("gemm_pm", pm)
    try:
        run_gemm_case(cuda_dev, 1700, 2304, 256, lowrank=True, bias=True, seed=pm * 10 + pn)
    finally:
        _lib.set_option("gemm_pn", 0); _lib.set_option("gemm_pm", 0)


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (128, 256, 256), (300, 512, 192), (1000, 768, 640), (2049, 1288, 384),
                                   (4608, 3072, 3072)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ew", [8, 16])
def test_gemm_cta_pair_kernel(cuda_dev, M, N, K, dtype, ew):
    """The cta_group::2 kernel forced on for every shape it accepts: odd numbers of 128-row tiles (one CTA of the
    last pair has no rows), ragged N, several tiles per pair, with and without the low-rank term; both epilogue
    widths (eight warps: long K; sixteen warps: short K) at every shape."""
    _lib.set_option("gemm_pair", 2); _lib.set_option("gemm_epi_warps", ew)
    try:
        run_gemm_case(cuda_dev, M, N, K, lowrank=True, bias=True, dtype=dtype, seed=M + N)
        run_gemm_case(cuda_dev, M, N, K, lowrank=False, bias=True, dtype=dtype, seed=M + N + 1)
        if ew == 16:                                 # the same tiles stored from registers instead of shared memory + TMA
            _lib.set_option("gemm_tma_store", 0)
            run_gemm_case(cuda_dev, M, N, K, lowrank=False, bias=True, dtype=dtype, seed=M + N + 1)
            _lib.set_option("gemm_tma_store", 1)
        _lib.set_option("gemm_max_ctas", 4)          # two pairs only: long per-pair tile sequences
        run_gemm_case(cuda_dev, M, N, K, lowrank=True, bias=False, dtype=dtype, seed=M + N + 2)
        run_gemm_case(cuda_dev, M, N, K, lowrank=False, bias=False, dtype=dtype, seed=M + N + 3)
    finally:
        _lib.set_option("gemm_pair", 1); _lib.set_option("gemm_max_ctas", 0); _lib.set_option("gemm_epi_warps", 0)
        _lib.set_option("gemm_tma_store", 1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_production_kernels_bit_equal_without_lowrank(cuda_dev, dtype):
    """The non-debug instantiations (what users run) against the fp32 restatement, no low-rank term: identical bits
    from every kernel variant."""
    g = torch.Generator().manual_seed(77)
    M, N, K = 900, 768, 384
    xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    sr = torch.rand(M, generator=g) * 0.05 + 0.001
    sc = torch.rand(N, generator=g) * 0.002 + 0.0001
    b = torch.randn(N, generator=g) * 0.01
    y32 = oracle.epilogue(oracle.int_mm(xq, wq), sr, sc, b, None, None, dtype)
    d = cuda_dev
    for pair, bn, ew in ((0, 256, 0), (0, 128, 0), (2, 0, 8), (2, 0, 16)):
        _lib.set_option("gemm_pair", pair); _lib.set_option("gemm_block_n", bn); _lib.set_option("gemm_epi_warps", ew)
        try:
            y = int8_exec.int8_gemm_fused(xq.to(d), sr.to(d), wq.to(d), sc.to(d), b.to(d), dtype)
        finally:
            _lib.set_option("gemm_pair", 1); _lib.set_option("gemm_block_n", 0); _lib.set_option("gemm_epi_warps", 0)
        assert torch.equal(y.cpu(), y32), (pair, bn, ew)


@pytest.mark.parametrize("pair", [0, 2])
def test_gemm_accumulators_beyond_24_bits_round_like_the_restatement(cuda_dev, pair):
    """Same-sign codes and K = 8192 give accumulators of 2^24 .. 2^27 with arbitrary low bits: the int32 -> fp32
    conversion of the epilogue has to round them to nearest-even exactly like the fp32 restatement.  Scales of 1 and
    no bias, fp16 and bf16 outputs of power-of-two-scaled sums expose the conversion's rounding at output ties."""
    g = torch.Generator().manual_seed(5)
    M, N, K = 512, 512, 8192
    xq = torch.randint(0, 128, (M, K), generator=g, dtype=torch.int8)
    wq = torch.randint(0, 128, (N, K), generator=g, dtype=torch.int8)
    wq[::2] = -wq[::2]
    acc = oracle.int_mm(xq, wq)
    assert int(acc.abs().max()) > 2 ** 24
    d = cuda_dev
    _lib.set_option("gemm_pair", pair)
    try:
        for dtype, sr_v in ((torch.bfloat16, 1.0), (torch.float16, 2.0 ** -12), (torch.bfloat16, 2.0 ** -7)):
            sr = torch.full((M,), sr_v); sc = torch.ones(N)
            want = oracle.epilogue(acc, sr, sc, None, None, None, dtype)
            got = int8_exec.int8_gemm_fused(xq.to(d), sr.to(d), wq.to(d), sc.to(d), None, dtype)
            assert torch.equal(got.cpu(), want), (pair, dtype)
    finally:
        _lib.set_option("gemm_pair", 1)


def test_gemm_cfg0_layer(cuda_dev):
    """BASELINE config 0: M=4608, K=N=3072, rank-32 branch and bias, through Int8Linear.forward."""
    L = oracle.make_layer(0, 4608, 3072, 3072)
    lin = nn.Linear(3072, 3072, bias=True).to(torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(L["w"]); lin.bias.copy_(L["bias"].to(torch.bfloat16))
    q = int8_exec.Int8Linear(lin, device=cuda_dev, lowrank=(L["lr_A"], L["lr_B"]))
    wq, ws = oracle.quant_weight(L["w"], where="cuda")
    assert torch.equal(q.weight_int8.cpu(), wq) and torch.equal(q.w_scale.cpu(), ws)
    x = L["x"].to(cuda_dev)
    y = q(x)
    assert y.dtype == torch.bfloat16 and y.shape == (4608, 3072)
    # integer stages bit-exact
    xq, sx = int8_exec.quant_rows(x)
    xqo, sxo = oracle.quant_rows(L["x"])
    assert torch.equal(xq.cpu(), xqo) and torch.equal(sx.cpu(), sxo)
    t_gpu = q._down(x)
    _, acc = ops.int8_gemm_debug(xq, sx, q.weight_int8, q.w_scale, q.bias, t_gpu, q.lr_B, torch.bfloat16)
    acc_ref = oracle.int_mm(xqo, wq)
    assert torch.equal(acc.cpu(), acc_ref)
    # output against the exact dequantised math and against the restated forward
    bias32 = lin.bias.detach().float()
    # the down-projection t = x @ lr_A (reference :390) accumulates in fp32 in another order than the CPU; its rounding
    # to bf16 may differ by one ulp, so the GEMM is judged on the t it was given and t on its own
    t_ref = (L["x"].float() @ L["lr_A"].float()).to(torch.bfloat16)
    assert bool(((t_gpu.cpu().float() - t_ref.float()).abs() <= t_ref.float().abs() * 2.0 ** -7 + 1e-3).all())
    ref64 = oracle.exact_dequant_f64(acc_ref, sxo, ws, bias32, t_gpu.cpu(), L["lr_B"])
    assert max_rel_err(y.cpu(), ref64) <= TOL
    y_or = oracle.int8_linear_forward(L["x"], wq, ws, bias32, L["lr_A"], L["lr_B"])
    rel_l2 = ((y.cpu().float() - y_or.float()).norm() / y_or.float().norm()).item()
    assert rel_l2 < 1e-3, rel_l2
    # 3-D input gives the same rows (reference self-test vi)
    y3 = q(x[:2048].reshape(8, 256, 3072))
    assert torch.equal(y3.reshape(2048, -1), q(x[:2048]))


def test_gemm_grouped_two_tiers(cuda_dev):
    g = torch.Generator().manual_seed(21)
    M, N, K, m_hi = 1000, 768, 512, 389
    xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w8 = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    s8 = torch.rand(N, generator=g) * 0.002 + 1e-4
    w4, s4 = oracle.nested4_from_int8(w8, s8)
    sr = torch.rand(M, generator=g) * 0.05 + 0.001
    b = torch.randn(N, generator=g) * 0.01
    t = torch.randn(M, 32, generator=g).to(torch.bfloat16)
    lb = (torch.randn(32, N, generator=g) * 0.02).to(torch.bfloat16)
    d = cuda_dev
    for mh in (m_hi, 0, M, 128):
        y = int8_exec.int8_gemm_grouped(xq.to(d), sr.to(d), w8.to(d), s8.to(d), w4.to(d), s4.to(d), b.to(d),
                                        t.to(d), lb.to(d), mh, torch.bfloat16).cpu()
        ref = torch.empty(M, N, dtype=torch.float64)
        ref[:mh] = oracle.exact_dequant_f64(oracle.int_mm(xq[:mh], w8), sr[:mh], s8, b, t[:mh], lb) if mh else ref[:mh]
        if mh < M:
            ref[mh:] = oracle.exact_dequant_f64(oracle.int_mm(xq[mh:], w4), sr[mh:], s4, b, t[mh:], lb)
        assert max_rel_err(y, ref) <= TOL, mh
        # the same call on the CTA-pair kernel (K-major low-rank factor given, kernel forced on): tiles of 256 rows
        # per tier, split rows not aligned to anything
        _lib.set_option("gemm_pair", 2)
        try:
            y2 = int8_exec.int8_gemm_grouped(xq.to(d), sr.to(d), w8.to(d), s8.to(d), w4.to(d), s4.to(d), b.to(d),
                                             t.to(d), lb.to(d), mh, torch.bfloat16, lb.t().contiguous().to(d)).cpu()
        finally:
            _lib.set_option("gemm_pair", 1)
        assert max_rel_err(y2, ref) <= TOL, mh


def test_shared_input_group(cuda_dev, monkeypatch):
    """Sibling layers on one input: one quantisation and one down-projection for the group, outputs identical to
    the same layers run alone on the same codes and the same slice of the shared down-projection."""
    g = torch.Generator().manual_seed(33)
    K, Ns, M = 512, (256, 512, 1024, 264), 700
    layers = []
    for i, N in enumerate(Ns):
        lin = nn.Linear(K, N, bias=(i != 1)).to(torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(N, K, generator=g) * 0.02)
        lr = None if i == 2 else ((torch.randn(K, 32, generator=g) * 0.02).to(torch.bfloat16),
                                  (torch.randn(32, N, generator=g) * 0.02).to(torch.bfloat16))
        layers.append(int8_exec.Int8Linear(lin, device=cuda_dev, lowrank=lr))
    x = (torch.randn(2, M // 2, K, generator=g)).to(torch.bfloat16).to(cuda_dev)
    alone = [m(x) for m in layers]
    grp = int8_exec.share_input_quantisation(layers)
    calls = {"n": 0}
    real = ops._quant_rows_impl

    def counting(x2):
        calls["n"] += 1
        return real(x2)
    monkeypatch.setattr(ops, "_quant_rows_impl", counting)
    together = [m(x) for m in layers]
    assert calls["n"] == 1
    x2 = x.reshape(-1, K)
    xq, sx = real(x2)
    _xq, _sx, T = grp.prepare(x2)                      # the group's own down-projection of width 32 x members
    assert T.shape == (M, 32 * sum(m.lr_A is not None for m in layers))
    t_wide = (x2.float() @ torch.cat([m.lr_A for m in layers if m.lr_A is not None], dim=1).float()).to(torch.bfloat16)
    assert bool(((T.float() - t_wide.float()).abs() <= t_wide.float().abs() * 2.0 ** -7 + 1e-3).all())
    off = 0
    for m, ya, yt in zip(layers, alone, together):
        assert yt.shape == ya.shape == (2, M // 2, m.out_features)
        if m.lr_A is None:
            assert torch.equal(yt, ya)
            continue
        exp = int8_exec.int8_gemm_lr(xq, sx, m.weight_int8, m.w_scale, m.bias, T[:, off:off + 32], m.lr_B, torch.bfloat16)
        off += 32
        assert torch.equal(yt.reshape(M, -1), exp)
        assert max_rel_err(yt.float().cpu(), ya.double().cpu()) <= TOL      # down-projection may round differently
    # a modified input (same storage) is quantised again; so is a new tensor
    x.mul_(0.5)
    _ = layers[0](x)
    assert calls["n"] == 2
    _ = layers[1](x)
    assert calls["n"] == 2
    _ = layers[1](x.clone())
    assert calls["n"] == 3
    grp.clear()


def _toy_layer(cuda_dev, g, K, N, lowrank=True, bias=True, dtype=torch.bfloat16):
    lin = nn.Linear(K, N, bias=bias).to(dtype)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(N, K, generator=g) * 0.05)
        if bias:
            lin.bias.copy_(torch.randn(N, generator=g) * 0.1)
    lr = ((torch.randn(K, 32, generator=g) * 0.05).to(dtype), (torch.randn(32, N, generator=g) * 0.05).to(dtype)) if lowrank else None
    return int8_exec.Int8Linear(lin, device=cuda_dev, lowrank=lr)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N,lowrank", [(768, True), (512, False), (264, True)])
def test_epilogue_variants(cuda_dev, dtype, N, lowrank):
    """GELU(tanh) and accumulate-into-output in the GEMM epilogue against the separate torch kernels on the layer's own
    output: the sum bit for bit; the activation within two units in the last place of the output type (hardware tanh).
    N = 264 is a shape the fused variants do not take: same results through the unfused sequence."""
    g = torch.Generator().manual_seed(N + (1 if lowrank else 0))
    K, M = 512, 700
    layer = _toy_layer(cuda_dev, g, K, N, lowrank=lowrank, dtype=dtype)
    x = (torch.randn(M, K, generator=g) * 1.5).to(dtype).to(cuda_dev)
    y = layer(x)
    ref_act = F.gelu(y, approximate="tanh")
    got_act = layer.forward_ex(x, ops.EPI_GELU_TANH)
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    err = (got_act.float() - ref_act.float()).abs()
    assert bool((err <= 2 * ulp * ref_act.float().abs() + 2e-3).all()), err.max().item()
    base = (torch.randn(M, N, generator=g)).to(dtype).to(cuda_dev)
    ref_sum = base + y
    out = base.clone()
    r = layer.forward_ex(x, ops.EPI_ACCUMULATE, out=out)
    assert r is out and torch.equal(out, ref_sum)
    both = base.clone()
    layer.forward_ex(x, ops.EPI_ACCUMULATE | ops.EPI_GELU_TANH, out=both)
    err = (both.float() - (base + ref_act).float()).abs()
    assert bool((err <= 4 * ulp * (base + ref_act).float().abs() + 4e-3).all()), err.max().item()


@pytest.mark.parametrize("M,K,N,lowrank,copies", [(700, 512, 768, True, 3), (1000, 256, 512, False, 7), (513, 3072, 1024, True, 1),
                                                  (300, 512, 264, True, 2)])
def test_gemm_stores_to_every_destination(cuda_dev, M, K, N, lowrank, copies):
    """`forward_into` (pq_int8_gemm_bcast): the epilogue writes each output tile to several buffers -- on several GPUs
    these are the peers' output buffers, here slices of larger local ones.  Every destination must equal the plain
    forward bit for bit and rows outside the slice must stay untouched.  N = 264 is a shape the kernel path does not
    take: same results through the copy path."""
    g = torch.Generator().manual_seed(M + copies)
    layer = _toy_layer(cuda_dev, g, K, N, lowrank=lowrank)
    x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16).to(cuda_dev)
    ref = layer(x)
    pad = 40
    bufs = [torch.full((M + 2 * pad, N), 7.0, dtype=torch.bfloat16, device=cuda_dev) for _ in range(copies + 1)]
    views = [b[pad: pad + M] for b in bufs]
    r = layer.forward_into(x, views[0], views[1:])
    torch.cuda.synchronize()
    ops.check_device_status(cuda_dev)
    assert r.data_ptr() == views[0].data_ptr()
    for b, v in zip(bufs, views):
        assert torch.equal(v, ref)
        assert bool((b[:pad] == 7.0).all()) and bool((b[pad + M:] == 7.0).all())


def test_peer_store_gather_on_one_rank(cuda_dev):
    """`parallel.PeerStoreGather` without a process group: one rank owns all rows, the result is the layer's output."""
    from pyraquant_b200 import parallel
    g = torch.Generator().manual_seed(11)
    M, K, N = 900, 512, 768
    layer = _toy_layer(cuda_dev, g, K, N, lowrank=True)
    x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16).to(cuda_dev)
    for chunks in (1, 3):
        og = parallel.PeerStoreGather(M, N, torch.bfloat16, cuda_dev, chunks=chunks)
        y = og.run(layer, x)
        assert y.shape == (M, N) and torch.equal(y, layer(x))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,T,K", [(1, 300, 3072), (2, 129, 640), (1, 70, 15360), (3, 50, 200), (1, 1, 1024)])
def test_adaln_quant_rows(cuda_dev, dtype, B, T, K):
    """LayerNorm + adaLN modulation + per-token quantisation in one kernel (flux/transformer_flux.py:236-239).  The
    quantisation of the modulated activations is exact; the modulated activations themselves equal the reference
    sequence (CPU restatement, and torch's own kernels on the GPU) except where the fp32 row statistics, summed in a
    different order, move a normalised value across a rounding boundary: a few elements in ten thousand, one unit in
    the last place of the products involved."""
    g = torch.Generator().manual_seed(B * 1000 + T + K)
    h = torch.randn(B, T, K, generator=g) * 2 + 0.3
    h[..., 5] *= 30.0
    h = h.to(dtype)
    scale = (torch.randn(B, K, generator=g) * 0.3).to(dtype)
    shift = (torch.randn(B, K, generator=g) * 0.2).to(dtype)
    hd, sc, sh = h.to(cuda_dev), scale.to(cuda_dev), shift.to(cuda_dev)
    q, s, z = ops.adaln_quant_rows(hd.reshape(-1, K), sc, sh, 1e-6, T)
    ops.check_device_status(cuda_dev)
    qo, so = oracle.quant_rows(z.cpu())
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    q2, s2, none = ops.adaln_quant_rows(hd.reshape(-1, K), sc, sh, 1e-6, T, want_modulated=False)
    assert none is None and torch.equal(q2, q) and torch.equal(s2, s)
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    refs = [oracle.adaln_modulate(h, scale, shift, 1e-6).reshape(-1, K),
            (F.layer_norm(hd, (K,), eps=1e-6) * (1 + sc[:, None]) + sh[:, None]).reshape(-1, K).cpu()]
    for zo in refs:
        diff = (z.cpu().float() - zo.float()).abs()
        bound = 4 * ulp * (zo.float().abs() + shift.float().abs().repeat_interleave(T, 0)) + 1e-6
        assert bool((diff <= bound).all()), (diff - bound).max().item()
        assert (z.cpu() != zo).float().mean().item() <= 2e-3


def test_forward_adaln(cuda_dev):
    """`Int8Linear.forward_adaln` against the separate sequence: torch's LayerNorm and modulation, then the layer."""
    g = torch.Generator().manual_seed(21)
    B, T, K, N = 2, 333, 1024, 768
    layer = _toy_layer(cuda_dev, g, K, N, lowrank=True)
    plain = _toy_layer(cuda_dev, g, K, N, lowrank=False)
    h = (torch.randn(B, T, K, generator=g) * 1.5).to(torch.bfloat16).to(cuda_dev)
    scale = (torch.randn(B, K, generator=g) * 0.3).to(torch.bfloat16).to(cuda_dev)
    shift = (torch.randn(B, K, generator=g) * 0.2).to(torch.bfloat16).to(cuda_dev)
    z_ref = F.layer_norm(h, (K,), eps=1e-6) * (1 + scale[:, None]) + shift[:, None]
    for m in (layer, plain):
        y, z = m.forward_adaln(h, scale, shift, return_modulated=True)
        assert y.shape == (B, T, N) and z.shape == h.shape
        assert (z != z_ref).float().mean().item() <= 2e-3
        assert torch.equal(y, m(z))                                  # the layer on the kernel's own modulated rows
        y_ref = m(z_ref)
        rel = ((y.float() - y_ref.float()).norm() / y_ref.float().norm()).item()
        assert rel < 2e-3, rel
        assert torch.equal(m.forward_adaln(h, scale, shift), y)
    # 2-D input with one modulation vector
    y2 = layer.forward_adaln(h[0], scale[0], shift[0])
    assert torch.equal(y2, layer.forward_adaln(h[:1], scale[:1], shift[:1])[0])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("K0,K1,lowrank", [(128, 160, True), (3072, 1024, True), (64, 16, False), (96, 160, True), (15360, 1024, False)])
def test_forward_on_two_sources(cuda_dev, dtype, K0, K1, lowrank):
    """`forward_cat(x0, x1)` == the layer on `torch.cat([x0, x1], -1)` (flux/transformer_flux.py:143-145), bit for bit:
    quantisation and down-projection read the two tensors in place.  K0 = 96 (seam off the 64-element grid) and
    K0 + K1 = 16384 (beyond the register-resident rows) take the concatenating route; row-strided views are consumed as
    they are.  Also through the gate-and-residual epilogue."""
    g = torch.Generator().manual_seed(K0 + K1)
    N, B, T = 256, 2, 150
    layer = _toy_layer(cuda_dev, g, K0 + K1, N, lowrank=lowrank, dtype=dtype)
    wide = (torch.randn(B, T, K0 + 40, generator=g) * 1.5).to(dtype).to(cuda_dev)
    x0 = wide[..., :K0]                                       # a view with a row stride of K0 + 40
    x1 = (torch.randn(B, T, K1, generator=g) * 0.7).to(dtype).to(cuda_dev)
    x1[..., 3] *= 25.0
    want = layer(torch.cat([x0, x1], dim=-1))
    got = layer.forward_cat(x0, x1)
    assert got.shape == want.shape and torch.equal(got, want)
    gate = (torch.randn(B, N, generator=g) * 0.5).to(dtype).to(cuda_dev)
    residual = torch.randn(B, T, N, generator=g).to(dtype).to(cuda_dev)
    ref = residual + gate.unsqueeze(1) * want
    res = residual.clone()
    layer.forward_gated_residual(x0, gate, res, x_more=x1)
    assert torch.equal(res, ref)
    ops.check_device_status(cuda_dev)


def test_shared_group_primed_by_adaln(cuda_dev, monkeypatch):
    """`SharedInputGroup.prime_adaln`: one pass produces the modulated activations and the members' shared codes; the
    members called on the result skip their own quantisation and give what they give ungrouped on the same tensor."""
    g = torch.Generator().manual_seed(41)
    B, T, K = 2, 200, 512
    layers = [_toy_layer(cuda_dev, g, K, n, lowrank=lr) for n, lr in ((768, True), (512, True), (256, False))]
    h = (torch.randn(B, T, K, generator=g) * 1.5).to(torch.bfloat16).to(cuda_dev)
    scale = (torch.randn(B, K, generator=g) * 0.3).to(torch.bfloat16).to(cuda_dev)
    shift = (torch.randn(B, K, generator=g) * 0.2).to(torch.bfloat16).to(cuda_dev)
    z_alone = ops.adaln_quant_rows(h.reshape(-1, K), scale, shift, 1e-6, T)[2].reshape(h.shape)
    want = [m(z_alone) for m in layers]
    grp = int8_exec.share_input_quantisation(layers)
    z = grp.prime_adaln(h, scale, shift)
    assert torch.equal(z, z_alone)
    calls = []
    real = ops._quant_rows_impl
    monkeypatch.setattr(ops, "_quant_rows_impl", lambda x2: (calls.append(1), real(x2))[1])
    got = [m(z) for m in layers]
    assert not calls, "members quantised again although the group was primed"
    for a, b, m in zip(got, want, layers):
        if m.lr_A is None:
            assert torch.equal(a, b)
        else:                                            # the shared down-projection is 64 columns wide: other fp32 summation order
            assert ((a.float() - b.float()).norm() / b.float().norm()).item() < 2e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("lowrank", [True, False])
def test_gated_residual_epilogue(cuda_dev, dtype, lowrank):
    """`residual + gate.unsqueeze(1) * Linear(x)` (flux/transformer_flux.py:145-149) in the GEMM epilogue: bit-identical to
    the layer followed by torch's multiply and add, two samples with their own gate vectors, fp16 sums clipped as the
    block clips them."""
    g = torch.Generator().manual_seed(31)
    B, T, K, N = 2, 333, 512, 768
    layer = _toy_layer(cuda_dev, g, K, N, lowrank=lowrank, dtype=dtype)
    x = (torch.randn(B, T, K, generator=g) * 1.5).to(dtype).to(cuda_dev)
    gate = (torch.randn(B, N, generator=g) * 0.7).to(dtype).to(cuda_dev)
    residual = (torch.randn(B, T, N, generator=g) * 3).to(dtype).to(cuda_dev)
    if dtype == torch.float16:
        residual[0, 0, :8] = 65000.0; residual[1, 5, :8] = -65000.0        # sums that leave the fp16 range
        gate[:, :8] = gate[:, :8].abs() + 40.0
    y = layer(x)
    want = residual + gate.unsqueeze(1) * y
    if dtype == torch.float16:
        want = want.clip(-65504, 65504)
    res = residual.clone()
    out = layer.forward_gated_residual(x, gate, res)
    assert out is res and torch.equal(res, want)
    # 2-D input, one gate vector
    res2 = residual[1].clone()
    layer.forward_gated_residual(x[1], gate[1], res2)
    assert torch.equal(res2, want[1])
    ops.check_device_status(cuda_dev)


def test_split_input_linear(cuda_dev):
    """y = L0(x[..., :in0]) + L1(x[..., in0:]) with the sum in the second GEMM's epilogue: identical to the two layers
    and a torch add (pyraquant/external_quant.py:191-192), 3-D input, strided halves."""
    g = torch.Generator().manual_seed(5)
    in0, in1, N = 256, 768, 512
    l0 = _toy_layer(cuda_dev, g, in0, N, lowrank=True, bias=False)
    l1 = _toy_layer(cuda_dev, g, in1, N, lowrank=True, bias=True)
    x = torch.randn(3, 333, in0 + in1, generator=g).to(torch.bfloat16).to(cuda_dev)
    ref = l0(x[..., :in0]) + l1(x[..., in0:])
    m = int8_exec.SplitInInt8Linear(l0, l1)
    y = m(x)
    assert y.shape == ref.shape and torch.equal(y, ref)


def test_forward_is_cuda_graph_capturable(cuda_dev):
    """After one warm-up call (library load, kernel attributes, tensor-map cache) a chain of Int8Linear forwards is
    captured into a CUDA graph and replayed on new input values: same bits as the eager calls."""
    g = torch.Generator().manual_seed(9)
    l0 = _toy_layer(cuda_dev, g, 512, 1024, lowrank=True)
    l1 = _toy_layer(cuda_dev, g, 1024, 512, lowrank=False)
    x = torch.randn(300, 512, generator=g).to(torch.bfloat16).to(cuda_dev)

    def chain():
        return l1(l0(x))
    chain(); chain()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = chain()
    for seed in (1, 2):
        x.copy_(torch.randn(300, 512, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y_static, chain())
    ops.check_device_status(cuda_dev)


def test_packed_low_tier(cuda_dev):
    """Four-bit storage of the low tier: pack -> device expansion returns the codes bit for bit (every nibble value
    at every position of a byte), and the routed Linear built with packed storage gives the same output as the one
    that keeps int8 codes."""
    g = torch.Generator().manual_seed(12)
    codes = torch.randint(-8, 8, (37, 96), generator=g, dtype=torch.int8)
    codes[0, :16] = torch.arange(-8, 8, dtype=torch.int8)
    codes[1, :32] = torch.arange(-8, 8, dtype=torch.int8).repeat_interleave(2)
    packed = ops.pack_int4(codes)
    assert packed.shape == (37, 48) and packed.dtype == torch.uint8
    assert torch.equal(ops.unpack_int4(packed.to(cuda_dev)).cpu(), codes)
    K, N, M = 512, 768, 600
    lin = nn.Linear(K, N, bias=True).to(torch.bfloat16)
    A = (torch.randn(K, 32, generator=g) * 0.02).to(torch.bfloat16)
    B = (torch.randn(32, N, generator=g) * 0.02).to(torch.bfloat16)
    plain = int8_exec.Int8LinearRouted(lin, device=cuda_dev, lowrank=(A, B))
    small = int8_exec.Int8LinearRouted(lin, device=cuda_dev, lowrank=(A, B), pack_lo=True)
    assert small.weight_lo_packed.numel() * 2 == plain.weight_lo.numel() and not hasattr(small, "weight_lo")
    assert torch.equal(ops.unpack_int4(small.weight_lo_packed), plain.weight_lo)
    x = rand_act(M, K, torch.bfloat16, 13).to(cuda_dev)
    for m_hi in (0, 250, M):
        assert torch.equal(small.forward_rows(x, m_hi), plain.forward_rows(x, m_hi))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,R", [(1, 64, 32), (63, 128, 32), (64, 200, 32), (129, 3072, 32), (1000, 1288, 32),
                                   (4608, 3072, 32), (65, 200, 64), (1000, 1288, 96), (129, 3072, 128),
                                   (9500, 3072, 128), (9500, 512, 64)])
def test_lowrank_down_projection(cuda_dev, M, K, R, dtype):
    """t = x @ A on the streaming tensor-core kernel against the fp64 product: within one unit in the last place of
    the output type (fp32 accumulation order differs from any reference), identical to torch's own matmul almost
    everywhere; row tails, K tails (K % 64 != 0), strided rows, one to four rank-32 factors side by side."""
    g = torch.Generator().manual_seed(M + K + R)
    xp = torch.randn(M, K + 8, generator=g).to(dtype)
    x = xp[:, :K]
    A = (torch.randn(K, R, generator=g) * 0.05).to(dtype)
    xd, Ad = xp.to(cuda_dev)[:, :K], A.to(cuda_dev)                   # row stride K + 8 on the device too
    assert xd.stride(0) == K + 8 or M == 1
    t = ops.lowrank_down(xd, Ad.t().contiguous()).cpu()
    ref = x.double() @ A.double()
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    err = (t.double() - ref).abs()
    mag = x.double().abs() @ A.double().abs()                        # bound of the fp32 accumulation error
    assert bool((err <= ulp * ref.abs() * 1.01 + 1e-6 * mag).all()), err.max().item()
    t_torch = (xd @ Ad).cpu()
    assert (t != t_torch).float().mean().item() < 0.02
    ops.check_device_status(cuda_dev)


def test_shared_input_group_uses_native_down_projection_for_many_rows(cuda_dev, monkeypatch):
    """A group of layers on one input takes ONE native down-projection of width 32 x members, and
    every member's output equals the ungrouped layer's wherever the two down-projections agree (they differ in fp32
    summation order only)."""
    from pyraquant_b200.int8_exec import share_input_quantisation
    g = torch.Generator().manual_seed(11)
    M, K = 32768 + 37, 256
    grouped = [_toy_layer(cuda_dev, g, K, n, lowrank=True) for n in (256, 512, 256)]
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_dev)
    alone = [m(x) for m in grouped]                                  # before grouping: one kernel call each
    t_alone = [m._down(x) for m in grouped]
    calls = []
    real = ops.lowrank_down

    def counting(x2, a_t):
        calls.append(tuple(a_t.shape))
        return real(x2, a_t)

    monkeypatch.setattr(ops, "lowrank_down", counting)
    grp = share_input_quantisation(grouped)
    outs = [m(x) for m in grouped]
    assert calls == [(96, K)], calls
    _, _, T = grp.prepare(x)
    for i, m in enumerate(grouped):
        same_t = (grp.t_of(m, T) == t_alone[i]).all(dim=1)
        assert same_t.float().mean().item() > 0.9
        assert torch.equal(outs[i][same_t], alone[i][same_t])
        assert (outs[i].float() - alone[i].float()).abs().max().item() <= 0.02 * alone[i].float().abs().max().item()
    ops.check_device_status(cuda_dev)


def test_int8linear_uses_native_down_projection_for_many_rows(cuda_dev, monkeypatch):
    """Int8Linear.forward takes the library's own down-projection kernel at small and large row counts: the output
    matches the exact dequantised math built on that kernel's t, and the kernel really is the one called."""
    g = torch.Generator().manual_seed(3)
    M, K, N = 32768 + 100, 256, 256
    layer = _toy_layer(cuda_dev, g, K, N, lowrank=True)
    x = (torch.randn(M, K, generator=g)).to(torch.bfloat16)
    calls = {"n": 0}
    real = ops.lowrank_down

    def counting(x2, a_t):
        calls["n"] += 1
        return real(x2, a_t)
    monkeypatch.setattr(ops, "lowrank_down", counting)
    xd = x.to(cuda_dev)
    y = layer(xd).cpu()
    assert calls["n"] == 1
    t = real(xd, layer._lr_At()).cpu()
    xq, sx = oracle.quant_rows(x)
    ref = oracle.exact_dequant_f64(oracle.int_mm(xq, layer.weight_int8.cpu()), sx, layer.w_scale.cpu(), layer.bias.cpu(),
                                   t, layer.lr_B.cpu())
    assert max_rel_err(y, ref) <= TOL


def test_dequant_epilogue_and_linear_2d(cuda_dev):
    L = oracle.make_layer(5, 300, 512, 256, lowrank=False)
    wq, ws = oracle.quant_weight(L["w"], where="cuda")
    xq, sx = oracle.quant_rows(L["x"])
    acc = oracle.int_mm(xq, wq)
    d = cuda_dev
    y = int8_exec.dequant_epilogue(acc.to(d), sx.to(d), ws.to(d), L["bias"].to(d), torch.bfloat16)
    assert torch.equal(y.cpu(), oracle.epilogue(acc, sx, ws, L["bias"], None, None, torch.bfloat16))
    for backend in (None, "triton", "cublas"):
        y2 = int8_exec.int8_linear_2d(L["x"].to(d), wq.to(d), ws.to(d), L["bias"].to(d), backend=backend)
        assert max_rel_err(y2.cpu(), oracle.exact_dequant_f64(acc, sx, ws, L["bias"], None, None)) <= TOL
    with pytest.raises(ValueError):
        int8_exec.int8_linear_2d(L["x"].to(d), wq.to(d), ws.to(d), None, backend="nope")


def test_reference_selftest_assertions(cuda_dev):
    """The reference's own numerical self-test (deploy/int8_exec.py:498-536) with its thresholds."""
    rep = int8_exec.selftest_and_bench(Ms=())["selftest"]
    assert rep["act_quant_mismatch_elems"] == 0 and rep["act_scale_max_rel_err"] == 0.0


# ------------------------------------------------------------------------------------------------ group-32 path
@pytest.mark.parametrize("M,K,N", [(128, 128, 128), (300, 640, 640), (257, 1280, 1280), (1000, 2560, 640),
                                   (77, 640, 5120), (512, 5120, 1280), (130, 256, 264)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_g32_matches_oracle(cuda_dev, M, K, N, dtype):
    """SDXL W8A8 group-32 shapes (config 3) in miniature: integer grid from the oracle, GEMM on the GPU."""
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    xq, sa = oracle.quant_rows_g32(x)
    wq, sw = oracle.quant_weight_g32(w, where="cuda")
    d = cuda_dev
    for bias in (b, None):
        y = int8_exec.int8_gemm_g32(xq.to(d), sa.to(d), wq.to(d), sw.t().contiguous().to(d),
                                    None if bias is None else bias.to(d), dtype).cpu()
        want = oracle.gemm_g32(xq, sa, wq, sw, bias, dtype)
        assert torch.equal(y, want)                  # exact partial sums and the same fp32 operation order
        assert max_rel_err(y, oracle.gemm_g32_f64(xq, sa, wq, sw, bias)) <= TOL


def test_int8linear_g32_module(cuda_dev):
    g = torch.Generator().manual_seed(33)
    lin = nn.Linear(640, 1280, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(1280, 640, generator=g) * 0.02); lin.bias.copy_(torch.randn(1280, generator=g) * 0.01)
    x = torch.randn(3, 77, 640, generator=g).to(torch.float16)
    q = int8_exec.Int8LinearG32(lin.to(torch.float16), device=cuda_dev)
    wq, sw = oracle.quant_weight_g32(lin.weight.detach().float(), where="cuda")
    assert torch.equal(q.weight_int8.cpu(), wq) and torch.equal(q.w_scale.cpu(), sw)
    y = q(x.to(cuda_dev)).cpu()
    xq, sa = oracle.quant_rows_g32(x.reshape(-1, 640))
    want = oracle.gemm_g32(xq, sa, wq, sw, lin.bias.detach().float(), torch.float16).reshape(3, 77, 1280)
    assert torch.equal(y, want)
    assert set(q.state_dict()) == {"weight_int8", "w_scale", "bias"}


# ------------------------------------------------------------------------------------------------ full-size properties
def test_full_size_quant_and_gemm_properties(cuda_dev):
    """BASELINE config 2 row count (M = 65536 + 512) at K = 3072 -> N = 3072: sizes the CPU oracle cannot
    finish quickly, so parity is checked through exact size-independent identities:
      column checksum  sum_m acc[m,:] == (sum_m xq[m,:]) @ w^T        (int64, exact)
      row checksum     sum_n acc[m,:] == xq[m,:] @ (sum_n w[n,:])     (int64, exact)
    plus the per-row quantisation identities |x - q*s| <= s/2 and max|q| == 127."""
    d = cuda_dev
    M, K, N = 66048, 3072, 3072
    g = torch.Generator(device=d).manual_seed(2)
    x = torch.randn(M, K, generator=g, device=d, dtype=torch.float32)
    x[:, ::211] *= 20.0
    x = x.to(torch.bfloat16)
    q, s = int8_exec.quant_rows(x)
    xf = x.float()
    amax = xf.abs().amax(1).clamp_min(1e-8)
    s_ref = amax / torch.full_like(amax, 127.0)            # tensor / tensor: IEEE division on CUDA as well
    assert torch.equal(s, s_ref)
    assert int(q.abs().amax(1).min()) == 127
    assert bool(((xf - q.float() * s[:, None]).abs() <= s[:, None] * 0.5001).all())
    del xf
    w = torch.randint(-127, 128, (N, K), generator=g, device=d, dtype=torch.int8)
    sc = torch.rand(N, generator=g, device=d) * 1e-3 + 1e-4
    out, acc = ops.int8_gemm_debug(q, s, w, sc, None, None, None, torch.bfloat16)
    col = acc.sum(0, dtype=torch.int64).cpu()
    row = acc.sum(1, dtype=torch.int64).cpu()
    qs = q.sum(0, dtype=torch.int64).cpu()
    ws = w.sum(0, dtype=torch.int64).cpu()
    assert torch.equal(col, w.cpu().to(torch.int64) @ qs)
    row_ref = torch.empty(M, dtype=torch.int64)
    qc = q.cpu()
    for i in range(0, M, 8192):
        row_ref[i:i + 8192] = qc[i:i + 8192].to(torch.int64) @ ws
    assert torch.equal(row, row_ref)
    # output = rounding of acc * (s_row*s_col): recompute from the verified accumulators in chunks
    for i in range(0, M, 16384):
        ref = (acc[i:i + 16384].float() * (s[i:i + 16384, None] * sc[None, :])).to(torch.bfloat16)
        assert torch.equal(out[i:i + 16384], ref)


# ------------------------------------------------------------------------------------------------ gather / scatter
def test_scatter_matches_reference_fixture(cuda_dev, golden):
    g = golden("routing_gather_scatter.npz")
    boxes = [tuple(b) for b in g["boxes"].tolist()]
    bg = from_bf16_bits(g["background_bits"])
    for prefix, halo, fb, bx, key in (("", 2, 1.0, boxes, "n_buckets"), ("h3_", 3, 0.75, boxes[:4], "h3_n_buckets")):
        plan = routing.build_route_plan((24, 24), bx, halo, fusion_beta=fb)
        y = torch.cat([from_bf16_bits(g[f"{prefix}bucket{i}_out_bits"]).reshape(-1, bg.shape[-1])
                       for i in range(int(g[key]))])
        fused = routing.fuse_rows(bg.to(cuda_dev), y.to(cuda_dev), plan)
        assert torch.equal(fused.cpu(), from_bf16_bits(g[f"{prefix}fused_bits"]))
    hidden = from_bf16_bits(g["hidden_bits"]).reshape(24 * 24, -1)
    plan = routing.build_route_plan((24, 24), boxes, 2)
    got = routing.gather_rows(hidden.to(cuda_dev), plan)
    want = torch.cat([from_bf16_bits(g[f"bucket{i}_hidden_bits"]).reshape(-1, hidden.shape[1])
                      for i in range(int(g["n_buckets"]))])
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_routed_gather_scatter_vs_oracle(cuda_dev, dtype):
    """64x64 token canvas, 8x8 leaves of 8 tokens, Bernoulli(0.3) selection, halo 2, C = 256."""
    H = W = 64; C = 256
    g = torch.Generator().manual_seed(4)
    sel = (torch.rand(8, 8, generator=g) < 0.3).float().numpy()
    boxes = routing.leaf_run_boxes(sel, 16)                     # leaf = 16 latent = 8 tokens
    canvas = torch.randn(1, H, W, C, generator=g).to(dtype)
    bg = torch.randn(1, H, W, C, generator=g).to(dtype)
    plan = routing.build_route_plan((H, W), boxes, 2, dtype=dtype)
    buckets = oracle.gather_buckets(canvas, boxes, 2)
    want_rows = torch.cat([t.reshape(-1, C) for _hw, t, _g in buckets])
    d = cuda_dev
    rows = routing.gather_rows(canvas.reshape(H * W, C).to(d), plan)
    assert torch.equal(rows.cpu(), want_rows)
    q, s = routing.gather_quant_rows(canvas.reshape(H * W, C).to(d), plan)
    qo, so = oracle.quant_rows(want_rows)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    outs, ys = [], []
    for hw, t, geoms in buckets:
        o = (torch.randn(t.shape, generator=g) * 2).to(dtype)
        # signed zeros in the routed rows (and a background of both signs): 0 * bg + y keeps or drops the sign of a zero
        # exactly as the reference's arithmetic does
        o.view(-1)[torch.randperm(o.numel(), generator=g)[: o.numel() // 50]] = -0.0
        o.view(-1)[torch.randperm(o.numel(), generator=g)[: o.numel() // 50]] = 0.0
        outs.append(((hw, geoms), o)); ys.append(o.reshape(-1, C))
    want = oracle.fuse_buckets(bg, outs, 1.0)
    got = routing.fuse_rows(bg.to(d), torch.cat(ys).to(d), plan)
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))       # bit patterns: -0 and +0 differ
    # untouched tokens are bit-identical to the background
    touched = torch.zeros(H * W, dtype=torch.bool); touched[torch.from_numpy(plan.tokens).long()] = True
    assert torch.equal(got.cpu().reshape(H * W, C)[~touched], bg.reshape(H * W, C)[~touched])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scatter_contributor_lists_of_every_kind(cuda_dev, dtype):
    """`pq_scatter_rows` on hand-made contributor lists that the routing plans of the other tests do not produce: one
    full-weight contributor (copied), fractional weights, weights that are not values of the canvas type (fp32
    arithmetic instead of the packed one), two and five contributors, more than 32 (the list is then walked from global
    memory), out-of-range row numbers (skipped), an all-invalid list (weight sum 0), signed zeros.  Checked bit for bit
    against the reference's sequence of roundings evaluated in fp32 with explicit rounding after every step."""
    g = torch.Generator().manual_seed(77)
    C, M_act, rows = 264, 64, 40
    y = (torch.randn(M_act, C, generator=g) * 2).to(dtype)
    y[3, :20] = -0.0; y[5, 7] = 0.0
    canvas = torch.randn(rows, C, generator=g).to(dtype)
    canvas[2, :9] = -0.0
    q = lambda v: float(torch.tensor(v).to(dtype))                     # a weight representable in the canvas type
    lists = [
        [(3, 1.0)],                                                       # copy, with -0 in the row
        [(7, q(0.37))],                                                   # one fractional weight: background keeps a share
        [(8, 0.3)],                                                       # 0.3 is not a bf16 / fp16 value
        [(1, 1.0), (2, q(0.25))],                                         # sum > 1, two contributors
        [(9, q(0.5)), (10, q(0.5))],                                      # power-of-two divisor
        [(11, q(0.2)), (12, q(0.3)), (13, q(0.1)), (14, q(0.15)), (15, q(0.05))],
        [(i % M_act, q(0.02)) for i in range(40)],                        # more than 32 entries
        [(-1, 1.0), (5, 1.0)],                                            # an invalid row number in front of a valid one
        [(M_act + 3, q(0.5))],                                            # nothing valid: weight sum 0
        [(20, 1.0), (-5, q(0.5)), (21, q(0.125))],
    ]
    tokens = torch.tensor([0, 2, 5, 6, 9, 17, 18, 30, 31, 39], dtype=torch.int32)
    ptr, src, beta = [0], [], []
    for lst in lists:
        src += [r for r, _ in lst]; beta += [b for _, b in lst]; ptr.append(len(src))
    rnd = lambda t: t.to(dtype).float()
    want = canvas.clone()
    for tok, lst in zip(tokens.tolist(), lists):
        local = torch.zeros(C); bsum = torch.zeros(())
        for r, b in lst:
            if r < 0 or r >= M_act:
                continue
            bt = torch.tensor(b, dtype=torch.float32)
            local = rnd(local + rnd(bt * y[r].float()))
            bsum = rnd(bsum + bt)
        bm = bsum.clamp(0.0, 1.0)
        denom = rnd(bsum.clamp_min(1e-8))
        om = rnd(1.0 - bm)
        c = rnd(local / denom) if bsum > 0 else torch.zeros(C)
        want[tok] = (rnd(om * canvas[tok].float()) + rnd(bm * c)).to(dtype)
    got = canvas.clone().to(cuda_dev)
    ops._scatter_rows_impl(y.to(cuda_dev), tokens.to(cuda_dev), torch.tensor(ptr, dtype=torch.int32, device=cuda_dev),
                           torch.tensor(src, dtype=torch.int32, device=cuda_dev),
                           torch.tensor(beta, dtype=torch.float32, device=cuda_dev), got)
    torch.cuda.synchronize()
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


def test_routed_two_tier_linear(cuda_dev):
    """Config-4 shape in miniature: routed rows -> Linear with per-leaf hi/lo weights -> scatter."""
    H = W = 32; K = 256; N = 512
    g = torch.Generator().manual_seed(8)
    sel = (torch.rand(4, 4, generator=g) < 0.4).float().numpy(); sel[0, 0] = 1; sel[1, 0] = 1
    scores = torch.rand(4, 4, generator=g).numpy()
    hi = routing.inner_split_median(scores, sel, 1.0)
    tmap = routing.leaf_tier_to_token_map(hi, (H, W))
    plan = routing.build_route_plan((H, W), routing.leaf_run_boxes(sel, 16), 2, token_tier_hi=tmap)
    canvas = rand_act(H * W, K, torch.bfloat16, 31)
    lin = nn.Linear(K, N, bias=True).to(torch.bfloat16)
    A = (torch.randn(K, 32, generator=g) * 0.02).to(torch.bfloat16)
    B = (torch.randn(32, N, generator=g) * 0.02).to(torch.bfloat16)
    q = int8_exec.Int8LinearRouted(lin, device=cuda_dev, lowrank=(A, B))
    y = q.forward_gathered(canvas.to(cuda_dev), plan.to(cuda_dev)["row_idx"], plan.m_hi).cpu()
    rows = canvas[torch.from_numpy(plan.row_idx).long()]
    w8, s8 = oracle.quant_weight(lin.weight.detach(), where="cuda")
    w4, s4 = oracle.nested4_from_int8(w8, s8)
    xq, sx = oracle.quant_rows(rows)
    t = q._down(rows.to(cuda_dev)).cpu()                      # the module's own down-projection
    b32 = lin.bias.detach().float()
    mh = plan.m_hi
    ref = torch.cat([oracle.exact_dequant_f64(oracle.int_mm(xq[:mh], w8), sx[:mh], s8, b32, t[:mh], B),
                     oracle.exact_dequant_f64(oracle.int_mm(xq[mh:], w4), sx[mh:], s4, b32, t[mh:], B)])
    assert 0 < mh < plan.n_rows
    assert max_rel_err(y, ref) <= TOL
    y2 = q.forward_rows(rows.to(cuda_dev), mh).cpu()
    assert max_rel_err(y2, ref) <= TOL


@pytest.mark.parametrize("case", ["rank16", "fp16_factors"])
def test_routed_linear_keeps_a_lowrank_branch_it_cannot_fuse(cuda_dev, case):
    """A low-rank branch outside the fused epilogue's reach (rank 16; factors in another dtype than the activations)
    is added after the two-tier GEMM instead of being dropped."""
    H = W = 16; K = 128; N = 256
    g = torch.Generator().manual_seed(90)
    sel = np.zeros((2, 2), np.float32); sel[0, 0] = sel[1, 1] = 1
    tmap = routing.leaf_tier_to_token_map(np.array([[1, 0], [0, 0]], np.float32), (H, W))
    plan = routing.build_route_plan((H, W), routing.leaf_run_boxes(sel, 16), 2, token_tier_hi=tmap)
    canvas = rand_act(H * W, K, torch.bfloat16, 91)
    lin = nn.Linear(K, N, bias=True).to(torch.bfloat16)
    R, fdt = (16, torch.bfloat16) if case == "rank16" else (32, torch.float16)
    A = (torch.randn(K, R, generator=g) * 0.05).to(fdt)
    B = (torch.randn(R, N, generator=g) * 0.05).to(fdt)
    q = int8_exec.Int8LinearRouted(lin, device=cuda_dev, lowrank=(A, B))
    rows = canvas[torch.from_numpy(plan.row_idx).long()]
    w8, s8 = oracle.quant_weight(lin.weight.detach(), where="cuda")
    w4, s4 = oracle.nested4_from_int8(w8, s8)
    xq, sx = oracle.quant_rows(rows)
    t = (rows.to(fdt).float() @ A.float()).to(fdt)
    b32 = lin.bias.detach().float()
    mh = plan.m_hi
    assert 0 < mh < plan.n_rows
    # the unfused sequence rounds twice (the GEMM output, then the sum), like the reference's own unfused branch
    # (deploy/int8_exec.py:394-407): the bar is the exact sum of the ROUNDED GEMM output and the exact low-rank term
    y_gemm = torch.cat([oracle.epilogue(oracle.int_mm(xq[:mh], w8), sx[:mh], s8, b32, None, None, torch.bfloat16),
                        oracle.epilogue(oracle.int_mm(xq[mh:], w4), sx[mh:], s4, b32, None, None, torch.bfloat16)])
    branch = t.double() @ B.double()
    ref = y_gemm.double() + branch
    assert float(branch.abs().mean() / y_gemm.double().abs().mean()) > 0.05      # the branch matters in this case
    # every rounding on the way (the factors and t converted to the activation dtype, GEMM output, the library's
    # product, the sum) is at most half a unit in the last place of its operand: the result stays within 2^-7 of the
    # operands' magnitudes of the exact sum, element by element
    bound = 2.0 ** -7 * (y_gemm.double().abs() + t.double().abs() @ B.double().abs()) + 1e-30

    def close(y):
        d = (y.double() - ref).abs()
        return bool((d <= bound).all()) and float(d.norm() / ref.norm()) < 4e-3

    y = q.forward_gathered(canvas.to(cuda_dev), plan.to(cuda_dev)["row_idx"], mh).cpu()
    assert close(y)
    assert max_rel_err(y, y_gemm.double()) > 5 * TOL               # i.e. the branch was not dropped
    y2 = q.forward_rows(rows.to(cuda_dev), mh).cpu()
    assert close(y2)


def test_shared_input_group_under_inference_mode_and_after_inplace_writes(cuda_dev, monkeypatch):
    """Inference tensors keep no version counter: grouped layers then run ungrouped instead of failing.  The
    library's own in-place write (accumulate epilogue) bumps the version of its target, so a cached quantisation of
    that tensor is not reused afterwards."""
    g = torch.Generator().manual_seed(34)
    K = 256
    a, b = _toy_layer(cuda_dev, g, K, 256), _toy_layer(cuda_dev, g, K, 256)
    x = rand_act(300, K, torch.bfloat16, 35).to(cuda_dev)
    alone = [a(x), b(x)]
    int8_exec.share_input_quantisation([a, b])
    with torch.inference_mode():
        xi = x.clone()
        assert xi.is_inference()
        got = [a(xi), b(xi)]
    assert torch.equal(got[0], alone[0]) and torch.equal(got[1], alone[1])
    # accumulate into a tensor the group has cached, then feed it to the group again
    calls = {"n": 0}
    real = ops._quant_rows_impl

    def counting(x2):
        calls["n"] += 1
        return real(x2)
    monkeypatch.setattr(ops, "_quant_rows_impl", counting)
    h = x.clone()
    y0 = a(h)                                                       # caches the quantisation of h
    n0 = calls["n"]
    v0 = h._version
    c = _toy_layer(cuda_dev, g, K, K, lowrank=False)
    c.forward_ex(x, ops.EPI_ACCUMULATE, out=h)                      # h += c(x), written by the GEMM epilogue
    assert h._version > v0
    y1 = b(h)
    assert calls["n"] == n0 + 2 and not torch.equal(h, x)         # c quantised x, b quantised the updated h
    monkeypatch.setattr(ops, "_quant_rows_impl", real)
    b.__dict__.pop("_shared_input"); a.__dict__.pop("_shared_input")
    assert torch.equal(y1, b(h))                                    # the fresh codes, not the stale ones
    del y0


def test_lean_path_follows_converted_buffers(cuda_dev):
    """Replacing or converting the float buffers (w_scale, bias, lr_B) while the int8 weight stays in place must not
    leave the fast path with stale addresses."""
    g = torch.Generator().manual_seed(36)
    m = _toy_layer(cuda_dev, g, 256, 512)
    x = rand_act(200, 256, torch.bfloat16, 37).to(cuda_dev)
    y0 = m(x)
    with torch.no_grad():
        new_scale = (m.w_scale * 2.0).clone()
        new_B = (m.lr_B.float() * 0.5).to(torch.bfloat16)
    m.w_scale = new_scale
    m.lr_B = new_B
    y1 = m(x)
    xq, sx = int8_exec.quant_rows(x)
    want = int8_exec.int8_gemm_lr(xq, sx, m.weight_int8, new_scale, m.bias, m._down(x), new_B, torch.bfloat16)
    assert torch.equal(y1, want) and not torch.equal(y1, y0)
    m.lr_B.mul_(2.0)                                               # in place: the K-major copy must follow
    want2 = int8_exec.int8_gemm_lr(xq, sx, m.weight_int8, new_scale, m.bias, m._down(x), m.lr_B, torch.bfloat16)
    assert torch.equal(m(x), want2)


def test_bounded_wait_runs_out_and_is_reported(cuda_dev):
    """A device-side wait that nothing ends: the kernel gives up after its budget (1 ms here), writes the status word
    and returns; the host turns the word into a RuntimeError, clears it, and the next GEMM on the same context is
    correct.  No trap, no endless loop, no fault."""
    lib = _lib.load()
    ws = ops.status_word(cuda_dev)
    ops.check_device_status(cuda_dev)
    rc = lib.pq_wait_probe(ws.data_ptr(), ws.numel() * 4, 1000, torch.cuda.current_stream(cuda_dev).cuda_stream)
    assert rc == 0
    with pytest.raises(RuntimeError, match="wait gave up"):
        ops.check_device_status(cuda_dev)
    ops.check_device_status(cuda_dev)                               # the word was cleared by the read above
    run_gemm_case(cuda_dev, 300, 512, 256, lowrank=True, bias=True, seed=5)
    run_gemm_case(cuda_dev, 2049, 768, 384, lowrank=False, bias=True, seed=6)
