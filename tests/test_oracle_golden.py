"""The CPU oracle against fixtures produced by running the reference's own CPU-runnable code
(tests/golden/make_golden.py).  Everything here is bit-exact."""
import numpy as np
import torch

from conftest import from_bf16_bits
from oracle import oracle


def test_weight_quant_matches_int8linear_ctor(golden):
    g = golden("int8linear_ctor.npz")
    w = from_bf16_bits(g["w_bits"])
    q, s = oracle.quant_weight(w)
    assert np.array_equal(q.numpy(), g["weight_int8"])
    assert np.array_equal(s.numpy(), g["w_scale"])
    # the all-zero channel takes the 1e-8 floor
    assert s[3].item() == np.float32(1e-8) / np.float32(127.0)
    assert (q[3] == 0).all()


def test_act_quant_matches_fakequant_a8(golden):
    g = golden("act_fakequant_a8.npz")
    x = from_bf16_bits(g["x_bits"])
    q, s = oracle.quant_rows(x)
    qdq = (q.float() * s[:, None]).to(torch.bfloat16)
    assert torch.equal(qdq, from_bf16_bits(g["qdq_bits"]))
    assert int(q.abs().max()) == 127 and (q[7] == 0).all()


def test_g32_weight_grid_matches_qdq_weight(golden):
    g = golden("qdq_weight_w8g32.npz")
    w = torch.from_numpy(g["w"])
    q, s = oracle.quant_weight_g32(w, 32)
    deq = (q.float().reshape(w.shape[0], -1, 32) * s[..., None]).reshape(w.shape)
    assert np.array_equal(deq.numpy(), g["qdq"])


def test_g32_act_grid_matches_dyn_group(golden):
    g = golden("act_dyn_group32.npz")
    x = torch.from_numpy(g["x"])
    q, s = oracle.quant_rows_g32(x, 32)
    deq = (q.float().reshape(x.shape[0], -1, 32) * s[..., None]).reshape(x.shape)
    assert np.array_equal(deq.numpy(), g["qdq"])


def test_nested4_matches_reference(golden):
    g = golden("nested4.npz")
    w = torch.from_numpy(g["w"])
    q8, s8 = oracle.quant_weight(w)
    c, s4 = oracle.nested4_from_int8(q8, s8)
    assert int(c.abs().max()) <= 7
    # reference dequantises as c * (127/7) * s8 with that association
    deq = c.float() * (127 / 7) * s8[:, None]
    assert np.array_equal(deq.numpy(), g["qdq_perchannel"])
    # group-32 flavour through the group grid
    q8g, s8g = oracle.quant_weight_g32(w, 32)
    cg = (q8g.float() * (7 / 127)).round().clamp(-7, 7).reshape(w.shape[0], -1, 32)
    deqg = (cg * (127 / 7) * s8g[..., None]).reshape(w.shape)
    assert np.array_equal(deqg.numpy(), g["qdq_g32"])


def test_nested4_lut_has_no_ties():
    q = torch.arange(-127, 128).float() * (7 / 127)
    assert ((q - q.floor() - 0.5).abs() > 1e-3).all()


def test_gather_matches_build_patch_buckets(golden):
    g = golden("routing_gather_scatter.npz")
    hidden = from_bf16_bits(g["hidden_bits"])
    H = W = 24
    grid = hidden.reshape(1, H, W, -1)
    buckets = oracle.gather_buckets(grid, [tuple(b) for b in g["boxes"].tolist()], 2)
    assert len(buckets) == int(g["n_buckets"])
    for i, (hw, tens, geoms) in enumerate(buckets):
        assert tuple(g[f"bucket{i}_hw"]) == hw
        assert torch.equal(tens, from_bf16_bits(g[f"bucket{i}_hidden_bits"]))
        assert np.array_equal(np.asarray([gm[1] for gm in geoms]), g[f"bucket{i}_halo_boxes"])


def test_scatter_matches_fuse_patch_predictions(golden):
    g = golden("routing_gather_scatter.npz")
    hidden = from_bf16_bits(g["hidden_bits"])
    background = from_bf16_bits(g["background_bits"])
    H = W = 24
    boxes = [tuple(b) for b in g["boxes"].tolist()]
    buckets = oracle.gather_buckets(hidden.reshape(1, H, W, -1), boxes, 2)
    outs = [((hw, geoms), from_bf16_bits(g[f"bucket{i}_out_bits"])) for i, (hw, _t, geoms) in enumerate(buckets)]
    fused = oracle.fuse_buckets(background, outs, 1.0)
    assert torch.equal(fused, from_bf16_bits(g["fused_bits"]))
    buckets3 = oracle.gather_buckets(hidden.reshape(1, H, W, -1), boxes[:4], 3)
    outs3 = [((hw, geoms), from_bf16_bits(g[f"h3_bucket{i}_out_bits"])) for i, (hw, _t, geoms) in enumerate(buckets3)]
    fused3 = oracle.fuse_buckets(background, outs3, 0.75)
    assert torch.equal(fused3, from_bf16_bits(g["h3_fused_bits"]))


def test_inner_split_median(golden):
    g = golden("inner_split_median.npz")
    hi = oracle.inner_split_median(torch.from_numpy(g["scores"]), torch.from_numpy(g["sel"]), 1.0)
    assert np.array_equal(hi.numpy(), g["hi"])


def test_int_mm_is_exact_beyond_fp32_range():
    # |acc| can reach K*127^2 > 2^24: an fp32 matmul would round, the oracle must not
    K = 4096
    xq = torch.full((32, K), 127, dtype=torch.int8)
    w = torch.full((8, K), 127, dtype=torch.int8)
    w[0, 0] = 126
    acc = oracle.int_mm(xq, w)
    assert acc[0, 1].item() == K * 127 * 127 and acc[0, 0].item() == K * 127 * 127 - 127
    small = oracle.int_mm(xq[:3], w)
    assert torch.equal(small, acc[:3])


def test_forward_agrees_with_reference_selftest_formula():
    # deploy/int8_exec.py:535 bound: fused vs unfused expression on the same codes, rel-L2 < 1e-3
    L = oracle.make_layer(0, 64, 256, 128, lowrank=False)
    wq, ws = oracle.quant_weight(L["w"])
    y = oracle.int8_linear_forward(L["x"], wq, ws, L["bias"]).float()
    xq, sx = oracle.quant_rows(L["x"])
    ref = oracle.selftest_unfused_reference(xq, sx, wq, ws, L["bias"]).float()
    assert ((y - ref).norm() / ref.norm()).item() < 1e-3


def test_adaln_modulate_follows_the_float64_formula():
    """The restatement of flux/transformer_flux.py:236-237 in the tensors' own type against float64 arithmetic."""
    g = torch.Generator().manual_seed(3)
    B, T, K = 2, 40, 256
    h = (torch.randn(B, T, K, generator=g) * 2 + 0.5).to(torch.bfloat16)
    scale = (torch.randn(B, K, generator=g) * 0.3).to(torch.bfloat16)
    shift = (torch.randn(B, K, generator=g) * 0.2).to(torch.bfloat16)
    z = oracle.adaln_modulate(h, scale, shift, 1e-6)
    hd = h.double()
    y = (hd - hd.mean(-1, keepdim=True)) / torch.sqrt(hd.var(-1, unbiased=False, keepdim=True) + 1e-6)
    want = y * (1 + scale.double()[:, None]) + shift.double()[:, None]
    assert z.dtype == torch.bfloat16 and z.shape == h.shape
    assert bool(((z.double() - want).abs() <= 2.0 ** -6 * (want.abs() + shift.double().abs()[:, None]) + 1e-3).all())
