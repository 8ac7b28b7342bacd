"""Host-side logic on CPU: the route plan (gather list + scatter contributor lists) against the
reference fixtures, and the drop-in module surface of int8_exec."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import from_bf16_bits
from oracle import oracle
from pyraquant_b200 import int8_exec, routing


def emulate_scatter(y, plan, canvas):
    """Torch-on-CPU walk of the CSR lists with the rounding points the CUDA kernel uses."""
    out = canvas.clone()
    dt = canvas.dtype
    r = lambda v: v.to(dt).float()
    for i, tok in enumerate(plan.tokens.tolist()):
        local = torch.zeros(canvas.shape[1]); bsum = torch.zeros(())
        for e in range(plan.ptr[i], plan.ptr[i + 1]):
            b = torch.tensor(float(plan.beta[e]))
            local = r(local + r(b * y[plan.src[e]].float()))
            bsum = r(bsum + b)
        bm = bsum.clamp(0, 1)
        denom = r(torch.maximum(bsum, torch.tensor(1e-8)))
        comb = r(local / denom) if bsum > 0 else torch.zeros_like(local)
        out[tok] = (r(r(1.0 - bm) * canvas[tok].float()) + r(bm * comb)).to(dt)
    return out


def test_leaf_run_boxes_known_answer():
    sel = np.array([[1, 1, 0, 1], [0, 0, 0, 0], [0, 1, 1, 1], [1, 0, 0, 0]], dtype=np.float32)
    got = routing.leaf_run_boxes(sel, 64)
    assert got == [(0, 64, 0, 128), (0, 64, 192, 256), (128, 192, 64, 256), (192, 256, 0, 64)]
    assert got == oracle.leaf_run_boxes(sel, 64)


def test_token_box_rules():
    assert routing.latent_box_to_token_box((0, 64, 64, 128)) == (0, 32, 32, 64)
    assert routing.latent_box_to_token_box((0, 64, 64, 128), 1) == (0, 33, 32, 65)
    for bad in [(-2, 4, 0, 4), (0, 3, 0, 4), (4, 4, 0, 2)]:
        with pytest.raises(ValueError):
            routing.latent_box_to_token_box(bad)
    with pytest.raises(ValueError):
        routing.latent_box_to_token_box((0, 2, 0, 2), 2)
    assert routing.expand_box((0, 8, 20, 24), 2, (24, 24)) == (0, 10, 18, 24)


def test_feather_weights_halo2_is_zero_one():
    w = routing.feather_weights((12, 12), (2, 10, 2, 10), torch.bfloat16)
    assert torch.equal(w, oracle.feather_mask((12, 12), (2, 10, 2, 10), torch.bfloat16))
    assert w[0].abs().max() == 0 and w[1, 1] == 1 and w[5, 5] == 1     # outer ring 0, inner ring 1


def test_feather_weights_match_reference_masks(golden):
    """Blend weights against masks made by the reference's halo_feather_mask (halo widths 1-6, clipped halos, all three
    profile shapes, powers 0.5/1/2, bf16 and fp16): bit-equal."""
    import sys
    sys.path.insert(0, str(__import__("pathlib").Path(__file__).parent / "golden"))
    from make_golden import FEATHER_CASES
    g = golden("feather_masks.npz")
    assert int(g["n"]) == len(FEATHER_CASES)
    for i, (hw, inner, mode, power) in enumerate(FEATHER_CASES):
        for tag, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
            want = torch.from_numpy(g[f"mask{i}_{tag}_bits"]).view(dt)
            got = routing.feather_weights(hw, inner, dt, 1.0, mode, power)
            assert torch.equal(got, want), (i, tag)
            if mode == "cosine" and power == 1.0:
                assert torch.equal(oracle.feather_mask(hw, inner, dt), want), (i, tag)
    with pytest.raises(ValueError):
        routing.feather_weights((4, 4), (1, 3, 1, 3), torch.bfloat16, mode="gaussian")


def test_plan_gather_matches_reference_buckets(golden):
    g = golden("routing_gather_scatter.npz")
    boxes = [tuple(b) for b in g["boxes"].tolist()]
    plan = routing.build_route_plan((24, 24), boxes, 2)
    hidden = from_bf16_bits(g["hidden_bits"]).reshape(24 * 24, -1)
    want = torch.cat([from_bf16_bits(g[f"bucket{i}_hidden_bits"]).reshape(-1, hidden.shape[1])
                      for i in range(int(g["n_buckets"]))])
    assert plan.n_rows == want.shape[0] and plan.m_hi == plan.n_rows
    assert torch.equal(hidden[torch.from_numpy(plan.row_idx).long()], want)
    assert [tuple(s) for s in plan.bucket_shapes] == [tuple(g[f"bucket{i}_hw"]) for i in range(int(g["n_buckets"]))]
    assert len(plan.patches) == 4                                        # the duplicate box was dropped


def test_plan_scatter_matches_reference_fusion(golden):
    g = golden("routing_gather_scatter.npz")
    boxes = [tuple(b) for b in g["boxes"].tolist()]
    bg = from_bf16_bits(g["background_bits"]).reshape(24 * 24, -1)
    for prefix, halo, fb, bx, key in (("", 2, 1.0, boxes, "n_buckets"), ("h3_", 3, 0.75, boxes[:4], "h3_n_buckets")):
        plan = routing.build_route_plan((24, 24), bx, halo, fusion_beta=fb)
        y = torch.cat([from_bf16_bits(g[f"{prefix}bucket{i}_out_bits"]).reshape(-1, bg.shape[1])
                       for i in range(int(g[key]))])
        got = emulate_scatter(y, plan, bg)
        assert torch.equal(got.reshape(1, 24, 24, -1), from_bf16_bits(g[f"{prefix}fused_bits"]))
        assert plan.ptr[-1] == plan.src.shape[0] and np.all(np.diff(plan.ptr) >= 1)


def test_plan_tier_ordering_keeps_scatter_result(golden):
    g = golden("routing_gather_scatter.npz")
    boxes = [tuple(b) for b in g["boxes"].tolist()]
    leaf_hi = np.array([[1, 0, 0], [0, 1, 0], [1, 0, 0]], dtype=np.float32)     # 3x3 leaves of 8 tokens
    tmap = routing.leaf_tier_to_token_map(leaf_hi, (24, 24))
    assert tmap.shape == (24, 24) and tmap[0, 0] and not tmap[0, 8] and tmap[8, 8]
    flat = routing.build_route_plan((24, 24), boxes, 2)
    tiered = routing.build_route_plan((24, 24), boxes, 2, token_tier_hi=tmap)
    assert sorted(tiered.row_idx.tolist()) == sorted(flat.row_idx.tolist())
    is_hi = tmap.reshape(-1)[tiered.row_idx]
    assert is_hi[:tiered.m_hi].all() and not is_hi[tiered.m_hi:].any() and 0 < tiered.m_hi < tiered.n_rows
    bg = from_bf16_bits(g["background_bits"]).reshape(24 * 24, -1)
    y_flat = torch.cat([from_bf16_bits(g[f"bucket{i}_out_bits"]).reshape(-1, bg.shape[1])
                        for i in range(int(g["n_buckets"]))])
    # the same per-row outputs, permuted like the rows, must blend to the same canvas
    perm = np.argsort(~tmap.reshape(-1)[flat.row_idx], kind="stable")
    got = emulate_scatter(y_flat[torch.from_numpy(perm)], tiered, bg)
    assert torch.equal(got.reshape(1, 24, 24, -1), from_bf16_bits(g["fused_bits"]))


def test_inner_split_median_matches_reference(golden):
    g = golden("inner_split_median.npz")
    assert np.array_equal(routing.inner_split_median(g["scores"], g["sel"], 1.0), g["hi"])


def test_empty_plan():
    plan = routing.build_route_plan((16, 16), [], 2)
    assert plan.n_rows == 0 and plan.tokens.shape[0] == 0 and plan.ptr.tolist() == [0]


# ---------------------------------------------------------------------------------------------- int8_exec surface
def test_module_surface_matches_reference_names():
    for name in ("BACKENDS", "DEFAULT_BACKEND", "BACKEND", "set_backend", "get_backend", "quant_rows",
                 "dequant_epilogue", "int8_gemm_fused", "int8_linear_2d", "int8_gemm_lr", "LOWRANK_A_ATTR",
                 "LOWRANK_B_ATTR", "Int8Linear", "is_bf16_whitelisted", "convert_linears_to_int8", "warm_kernels",
                 "FLUX_TOKEN_SHAPES", "selftest_and_bench", "_m_bucket", "_bench"):
        assert hasattr(int8_exec, name), name
    assert int8_exec.BACKENDS == ("triton", "cublas") and int8_exec.DEFAULT_BACKEND == "triton"
    assert int8_exec.FLUX_TOKEN_SHAPES[(3072, 3072)] == 19 * 8 + 38 * 3
    assert [int8_exec._m_bucket(m) for m in (1, 8191, 8192, 32767, 32768)] == [0, 0, 1, 1, 2]


def test_set_backend_contract():
    assert int8_exec.set_backend("cublas") == "cublas" and int8_exec.get_backend() == "cublas"
    assert int8_exec.set_backend("triton") == "triton"
    with pytest.raises(ValueError):
        int8_exec.set_backend("cutlass")


def test_int8linear_ctor_matches_reference(golden):
    g = golden("int8linear_ctor.npz")
    lin = nn.Linear(96, 40, bias=True).to(torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(from_bf16_bits(g["w_bits"]))
        lin.bias.copy_(from_bf16_bits(g["bias_bits"]))
    A, B = from_bf16_bits(g["lr_A_bits"]), from_bf16_bits(g["lr_B_bits"])
    setattr(lin, int8_exec.LOWRANK_A_ATTR, A); setattr(lin, int8_exec.LOWRANK_B_ATTR, B)   # attribute route
    q = int8_exec.Int8Linear(lin)
    assert np.array_equal(q.weight_int8.numpy(), g["weight_int8"])
    assert np.array_equal(q.w_scale.numpy(), g["w_scale"])
    assert np.array_equal(q.bias.numpy(), g["bias_f32"])
    assert torch.equal(q.lr_A, A) and torch.equal(q.lr_B, B)
    assert q.in_features == 96 and q.out_features == 40
    sd = q.state_dict()
    assert set(sd) == {"weight_int8", "w_scale", "bias", "lr_A", "lr_B"}
    nb = int8_exec.Int8Linear(nn.Linear(32, 16, bias=False))
    assert nb.bias is None and nb.lr_A is None and set(nb.state_dict()) == {"weight_int8", "w_scale"}


def test_cpu_forward_is_refused_like_the_reference():
    q = int8_exec.Int8Linear(nn.Linear(64, 32).to(torch.bfloat16))
    with pytest.raises(AssertionError):
        q(torch.randn(4, 64).to(torch.bfloat16))
    with pytest.raises(AssertionError):
        int8_exec.quant_rows(torch.randn(4, 64).to(torch.bfloat16))


def test_whitelist_and_conversion_stats():
    assert int8_exec.is_bf16_whitelisted("x_embedder")
    assert int8_exec.is_bf16_whitelisted("transformer_blocks.3.norm1_context.linear")
    assert int8_exec.is_bf16_whitelisted("single_transformer_blocks.0.norm.linear")
    assert not int8_exec.is_bf16_whitelisted("transformer_blocks.3.attn.to_q")
    assert not int8_exec.is_bf16_whitelisted("transformer_blocks.3.ff.net.2")

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn = nn.Linear(32, 32)
            self.norm1 = nn.Sequential()
            self.norm1.linear = nn.Linear(32, 64)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.x_embedder = nn.Linear(8, 32)
            self.blocks = nn.ModuleList([Block(), Block()])
            self.proj_out = nn.Linear(32, 8)

    net = Net()
    st = int8_exec.convert_linears_to_int8(net, device=None)
    assert st["n_int8_linear"] == 2 and st["n_bf16_linear_kept"] == 4
    assert st["params_int8"] == 2 * 32 * 32 and st["bf16_equiv_gib"] == st["int8_weight_gib"] * 2
    assert isinstance(net.blocks[0].attn, int8_exec.Int8Linear) and isinstance(net.blocks[0].norm1.linear, nn.Linear)
    assert set(st) == {"n_int8_linear", "n_bf16_linear_kept", "params_int8", "params_bf16_linear_kept",
                       "bf16_kept_names", "int8_weight_gib", "bf16_equiv_gib"}


def test_nested4_codes_match_oracle():
    w = torch.randn(16, 64) * 0.02
    q8, s8 = oracle.quant_weight(w)
    c, s4 = int8_exec.nested4_codes(q8, s8)
    co, so = oracle.nested4_from_int8(q8, s8)
    assert torch.equal(c, co) and torch.equal(s4, so)


def test_group_shared_inputs_on_flux_like_blocks():
    """Sibling layers that read the same tensor are tied into groups by relative path; a layer joins one group only."""
    import torch.nn as nn
    from pyraquant_b200 import int8_exec

    class Attn(nn.Module):
        def __init__(self, ctx):
            super().__init__()
            self.to_q = nn.Linear(64, 64); self.to_k = nn.Linear(64, 64); self.to_v = nn.Linear(64, 64)
            if ctx:
                self.add_q_proj = nn.Linear(64, 64); self.add_k_proj = nn.Linear(64, 64); self.add_v_proj = nn.Linear(64, 64)

    class Single(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj_mlp = nn.Linear(64, 256); self.attn = Attn(False); self.proj_out = nn.Linear(320, 64)

    class Double(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn = Attn(True)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.single = nn.ModuleList([Single(), Single()]); self.dual = nn.ModuleList([Double()])

    net = Net()
    stats = int8_exec.convert_linears_to_int8(net, device=None, whitelist=lambda n: False,
                                              shared_input_groups=int8_exec.FLUX_SHARED_INPUT_GROUPS)
    # 2 single blocks (proj_mlp + q/k/v) + 1 double block (q/k/v and add_q/k/v)
    assert stats["n_shared_input_groups"] == 4
    g = net.single[0].proj_mlp.__dict__["_shared_input"]
    assert [m for m in g.layers] == [net.single[0].proj_mlp, net.single[0].attn.to_q, net.single[0].attn.to_k,
                                     net.single[0].attn.to_v]
    assert "_shared_input" not in net.single[0].proj_out.__dict__
    assert net.dual[0].attn.to_q.__dict__["_shared_input"] is not net.dual[0].attn.add_q_proj.__dict__["_shared_input"]
    # the reference's statistics keys are untouched when the option is not used
    stats2 = int8_exec.convert_linears_to_int8(Net(), device=None, whitelist=lambda n: False)
    assert "n_shared_input_groups" not in stats2


def test_fuse_split_inputs_replaces_reference_layout():
    import torch.nn as nn
    from pyraquant_b200 import int8_exec

    class SplitInLinear(nn.Module):          # the layout of pyraquant/external_quant.py:174-192
        def __init__(self, in0, in1, out):
            super().__init__()
            self.linears = nn.ModuleList([nn.Linear(in0, out, bias=False), nn.Linear(in1, out)]); self.in0 = in0

        def forward(self, x):
            return self.linears[0](x[..., : self.in0]) + self.linears[1](x[..., self.in0:])

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj_out = SplitInLinear(64, 128, 32); self.other = nn.Linear(32, 32)

    net = nn.Sequential(Block(), Block())
    stats = int8_exec.convert_linears_to_int8(net, device=None, whitelist=lambda n: False, fuse_split=True)
    assert stats["n_int8_linear"] == 6 and stats["n_split_fused"] == 2
    m = net[0].proj_out
    assert isinstance(m, int8_exec.SplitInInt8Linear) and m.in0 == 64 and m.in_features == 192 and m.out_features == 32
    assert isinstance(net[0].other, int8_exec.Int8Linear)


def test_pack_int4_layout():
    """Element 2b in the low nibble of byte b, element 2b+1 in the high nibble, two's complement; out-of-range codes refused."""
    import pytest
    from pyraquant_b200 import ops
    c = torch.tensor([[-8, 7, 0, -1, 3, -4, 1, 2]], dtype=torch.int8)
    p = ops.pack_int4(c)
    assert p.tolist() == [[0x78, 0xF0, 0xC3, 0x21]]
    with pytest.raises(AssertionError):
        ops.pack_int4(torch.tensor([[8, 0]], dtype=torch.int8))
