"""Generates the golden fixtures in this directory by RUNNING the reference's own CPU-runnable code.

    python tests/golden/make_golden.py /path/to/PyraQuant [feather]

Only works where the reference checkout is available (the build container); the fixtures it writes
(small .npz files) are committed and are what the tests read.  Inputs are seeded; bf16 tensors are
stored as their raw 16-bit patterns (numpy has no bfloat16).
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


FEATHER_CASES = [  # (patch_hw, inner box in the patch, mode, power)
    ((12, 12), (2, 10, 2, 10), "cosine", 1.0), ((20, 36), (2, 18, 2, 34), "cosine", 1.0),
    ((11, 19), (3, 11, 3, 16), "cosine", 1.0), ((9, 9), (1, 8, 1, 8), "cosine", 1.0),
    ((26, 14), (5, 21, 0, 9), "cosine", 1.0), ((16, 16), (4, 12, 4, 12), "cosine", 2.0),
    ((16, 16), (4, 12, 4, 12), "smoothstep", 1.0), ((13, 17), (3, 10, 6, 11), "linear", 0.5),
]


def feather_fixture(ref_root: str) -> None:
    """halo_feather_mask (flux/routing.py:34-75) for a few patch geometries, profile shapes and powers, in bf16
    and fp16."""
    sys.path.insert(0, str(Path(ref_root) / "flux"))
    import routing as ref_routing
    save = {"n": np.int64(len(FEATHER_CASES))}
    for i, (hw, inner, mode, power) in enumerate(FEATHER_CASES):
        for tag, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
            m = ref_routing.halo_feather_mask(hw, inner, device=torch.device("cpu"), dtype=dt, mode=mode, power=power)
            save[f"mask{i}_{tag}_bits"] = m.contiguous().view(torch.int16).numpy().copy()
    np.savez(HERE / "feather_masks.npz", **save)
    print("feather_masks.npz written")


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    for p in (ref, ref / "deploy", ref / "flux"):
        sys.path.insert(0, str(p))
    import torch.nn as nn
    import int8_exec as ref_exec                                   # deploy/int8_exec.py
    from pyraquant.quant_unet import _ActFakeQuant
    from pyraquant.quantizers_weight import qdq_weight, nested4_qdq_weight
    from pyraquant.external_quant import ExtActQuant, ExtState
    import routing as ref_routing                                  # flux/routing.py

    g = torch.Generator().manual_seed(1234)

    # ---- 1. Int8Linear.__init__: weight codes / scales / bias / low-rank buffers
    lin = nn.Linear(96, 40, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(40, 96, generator=g) * 0.02)
        lin.weight[3].zero_()                                      # all-zero channel -> clamp_min path
        lin.bias.copy_(torch.randn(40, generator=g) * 0.01)
    lin = lin.to(torch.bfloat16)
    A = (torch.randn(96, 32, generator=g) * 0.02).to(torch.bfloat16)
    B = (torch.randn(32, 40, generator=g) * 0.02).to(torch.bfloat16)
    q = ref_exec.Int8Linear(lin, device=None, lowrank=(A, B))
    np.savez(HERE / "int8linear_ctor.npz", w_bits=bf16_bits(lin.weight.detach()), bias_bits=bf16_bits(lin.bias.detach()),
             weight_int8=q.weight_int8.numpy(), w_scale=q.w_scale.numpy(), bias_f32=q.bias.numpy(),
             lr_A_bits=bf16_bits(q.lr_A), lr_B_bits=bf16_bits(q.lr_B))

    # ---- 2. per-token A8 fake quant (_ActFakeQuant(8)): QDQ output in bf16
    x = torch.randn(37, 96, generator=g)
    x[:, 5] *= 30.0
    x[7].zero_()                                                    # all-zero token
    x = x.to(torch.bfloat16)
    (xq,) = _ActFakeQuant(8)(None, (x,))
    np.savez(HERE / "act_fakequant_a8.npz", x_bits=bf16_bits(x), qdq_bits=bf16_bits(xq))

    # ---- 3. group-32 weight grid: qdq_weight(w, 8, 32) in fp32
    w = torch.randn(24, 128, generator=g) * 0.02
    np.savez(HERE / "qdq_weight_w8g32.npz", w=w.numpy(), qdq=qdq_weight(w, 8, 32).numpy())

    # ---- 4. nested W4 from W8 codes, per-output-channel groups (group_size=None) and group 32
    np.savez(HERE / "nested4.npz", w=w.numpy(), qdq_perchannel=nested4_qdq_weight(w, None).numpy(),
             qdq_g32=nested4_qdq_weight(w, 32).numpy())

    # ---- 5. ExtActQuant dyn_group, group 32, 8 bits signed
    st = ExtState() if callable(ExtState) else None
    hook = ExtActQuant("probe", {"bits": 8, "mode": "dyn_group", "group": 32}, {}, st)
    xg = torch.randn(19, 128, generator=g)
    xg[:, 40] *= 25.0
    np.savez(HERE / "act_dyn_group32.npz", x=xg.numpy(), qdq=hook._qdq_rows(xg.clone()).numpy())

    # ---- 6. gather (build_patch_buckets) and scatter (fuse_patch_predictions) on a 24x24 token canvas
    H = W = 24
    C = 16
    hidden = torch.randn(1, H * W, C, generator=g).to(torch.bfloat16)
    ys, xs = torch.meshgrid(torch.arange(H), torch.arange(W), indexing="ij")
    img_ids = torch.stack([torch.zeros_like(ys), ys, xs], dim=-1).reshape(H * W, 3).float()
    boxes = [(0, 16, 0, 32), (16, 32, 16, 32), (32, 48, 0, 16), (32, 48, 32, 48), (16, 32, 16, 32)]  # latent coords; last = duplicate
    buckets = ref_routing.build_patch_buckets(hidden, img_ids, token_hw=(H, W), route_boxes_unpacked=boxes,
                                              halo_tokens=2, packing_offset_latent=0)
    background = torch.randn(1, H, W, C, generator=g).to(torch.bfloat16)
    outs = []
    save = {"hidden_bits": bf16_bits(hidden), "background_bits": bf16_bits(background),
            "boxes": np.asarray(boxes, dtype=np.int64), "n_buckets": np.int64(len(buckets))}
    for i, b in enumerate(buckets):
        o = (torch.randn(b.hidden_states.shape, generator=g) * 1.5).to(torch.bfloat16)
        outs.append((b, o))
        save[f"bucket{i}_hw"] = np.asarray(b.patch_hw, dtype=np.int64)
        save[f"bucket{i}_hidden_bits"] = bf16_bits(b.hidden_states)
        save[f"bucket{i}_ids"] = b.img_ids.numpy()
        save[f"bucket{i}_out_bits"] = bf16_bits(o)
        save[f"bucket{i}_halo_boxes"] = np.asarray([gm.halo_box for gm in b.geometries], dtype=np.int64)
    fused = ref_routing.fuse_patch_predictions(background, outs, fusion_beta=1.0, feather_mode="cosine", feather_power=1.0)
    save["fused_bits"] = bf16_bits(fused)
    # a second blend with a wider halo and fusion_beta < 1 exercises fractional weights
    buckets3 = ref_routing.build_patch_buckets(hidden, img_ids, token_hw=(H, W), route_boxes_unpacked=boxes[:4],
                                               halo_tokens=3, packing_offset_latent=0)
    outs3 = []
    save["h3_n_buckets"] = np.int64(len(buckets3))
    for i, b in enumerate(buckets3):
        o = (torch.randn(b.hidden_states.shape, generator=g) * 1.5).to(torch.bfloat16)
        outs3.append((b, o))
        save[f"h3_bucket{i}_out_bits"] = bf16_bits(o)
        save[f"h3_bucket{i}_hw"] = np.asarray(b.patch_hw, dtype=np.int64)
    fused3 = ref_routing.fuse_patch_predictions(background, outs3, fusion_beta=0.75, feather_mode="cosine", feather_power=1.0)
    save["h3_fused_bits"] = bf16_bits(fused3)
    np.savez(HERE / "routing_gather_scatter.npz", **save)

    # ---- 7. inner_split_median (flux/run_flux.py): needs the module to import; skipped when its heavy imports are absent
    try:
        import run_flux as ref_run_flux                            # flux/run_flux.py
        sc = torch.rand(8, 8, generator=g)
        sel = (torch.rand(8, 8, generator=g) < 0.3).float()
        hi = ref_run_flux.inner_split_median(sc, sel, 1.0)
        np.savez(HERE / "inner_split_median.npz", scores=sc.numpy(), sel=sel.numpy(), hi=hi.numpy())
    except Exception as e:                                         # noqa: BLE001
        print("inner_split_median fixture skipped:", repr(e))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[2] == "feather":
        feather_fixture(sys.argv[1])                                # only feather_masks.npz
    elif len(sys.argv) == 2:
        main(sys.argv[1])
        feather_fixture(sys.argv[1])
    else:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/PyraQuant [feather]")
