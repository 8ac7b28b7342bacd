"""The assembled forward (quantise -> INT8 GEMM -> dequantise + low-rank + bias) against vectors produced by the
reference's own GPU code: tests/golden/forward_reference_gpu.npz holds what the unmodified reference module
(deploy/int8_exec.py: Int8Linear.forward :382-393, quant_rows :216-230) returned on a B200 for the seeded inputs of
tests/golden/make_golden_gpu.py.  The CPU oracle is checked here without a GPU; the CUDA path with one.

Bars: activation codes may differ from the reference's in at most 1e-4 of the elements (the reference's own bar for
its kernel against torch, :534: its kernel forms the scale with an approximate division, so a value that sits on a
rounding tie can fall the other way), scales to 1e-6 relative.  Outputs: relative L2 below 3e-3 over all sampled rows,
and max-rel-err 1e-2 (|y - ref| / max(|ref|, 1e-3 max|ref|)) on every sampled row whose codes equal the reference's
(one differing code moves a whole output row by about s_row * |w| * s_col, which is the quantisation step, not an
error of the forward).  The fixture records which of the reference's two backends produced it
(`reference_backend`).  Its "cublas" backend adds the low-rank branch with a separate in-place addmm AFTER the GEMM
output was rounded to 16 bits (:394-407), so there the reference itself carries one extra rounding of the
intermediate: the bar for that case allows one unit in the last place of the intermediate on top.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
from make_golden_gpu import FORWARD_CASES, forward_case, sha   # noqa: E402

TOL = 1e-2
CASE_IDS = [c[0] for c in FORWARD_CASES]


def output_error(y, y_ref, c, rows, fix, same_codes):
    """max over the elements of rows with identical codes of |y - ref| / max(|ref|, 1e-3 max|ref|), after the allowance
    for the reference's own extra rounding where its unfused low-rank path produced the vector."""
    assert int(same_codes.sum()) >= len(rows) // 2, "too few sampled rows with codes identical to the reference's"
    err = (y.double() - y_ref.double()).abs()
    if "A" in c and str(fix["reference_backend"]) == "cublas":
        # the unfused branch: t = x @ A rounded to 16 bits by a library GEMM (summation order may move an element of t by
        # one unit in the last place), the GEMM output rounded to 16 bits, and their sum t @ B + y rounded again.  Where
        # the two terms cancel, the result is small but carries those roundings of the large terms.
        xs = c["x"][rows]
        t = (xs.float() @ c["A"].float()).to(c["A"].dtype).double()
        ulp = 2.0 ** -8 if y_ref.dtype == torch.bfloat16 else 2.0 ** -11
        err = (err - ulp * (2.0 * y_ref.double().abs() + 2.0 * t.abs() @ c["B"].double().abs())).clamp_min(0.0)
    denom = torch.maximum(y_ref.double().abs(), 1e-3 * y_ref.double().abs().max())
    return float((err / denom)[same_codes].max())


def load_case(fix, case):
    name, M, K, N, dtype, lowrank, _n, seed = case
    c = forward_case(name, M, K, N, dtype, lowrank, seed)
    for k, v in c.items():
        assert sha(v) == str(fix[f"{name}_sha_{k}"]), f"input {k} of case {name} differs from the one the fixture was made with"
    rows = torch.from_numpy(fix[f"{name}_rows"]).long()
    y_ref = torch.from_numpy(fix[f"{name}_y_bits"]).view(dtype)
    return c, rows, y_ref, torch.from_numpy(fix[f"{name}_codes"]), torch.from_numpy(fix[f"{name}_scales"])


@pytest.fixture(scope="module")
def fix():
    return np.load(GOLDEN / "forward_reference_gpu.npz")


@pytest.mark.parametrize("case", FORWARD_CASES, ids=CASE_IDS)
def test_oracle_forward_matches_reference_gpu_vector(fix, case):
    c, rows, y_ref, codes_ref, scales_ref = load_case(fix, case)
    xs = c["x"][rows]
    # weight grid as the reference's constructor made it ON THE GPU: scales bit for bit, codes through their row sums
    wq, ws = oracle.quant_weight(c["w"], where="cuda")
    assert torch.equal(ws, torch.from_numpy(fix[f"{case[0]}_w_scale"]))
    assert torch.equal(wq.sum(1, dtype=torch.int64), torch.from_numpy(fix[f"{case[0]}_w_codes_rowsum"]))
    xq, sx = oracle.quant_rows(xs)
    assert float((xq != codes_ref).float().mean()) <= 1e-4
    assert float(((sx - scales_ref[rows]).abs() / scales_ref[rows]).max()) <= 1e-6
    y = oracle.int8_linear_forward(xs, wq, ws, c["b"].float(), c.get("A"), c.get("B"))
    assert output_error(y, y_ref, c, rows, fix, (xq == codes_ref).all(1)) <= TOL
    assert float((y.float() - y_ref.float()).norm() / y_ref.float().norm()) < 3e-3


@pytest.mark.gpu
@pytest.mark.parametrize("case", FORWARD_CASES, ids=CASE_IDS)
def test_cuda_forward_matches_reference_gpu_vector(cuda_dev, fix, case):
    from pyraquant_b200 import int8_exec, ops
    name, M, K, N, dtype, lowrank, _n, _seed = case
    c, rows, y_ref, codes_ref, scales_ref = load_case(fix, case)
    lin = nn.Linear(K, N, bias=True).to(dtype)
    with torch.no_grad():
        lin.weight.copy_(c["w"]); lin.bias.copy_(c["b"])
    layer = int8_exec.Int8Linear(lin, device=cuda_dev, lowrank=(c["A"], c["B"]) if lowrank else None)
    # converted on the GPU like the reference's layer: identical weight grid
    assert torch.equal(layer.w_scale.cpu(), torch.from_numpy(fix[f"{name}_w_scale"]))
    assert torch.equal(layer.weight_int8.sum(1, dtype=torch.int64).cpu(), torch.from_numpy(fix[f"{name}_w_codes_rowsum"]))
    x = c["x"].to(cuda_dev)
    y = layer(x)
    xq, sx = int8_exec.quant_rows(x)
    ops.check_device_status(cuda_dev)
    r = rows.to(cuda_dev)
    assert float((xq[r].cpu() != codes_ref).float().mean()) <= 1e-4
    assert float(((sx.cpu() - scales_ref).abs() / scales_ref).max()) <= 1e-6
    assert output_error(y[r].cpu(), y_ref, c, rows, fix, (xq[r].cpu() == codes_ref).all(1)) <= TOL
    assert float((y[r].cpu().float() - y_ref.float()).norm() / y_ref.float().norm()) < 3e-3
