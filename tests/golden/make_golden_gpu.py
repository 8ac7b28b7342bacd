"""Generates forward_reference_gpu.npz by RUNNING the reference's own GPU code (its Triton kernels) on a CUDA
device, and optionally times those kernels on the benchmark's layers.

    python tests/golden/make_golden_gpu.py /path/to/PyraQuant [--bench out.json] [--no-fixture]

The reference's forward (deploy/int8_exec.py:382-393) asserts CUDA tensors, so this is the only way to obtain
a reference-made vector for the ASSEMBLED path (quantise -> INT8 GEMM -> dequantise + low-rank + bias).  Needs a
CUDA GPU, Triton and a checkout of the reference (only deploy/int8_exec.py is imported, unmodified).

Backends.  The reference has two (set_backend, :58-74): "triton" (its fused GEMM kernels, the default) and "cublas"
(its quantisation kernel + torch._int_mm + its dequantisation kernel + an in-place addmm for the low-rank branch,
:246-261, :394-407).  Its fused GEMM kernels were written for Triton 3.2; where the installed Triton refuses them,
the error is recorded in the outputs (`triton_backend_error`) and the run continues on the reference's own "cublas"
backend, still through its unmodified Int8Linear.forward.

Inputs are drawn from seeded CPU generators (`forward_cases()`), so the tests rebuild identical bits without the
reference; the fixture stores a SHA-256 of every input next to the reference's outputs.  To keep the fixture
small, outputs and codes are stored for a sample of rows (first, last and evenly spread) and row scales for all.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
import time
from pathlib import Path

import numpy as np
import torch
import torch.nn as nn

HERE = Path(__file__).resolve().parent

# name, M, K, N, dtype, low-rank branch, sampled rows, seed
FORWARD_CASES = [
    ("flux_lr", 512, 3072, 3072, torch.bfloat16, True, 64, 501),       # rank-32 branch + bias (int8_gemm_lr, :327-336)
    ("selftest", 4352, 3072, 12288, torch.bfloat16, False, 24, 502),    # the self-test's shape and outlier channel (:498-501)
    ("sdxl_fp16", 154, 640, 1280, torch.float16, False, 48, 503),       # fp16 in/out, ragged row count
]


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def sample_rows(M: int, n: int) -> np.ndarray:
    idx = np.unique(np.concatenate([np.arange(min(4, M)), np.arange(max(0, M - 4), M),
                                    np.linspace(0, M - 1, n).round().astype(np.int64)]))
    return idx.astype(np.int64)


def forward_case(name, M, K, N, dtype, lowrank, seed):
    """Seeded inputs of one case, on the CPU: x (one channel scaled by 30, as in the reference's self-test, plus 0.5 %
    of the channels scaled by 20), Linear weight and bias, rank-32 factors."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 2
    x[:, 5] *= 30.0
    x[:, torch.randperm(K, generator=g)[: max(1, K // 200)]] *= 20.0
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    out = {"x": x.to(dtype), "w": w.to(dtype), "b": b.to(dtype)}
    if lowrank:
        out["A"] = (torch.randn(K, 32, generator=g) * 0.02).to(dtype)
        out["B"] = (torch.randn(32, N, generator=g) * 0.02).to(dtype)
    return out


def pick_backend(ref_exec) -> dict:
    """Runs one small forward with a rank-32 branch on the reference's default backend; falls back to its "cublas"
    backend when the fused Triton GEMM does not compile or run.  Returns {"backend", "triton_backend_error"}."""
    dev = torch.device("cuda", 0)
    lin = nn.Linear(256, 256, bias=True).to(torch.bfloat16)
    A = torch.zeros(256, 32, dtype=torch.bfloat16); B = torch.zeros(32, 256, dtype=torch.bfloat16)
    x = torch.randn(64, 256).to(torch.bfloat16).to(dev)
    info = {"backend": ref_exec.get_backend(), "triton_backend_error": ""}
    try:
        ref_exec.Int8Linear(lin, device=dev, lowrank=(A, B))(x)
        ref_exec.Int8Linear(lin, device=dev)(x)
        torch.cuda.synchronize()
    except Exception as e:                                          # noqa: BLE001 - whatever the compiler raises
        info["triton_backend_error"] = f"{type(e).__name__}: {str(e).strip().splitlines()[-1] if str(e).strip() else ''}"[:400]
        cause = e.__cause__
        if cause is not None:
            info["triton_backend_error"] += f" (caused by {type(cause).__name__} in tl.dot: {cause})"[:300]
        ref_exec.set_backend("cublas")
        info["backend"] = ref_exec.get_backend()
        ref_exec.Int8Linear(lin, device=dev, lowrank=(A, B))(x)
        torch.cuda.synchronize()
    print("[golden-gpu] reference backend:", info, flush=True)
    return info


def make_fixture(ref_exec, info: dict) -> None:
    dev = torch.device("cuda", 0)
    save = {"reference_backend": np.array(info["backend"]), "triton_backend_error": np.array(info["triton_backend_error"])}
    for name, M, K, N, dtype, lowrank, n_rows, seed in FORWARD_CASES:
        c = forward_case(name, M, K, N, dtype, lowrank, seed)
        lin = nn.Linear(K, N, bias=True).to(dtype)
        with torch.no_grad():
            lin.weight.copy_(c["w"]); lin.bias.copy_(c["b"])
        q = ref_exec.Int8Linear(lin, device=dev, lowrank=(c["A"], c["B"]) if lowrank else None)
        xd = c["x"].to(dev)
        y = q(xd)                                                     # the reference's forward, unmodified
        xq, sx = ref_exec.quant_rows(xd)                              # its quantisation kernel
        torch.cuda.synchronize()
        rows = sample_rows(M, n_rows)
        r = torch.from_numpy(rows).to(dev)
        save[f"{name}_rows"] = rows
        save[f"{name}_y_bits"] = y[r].contiguous().view(torch.int16).cpu().numpy()
        save[f"{name}_codes"] = xq[r].cpu().numpy()
        save[f"{name}_scales"] = sx.cpu().numpy()
        save[f"{name}_w_scale"] = q.w_scale.cpu().numpy()
        save[f"{name}_w_codes_rowsum"] = q.weight_int8.sum(1, dtype=torch.int64).cpu().numpy()
        for k, v in c.items():
            save[f"{name}_sha_{k}"] = np.array(sha(v))
        print(f"[golden-gpu] {name}: M={M} K={K} N={N} {dtype} lowrank={lowrank} rows={len(rows)}", flush=True)
    save["torch_version"] = np.array(torch.__version__)
    save["gpu"] = np.array(torch.cuda.get_device_name())
    np.savez_compressed(HERE / "forward_reference_gpu.npz", **save)
    print("[golden-gpu] wrote", HERE / "forward_reference_gpu.npz")


def bench_reference(ref_exec, info: dict, out_path: str, rows: int, iters: int) -> None:
    """CUDA-event times of the reference's quantisation kernel and of its whole Int8Linear.forward (rank 32 + bias) on
    the two layers of the FLUX 4K single-block set, on the backend `pick_backend` chose; with the "triton" backend
    also of int8_gemm_lr alone (its first call per shape runs Triton's autotuner)."""
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(7)
    res = {"gpu": torch.cuda.get_device_name(), "rows": rows, "iters": iters, "layers": [], **info}

    def timed(fn):
        fn(); fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); a.record()
        for _ in range(iters):
            fn()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e3

    for K, N in ((3072, 21504), (15360, 3072)):
        lin = nn.Linear(K, N, bias=True, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(N, K, generator=g, device=dev) * 0.02)
        A = (torch.randn(K, 32, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        B = (torch.randn(32, N, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        q = ref_exec.Int8Linear(lin, device=dev, lowrank=(A, B))
        x = torch.randn(rows, K, generator=g, device=dev)
        x[:, torch.randperm(K, generator=g, device=dev)[: max(1, round(K * 0.005))]] *= 20.0
        x = x.to(torch.bfloat16)
        t0 = time.time()
        q(x)
        torch.cuda.synchronize()
        item = {"layer": f"{K}->{N}", "first_call_s": time.time() - t0,
                "quant_us": timed(lambda: ref_exec.quant_rows(x)),
                "forward_us": timed(lambda: q(x))}
        item["forward_tops"] = 2.0 * rows * K * N / item["forward_us"] / 1e6
        xq, sx = ref_exec.quant_rows(x)
        if info["backend"] == "triton":
            t = (x @ q.lr_A).contiguous()
            item["gemm_lr_us"] = timed(lambda: ref_exec.int8_gemm_lr(xq, sx, q.weight_int8, q.w_scale, q.bias, t, q.lr_B,
                                                                     torch.bfloat16))
            item["gemm_lr_tops"] = 2.0 * rows * K * N / item["gemm_lr_us"] / 1e6
            del t
        else:
            wt = q.weight_int8.t()
            acc = torch._int_mm(xq, wt)
            item["int_mm_us"] = timed(lambda: torch._int_mm(xq, wt))
            item["int_mm_tops"] = 2.0 * rows * K * N / item["int_mm_us"] / 1e6
            item["dequant_epilogue_us"] = timed(lambda: ref_exec.dequant_epilogue(acc, sx, q.w_scale, q.bias, torch.bfloat16))
            del acc
        res["layers"].append(item)
        print("[golden-gpu] bench", json.dumps(item), flush=True)
        del lin, q, x, xq, sx
        torch.cuda.empty_cache()
    Path(out_path).write_text(json.dumps(res, indent=1))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("ref_root")
    ap.add_argument("--bench", default=None, help="also time the reference's kernels; JSON written here")
    ap.add_argument("--rows", type=int, default=65536 + 512)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-fixture", action="store_true")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.ref_root) / "deploy"))
    import int8_exec as ref_exec                                      # the reference's module, as it is
    assert Path(ref_exec.__file__).resolve().parent == (Path(a.ref_root) / "deploy").resolve(), ref_exec.__file__
    info = pick_backend(ref_exec)
    if not a.no_fixture:
        make_fixture(ref_exec, info)
    if a.bench:
        bench_reference(ref_exec, info, a.bench, a.rows, a.iters)
