"""Benchmark of the Int8Linear hot path on the FLUX 4K single-block linear set.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--allgather]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one "step"): the two Int8Linear layers of a FLUX single-stream block at the 4K stage,
M = 65536 + 512 token rows: fused QKV+MLP-in 3072 -> 21504 and proj-out 15360 -> 3072, each with a
rank-32 low-rank branch and bias, bf16 in/out.  Rows are sharded ceil(M / N) per GPU with replicated
weights (strong scaling: the row count is fixed); the optional output all-gather is off unless
--allgather.  Inputs are synthetic: X ~ N(0,1) with 0.5 % of the channels scaled x20, W ~ N(0,0.02),
low-rank factors ~ N(0,0.02), bias ~ N(0,0.01), seeded.

Printed (rank 0, one JSON line): effective TOPS = 2*M*N*K summed over both layers / step time, with the
step = down-projection + per-token quantisation + fused GEMM of both layers (three kernels of this library per layer); `roofline` for the GEMM
kernel (CUDA-event time per launch), `e2e` through host buffers, `cpu_baseline` (the CPU oracle on a
bounded row sample), clocks sampled during the timed region.

`roofline.peak` is the INT8 tensor-pipe ceiling measured in the same run (tcgen05.mma kind::i8 issued back to back on
pseudo-random operand bytes that stay in shared memory, sustained for seconds: what the GPU's tensor cores deliver under
its power cap before any operand has to move); the datasheet figure and the 2 x bf16 proxy are secondary keys.
`gpu_baseline` (one GPU, when the git-ignored baseline/_ref copy of the reference's deploy/int8_exec.py is present) is
the reference's own unmodified Int8Linear.forward on the same GPU, same shapes: its Triton GEMM kernels where the
installed Triton compiles them, else its "cublas" backend.

--impl reference times the reference's algorithm on the host CPU cores (the CPU restatement in
oracle/; the reference's own forward cannot run without CUDA + Triton kernels).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

M_TOTAL = 65536 + 512
LAYERS = [  # (name, K, N)
    ("qkv_mlp_in", 3072, 21504),
    ("proj_out", 15360, 3072),
]
RANK = 32
METRIC = "int8linear_effective_tops_flux4k"
DATASHEET_INT8_TOPS = 4500.0   # NVIDIA B200 dense INT8 tensor peak per GPU (spec sheet figure)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16": d.get("bf16_tflops"), "bf16_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def step_ops(rows: int) -> float:
    return sum(2.0 * rows * K * N for _n, K, N in LAYERS)


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """nvidia-smi sampled every 50 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); smax.append(float(r[1])); pw.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # the samples under load are the ones that matter: keep those above 60 % of the highest power seen
        if pw:
            thr = 0.6 * max(pw)
            sm_load = [s for s, p in zip(sm, pw) if p >= thr] or sm
        else:
            sm_load = sm
        return {"sm_mhz": statistics.median(sm_load) if sm_load else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_reference_step(layers_cpu, rows: int):
    """One pass of the CPU restatement over `rows` rows of every layer; returns seconds."""
    from oracle import oracle
    t0 = time.perf_counter()
    for L in layers_cpu:
        oracle.int8_linear_forward(L["x"][:rows], L["wq"], L["ws"], L["bias"], L["lr_A"], L["lr_B"])
    return time.perf_counter() - t0


def make_cpu_layers(rows: int):
    from oracle import oracle
    out = []
    for i, (_name, K, N) in enumerate(LAYERS):
        L = oracle.make_layer(2 + i, rows, K, N)
        wq, ws = oracle.quant_weight(L["w"])
        out.append({"x": L["x"], "wq": wq, "ws": ws, "bias": L["bias"], "lr_A": L["lr_A"], "lr_B": L["lr_B"]})
    return out


def measure_issue_ceiling(dev, sustain_s: float = 3.0):
    """Measured ceiling of the INT8 tensor pipe on this GPU: one CTA per SM issues tcgen05.mma kind::i8 128x256x32 back
    to back on operands that stay in shared memory (no global traffic at all).  Reported: a short burst on an idle GPU,
    and the rate over the last quarter of `sustain_s` seconds of back-to-back launches, once with constant operands
    (the pipe's rate at the clock the GPU can hold with little switching activity) and once with pseudo-random operands
    (tensor-core power is data dependent: with random bytes the power cap alone pulls the clock down)."""
    import torch
    from pyraquant_b200 import _lib, ops
    lib = _lib.load()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    cycles = torch.zeros(sms, dtype=torch.int64, device=dev)
    ws = ops.status_word(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    ops_per_iter = 4 * 2.0 * 128 * 256 * 32 * sms

    def launch(iters):
        rc = lib.pq_i8_mma_issue_loop(sms, iters, cycles.data_ptr(), ws.data_ptr(), ws.numel() * 4, stream)
        _lib.check(rc, "pq_i8_mma_issue_loop")

    def sustained(sign):
        it_long = 200000
        t_end = time.time() + sustain_s
        marks = []
        while time.time() < t_end:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); launch(sign * it_long); b.record()
            marks.append((a, b))
            torch.cuda.synchronize(dev)
        tail = marks[-max(1, len(marks) // 4):]
        return ops_per_iter * it_long * len(tail) / (sum(a.elapsed_time(b) for a, b in tail) * 1e-3) / 1e12

    launch(2000)
    torch.cuda.synchronize(dev)
    time.sleep(0.5)                                    # let the clocks recover from whatever ran before
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    it_burst = 20000
    e0.record(); launch(it_burst); e1.record()
    torch.cuda.synchronize(dev)
    burst = ops_per_iter * it_burst / (e0.elapsed_time(e1) * 1e-3) / 1e12
    cyc_per_mma = float(cycles.double().mean().item()) / (4.0 * it_burst)
    s_const = sustained(1)
    s_rand = sustained(-1)                             # negative iteration count = pseudo-random operand bytes
    ops.check_device_status(dev)
    return {"burst_tops": burst, "sustained_tops": s_const, "sustained_random_operands_tops": s_rand,
            "cycles_per_mma_128x256x32": cyc_per_mma, "sustain_seconds": sustain_s, "ctas": sms}


def run_gpu_baseline(dev, xs, iters: int):
    """The reference's own GPU path on this GPU: unmodified deploy/int8_exec.py (staged under baseline/_ref by the build
    step), Int8Linear.forward with rank-32 branch and bias on the benchmark's two layers and activations.  Returns None
    when the copy is absent, {"unavailable": why} when it cannot run."""
    ref_dir = ROOT / "baseline" / "_ref" / "deploy"
    if not (ref_dir / "int8_exec.py").is_file():
        return None
    import importlib.util
    import torch.nn as nn
    try:
        spec = importlib.util.spec_from_file_location("pyraquant_reference_int8_exec", ref_dir / "int8_exec.py")
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
    except Exception as e:                                          # noqa: BLE001
        return {"unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}
    g = torch.Generator(device=dev).manual_seed(7)
    info = {"backend": ref.get_backend(), "triton_backend_error": None}
    layers = []
    try:
        probe = nn.Linear(256, 256, bias=True, device=dev, dtype=torch.bfloat16)
        pa = torch.zeros(256, 32, device=dev, dtype=torch.bfloat16); pb = torch.zeros(32, 256, device=dev, dtype=torch.bfloat16)
        px = torch.randn(64, 256, device=dev).to(torch.bfloat16)
        try:
            ref.Int8Linear(probe, device=dev, lowrank=(pa, pb))(px)
            torch.cuda.synchronize(dev)
        except Exception as e:                                      # noqa: BLE001  (Triton compile errors of any kind)
            info["triton_backend_error"] = (f"{type(e).__name__} at tl.dot of the fused GEMM kernels "
                                            f"({type(e.__cause__).__name__ if e.__cause__ else 'no cause'})")
            ref.set_backend("cublas")
            info["backend"] = ref.get_backend()
            ref.Int8Linear(probe, device=dev, lowrank=(pa, pb))(px)
            torch.cuda.synchronize(dev)
        total_ms = 0.0
        for (name, K, N), x in zip(LAYERS, xs):
            lin = nn.Linear(K, N, bias=True, device=dev, dtype=torch.bfloat16)
            with torch.no_grad():
                lin.weight.copy_(torch.randn(N, K, generator=g, device=dev) * 0.02)
            A = (torch.randn(K, RANK, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            B = (torch.randn(RANK, N, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            q = ref.Int8Linear(lin, device=dev, lowrank=(A, B))
            del lin
            for _ in range(2):
                q(x)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev); e0.record()
            for _ in range(iters):
                q(x)
            e1.record(); torch.cuda.synchronize(dev)
            ms = e0.elapsed_time(e1) / iters
            total_ms += ms
            layers.append({"layer": name, "forward_us": ms * 1e3, "forward_tops": 2.0 * x.shape[0] * K * N / (ms * 1e-3) / 1e12})
            del q, A, B
            torch.cuda.empty_cache()
        rows = xs[0].shape[0]
        return {"value": step_ops(rows) / (total_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": total_ms,
                "what": "the reference's unmodified Int8Linear.forward (deploy/int8_exec.py:382-408) on this GPU, same layers and "
                        "activations, rank-32 branch + bias, CUDA events", "layers": layers, **info}
    except Exception as e:                                          # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"[:300], **info}


def run_cpu_baseline(sample_rows: int, reps: int):
    torch.set_num_threads(os.cpu_count() or 1)
    layers = make_cpu_layers(sample_rows)
    cpu_reference_step(layers, min(sample_rows, 64))          # warm-up of the thread pool
    times = [cpu_reference_step(layers, sample_rows) for _ in range(reps)]
    t = statistics.median(times)
    return {"value": step_ops(sample_rows) / t / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_rows} of {M_TOTAL} rows of both layers, median of {reps} passes, "
                      f"{t * 1e3:.0f} ms per pass; torch CPU restatement (torch._int_mm + fp32 epilogue)"}, t


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = args.cpu_sample_rows
    torch.set_num_threads(os.cpu_count() or 1)
    layers = make_cpu_layers(rows)
    for _ in range(max(1, args.warmup)):
        cpu_reference_step(layers, min(rows, 256))
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(layers, rows)
    dt = (time.perf_counter() - t0) / args.steps
    val = step_ops(rows) / dt / 1e12
    sample = (f"each step = {rows} of {M_TOTAL} rows of both layers on the host CPU (the forward needs CUDA in the "
              f"reference, so its algorithm runs as the torch CPU restatement in oracle/)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "FLUX 4K single-block linear set (configs[2])", "rows_total": M_TOTAL, "rows_per_step": rows,
                   "layers": [f"{K}->{N}" for _n, K, N in LAYERS], "lowrank": RANK},
        "cpu_baseline": {"value": val, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------ GPU arm
def main_ours(args):
    import torch.distributed as dist
    import torch.nn as nn
    from pyraquant_b200 import int8_exec, ops, parallel
    from pyraquant_b200.host_pipeline import HostRowPipeline

    rank, local, world = parallel.init_from_env("cuda")
    dev = torch.device("cuda", local)
    a, b = parallel.shard_rows(M_TOTAL, world, rank)
    rows = b - a
    peaks = measured_peaks()

    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    gw = torch.Generator(device=dev).manual_seed(7)          # weights identical on every rank (replicated)
    mods, xs = [], []
    for _name, K, N in LAYERS:
        lin = nn.Linear(K, N, bias=True, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(N, K, generator=gw, device=dev) * 0.02)
            lin.bias.copy_(torch.randn(N, generator=gw, device=dev) * 0.01)
        A = (torch.randn(K, RANK, generator=gw, device=dev) * 0.02).to(torch.bfloat16)
        B = (torch.randn(RANK, N, generator=gw, device=dev) * 0.02).to(torch.bfloat16)
        mods.append(int8_exec.Int8Linear(lin, device=dev, lowrank=(A, B)))
        del lin
        x = torch.randn(rows, K, generator=g, device=dev, dtype=torch.float32)
        ch = torch.randperm(K, generator=gw, device=dev)[: max(1, round(K * 0.005))]
        x[:, ch] *= 20.0
        xs.append(x.to(torch.bfloat16))
        del x
    torch.cuda.empty_cache()

    def step():
        outs = [m(x) for m, x in zip(mods, xs)]
        if args.allgather and world > 1:
            outs = [parallel.all_gather_rows(o, M_TOTAL) for o in outs]
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    ops.check_device_status(dev)

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    t = torch.tensor([ms_total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps

    # ---- the optional output all-gather, measured next to the figure without it (north star: "optional NCCL NVLink
    # all-gather of outputs"): once as a plain gather after each layer, once hidden behind the computation
    gather = None
    if world > 1 and not args.no_gather:
        from pyraquant_b200 import _lib

        def timed_steps(fn, n):
            fn(); fn()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(n):
                fn()
            a1.record()
            barrier()
            tt = torch.tensor([a0.elapsed_time(a1) / n], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())

        n_g = max(3, min(args.steps, 10))
        seq_ms = timed_steps(lambda: [parallel.all_gather_rows(m(x), M_TOTAL) for m, x in zip(mods, xs)], n_g)
        seq_out = [parallel.all_gather_rows(m(x), M_TOTAL) for m, x in zip(mods, xs)]
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        classes = {"push": parallel.PeerPushGather, "pushcopy": parallel.PeerPushGather, "nccl": parallel.OverlappedRowGather, "store": parallel.PeerStoreGather}
        # candidates (mode, chunks per rank): more chunks start the transfers earlier but cost smaller launches and more
        # copies in flight (measured: two chunks win on 2 GPUs, one chunk -- only the next layer computes behind the
        # transfers -- on 8); the store mode needs no chunks: tiles leave from the GEMM epilogue as they are finished
        if args.gather_mode == "auto":
            cands = [("store", 1), ("push", 1), ("push", 2), ("push", 4)] + ([("pushcopy", 1), ("pushcopy", 2)] if args.gather_try_copy else [])
        elif args.gather_mode == "store":
            cands = [("store", max(1, args.gather_chunks))]
        else:
            cands = [(args.gather_mode, ch) for ch in ([args.gather_chunks] if args.gather_chunks > 0 else [1, 2])]
        best = None
        tried = []
        for mode, chunks in cands:
            c = parallel.cyclic_block_rows(M_TOTAL, world, chunks)
            kw = {"direct": False} if mode == "pushcopy" else {}
            ogs = [classes[mode](M_TOTAL, N, torch.bfloat16, dev, chunks=chunks, **kw) for _n, _K, N in LAYERS]
            xl = []
            for x in xs:                               # this rank's rows, block after block (synthetic rows: any will do)
                xp = x.new_zeros((chunks * c, x.shape[1]))
                xp[: min(x.shape[0], chunks * c)] = x[: chunks * c]
                xl.append(xp)

            def gather_step():
                for og, m, x in zip(ogs, mods, xl):            # the next layer computes behind the last transfers of this one
                    og.run(m, x, local=True, wait=False)
                for og in ogs:
                    og.finish()
            for spare in ([args.gather_sms] if args.gather_sms >= 0 else ([0, 8, 16] if mode == "nccl" else [0])):
                # NCCL's copy kernels need SMs, which the persistent GEMM otherwise holds for the length of a chunk
                _lib.set_option("gemm_max_ctas", sms - spare if spare > 0 else 0)
                ms = timed_steps(gather_step, n_g)
                tried.append({"mode": mode, "chunks": chunks, "spare_sms": spare, "ms_per_step": ms})
                if best is None or ms < best[0]:
                    best = (ms, spare, chunks, mode)
            _lib.set_option("gemm_max_ctas", 0)
            if chunks == 1:
                # with one block per rank the row layout is the sequential gather's: the results must be the same tensors
                gather_step()
                barrier()
                for og, ref in zip(ogs, seq_out):
                    assert torch.equal(og.full[:M_TOTAL], ref), f"gathered output differs from the sequential all-gather ({mode})"
            del ogs, xl
            torch.cuda.empty_cache()
        del seq_out
        chunks, mode = best[2], best[3]
        recv = (world - 1) / world * sum(M_TOTAL * N * 2.0 for _n, _K, N in LAYERS)
        how = {"pushcopy": "as push, through a staging tensor",
               "push": f"rows dealt out block-cyclically in {chunks} chunks per rank, chunk i pushed into every peer's output buffer by "
                       f"device-to-device copies (copy engines over NVLink, symmetric-memory buffers) while the next chunk or layer "
                       f"computes; two one-element all-reduces order the step",
               "store": "the GEMM epilogue stores every output tile into this GPU's and every peer's output buffer (plain vector stores to "
                        "peer memory, symmetric-memory buffers): tiles cross NVLink while the tensor cores work on the next ones; two "
                        "one-element all-reduces order the step",
               "nccl": f"rows dealt out block-cyclically in {chunks} chunks per rank, chunk i gathered (NCCL, asynchronous) while chunk "
                       f"i+1 computes, {best[1]} SMs left free for NCCL's kernels"}[mode]
        gather = {"ms_per_step": best[0], "tops": step_ops(M_TOTAL) / (best[0] * 1e-3) / 1e12,
                  "mode": f"{mode}: {how}", "tried": tried,
                  "bytes_recv_per_gpu": recv, "gbps": recv / (best[0] * 1e-3) / 1e9,
                  "sequential_ms_per_step": seq_ms, "sequential_tops": step_ops(M_TOTAL) / (seq_ms * 1e-3) / 1e12,
                  "compute_only_ms_per_step": ms_step,
                  "bound_ms": max(ms_step, recv / 0.9e12 * 1e3)}

    # ---- per-kernel device times (CUDA events on the launching stream): quantisation and GEMM of each layer
    def time_ms(fn, iters):
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); e0.record()
        for _ in range(iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    # Instrumented steps: the step's own kernel sequence (down-projection, quantisation, GEMM per layer, as
    # Int8Linear.forward launches them), every launch bracketed by CUDA events on the launching stream.  The GEMM's time
    # for the roofline is taken here, inside a running step, where the memory-bound kernels between the GEMMs give power
    # budget back; the same launch repeated back to back for seconds settles lower (kernels[].gemm_back_to_back_us).
    n_inst = max(3, args.steps)
    inst = [[] for _ in LAYERS]

    def instrumented_step(keep):
        for li, (m, x) in enumerate(zip(mods, xs)):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
            t_lr = m._down(x)
            ev[1].record()
            xq, sx = int8_exec.quant_rows(x)
            ev[2].record()
            int8_exec.int8_gemm_lr(xq, sx, m.weight_int8, m.w_scale, m.bias, t_lr, m.lr_B, torch.bfloat16, m._lr_Bt())
            ev[3].record()
            if keep:
                inst[li].append(ev)
    instrumented_step(False); instrumented_step(False)
    torch.cuda.synchronize()
    for _ in range(n_inst):
        instrumented_step(True)
    torch.cuda.synchronize()

    kern = []
    gemm_ms_sum = 0.0
    for li, ((name, K, N), m, x) in enumerate(zip(LAYERS, mods, xs)):
        d_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in inst[li])
        q_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in inst[li])
        g_ms = statistics.mean(e[2].elapsed_time(e[3]) for e in inst[li])
        t_lr = m._down(x)
        xq, sx = int8_exec.quant_rows(x)
        gb_ms = time_ms(lambda: int8_exec.int8_gemm_lr(xq, sx, m.weight_int8, m.w_scale, m.bias, t_lr, m.lr_B,
                                                       torch.bfloat16), args.steps)
        # the same launch on codes uniform in [-127, 127]: the workload's own codes are small (the x20 outlier channels
        # set the row scale, ordinary channels land within a few units of zero), and tensor-core power follows the data
        xq_full = torch.randint(-127, 128, xq.shape, generator=g, device=dev, dtype=torch.int8)
        gf_ms = time_ms(lambda: int8_exec.int8_gemm_lr(xq_full, sx, m.weight_int8, m.w_scale, m.bias, t_lr, m.lr_B,
                                                       torch.bfloat16), args.steps)
        del xq_full
        gemm_ms_sum += g_ms
        kern.append({"layer": name, "rows": rows, "K": K, "N": N, "gemm_us": g_ms * 1e3,
                     "gemm_tops": 2.0 * rows * K * N / (g_ms * 1e-3) / 1e12,
                     "gemm_back_to_back_us": gb_ms * 1e3,
                     "gemm_back_to_back_tops": 2.0 * rows * K * N / (gb_ms * 1e-3) / 1e12,
                     "gemm_full_range_codes_us": gf_ms * 1e3,
                     "gemm_full_range_codes_tops": 2.0 * rows * K * N / (gf_ms * 1e-3) / 1e12,
                     "mean_abs_code": float(xq.float().abs().mean().item()),
                     "quant_us": q_ms * 1e3, "quant_gbs": (3.0 * rows * K + 4 * rows) / (q_ms * 1e-3) / 1e9,
                     "lowrank_down_us": d_ms * 1e3})
        del xq, sx, t_lr
    del inst
    clocks = sampler.stop() if sampler else None
    ops.check_device_status(dev)

    # ---- end to end through host buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        # about eight chunks per rank so that the three pipeline stages overlap at every GPU count
        chunk = min(8192, max(1024, ((rows + 7) // 8 + 255) // 256 * 256))
        pipes = [HostRowPipeline(m, K, torch.bfloat16, dev, chunk) for (_n, K, _N), m in zip(LAYERS, mods)]
        hx = [torch.empty((rows, K), dtype=torch.bfloat16).pin_memory() for _n, K, _N in LAYERS]
        hy = [torch.empty((rows, N), dtype=torch.bfloat16).pin_memory() for _n, _K, N in LAYERS]
        for h, x in zip(hx, xs):
            h.copy_(x)
        def e2e_step():
            # both layers' pipelines are enqueued before either is awaited: the 15360->3072 layer is read-heavy, the
            # 3072->21504 layer write-heavy, so their host copies use the two PCIe directions at the same time
            for pipe, h_in, h_out in zip(pipes, hx, hy):
                pipe.start(h_in, h_out)
            for pipe in pipes:
                pipe.finish()
        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(1, min(args.steps, 3))
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1) / n_e2e], device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        # copy-only leg: the same pinned buffers, chunks and streams with the kernels left out (each chunk "computes" by
        # handing back a resident device buffer): what host<->device copies alone cost on this box at this GPU count
        ybufs = [torch.empty((chunk, N), dtype=torch.bfloat16, device=dev) for _n, _K, N in LAYERS]
        copy_pipes = [HostRowPipeline((lambda buf, yb=yb: yb[: buf.shape[0]]), K, torch.bfloat16, dev, chunk)
                      for (_n, K, _N), yb in zip(LAYERS, ybufs)]
        def copy_step():
            for pipe, h_in, h_out in zip(copy_pipes, hx, hy):
                pipe.start(h_in, h_out)
            for pipe in copy_pipes:
                pipe.finish()
        copy_step()
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(n_e2e):
            copy_step()
        c1.record()
        barrier()
        tc = torch.tensor([c0.elapsed_time(c1) / n_e2e], device=dev)
        if world > 1:
            dist.all_reduce(tc, op=dist.ReduceOp.MAX)
        del copy_pipes, ybufs
        e2e = {"value": step_ops(M_TOTAL) / (float(te.item()) * 1e-3) / 1e12, "unit": "TOPS",
               "h2d_bytes_per_step": int(sum(rows * K * 2 for _n, K, _N in LAYERS)),
               "d2h_bytes_per_step": int(sum(rows * N * 2 for _n, _K, N in LAYERS)),
               "ms_per_step": float(te.item()), "chunk_rows": chunk, "steps": n_e2e,
               "copy_only_ms_per_step": float(tc.item()),
               "copy_only_gbs_per_gpu": (sum(rows * K * 2 for _n, K, _N in LAYERS) + sum(rows * N * 2 for _n, _K, N in LAYERS))
                                        / (float(tc.item()) * 1e-3) / 1e9,
               "frac_of_copy_ceiling": float(tc.item()) / float(te.item())}
        del hx, hy, pipes

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    value = step_ops(M_TOTAL) / (ms_step * 1e-3) / 1e12
    gemm_ops = step_ops(rows)
    achieved = gemm_ops / (gemm_ms_sum * 1e-3) / 1e12
    proxy = 2.0 * float(peaks["bf16_sustained"])
    ceil = None
    if not args.no_ceiling and not args.no_cpu:                      # diagnostic runs (--no-cpu) skip it too
        ceil = measure_issue_ceiling(dev)
    if ceil is not None:
        peak = ceil["sustained_random_operands_tops"]
        basis = ("INT8 tensor-pipe ceiling measured in this run on this GPU: tcgen05.mma kind::i8 128x256x32 issued back to "
                 "back by one CTA per SM on pseudo-random operand bytes resident in shared memory (no global traffic), rate "
                 "over the last quarter of 3 s; MEASURED_PEAKS.json holds no INT8 figure")
    else:
        peak = DATASHEET_INT8_TOPS
        basis = "datasheet dense INT8 figure (the measured ceiling was skipped in this run)"
    # DRAM traffic of the GEMM launches of one step, from ncu captures of the same kernel at 8192, 16384 and 66048 rows
    # (committed summary), interpolated linearly between the captured row counts; it does not grow in proportion to the
    # rows (the weights' share and the number of sweeps over the activations change with them)
    traffic = None
    tp = ROOT / "profiles" / "gemm_fused_pair_flux4k_rows8192_full.md"
    if tp.exists():
        pts = {}
        for ln in tp.read_text().splitlines():
            if ln.startswith("TRAFFIC_POINT"):
                _tag, name, r_, b_ = ln.split()
                pts.setdefault(name, []).append((float(r_), float(b_)))
        if all(len(pts.get(n, [])) >= 2 for n, _K, _N in LAYERS):
            def at(points, r):
                points = sorted(points)
                for (r0, b0), (r1, b1) in zip(points, points[1:]):
                    if r <= r1 or (r1, b1) == points[-1]:
                        return b0 + (b1 - b0) * (r - r0) / (r1 - r0)
            traffic = sum(at(pts[n], float(rows)) for n, _K, _N in LAYERS)
    min_bytes = sum(rows * K + N * K + 2.0 * rows * N + 64.0 * (rows + N) for _n, K, N in LAYERS)
    line = {
        "metric": METRIC, "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": "FLUX 4K single-block linear set (configs[2])", "rows_total": M_TOTAL, "rows_per_gpu": rows,
                   "layers": [f"{K}->{N}" for _n, K, N in LAYERS], "lowrank": RANK, "bias": True, "out": "bf16",
                   "parallelism": f"row-sharded x{world}, weights replicated", "allgather": bool(args.allgather and world > 1),
                   "l2": "inputs (2.4 GB) and outputs (3.2 GB) exceed L2; no flush needed",
                   "codes": "activation codes are small: 0.5 % of the channels are scaled x20 and set each row's scale, so "
                            "ordinary channels quantise to a few units around zero (kernels[].mean_abs_code); tensor-core "
                            "power and with it the sustained clock depend on the data, see kernels[].gemm_full_range_codes_*"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOPS", "frac": achieved / peak,
                     "traffic": traffic, "traffic_basis": "ncu dram__bytes_read + dram__bytes_write of the two GEMM launches, captured at 8192, 16384 and 66048 "
                                                         "rows and interpolated to this launch's rows",
                     "algorithmic_min_bytes": min_bytes,
                     "kernel": "pq_int8_gemm_fused_pair_kernel (both launches of a step)",
                     "timing": f"CUDA events around every GEMM launch inside {n_inst} running steps (down-projection, quantisation, "
                               "GEMM per layer, as the forward launches them); the launch repeated back to back: kernels[].gemm_back_to_back_*",
                     "achieved_back_to_back": gemm_ops / (sum(k["gemm_back_to_back_us"] for k in kern) * 1e-6) / 1e12,
                     "peak_basis": basis,
                     "frac_of_datasheet_4500": achieved / DATASHEET_INT8_TOPS,
                     "frac_of_2x_bf16_sustained": achieved / proxy,
                     "proxy_2x_bf16_sustained_tops": proxy, "proxy_source": peaks["source"],
                     "ops_per_launch": [2.0 * rows * K * N for _n, K, N in LAYERS]},
        "kernels": kern,
        "clocks": clocks,
        # this library's kernels per step and layer: quantisation, GEMM and the down-projection where the library's own
        # kernel takes it (ops.lowrank_down_ok)
        "gpu_launches": sum(2 + (1 if ops.lowrank_down_ok(x) else 0) for x in xs) * args.steps,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if gather is not None:
        line["allgather"] = gather
    if ceil is not None:
        line["roofline"]["int8_issue_ceiling"] = ceil
        line["roofline"]["frac_of_issue_ceiling_constant_operands"] = achieved / ceil["sustained_tops"]
    if world == 1 and not args.no_cpu and not args.no_gpu_baseline:
        gb = run_gpu_baseline(dev, xs, max(3, min(args.steps, 10)))
        if gb is not None:
            line["gpu_baseline"] = gb
    if world == 1 and not args.no_cpu:
        cb, _t = run_cpu_baseline(args.cpu_sample_rows, 3)
        line["cpu_baseline"] = cb
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main_other(args) -> None:
    """Secondary workloads (one GPU, one JSON line each, not the contract line): the other configurations of the path
    measured with the same hygiene -- interleaved repetitions, CUDA events, median per item.

    flux2k    FLUX double-block linear set at the 2K stage (M = 16896, four layers, rank 32 + bias)
    sdxl_pc   SDXL 4K-stage linears as the reference deploys them: per-channel / per-token scales, fp16 (six shapes)
    sdxl_g32  SDXL 4K-stage linears, group-32 scales on both operands (six shapes, fp16)
    routed4k  routed nested-precision FLUX MLP at the 4K stage: gather + quantise from the canvas, two-tier GEMMs
              3072 -> 12288 -> 3072, feathered scatter back (16x16-token leaves, ~30 % active, halo 2)"""
    import numpy as np
    import torch.nn as nn
    from pyraquant_b200 import int8_exec, ops, routing
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(1)

    BURST = 4

    def interleaved(items, reps):
        """items: list of (name, fn); fn takes a call counter (to rotate between input copies).  Returns {name: median
        microseconds per call}; the repetitions of the items are interleaved.  Each measurement is a burst of BURST calls
        back to back between two events.  The burst of every item is captured once into a CUDA graph and replayed, so
        that the device runs the calls back to back and the host-side cost of a call (10-50 us of Python and launch
        latency) is not mistaken for device time of kernels that take 15-100 us; an item that cannot be captured is
        timed as a plain burst (the host enqueues the next launch while the previous one runs)."""
        n = 0
        for _n, fn in items:
            fn(0); fn(1)
        torch.cuda.synchronize()
        graphs = {}
        if not args.no_graph:
            side = torch.cuda.Stream(dev)
            for name, fn in items:
                try:
                    gr = torch.cuda.CUDAGraph()
                    side.wait_stream(torch.cuda.current_stream(dev))
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(gr, stream=side):
                            for j in range(BURST):
                                fn(j)
                    graphs[name] = gr
                except Exception as e:                      # noqa: BLE001 - capture is an optimisation of the timing only
                    print(f"[bench] {name}: not captured ({type(e).__name__}), timed as plain bursts", file=sys.stderr)
                    torch.cuda.synchronize()
            torch.cuda.current_stream(dev).wait_stream(side)
            for gr in graphs.values():
                gr.replay()
            torch.cuda.synchronize()
        ev = {name: [] for name, _ in items}
        for _ in range(reps):
            for name, fn in items:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                if name in graphs:
                    graphs[name].replay()
                else:
                    for _j in range(BURST):
                        fn(n); n += 1
                b.record()
                ev[name].append((a, b))
            torch.cuda.synchronize()
        return {name: statistics.median(a.elapsed_time(b) for a, b in v) * 1e3 / BURST for name, v in ev.items()}

    def copies(x, total_bytes):
        """Enough copies of x that rotating through them defeats L2 (the working set of the copies exceeds 3 x L2)."""
        k = max(1, min(6, int(3 * 126e6 // max(1, total_bytes)) + 1))
        return [x] + [x.clone() for _ in range(k - 1)]

    def act(M, K, dtype):
        x = torch.randn(M, K, generator=g, device=dev)
        ch = torch.randperm(K, generator=g, device=dev)[: max(1, round(K * 0.005))]
        x[:, ch] *= 20.0
        return x.to(dtype)

    def layer(K, N, dtype, routed=False):
        lin = nn.Linear(K, N, bias=True, device=dev, dtype=dtype)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(N, K, generator=g, device=dev) * 0.02)
            lin.bias.copy_(torch.randn(N, generator=g, device=dev) * 0.01)
        A = (torch.randn(K, RANK, generator=g, device=dev) * 0.02).to(dtype)
        B = (torch.randn(RANK, N, generator=g, device=dev) * 0.02).to(dtype)
        cls = int8_exec.Int8LinearRouted if routed else int8_exec.Int8Linear
        return cls(lin, device=dev, lowrank=(A, B))

    reps = max(5, args.steps)

    def wanted(M, K, N):
        """--shape MxKxN restricts the SDXL workloads to one layer (profiler captures)."""
        return args.shape is None or args.shape == f"{M}x{K}x{N}"

    out = {"workload": args.workload, "n_gpus": 1,
           "unit_time": f"us per call (median over interleaved repetitions of bursts of {BURST} back-to-back calls" + (")" if args.no_graph else ", each burst replayed from a CUDA graph)"), "reps": reps,
           "data": "synthetic", "items": []}
    if args.workload == "flux2k":
        M = 16384 + 512
        for K, N in ((3072, 9216), (3072, 3072), (3072, 12288), (12288, 3072)):
            m = layer(K, N, torch.bfloat16)
            x = act(M, K, torch.bfloat16)
            xq, sx = int8_exec.quant_rows(x)
            t = x @ m.lr_A
            xc = copies(x, 3 * M * K)
            r = interleaved([("forward", lambda i: m(xc[i % len(xc)])), ("quant", lambda i: int8_exec.quant_rows(xc[i % len(xc)])),
                             ("down", lambda i: m._down(xc[i % len(xc)])),
                             ("gemm", lambda i: int8_exec.int8_gemm_lr(xq, sx, m.weight_int8, m.w_scale, m.bias, t, m.lr_B,
                                                                       torch.bfloat16, m._lr_Bt()))], reps)
            opsn = 2.0 * M * K * N
            out["items"].append({"layer": f"{K}->{N}", "rows": M, "forward_us": r["forward"], "forward_tops": opsn / r["forward"] / 1e6,
                                 "gemm_us": r["gemm"], "gemm_tops": opsn / r["gemm"] / 1e6, "quant_us": r["quant"],
                                 "quant_gbs": (3.0 * M * K + 4 * M) / r["quant"] / 1e3,
                                 "lowrank_down_us": r["down"], "lowrank_down_gbs": 2.0 * M * K / r["down"] / 1e3})
            del m, x, xq, sx, t, xc
        # adaLN prologue of the feed-forward's first Linear (flux/transformer_flux.py:236-240): LayerNorm, modulation and
        # quantisation as one kernel, against torch's three kernels followed by the plain quantisation
        K, N = 3072, 12288
        m = layer(K, N, torch.bfloat16)
        hc = copies(act(M, K, torch.bfloat16), 5 * M * K)
        sc = (torch.randn(1, K, generator=g, device=dev) * 0.3).to(torch.bfloat16)
        sh = (torch.randn(1, K, generator=g, device=dev) * 0.2).to(torch.bfloat16)
        F = torch.nn.functional

        def unfused(h):
            z = F.layer_norm(h, (K,), eps=1e-6) * (1 + sc) + sh
            return int8_exec.quant_rows(z)
        r = interleaved([("fused", lambda i: ops.adaln_quant_rows(hc[i % len(hc)], sc, sh, 1e-6)),
                         ("fused_codes_only", lambda i: ops.adaln_quant_rows(hc[i % len(hc)], sc, sh, 1e-6, want_modulated=False)),
                         ("unfused", lambda i: unfused(hc[i % len(hc)])),
                         ("forward_adaln", lambda i: m.forward_adaln(hc[i % len(hc)], sc[0], sh[0])),
                         ("forward_unfused", lambda i: m(F.layer_norm(hc[i % len(hc)], (K,), eps=1e-6) * (1 + sc) + sh))], reps)
        out["adaln"] = {"rows": M, "K": K, "N": N, "fused_us": r["fused"], "fused_gbs": 5.0 * M * K / r["fused"] / 1e3,
                        "fused_codes_only_us": r["fused_codes_only"], "fused_codes_only_gbs": 3.0 * M * K / r["fused_codes_only"] / 1e3,
                        "torch_layernorm_mul_add_then_quant_us": r["unfused"],
                        "forward_adaln_us": r["forward_adaln"], "forward_after_torch_modulation_us": r["forward_unfused"]}
        del m, hc
        # tail of a block (flux/transformer_flux.py:145-149): residual + gate * Linear(x), in the GEMM epilogue against
        # the layer followed by torch's multiply and add
        K, N = 12288, 3072
        m = layer(K, N, torch.bfloat16)
        xc = copies(act(M, K, torch.bfloat16), 3 * M * K)
        gate = (torch.randn(N, generator=g, device=dev) * 0.5).to(torch.bfloat16)
        resid = [torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]
        r = interleaved([("fused", lambda i: m.forward_gated_residual(xc[i % len(xc)], gate, resid[i % 3])),
                         ("unfused", lambda i: resid[i % 3].add_(gate * m(xc[i % len(xc)]))),
                         ("linear", lambda i: m(xc[i % len(xc)]))], reps)
        out["gated_residual"] = {"rows": M, "K": K, "N": N, "fused_us": r["fused"], "linear_then_torch_mul_add_us": r["unfused"],
                                 "linear_alone_us": r["linear"]}
        del m, xc, resid
    elif args.workload == "sdxl_pc":
        # the reference's SDXL deployment arm: per-channel weights, per-token activations, fp16, no low-rank branch
        # (deploy/run_sdxl_latency.py:214-224, shapes :280)
        for M, K, N in ((65536, 640, 640), (65536, 640, 5120), (65536, 2560, 640), (16384, 1280, 1280), (16384, 1280, 10240),
                        (16384, 5120, 1280)):
            if not wanted(M, K, N):
                continue
            lin = nn.Linear(K, N, bias=True, device=dev, dtype=torch.float16)
            with torch.no_grad():
                lin.weight.copy_(torch.randn(N, K, generator=g, device=dev) * 0.02)
            m = int8_exec.Int8Linear(lin, device=dev)
            x = torch.randn(M, K, generator=g, device=dev).to(torch.float16)
            xq, sx = int8_exec.quant_rows(x)
            xc = copies(x, 3 * M * K)
            r = interleaved([("forward", lambda i: m(xc[i % len(xc)])), ("quant", lambda i: int8_exec.quant_rows(xc[i % len(xc)])),
                             ("gemm", lambda i: int8_exec.int8_gemm_fused(xq, sx, m.weight_int8, m.w_scale, m.bias, torch.float16)),
                             ("fp16", lambda i: torch.nn.functional.linear(xc[i % len(xc)], lin.weight, lin.bias))], reps)
            opsn = 2.0 * M * K * N
            out["items"].append({"layer": f"{K}->{N}", "rows": M, "forward_us": r["forward"], "forward_tops": opsn / r["forward"] / 1e6,
                                 "gemm_us": r["gemm"], "gemm_tops": opsn / r["gemm"] / 1e6, "quant_us": r["quant"],
                                 "quant_gbs": (3.0 * M * K + 4 * M) / r["quant"] / 1e3, "torch_fp16_linear_us": r["fp16"]})
            del m, x, lin, xq, sx, xc
    elif args.workload == "sdxl_g32":
        for M, K, N in ((65536, 640, 640), (65536, 640, 5120), (65536, 2560, 640), (16384, 1280, 1280), (16384, 1280, 10240),
                        (16384, 5120, 1280)):
            if not wanted(M, K, N):
                continue
            lin = nn.Linear(K, N, bias=True, device=dev, dtype=torch.float16)
            with torch.no_grad():
                lin.weight.copy_(torch.randn(N, K, generator=g, device=dev) * 0.02)
            m = int8_exec.Int8LinearG32(lin, device=dev)
            x = torch.randn(M, K, generator=g, device=dev).to(torch.float16)
            xc = copies(x, 3 * M * K)
            r = interleaved([("forward", lambda i: m(xc[i % len(xc)])), ("quant", lambda i: int8_exec.quant_rows_g32(xc[i % len(xc)]))], reps)
            opsn = 2.0 * M * K * N
            out["items"].append({"layer": f"{K}->{N}", "rows": M, "forward_us": r["forward"], "forward_tops": opsn / r["forward"] / 1e6,
                                 "quant_g32_us": r["quant"], "quant_g32_gbs": (3.0 * M * K + 4.0 * M * K / 32) / r["quant"] / 1e3,
                                 "gemm_g32_us": r["forward"] - r["quant"],
                                 "gemm_g32_tops": opsn / max(r["forward"] - r["quant"], 1e-3) / 1e6})
            del m, x, lin, xc
    elif args.workload == "block4k":
        # The Linear path of one FLUX single-stream block at the 4K stage (flux/transformer_flux.py:126-150), attention
        # left out (its output is stood in for by the query projection): the reference's call sequence on this
        # library's drop-in layers against the same block with the block-level fusions (adaLN prologue shared by the four
        # sibling projections, GELU in the epilogue, proj_out reading its two sources in place, gate and residual in the
        # epilogue).
        M, D, H4 = 65536 + 512, 3072, 12288
        F = torch.nn.functional
        proj_mlp, to_q, to_k, to_v = layer(D, H4, torch.bfloat16), layer(D, D, torch.bfloat16), layer(D, D, torch.bfloat16), layer(D, D, torch.bfloat16)
        proj_out = layer(D + H4, D, torch.bfloat16)
        h = act(M, D, torch.bfloat16)
        shift, scale, gate = [(torch.randn(1, D, generator=g, device=dev) * 0.3).to(torch.bfloat16) for _ in range(3)]

        def unfused(_i):
            z = F.layer_norm(h, (D,), eps=1e-6) * (1 + scale) + shift
            mlp = F.gelu(proj_mlp(z), approximate="tanh")
            q_, k_, v_ = to_q(z), to_k(z), to_v(z)
            cat = torch.cat([q_, mlp], dim=-1)
            return h + gate * proj_out(cat), k_, v_
        grp = int8_exec.share_input_quantisation([proj_mlp, to_q, to_k, to_v])
        res = [h.clone() for _ in range(2)]        # the residual stream is updated in place (the block's input is dead after it)

        def fused(i):
            z = grp.prime_adaln(h, scale[0], shift[0])
            mlp = proj_mlp.forward_ex(z, ops.EPI_GELU_TANH)
            q_, k_, v_ = to_q(z), to_k(z), to_v(z)
            return proj_out.forward_gated_residual(q_, gate[0], res[i % 2], x_more=mlp), k_, v_     # no concatenated tensor
        a, b = unfused(0), fused(0)
        torch.cuda.synchronize()
        rel = ((a[0].float() - b[0].float()).norm() / a[0].float().norm()).item()
        del a, b
        res[0].copy_(h)
        r = interleaved([("unfused", unfused), ("fused", fused)], reps)
        opsn = 2.0 * M * (D * H4 + 3 * D * D + (D + H4) * D)
        out["items"] = [{"item": "single-stream block, Linear path, reference call sequence on the drop-in layers", "us": r["unfused"],
                         "tops": opsn / r["unfused"] / 1e6},
                        {"item": "same block with the block-level fusions", "us": r["fused"], "tops": opsn / r["fused"] / 1e6,
                         "rel_l2_vs_unfused": rel}]
        out.update({"rows": M, "dim": D, "mlp_dim": H4})
    else:
        H = W = 256
        C, F = 3072, 12288
        rng = np.random.default_rng(4)
        sel = (rng.random((16, 16)) < 0.3).astype(np.float32)
        hi = routing.inner_split_median(rng.random((16, 16)), sel, 1.0)
        plan = routing.build_route_plan((H, W), routing.leaf_run_boxes(sel, 32), 2,
                                        token_tier_hi=routing.leaf_tier_to_token_map(hi, (H, W)))
        d = plan.to(dev)
        M, mh = plan.n_rows, plan.m_hi
        canvas = act(H * W, C, torch.bfloat16)
        up, down = layer(C, F, torch.bfloat16, routed=True), layer(F, C, torch.bfloat16, routed=True)
        hmid = up.forward_gathered(canvas, d["row_idx"], mh)
        y = down.forward_rows(hmid, mh)
        cv = [canvas, canvas.clone()]                       # 2 x 403 MB: rotating defeats L2
        # plain device copies that move as many bytes as the two memory-bound kernels (half read, half written): what
        # the memory system gives a kernel of this size in the same timing loop
        gq_bytes, sc_bytes = 3.0 * M * C + 8.0 * M, 2.0 * C * (int(plan.src.shape[0]) + int(plan.tokens.shape[0]))
        n_gq, n_sc = int(gq_bytes) // 8, int(sc_bytes) // 8                   # int32 elements of each half
        cp_src = [torch.empty(max(n_gq, n_sc) + 1024, dtype=torch.int32, device=dev) for _ in range(2)]
        cp_dst = [torch.empty_like(t) for t in cp_src]
        r = interleaved([("copy_gq", lambda i: cp_dst[i % 2][:n_gq].copy_(cp_src[i % 2][:n_gq])),
                         ("copy_sc", lambda i: cp_dst[i % 2][:n_sc].copy_(cp_src[i % 2][:n_sc])),
                         ("gather_quant", lambda i: routing.gather_quant_rows(cv[i % 2], plan)),
                         ("up", lambda i: up.forward_gathered(cv[i % 2], d["row_idx"], mh)),
                         ("down", lambda i: down.forward_rows(hmid, mh)),
                         ("scatter", lambda i: routing.scatter_rows_(y, plan, cv[i % 2]))], reps)
        nt, nnz = int(plan.tokens.shape[0]), int(plan.src.shape[0])
        # canvas rows the scatter has to read: tokens whose accumulated blend weight stays below one (the others take
        # nothing from the background)
        n_bg = int((np.add.reduceat(plan.beta.astype(np.float64), plan.ptr[:-1].astype(np.int64)) < 1.0).sum()) if nnz else nt
        out.update({"rows_gathered": M, "rows_hi": mh, "touched_tokens": nt, "canvas": [H * W, C]})
        out["items"] = [
            {"item": "gather+quantise", "us": r["gather_quant"], "gbs": (3.0 * M * C + 8.0 * M) / r["gather_quant"] / 1e3,
             "plain_copy_same_bytes_us": r["copy_gq"]},
            {"item": f"routed Linear {C}->{F} (gather, quantise, down-projection, two-tier GEMM)", "us": r["up"],
             "tops": 2.0 * M * C * F / r["up"] / 1e6},
            {"item": f"routed Linear {F}->{C} (quantise, down-projection, two-tier GEMM)", "us": r["down"],
             "tops": 2.0 * M * C * F / r["down"] / 1e6},
            {"item": "feathered scatter", "us": r["scatter"], "gbs": 2.0 * C * (nnz + nt + n_bg) / r["scatter"] / 1e3,
             "rows_read": nnz, "canvas_rows_written": nt, "canvas_rows_read": n_bg,
             "plain_copy_same_bytes_us": r["copy_sc"] * (nnz + nt + n_bg) / (nnz + nt)}]
    ops.check_device_status(dev)
    out["peaks"] = {"hbm_gbs": peaks["hbm_gbs"], "int8_proxy_tops": 2.0 * float(peaks["bf16_sustained"]), "source": peaks["source"]}
    print(json.dumps(out))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--allgather", action="store_true", help="also all-gather the outputs over NCCL inside the step")
    ap.add_argument("--cpu-sample-rows", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=M_TOTAL,
                    help="total token rows (default: the 4K stage's 66048); smaller values are for profiler captures only")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="secondary workloads: time plain bursts instead of CUDA-graph replays")
    ap.add_argument("--no-gather", action="store_true", help="N > 1: skip the measurement of the optional output all-gather")
    ap.add_argument("--gather-chunks", type=int, default=0, help="chunks per rank of the overlapped all-gather (0: try 1 and 2)")
    ap.add_argument("--gather-mode", choices=("auto", "store", "push", "nccl"), default="auto",
                    help="all-gather hidden behind the compute: stores to peers from the GEMM epilogue, copy-engine pushes into "
                         "peers' buffers, NCCL per chunk; auto tries the first two and reports the faster")
    ap.add_argument("--gather-try-copy", action="store_true", help="also try the push mode with a local staging copy")
    ap.add_argument("--gather-sms", type=int, default=-1,
                    help="SMs the GEMM leaves free while NCCL gathers (-1: try 0, 8 and 16 and report the best)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-ceiling", action="store_true", help="skip the tensor-pipe issue-loop ceiling measurement")
    ap.add_argument("--no-gpu-baseline", action="store_true", help="skip the reference's own GPU forward (baseline/_ref)")
    ap.add_argument("--shape", default=None, help="MxKxN: only this layer of the sdxl_pc / sdxl_g32 workloads")
    ap.add_argument("--workload", choices=("flux4k", "flux2k", "sdxl_pc", "sdxl_g32", "routed4k", "block4k"), default="flux4k",
                    help="flux4k (default) is the benchmark contract; the others print one JSON line of per-item "
                         "measurements for the remaining configurations of the path (one GPU)")
    args = ap.parse_args()
    M_TOTAL = int(args.rows)
    if args.workload != "flux4k":
        main_other(args)
    elif args.impl == "reference":
        main_reference(args)
    else:
        main_ours(args)
