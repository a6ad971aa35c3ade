"""Benchmark of the block-sparse Linear hot path (pack + fwd + dgrad + wgrad of one layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--precision P]
    python bench.py --impl reference ...      # the reference's CPU path (to_dense + matmul) on host cores

One step = one pass of the hot path over one batch of synthetic activations:
weight packing (the per-step replacement of the reference's transposed weight copy), forward
y = x W^T + b, dgrad dx = dy W and the sparse-output wgrad.  With N > 1 ranks the layer runs
token-data-parallel (every rank its own tokens, same weights) and the step ends with an NCCL
all-reduce of the nnz-block gradient buffer.  Prints ONE JSON line on rank 0.

metric = effective TFLOP/s = 3 * (2 * M * nnz * 1024) FLOP per step / time, the work of the
non-zero blocks only (extra tensor-core passes of the 3xTF32 split and padding do not count).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "block_sparse_linear_fwd_bwd_effective_tflops"
UNIT = "TFLOP/s"

# single-layer workloads of the benchmark configurations (tokens M, out N, in K, density)
WORKLOADS = {
    "c3_d0.25": dict(m=16384, n=4096, k=4096, density=0.25),  # headline: density sweep, d = 0.25
    "c3_d0.10": dict(m=16384, n=4096, k=4096, density=0.10),
    "c3_d0.50": dict(m=16384, n=4096, k=4096, density=0.50),
    "c3_d0.75": dict(m=16384, n=4096, k=4096, density=0.75),
    "c2_up": dict(m=4096, n=3072, k=768, density=0.5),  # RoBERTa-base FFN 768 -> 3072
    "c2_down": dict(m=4096, n=768, k=3072, density=0.5),  # RoBERTa-base FFN 3072 -> 768
    "c1": dict(m=256, n=256, k=1024, density=0.5),  # the reference's CPU-runnable case
    # one GPU's block-row shard of the large column-parallel layer (65536 tokens, 32768 x 8192 at density 0.1, 8 GPUs)
    "c5_shard": dict(m=65536, n=4096, k=8192, density=0.1),
}


def nnz_of(cfg):
    return int(cfg["density"] * cfg["n"] * cfg["k"] / 1024)


def flops_per_op(cfg):
    return 2.0 * cfg["m"] * nnz_of(cfg) * 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], bf16_tflops_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {
            "sm_mhz": sm[len(sm) // 2] if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


# --------------------------------------------------------------------------- CPU reference path
def cpu_reference_step(cfg, sample_m, seed=0):
    """Build the seeded sample once; return a callable running fwd+dgrad+wgrad the way the reference's
    CPU path does (to_dense + matmul in fp32), restated in numpy by the oracle."""
    import numpy as np

    from oracle import block_sparse_oracle as orc

    rng = np.random.RandomState(seed)
    np.random.seed(seed)
    shape = (cfg["n"], cfg["k"])
    mask = orc.random_mask(shape, nnz_of(cfg))
    idx = orc.build_indices(mask)
    data = (rng.standard_normal((nnz_of(cfg) * 32, 32)) * 0.02).astype(np.float32)
    x = rng.standard_normal((sample_m, cfg["k"])).astype(np.float32)
    dy = rng.standard_normal((sample_m, cfg["n"])).astype(np.float32)
    bias = (rng.standard_normal(cfg["n"]) * 0.02).astype(np.float32)

    def step():
        y = orc.forward(x, shape, idx["blocks"], data, bias, dtype=np.float32)
        dx = orc.dgrad(dy, shape, idx["blocks"], data, dtype=np.float32)
        dw = orc.wgrad(dy, x, shape, idx["blocks"], dtype=np.float32)
        return y, dx, dw

    return step


def time_cpu_reference(cfg, target_seconds, reps):
    """Effective TFLOP/s of the CPU path on a bounded token sample sized for ~target_seconds."""
    probe_m = min(cfg["m"], 256)
    step = cpu_reference_step(cfg, probe_m)
    step()
    t0 = time.perf_counter()
    step()
    probe = time.perf_counter() - t0
    per_token = max(probe / probe_m, 1e-9)
    sample_m = int(min(cfg["m"], max(probe_m, target_seconds / reps / per_token)))
    sample_m = max(32, sample_m // 32 * 32)
    step = cpu_reference_step(cfg, sample_m)
    step()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    value = 3 * 2.0 * sample_m * nnz_of(cfg) * 1024 / med / 1e12
    return value, sample_m, med


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    probe_m = min(cfg["m"], 256)
    step = cpu_reference_step(cfg, probe_m)
    step()
    t0 = time.perf_counter()
    step()
    per_token = max((time.perf_counter() - t0) / probe_m, 1e-9)
    budget = 60.0 / max(1, args.steps + args.warmup)  # whole run within about a minute of compute
    sample_m = int(min(cfg["m"], max(probe_m, budget / per_token)))
    sample_m = max(32, sample_m // 32 * 32)
    step = cpu_reference_step(cfg, sample_m)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    ms = elapsed / args.steps * 1e3
    value = 3 * 2.0 * sample_m * nnz_of(cfg) * 1024 / (ms / 1e3) / 1e12
    sample = "first %d of %d tokens per step; to_dense + fp32 matmul for fwd, dgrad, wgrad" % (sample_m, cfg["m"])
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": dict(workload=args.workload, nnz=nnz_of(cfg), sample_tokens=sample_m, **cfg),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args, cfg):
    import numpy as np
    import torch
    import torch.distributed as dist

    from pytorch_block_sparse_b200 import BlockSparseLinear, BlockSparseMatrix, native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    prec_name = args.precision
    prec = native.resolve_precision(prec_name)
    native.set_default_precision(prec_name)
    m, n, k = cfg["m"], cfg["n"], cfg["k"]
    nnz = nnz_of(cfg)

    # same pattern and weights on every rank (token-data-parallel), different tokens per rank
    np.random.seed(1234)
    torch.manual_seed(1234)
    lin = BlockSparseLinear(k, n, bias=True, density=cfg["density"])
    with torch.no_grad():
        lin.weight.data.copy_((torch.randn(lin.weight.data.shape) * 0.02).to(dev))
        lin.bias.copy_((torch.randn(n) * 0.02).to(dev))
    w = lin.weight
    assert w.data.shape[0] == nnz * 32
    g = torch.Generator().manual_seed(99 + rank)
    x_host = torch.randn(m, k, generator=g).pin_memory()
    dy_host = torch.randn(m, n, generator=g).pin_memory()
    x = x_host.to(dev)
    dy = dy_host.to(dev)
    y = torch.empty(m, n, device=dev)
    dx = torch.empty(m, k, device=dev)
    dw = torch.empty_like(w.data)
    plan_f, plan_d, plan_w = w._plan(True), w._plan(False), w._sddmm_plan()
    bias = lin.bias.detach()
    data = w.data.detach()

    launches_per_step = [0]

    def step(count=False):
        packed = native.pack_weights(data, prec)
        native.dsd_matmul(x, plan_f, packed, n, True, bias=bias, out=y)
        native.dsd_matmul(dy, plan_d, packed, k, False, out=dx)
        native.sddmm(dy, True, x, True, w.blocks, dw, precision=prec, plan=plan_w)
        if world > 1:
            dist.all_reduce(dw)
        return packed

    # kernels of this library launched per step: pack, fwd, dgrad, wgrad (+ its token-range reduction)
    launches_per_step = 5 if native.load().bsmm_sddmm_workspace_bytes(n, k, m, nnz, prec) > 0 else 4

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert native.device_status() == 0, "a kernel abandoned a bounded wait during warm-up"

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = elapsed_ms / args.steps
    f_op = flops_per_op(cfg)
    value = world * 3 * f_op / (ms_per_step / 1e3) / 1e12

    # ---- per-kernel timings (same stream, CUDA events, inputs larger than L2) ----
    def time_op(fn, reps):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    packed = native.pack_weights(data, prec)
    reps = max(3, min(20, args.steps))
    kernels = {
        "pack_ms": time_op(lambda: native.pack_weights(data, prec), reps),
        "fwd_ms": time_op(lambda: native.dsd_matmul(x, plan_f, packed, n, True, bias=bias, out=y), reps),
        "dgrad_ms": time_op(lambda: native.dsd_matmul(dy, plan_d, packed, k, False, out=dx), reps),
        "wgrad_ms": time_op(lambda: native.sddmm(dy, True, x, True, w.blocks, dw, precision=prec, plan=plan_w), reps),
    }

    # ---- end to end through the public layer API with host buffers ----
    y_host = torch.empty(m, n).pin_memory()
    dx_host = torch.empty(m, k).pin_memory()
    dw_host = torch.empty(w.data.shape).pin_memory()

    # Every step copies its inputs from pinned host memory and its results back.  The copies of consecutive
    # steps are pipelined over two extra streams (PCIe is full duplex): step i+1's inputs travel while step i
    # computes and step i-1's results return.  Device input buffers are double-buffered.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    x_dev = [torch.empty(m, k, device=dev) for _ in range(2)]
    dy_dev = [torch.empty(m, n, device=dev) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    for ev in in_free:
        ev.record()

    def e2e_step(i):
        buf = i & 1
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[buf])
            x_dev[buf].copy_(x_host, non_blocking=True)
            dy_dev[buf].copy_(dy_host, non_blocking=True)
            in_ready[buf].record(s_in)
        cur.wait_event(in_ready[buf])
        xd = x_dev[buf].detach().requires_grad_(True)
        lin.weight.data.grad = None
        out = lin(xd)
        out.backward(dy_dev[buf])
        if world > 1:
            dist.all_reduce(lin.weight.data.grad)
        in_free[buf].record(cur)
        done = torch.cuda.Event()
        done.record(cur)
        results = (out.detach(), xd.grad, lin.weight.data.grad)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for host, t in zip((y_host, dx_host, dw_host), results):
                host.copy_(t, non_blocking=True)
                t.record_stream(s_out)

    e2e_steps = max(4, min(args.steps, 8))
    for i in range(2):
        e2e_step(i)
    torch.cuda.current_stream().wait_stream(s_out)
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.current_stream().wait_stream(s_out)  # the last step's results are on the host
    b.record()
    barrier()
    e2e_ms = a.elapsed_time(b) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * 3 * f_op / (e2e_ms / 1e3) / 1e12
    h2d = (x_host.numel() + dy_host.numel()) * 4
    d2h = (y_host.numel() + dx_host.numel() + dw_host.numel()) * 4
    status = native.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- comparators: cuBLAS dense nn.Linear fwd+bwd on the same shape ----
    comparators = {}
    if not args.no_comparators:
        wd = torch.randn(n, k, device=dev) * 0.02

        def dense_step():
            torch.addmm(bias, x, wd.t(), out=y)
            torch.mm(dy, wd, out=dx)
            torch.mm(dy.t(), x)

        for name, tf32 in (("cublas_dense_tf32_ms", True), ("cublas_dense_fp32_ms", False)):
            torch.backends.cuda.matmul.allow_tf32 = tf32
            comparators[name] = time_op(dense_step, 3)
        torch.backends.cuda.matmul.allow_tf32 = False
        xb, dyb, wb = x.bfloat16(), dy.bfloat16(), wd.bfloat16()
        yb, dxb = torch.empty(m, n, device=dev, dtype=torch.bfloat16), torch.empty(m, k, device=dev, dtype=torch.bfloat16)

        def dense_bf16():
            torch.mm(xb, wb.t(), out=yb)
            torch.mm(dyb, wb, out=dxb)
            torch.mm(dyb.t(), xb)

        comparators["cublas_dense_bf16_ms"] = time_op(dense_bf16, 3)
        del xb, dyb, wb, yb, dxb, wd

        # the reference's own SIMT kernels rebuilt for sm_100a (oracle/_ref, built by oracle/build_ref.py);
        # they launch on the legacy default stream, which is the stream timed here
        from oracle import ref_cuda

        if ref_cuda.available() and m * max(n, k) < 2 ** 31:
            def reference_step():
                ref_cuda.reverse_matmul(w, x, True)
                ref_cuda.reverse_matmul(w, dy, False)
                ref_cuda.sddmm(w, dy, x)

            comparators["reference_cuda_kernels_ms"] = time_op(reference_step, 3)

    # ---- roofline of the dominant kernel ----
    peaks = measured_peaks()
    op_names = {"fwd_ms": "dsd forward", "dgrad_ms": "dsd dgrad", "wgrad_ms": "sddmm wgrad"}
    dom = max(op_names, key=lambda key: kernels[key])
    achieved = f_op / (kernels[dom] / 1e3) / 1e12
    # tcgen05 kind::tf32 runs at half the bf16 rate; the measured dense bf16 peak (sustained, the
    # kernel is timed inside a long loop) halved is the single-pass TF32 ceiling used here
    peak = peaks["bf16_tflops_sustained"] / 2.0 if prec_name != "bf16" else peaks["bf16_tflops_sustained"]
    # DRAM bytes (read + write) of one launch of that kernel from an ncu capture of this workload; null
    # where no capture was taken (the summaries with the commands are under profiles/)
    ncu_traffic = {
        ("c3_d0.25", "tf32x3", "wgrad_ms"): (666.8e6, "profiles/sddmm_umma_tf32x3_c3_d0.25.md"),
        ("c3_d0.25", "tf32x3", "fwd_ms"): (624.0e6, "profiles/dsd_umma_tf32x3_c3_d0.25.md"),
    }.get((args.workload, prec_name, dom), (None, None))
    roofline = {
        "kernel": op_names[dom], "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak, "traffic": ncu_traffic[0], "traffic_source": ncu_traffic[1],
        "peak_source": "%s bf16 sustained %.1f TFLOP/s %s" % (peaks["source"], peaks["bf16_tflops_sustained"], "/ 2 (tf32)" if prec_name != "bf16" else ""),
        "algorithmic_flops_per_launch": f_op,
    }

    if world == 1:
        cpu_value, cpu_m, cpu_t = time_cpu_reference(cfg, target_seconds=args.cpu_seconds, reps=3)
        cpu_sample = "first %d of %d tokens, median of 3; numpy to_dense + fp32 matmul" % (cpu_m, m)
    else:  # the host cores are timed in the single-GPU run only
        cpu_value, cpu_sample = None, "not timed when n_gpus > 1"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": prec_name, "data": "synthetic",
        "config": dict(workload=args.workload, nnz=nnz, parallelism="token-dp%d" % world,
                       cache=("x and dy are %d and %d MiB, larger than the 126 MB L2" % (m * k * 4 >> 20, m * n * 4 >> 20))
                       if min(m * k, m * n) * 4 > (126 << 20) else
                       ("x and dy (%d and %d MiB) fit the 126 MB L2 and are not flushed between steps"
                        % (m * k * 4 >> 20, m * n * 4 >> 20)), **cfg),
        "roofline": roofline,
        "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                         "sample": cpu_sample},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "kernels": kernels,
        "comparators": comparators,
        "device_status": status,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3_d0.25", choices=sorted(WORKLOADS))
    ap.add_argument("--precision", default="tf32x3", choices=["tf32x3", "tf32", "bf16", "fp32"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-comparators", action="store_true")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_gpu_arm(args, cfg)


if __name__ == "__main__":
    main()
