"""Benchmark of the block-sparse Linear hot path (pack + fwd + dgrad + wgrad of one layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--precision P] [--legs sweep,c5,c4]
    python bench.py --impl reference ...      # the reference's CPU path (to_dense + matmul) on host cores

One step = one pass of the hot path over one batch of synthetic activations:
weight packing (the per-step replacement of the reference's transposed weight copy), forward
y = x W^T + b, the sparse-output wgrad and dgrad dx = dy W.  With N > 1 ranks the layer runs
token-data-parallel (every rank its own tokens, same weights): the NCCL all-reduce of the nnz-block gradient
buffer runs on a side stream while dgrad computes.  Prints ONE JSON line on rank 0.

metric = effective TFLOP/s = 3 * (2 * M * nnz * 1024) FLOP per step / time, the work of the
non-zero blocks only (extra tensor-core passes of the 3xTF32 split and padding do not count).

Extra legs in the same line (each timed after the headline region, never inside it):
  sweep  ms per step of the other benchmark configurations and precisions on this GPU
  c5     the large column-parallel layer (32768 x 8192, density 0.1, 65536 tokens) sharded by block-rows over the
         N ranks, strong scaling: compute alone and with the output all-gather + input-gradient all-reduce
  c4     RoBERTa-base (12 layers) patched by BlockSparseModelPatcher at density 0.5, MLM loss, AdamW,
         token-data-parallel over the N ranks: training tokens/s beside the dense model
"""
import argparse
import json
import os
import re
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
C5 = dict(m=65536, n=32768, k=8192, density=0.1)
# what the sweep leg times beside the headline (workload, precision)
# ("bf16io" = 'bf16' precision on bf16 activation / output tensors: half the activation bytes in HBM;
#  "bf16x3" = the other fp32-class mode: forward and dgrad split into bf16 pairs, wgrad as in 3xTF32)
SWEEP = [("c3_d0.25", "bf16x3"), ("c3_d0.25", "tf32"), ("c3_d0.25", "bf16"), ("c3_d0.25", "bf16io"), ("c3_d0.10", "tf32x3"), ("c3_d0.10", "bf16io"),
         ("c3_d0.50", "tf32x3"), ("c3_d0.50", "bf16x3"), ("c3_d0.75", "tf32x3"), ("c2_up", "tf32x3"), ("c2_down", "tf32x3"),
         ("c5_shard", "tf32x3"), ("c5_shard", "bf16io")]


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


def profile_traffic(kernel, precision, workload):
    """DRAM read + write bytes of one launch of `kernel`, from the committed ncu summary of that kernel, precision
    and workload (a line `traffic_bytes_per_launch: <number>`); (None, None) where no capture was taken."""
    path = os.path.join(ROOT, "profiles", "%s_%s_%s.md" % (kernel, precision, workload))
    if not os.path.exists(path):
        return None, None
    with open(path) as f:
        m = re.search(r"traffic_bytes_per_launch\s*:\s*([0-9.eE+]+)", f.read())
    return (float(m.group(1)), os.path.relpath(path, ROOT)) if m else (None, None)


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
def reference_package():
    """The unmodified reference package when it was pip-installed into the git-ignored baseline/_ref, else None."""
    site = os.environ.get("BSMM_REFERENCE_SITE", os.path.join(ROOT, "baseline", "_ref"))
    if not os.path.isdir(os.path.join(site, "pytorch_block_sparse")):
        return None
    sys.path.insert(0, site)
    try:
        import pytorch_block_sparse as ref
    except Exception:
        return None
    finally:
        sys.path.remove(site)
    return ref


def cpu_reference_step(cfg, sample_m, seed=0):
    """Build the seeded sample once; return (step, kind).  `step` runs fwd + dgrad + wgrad the way the
    reference's CPU path does: BlockSparseMatrix.to_dense() followed by fp32 matmuls, the weight gradient masked
    to the stored blocks.  kind "reference": the reference's own classes and torch.matmul on all host cores;
    kind "port": the numpy restatement under oracle/ (where the reference package is not installed)."""
    import numpy as np

    cores = os.cpu_count() or 1
    shape = (cfg["n"], cfg["k"])
    ref = reference_package()
    if ref is not None:
        import torch

        torch.set_num_threads(cores)
        np.random.seed(seed)
        torch.manual_seed(seed)
        w = ref.BlockSparseMatrix.zeros(shape, n_blocks=nnz_of(cfg), device="cpu")
        with torch.no_grad():
            w.data.normal_(0, 0.02)
        x = torch.randn(sample_m, cfg["k"])
        dy = torch.randn(sample_m, cfg["n"])
        bias = torch.randn(cfg["n"]) * 0.02
        ones = torch.ones_like(w.data)

        def step():
            with torch.no_grad():
                y = x @ w.to_dense().t() + bias
                dx = dy @ w.to_dense()
                dw = (dy.t() @ x) * w.to_dense(data_replace=ones)
            return y, dx, dw

        return step, "reference"

    from threadpoolctl import threadpool_limits

    from oracle import block_sparse_oracle as orc

    threadpool_limits(limits=cores)
    rng = np.random.RandomState(seed)
    np.random.seed(seed)
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

    return step, "port"


def sized_cpu_sample(cfg, seconds_per_step):
    """A token count whose CPU step takes about `seconds_per_step` (a probe on 256 tokens sets the rate)."""
    probe_m = min(cfg["m"], 256)
    step, _ = cpu_reference_step(cfg, probe_m)
    step()
    t0 = time.perf_counter()
    step()
    per_token = max((time.perf_counter() - t0) / probe_m, 1e-9)
    sample_m = int(min(cfg["m"], max(probe_m, seconds_per_step / per_token)))
    return max(32, sample_m // 32 * 32)


def time_cpu_reference(cfg, target_seconds, reps):
    """Effective TFLOP/s of the CPU path on a bounded token sample sized for ~target_seconds."""
    sample_m = sized_cpu_sample(cfg, target_seconds / reps)
    step, kind = cpu_reference_step(cfg, sample_m)
    step()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    value = 3 * 2.0 * sample_m * nnz_of(cfg) * 1024 / med / 1e12
    return value, sample_m, kind


def run_reference_arm(args, cfg):
    """The reference's own CPU implementation of the path on the host cores.  It has no multi-GPU form: under
    torchrun rank 0 alone runs it (with every host core, whatever OMP_NUM_THREADS the launcher exported)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    os.environ["MKL_NUM_THREADS"] = str(cores)
    budget = 60.0 / max(1, args.steps + args.warmup)  # whole run within about a minute of compute
    sample_m = sized_cpu_sample(cfg, budget)
    step, kind = cpu_reference_step(cfg, sample_m)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    ms = elapsed / args.steps * 1e3
    value = 3 * 2.0 * sample_m * nnz_of(cfg) * 1024 / (ms / 1e3) / 1e12
    how = ("the reference package's BlockSparseMatrix.to_dense + torch.matmul" if kind == "reference"
           else "numpy restatement of to_dense + fp32 matmul")
    sample = "first %d of %d tokens per step; %s for fwd, dgrad, wgrad" % (sample_m, cfg["m"], how)
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": dict(workload=args.workload, nnz=nnz_of(cfg), sample_tokens=sample_m,
                       note="CPU path: one process on the host cores whatever --gpus says", **cfg),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU helpers
def time_op(fn, reps, warm=2):
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def measure_gemm_peaks(dev):
    """cuBLAS 8192^3 GEMMs on this GPU, best of 5 launches each: the TF32 figure is the roofline's denominator for
    the tf32 kernels (single pass; the 3xTF32 default does three times the tensor work per useful FLOP)."""
    import torch

    n = 8192
    a = torch.randn(n, n, device=dev)
    b = torch.randn(n, n, device=dev)
    c = torch.empty(n, n, device=dev)
    out = {}
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    best = min(time_op(lambda: torch.mm(a, b, out=c), 1, warm=1) for _ in range(5))
    out["tf32_tflops"] = 2.0 * n ** 3 / (best / 1e3) / 1e12
    torch.backends.cuda.matmul.allow_tf32 = old
    ab, bb = a.bfloat16(), b.bfloat16()
    cb = torch.empty(n, n, device=dev, dtype=torch.bfloat16)
    best = min(time_op(lambda: torch.mm(ab, bb, out=cb), 1, warm=1) for _ in range(5))
    out["bf16_tflops"] = 2.0 * n ** 3 / (best / 1e3) / 1e12
    return out


class LayerCase:
    """One BlockSparseLinear workload resident on the device: seeded pattern, weights and activations."""

    def __init__(self, cfg, dev, rank=0, host_buffers=False):
        import numpy as np
        import torch

        from pytorch_block_sparse_b200 import BlockSparseLinear

        self.cfg = cfg
        m, n, k = cfg["m"], cfg["n"], cfg["k"]
        # same pattern and weights on every rank (token-data-parallel), different tokens per rank
        np.random.seed(1234)
        torch.manual_seed(1234)
        self.lin = BlockSparseLinear(k, n, bias=True, density=cfg["density"])
        with torch.no_grad():
            self.lin.weight.data.copy_((torch.randn(self.lin.weight.data.shape) * 0.02).to(dev))
            self.lin.bias.copy_((torch.randn(n) * 0.02).to(dev))
        self.w = self.lin.weight
        assert self.w.data.shape[0] == nnz_of(cfg) * 32
        g = torch.Generator().manual_seed(99 + rank)
        if host_buffers:
            self.x_host = torch.randn(m, k, generator=g).pin_memory()
            self.dy_host = torch.randn(m, n, generator=g).pin_memory()
            self.x, self.dy = self.x_host.to(dev), self.dy_host.to(dev)
        else:
            gd = torch.Generator(device=dev).manual_seed(99 + rank)
            self.x = torch.randn(m, k, generator=gd, device=dev)
            self.dy = torch.randn(m, n, generator=gd, device=dev)
        self.y = torch.empty(m, n, device=dev)
        self.dx = torch.empty(m, k, device=dev)
        self.dw = torch.empty_like(self.w.data)
        self.plans = (self.w._plan(True), self.w._plan(False), self.w._sddmm_plan())
        self.bias = self.lin.bias.detach()
        self.data = self.w.data.detach()

    def ops(self, prec, io_bf16=False):
        """(pack, fwd, dgrad, wgrad) closures for one precision; io_bf16: on bf16 copies of the activations, with
        bf16 outputs."""
        import torch

        from pytorch_block_sparse_b200 import native

        n, k = self.cfg["n"], self.cfg["k"]
        plan_f, plan_d, plan_w = self.plans
        state = {}
        x, dy, y, dx = self.x, self.dy, self.y, self.dx
        if io_bf16:
            x, dy = x.bfloat16(), dy.bfloat16()
            y, dx = torch.empty_like(y, dtype=torch.bfloat16), torch.empty_like(dx, dtype=torch.bfloat16)

        def pack():
            state["packed"] = native.pack_weights(self.data, prec)

        def fwd():
            native.dsd_matmul(x, plan_f, state["packed"], n, True, bias=self.bias, out=y)

        def dgrad():
            native.dsd_matmul(dy, plan_d, state["packed"], k, False, out=dx)

        def wgrad():
            native.sddmm(dy, True, x, True, self.w.blocks, self.dw, precision=prec, plan=plan_w)

        return pack, fwd, dgrad, wgrad


def run_sweep(dev, steps):
    """ms per fwd+bwd step of the other benchmark configurations / precisions (one GPU, inputs resident)."""
    import torch

    from pytorch_block_sparse_b200 import native

    out = {}
    cases = {}
    for workload, prec_name in SWEEP:
        if workload not in cases:
            cases.clear()  # one workload resident at a time
            torch.cuda.empty_cache()
            cases[workload] = LayerCase(WORKLOADS[workload], dev)
        case = cases[workload]
        io16 = prec_name == "bf16io"
        pack, fwd, dgrad, wgrad = case.ops(native.resolve_precision("bf16" if io16 else prec_name), io_bf16=io16)

        def step():
            pack(); fwd(); wgrad(); dgrad()

        ms = time_op(step, max(3, min(steps, 10)), warm=3)
        entry = {"ms_per_step": ms, "effective_tflops": 3 * flops_per_op(case.cfg) / (ms / 1e3) / 1e12}
        if io16:  # these are the HBM-bound cases: activation bytes in + out, weight images, fp32 weight gradient
            c = case.cfg
            nbytes = 2 * (3 * c["m"] * c["k"] + 3 * c["m"] * c["n"]) + nnz_of(c) * (2 * 2048 + 4096 + 4096)
            entry["algorithmic_gbs"] = nbytes / (ms / 1e3) / 1e9
            entry["frac_of_measured_hbm"] = entry["algorithmic_gbs"] / measured_peaks()["hbm_gbs"]
        out["%s/%s" % (workload, prec_name)] = entry
        del pack, fwd, dgrad, wgrad
    # the headline shape with 64x64 blocks at the same density (the reference sends such shapes to its dense-masked
    # emulator; here they run on the same kernels through their 32x32 expansion)
    cases.clear()
    torch.cuda.empty_cache()
    import numpy as np

    from pytorch_block_sparse_b200 import BlockSparseMatrix

    c = WORKLOADS["c3_d0.25"]
    np.random.seed(64)
    torch.manual_seed(64)
    w64 = BlockSparseMatrix.zeros((c["n"], c["k"]), n_blocks=nnz_of(c) // 4, block_shape=(64, 64), device=dev)
    with torch.no_grad():
        w64.data.normal_(0, 0.02)
    x64 = torch.randn(c["m"], c["k"], device=dev)
    dy64 = torch.randn(c["m"], c["n"], device=dev)

    def step64():
        packed = w64.packed_weights()
        w64.reverse_matmul(x64, transpose=True, packed=packed)
        w64.matmul_with_output_sparse_support(dy64, x64)
        w64.reverse_matmul(dy64, transpose=False, packed=packed)

    ms = time_op(step64, max(3, min(steps, 10)), warm=3)
    out["c3_d0.25_blocks64/tf32x3"] = {"ms_per_step": ms, "effective_tflops": 3 * flops_per_op(c) / (ms / 1e3) / 1e12}
    del w64, x64, dy64
    torch.cuda.empty_cache()
    # host-side cost of one call: the smallest configuration is launch-bound, so the wall time of a long run of
    # back-to-back asynchronous calls is what the Python layer, ctypes, the tensor-map encoding and the launch cost
    import time as _time

    case = LayerCase(WORKLOADS["c1"], dev)
    pack, fwd, dgrad, wgrad = case.ops(native.resolve_precision("tf32x3"))
    pack()
    for name, fn in (("dsd", fwd), ("sddmm", wgrad), ("pack", pack)):
        for _ in range(20):
            fn()
        torch.cuda.synchronize()
        t0 = _time.perf_counter()
        for _ in range(300):
            fn()
        host = (_time.perf_counter() - t0) / 300
        torch.cuda.synchronize()
        out["host_us_per_call/c1/" + name] = host * 1e6
    del case, pack, fwd, dgrad, wgrad
    torch.cuda.empty_cache()
    # one step of the sparsity optimizer (pruning + regrowth of 10 % of the blocks, Adam state attached) on the
    # headline layer: statistic kernel, k-smallest selection, sampling of empty positions, index rebuild
    cases.clear()
    torch.cuda.empty_cache()
    from pytorch_block_sparse_b200 import SparseOptimizer

    case = LayerCase(WORKLOADS["c3_d0.25"], dev)
    adam = torch.optim.Adam([case.w.data], lr=1e-3)
    case.w.data.grad = torch.zeros_like(case.w.data)
    adam.step()
    so = SparseOptimizer([case.w], lr=0.1, seed=1)
    so.attach_optimizer(adam)
    out["sparse_optimizer_step_ms/c3_d0.25"] = time_op(so.step, 5, warm=2)
    del case, adam, so
    torch.cuda.empty_cache()
    return out


def run_c5(dev, world, rank, steps, precisions):
    """Benchmark configuration 5: one 32768 x 8192 layer at density 0.1 on 65536 tokens, its block-rows split over
    the ranks (strong scaling: the whole layer's work is fixed).  Per step and rank: pack, forward of the shard,
    all-gather of the output shards (side stream, overlapping what follows), local wgrad, dgrad to a partial
    input gradient, all-reduce of that partial gradient."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from pytorch_block_sparse_b200 import BlockSparseMatrix, native
    from pytorch_block_sparse_b200.distributed import shard_block_rows

    m, n, k = C5["m"], C5["n"], C5["k"]
    nnz = nnz_of(C5)
    np.random.seed(555)
    torch.manual_seed(555)
    full = BlockSparseMatrix.zeros((n, k), n_blocks=nnz, device=dev)
    with torch.no_grad():
        full.data.normal_(0, 0.02)
    w = shard_block_rows(full, rank, world) if world > 1 else full
    del full
    n_local = w.shape[0]
    gd = torch.Generator(device=dev).manual_seed(77)
    x = torch.randn(m, k, generator=gd, device=dev)            # replicated input
    dy = torch.randn(m, n_local, generator=gd, device=dev)     # this rank's slice of the output gradient
    bias = torch.zeros(n_local, device=dev)
    y = torch.empty(m, n_local, device=dev)
    dx = torch.empty(m, k, device=dev)
    dw = torch.empty_like(w.data)
    y_all = torch.empty(world, m, n_local, device=dev) if world > 1 else None  # rank-major gather, no interleave copy
    plan_f, plan_d, plan_w = w._plan(True), w._plan(False), w._sddmm_plan()
    side = torch.cuda.Stream(device=dev)
    data = w.data.detach()
    out = {"shape": dict(C5, nnz=nnz), "block_rows_per_rank": n_local // 32, "scaling": "strong"}
    f_total = 3 * 2.0 * m * nnz * 1024
    tensors32 = (x, dy, y, dx, y_all)
    for prec_name in precisions:
        prec = native.resolve_precision(prec_name)
        if prec_name == "bf16":  # the configuration says "X bf16": bf16 activations and outputs in HBM
            x, dy = tensors32[0].bfloat16(), tensors32[1].bfloat16()
            y, dx = torch.empty_like(tensors32[2], dtype=torch.bfloat16), torch.empty_like(tensors32[3], dtype=torch.bfloat16)
            y_all = torch.empty(world, m, n_local, device=dev, dtype=torch.bfloat16) if world > 1 else None
        else:
            x, dy, y, dx, y_all = tensors32
        elem = 2 if prec_name == "bf16" else 4

        def step(collectives):
            packed = native.pack_weights(data, prec)
            native.dsd_matmul(x, plan_f, packed, n_local, True, bias=bias, out=y)
            if collectives and world > 1:
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    dist.all_gather_into_tensor(y_all, y)
            native.sddmm(dy, True, x, True, w.blocks, dw, precision=prec, plan=plan_w)
            native.dsd_matmul(dy, plan_d, packed, k, False, out=dx)
            if collectives and world > 1:
                dist.all_reduce(dx)
                torch.cuda.current_stream().wait_stream(side)

        # the same step with the all-gather fused into the forward kernel: its epilogue stores this rank's columns into
        # every rank's full-width output over NVLink peer mappings (symmetric memory) while it computes
        fused_state = {}

        def fused_step(reduce_too):
            if "buf" not in fused_state:
                from pytorch_block_sparse_b200.distributed import PeerOutputs

                fused_state["outputs"] = PeerOutputs()
                full_y, handle = fused_state["outputs"].get(m, world * n_local, y.dtype, dev)
                fused_state["buf"], fused_state["handle"] = full_y, handle
                fused_state["peers"] = [int(handle.buffer_ptrs[r]) for r in range(world) if r != rank]
            if reduce_too and "parts" not in fused_state:
                parts, hp = fused_state["outputs"].get(m, k, torch.float32, dev, tag="dx_parts")
                total, ht = fused_state["outputs"].get(m, k, torch.float32, dev, tag="dx_sum")
                fused_state["parts"], fused_state["hp"], fused_state["ht"] = parts.view(world, m // world, k), hp, ht
                fused_state["part_ptrs"] = [int(hp.buffer_ptrs[r]) for r in range(world)]
                fused_state["sum_ptrs"] = [int(ht.buffer_ptrs[r]) for r in range(world)]
            handle = fused_state["handle"]
            packed = native.pack_weights(data, prec)
            handle.barrier()  # every rank is done with the previous step's outputs, parts and sums
            native.dsd_matmul(x, plan_f, packed, n_local, True, bias=bias, out=fused_state["buf"],
                              out_col0=rank * n_local, peer_outs=fused_state["peers"])
            native.sddmm(dy, True, x, True, w.blocks, dw, precision=prec, plan=plan_w)
            if reduce_too:
                # dgrad fused with the reduce-scatter half of the all-reduce: completed tiles go to this rank's slot on
                # the rank owning their tokens; each rank then adds its slots and stores the sums to every rank
                native.dsd_scatter(dy, plan_d, packed, k, False, fused_state["part_ptrs"], rank, scratch=dx)
                handle.barrier()  # every rank's columns and parts have arrived
                native.sum_row_slots(fused_state["parts"], fused_state["sum_ptrs"], rank * (m // world))
                handle.barrier()  # every rank's rows of the summed gradient have arrived
            else:
                native.dsd_matmul(dy, plan_d, packed, k, False, out=dx)
                dist.all_reduce(dx)
                handle.barrier()

        def step_fused(_):
            fused_step(False)

        def step_fused_both(_):
            fused_step(True)

        res = {}
        legs_c5 = [("compute_ms", step, False), ("with_collectives_ms", step, True)]
        if world > 1:
            legs_c5.append(("with_fused_gather_ms", step_fused, True))
            if prec_name != "bf16" and m % (128 * world) == 0:
                legs_c5.append(("with_fused_gather_and_reduce_scatter_ms", step_fused_both, True))
        for name, fn, coll in legs_c5:
            if coll and world == 1:
                res[name] = res["compute_ms"]
                continue
            if world > 1:
                dist.barrier()
            try:
                ms = time_op(lambda: fn(coll), max(2, min(steps, 5)), warm=2)
            except Exception as exc:  # symmetric memory may be unavailable on a box without peer access
                if fn is step_fused or fn is step_fused_both:
                    res[name] = None
                    res["fused_gather_unavailable"] = str(exc)[:200]
                    continue
                raise
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            res[name] = ms
        res["tensors"] = "bf16 activations and outputs" if elem == 2 else "fp32"
        res["all_gather_bytes_per_rank"] = (world - 1) * m * n_local * elem if world > 1 else 0
        res["all_reduce_bytes"] = m * k * elem if world > 1 else 0
        fused_state.clear()
        res["effective_tflops"] = f_total / (res["with_collectives_ms"] / 1e3) / 1e12
        if res.get("with_fused_gather_ms"):
            res["effective_tflops_fused_gather"] = f_total / (res["with_fused_gather_ms"] / 1e3) / 1e12
        if res.get("with_fused_gather_and_reduce_scatter_ms"):
            res["effective_tflops_fused_both"] = f_total / (res["with_fused_gather_and_reduce_scatter_ms"] / 1e3) / 1e12
        res["effective_tflops_compute_only"] = f_total / (res["compute_ms"] / 1e3) / 1e12
        out[prec_name] = res
    return out


def run_c4(dev, world, rank, steps):
    """Benchmark configuration 4: RoBERTa-base, three Linear kinds per layer made block-sparse at density 0.5 by
    BlockSparseModelPatcher, batch 32 x 512 random token ids per GPU, MLM loss, AdamW; token-data-parallel
    (gradients summed over the ranks; the sparse layers contribute only their stored blocks)."""
    import contextlib
    import io

    import numpy as np
    import torch
    import torch.distributed as dist

    try:
        from transformers import RobertaConfig, RobertaForMaskedLM
    except Exception as exc:  # pragma: no cover - the image has transformers
        return {"unavailable": "transformers not importable: %s" % exc}
    from pytorch_block_sparse_b200 import BlockSparseModelPatcher
    from pytorch_block_sparse_b200.block_sparse import BlockSparseMatrixBase

    batch, seq = 32, 512
    cfg = RobertaConfig(vocab_size=50265, hidden_size=768, num_hidden_layers=12, num_attention_heads=12,
                        intermediate_size=3072, max_position_embeddings=514, type_vocab_size=1,
                        hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, attn_implementation="sdpa")
    g = torch.Generator().manual_seed(4 + rank)
    ids = torch.randint(0, 50265, (batch, seq), generator=g).to(dev)
    labels = ids.clone()
    labels[torch.rand(batch, seq, generator=g).to(dev) > 0.15] = -100

    def build(sparse):
        torch.manual_seed(44)
        np.random.seed(44)
        model = RobertaForMaskedLM(cfg).to(dev)
        if sparse:
            mp = BlockSparseModelPatcher()
            for kind in ("intermediate", "output", "attention\\.output"):
                mp.add_pattern("roberta\\.encoder\\.layer\\.[0-9]+\\.%s\\.dense" % kind, {"density": 0.5})
            with contextlib.redirect_stdout(io.StringIO()):
                mp.patch_model(model)
        model.train()
        return model

    def train_ms(model, tf32):
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
        sparse_data = {id(mod.data) for mod in model.modules() if isinstance(mod, BlockSparseMatrixBase)}
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = tf32

        def step():
            opt.zero_grad(set_to_none=True)
            loss = model(input_ids=ids, labels=labels).loss
            loss.backward()
            if world > 1:
                grads = [p.grad for p in model.parameters() if p.grad is not None]
                flat = torch.cat([gr.reshape(-1) for gr in grads])
                dist.all_reduce(flat)
                flat /= world
                off = 0
                for gr in grads:
                    gr.copy_(flat[off:off + gr.numel()].view_as(gr))
                    off += gr.numel()
            opt.step()
            return loss

        if world > 1:
            dist.barrier()
        ms = time_op(step, max(2, min(steps, 4)), warm=2)
        torch.backends.cuda.matmul.allow_tf32 = old
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        grad_bytes = sum(p.numel() * 4 for p in model.parameters())
        sparse_bytes = sum(p.numel() * 4 for p in model.parameters() if id(p) in sparse_data)
        return ms, grad_bytes, sparse_bytes, float(step().item())

    out = {"model": "RoBERTa-base 12 x 768/3072, vocab 50265", "tokens_per_gpu_step": batch * seq,
           "patched": "intermediate.dense, output.dense, attention.output.dense at density 0.5"}
    # the patched model twice: with cuBLAS TF32 for the layers that stayed dense (QKV projections, LM head), as
    # beside "dense_tf32", and with strict fp32 there, as beside "dense_fp32"; the sparse layers run in the
    # library's precision either way -- once more with the other fp32-class mode ("bf16x3") and once with
    # single-pass TF32 in the sparse layers too, the like-for-like partner of "dense_tf32"
    from pytorch_block_sparse_b200 import native

    model = build(True)
    default_precision = native.default_precision()
    for name, tf32, sparse_prec in (("sparse", True, default_precision), ("sparse_fp32_rest", False, default_precision),
                                    ("sparse_bf16x3", True, "bf16x3"), ("sparse_tf32", True, "tf32")):
        native.set_default_precision(sparse_prec)
        try:
            ms, grad_bytes, sparse_bytes, loss = train_ms(model, tf32=tf32)
        finally:
            native.set_default_precision(default_precision)
        out[name] = {"ms_per_step": ms, "tokens_per_s": world * batch * seq / (ms / 1e3), "loss": loss,
                     "dense_layers_allow_tf32": tf32, "sparse_layers_precision": sparse_prec,
                     "parameters": sum(p.numel() for p in model.parameters()),
                     "grad_bytes_per_step": grad_bytes, "of_which_sparse_layers": sparse_bytes}
    del model
    torch.cuda.empty_cache()
    model = build(False)
    for name, tf32 in (("dense_tf32", True), ("dense_fp32", False)):
        ms, grad_bytes, _, loss = train_ms(model, tf32=tf32)
        out[name] = {"ms_per_step": ms, "tokens_per_s": world * batch * seq / (ms / 1e3), "loss": loss,
                     "parameters": sum(p.numel() for p in model.parameters()), "grad_bytes_per_step": grad_bytes}
    del model
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args, cfg):
    import torch
    import torch.distributed as dist

    from pytorch_block_sparse_b200 import native

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
    legs = set(filter(None, args.legs.split(","))) - {"none"}

    case = LayerCase(cfg, dev, rank, host_buffers=True)
    lin, w = case.lin, case.w
    x, dy, y, dx, dw = case.x, case.dy, case.y, case.dx, case.dw
    side = torch.cuda.Stream(device=dev)
    reducer, allreduce_kind = None, "none"
    if world > 1:
        # the nnz-block gradient is summed over the ranks by this library's own peer-memory kernel (the gradient
        # buffer lives in symmetric memory); NCCL where symmetric memory is not available
        allreduce_kind = "nccl"
        if not args.nccl_allreduce:
            try:
                from pytorch_block_sparse_b200.distributed import PeerAllReduce

                reducer = PeerAllReduce(case.dw.numel(), dev)
                case.dw = dw = reducer.buffer[: dw.numel()].view_as(dw)
                allreduce_kind = "bsmm_allreduce_peers over symmetric memory"
            except Exception as exc:  # noqa: BLE001
                allreduce_kind = "nccl (symmetric memory unavailable: %s)" % str(exc)[:120]
    pack, fwd, dgrad, wgrad = case.ops(prec)

    def step():
        # the weight gradient first: its all-reduce (N > 1) then travels while dgrad computes
        pack()
        fwd()
        wgrad()
        if world > 1:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                if reducer is not None:
                    reducer()
                else:
                    dist.all_reduce(dw)
        dgrad()
        if world > 1:
            torch.cuda.current_stream().wait_stream(side)

    # kernels of this library launched per step: pack, fwd, dgrad, wgrad (+ its token-range reduction)
    launches_per_step = 5 if native.load().bsmm_sddmm_workspace_bytes(n, k, m, nnz, prec) > 0 else 4
    if reducer is not None:
        launches_per_step += 1  # the peer-memory all-reduce kernel (the two barriers around it are torch's)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
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
    pack()
    reps = max(3, min(20, args.steps))
    kernels = {"pack_ms": time_op(pack, reps), "fwd_ms": time_op(fwd, reps), "dgrad_ms": time_op(dgrad, reps),
               "wgrad_ms": time_op(wgrad, reps)}

    # ---- end to end through the public layer API with host buffers ----
    x_host, dy_host = case.x_host, case.dy_host
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

    e2e_steps = max(4, args.steps)
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
    del x_dev, dy_dev, y_host, dx_host, dw_host

    # ---- comparators (rank 0): cuBLAS dense nn.Linear fwd+bwd on the same shape, the reference's CUDA kernels ----
    comparators, peaks_here = {}, None
    if rank == 0 and not args.no_comparators:
        peaks_here = measure_gemm_peaks(dev)
        wd = torch.randn(n, k, device=dev) * 0.02
        bias = case.bias

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

    # ---- extra legs ----
    extra = {}
    if "sweep" in legs and world == 1:
        del case, lin, w, x, dy, y, dx, dw, pack, fwd, dgrad, wgrad, x_host, dy_host
        torch.cuda.empty_cache()
        extra["sweep"] = run_sweep(dev, args.steps)
    else:
        del case, lin, w, x, dy, y, dx, dw, pack, fwd, dgrad, wgrad, x_host, dy_host
        torch.cuda.empty_cache()
    if "c5" in legs:
        extra["c5"] = run_c5(dev, world, rank, args.steps, sorted({prec_name, "bf16"}))
        torch.cuda.empty_cache()
    if "c4" in legs:
        extra["c4"] = run_c4(dev, world, rank, args.steps)
        torch.cuda.empty_cache()
    status |= native.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel ----
    peaks = measured_peaks()
    op_names = {"fwd_ms": ("dsd forward", "dsd_umma"), "dgrad_ms": ("dsd dgrad", "dsd_umma"), "wgrad_ms": ("sddmm wgrad", "sddmm_umma")}
    dom = max(op_names, key=lambda key: kernels[key])
    achieved = f_op / (kernels[dom] / 1e3) / 1e12
    if peaks_here is not None:
        # the denominator is cuBLAS on this GPU in this run: TF32 for the tf32 kernels, bf16 for the bf16 mode
        peak = peaks_here["bf16_tflops"] if prec_name == "bf16" else peaks_here["tf32_tflops"]
        peak_source = "measured in this run: cuBLAS %s 8192^3, best of 5" % ("bf16" if prec_name == "bf16" else "TF32 (allow_tf32)")
    else:
        peak = peaks["bf16_tflops"] if prec_name == "bf16" else peaks["bf16_tflops"] / 2.0
        peak_source = "%s bf16 burst %.1f TFLOP/s%s (comparators switched off: no TF32 GEMM was timed)" % (
            peaks["source"], peaks["bf16_tflops"], "" if prec_name == "bf16" else " / 2")
    traffic, traffic_source = profile_traffic(op_names[dom][1], prec_name, args.workload)
    roofline = {
        "kernel": op_names[dom][0], "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_source, "peak_source": peak_source,
        "algorithmic_flops_per_launch": f_op,
    }
    if prec_name == "tf32x3":
        # three tensor-core products per useful one: the ceiling of this mode on effective FLOPs
        roofline["frac_of_3xtf32_ceiling"] = achieved / (peak / 3.0)
    if peaks_here is not None:
        roofline["gemm_peaks_this_run"] = peaks_here
    roofline["step_frac"] = (3 * f_op / (ms_per_step / 1e3) / 1e12) / world / peak * world  # whole step vs the same peak

    def ratio(key):  # > 1: this library's step is the faster one
        return comparators[key] / ms_per_step if key in comparators else None

    if world == 1:
        cpu_value, cpu_m, cpu_kind = time_cpu_reference(cfg, target_seconds=args.cpu_seconds, reps=3)
        cpu_sample = "first %d of %d tokens, median of 3; to_dense + fp32 matmul (%s)" % (
            cpu_m, m, "the reference package on torch CPU" if cpu_kind == "reference" else "numpy restatement")
    else:  # the host cores are timed in the single-GPU run only
        cpu_value, cpu_sample, cpu_kind = None, "not timed when n_gpus > 1", "port"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": prec_name, "data": "synthetic",
        "config": dict(workload=args.workload, nnz=nnz, parallelism="token-dp%d" % world, grad_allreduce=allreduce_kind,
                       cache=("x and dy are %d and %d MiB, larger than the 126 MB L2" % (m * k * 4 >> 20, m * n * 4 >> 20))
                       if min(m * k, m * n) * 4 > (126 << 20) else
                       ("x and dy (%d and %d MiB) fit the 126 MB L2 and are not flushed between steps"
                        % (m * k * 4 >> 20, m * n * 4 >> 20)), **cfg),
        "roofline": roofline,
        "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": os.cpu_count(), "kind": cpu_kind,
                         "sample": cpu_sample},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "kernels": kernels,
        "comparators": comparators,
        "vs_cublas_tf32": ratio("cublas_dense_tf32_ms"),
        "vs_cublas_bf16": ratio("cublas_dense_bf16_ms"),
        "vs_cublas_fp32": ratio("cublas_dense_fp32_ms"),
        "vs_reference_cuda": ratio("reference_cuda_kernels_ms"),
        "device_status": status,
    }
    line.update(extra)
    # the other fp32-class precision on the headline workload (timed in the sweep leg) beside dense cuBLAS TF32
    other = extra.get("sweep", {}).get("%s/bf16x3" % args.workload)
    if other is not None and prec_name == "tf32x3" and "cublas_dense_tf32_ms" in comparators:
        line["bf16x3"] = {"ms_per_step": other["ms_per_step"], "effective_tflops": other["effective_tflops"],
                          "vs_cublas_tf32": comparators["cublas_dense_tf32_ms"] / other["ms_per_step"],
                          "note": "fp32-class (error 5e-6, bound 1e-5): three products of bf16 hi and lo parts"}
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
    ap.add_argument("--precision", default="tf32x3", choices=["tf32x3", "bf16x3", "tf32", "bf16", "fp32"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-comparators", action="store_true")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="N > 1: sum the weight gradients with NCCL instead of the library's peer-memory kernel")
    ap.add_argument("--legs", default="sweep,c5,c4",
                    help="comma list of extra legs timed after the headline: sweep (1 GPU only), c5, c4; 'none' for none")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_gpu_arm(args, cfg)


if __name__ == "__main__":
    main()
