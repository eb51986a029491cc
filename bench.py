#!/usr/bin/env python
"""Benchmarks of the MXFP8 dense / MoE hot path on B200. Prints ONE JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Workloads (``--workload``):

  dense     (default) the headline: one step = one pass of ``fso.dense.linear`` (1x32 activation quantizer, then the
            tcgen05 block-scaled GEMM) over the Llama-3-8B gate_up projection, M=8192, N=28672, K=4096. Operands and
            output exceed L2, so every step streams them from HBM. With N > 1 (torch.distributed.run, one rank per
            GPU) the weight rows are split N ways (column parallel, no data-path collective); ``value`` is the whole
            job's 2*M*N*K over the slowest rank's device time. Unless ``--no-moe`` is given, the same run then
            measures the ``moe`` workload below with fewer steps and attaches it as the line's ``"moe"`` object
            (the second half of the headline metric: MoE layer tokens/s at 1/2/4/8 GPUs).
  moe       one DeepSeek-V3-shaped MoE layer (256 experts, top-8, H=7168, I=2048), 4096 tokens per GPU, experts
            sharded 256/N per GPU, token rows exchanged by the library's kernels over peer memory (weak scaling;
            ``FSO_B200_EP_TRANSPORT=collective`` uses NCCL all-to-all-v instead); ``--moe-config mixtral``
            runs the 8-expert top-2 H=4096 I=14336 layer on one GPU. Metric: tokens/s.
  decode    dense linears at M=16 over the four Llama-3-8B shapes, CUDA-graph replay over rotated weight copies
            (cold weights). Metric: achieved weight-stream GB/s (worst of the four shapes).
  quantize  the activation quantizer alone on [8192, 4096]. Metric: GB/s.
  requant   the block-FP8 -> MXFP8 requantization kernel of prepare_weight alone on [24576, 7168]. Metric: GB/s.
  bsfp8     BASELINE.json configs[2]: prepare_weight(format="bsfp8") on the three DeepSeek-V3 dense shapes and the
            linears at M in {16, 512, 4096} on the prepared weights (CUDA-graph replay).
  sweep     BASELINE.json configs[1] as one table: the four Llama-3-8B shapes x M in {1, 16, 128, 1024, 8192} with
            cuBLAS' MXFP8 GEMM and a bf16 matmul in the same run.

``--impl reference`` times the reference's CPU statement of the same workload (the fp32 dequantize-then-matmul
oracle under ``oracle/``, the only thing that runs there) on this box's host cores, on a bounded sample, and prints
the same line with ``"impl": "reference"``.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA = {"qkv": (6144, 4096), "gate_up": (28672, 4096), "o_proj": (4096, 4096), "down": (4096, 14336)}
MOE_CONFIGS = {"dsv3": dict(E=256, k=8, H=7168, I=2048, T=4096, renorm=False),
               "mixtral": dict(E=8, k=2, H=4096, I=14336, T=8192, renorm=True),
               # a quarter of the DeepSeek-V3 layer with the same 128 rows expected per expert: 2.8 GB of weights,
               # small enough for a multi-pass profiler capture and still far larger than L2
               "dsv3_e64": dict(E=64, k=8, H=7168, I=2048, T=1024, renorm=False)}
L2_BYTES = 126e6


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_burst": float(p["bf16_tflops"]),
                "bf16_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - clocks are reported as unavailable, the run goes on
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(0.005)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


class Dist:
    """The process group of this run (one rank per GPU under torch.distributed.run, or a single process)."""

    def __init__(self, torch):
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (B200); this arm has no CPU path")
        torch.cuda.set_device(self.local)
        self.keep = False
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, dtype=self.torch.float64, device="cuda")
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def close(self):
        """Ends the process group, unless another workload of this run still needs it (``keep``)."""
        if self.keep:
            return
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


_SHARED_DIST = None


def shared_dist(torch) -> "Dist":
    """One process group per run: the default run measures two workloads one after the other."""
    global _SHARED_DIST
    if _SHARED_DIST is None:
        _SHARED_DIST = Dist(torch)
    return _SHARED_DIST


def device_allocs(torch) -> int:
    """cudaMalloc calls the caching allocator has made so far on this device."""
    return int(torch.cuda.memory_stats().get("num_device_alloc", 0))


def timed_steps(torch, d: Dist, step, steps: int, warmup: int, per_step_events: bool = False, finish=None, stats=None):
    """W untimed steps, then exactly K steps between barrier + synchronize on both sides, timed with CUDA events on
    the launching stream. ``finish`` (optional) runs after the last step and before the closing event: it makes the
    launching stream wait for work the steps put on other streams. ``stats`` (optional dict) receives the number of
    device allocations the caching allocator made inside the timed region. Returns (total ms, clocks summary,
    [per-step event pairs])."""
    stream = torch.cuda.current_stream()
    for _ in range(warmup):
        step(None)
    if finish is not None:
        finish()
    d.barrier()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)] \
        if per_step_events else None
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(d.local) as clocks:
        d.barrier()
        allocs0 = device_allocs(torch)
        t0.record(stream)
        for i in range(steps):
            step(pairs[i] if pairs else None)
        if finish is not None:
            finish()
        t1.record(stream)
        if stats is not None:
            stats["device_allocs"] = device_allocs(torch) - allocs0
        d.barrier()
    return t0.elapsed_time(t1), clocks.summary(), pairs


def timed_e2e(torch, d: Dist, pipe, steps: int, warmup: int = 3, attempts: int = 3):
    """The end-to-end leg: ``timed_steps`` over the host pipeline, measured again (at most ``attempts`` times) while
    the caching allocator still obtained device memory inside the timed region. The pipeline keeps results alive
    until their copy to the host has finished, so its first steps grow the allocator's pool, and a cudaMalloc stalls
    the device for milliseconds; a steady-state step allocates nothing. Returns (total ms of the last region,
    every measured region as [ms per step, max over ranks, allocations]); the last one counts."""
    ms, tried = 0.0, []
    for _ in range(attempts):
        st = {}
        ms, _, _ = timed_steps(torch, d, pipe.step, steps, warmup, finish=pipe.finish, stats=st)
        ms_max, grew = d.max_over_ranks([ms, float(st["device_allocs"])])
        tried.append([round(ms_max / steps, 4), int(grew)])
        if grew == 0:
            break
    return ms, tried


def parse_cpulist(text: str):
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11}."""
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


class NearGpu:
    """Runs its block on the CPUs next to one GPU's PCIe root (``local_cpulist`` of the device in sysfs), so that the
    pinned host buffers allocated inside are placed by first touch on that NUMA node; the affinity the process had
    is put back afterwards (the CPU baseline keeps every core). Best effort: without the sysfs entry, or when the
    list would not narrow the affinity, nothing changes. ``note`` says what happened."""

    def __init__(self, torch, device_index: int, sysfs: str = "/sys/bus/pci/devices"):
        self.note, self._cpus, self._old = "host buffers pinned where the process ran (no NUMA information)", None, None
        try:
            pr = torch.cuda.get_device_properties(device_index)
            dev = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            with open(os.path.join(sysfs, dev, "local_cpulist")) as f:
                text = f.read().strip()
            old = os.sched_getaffinity(0)
            near = parse_cpulist(text) & old
            if near and near != old:
                self._cpus, self._old = near, old
                self.note = f"host buffers pinned on the GPU's NUMA node (cpus {text})"
            elif near:
                self.note = "host buffers pinned where the process ran (one NUMA node)"
        except (OSError, ValueError, AttributeError, RuntimeError):
            pass

    def __enter__(self):
        if self._cpus:
            os.sched_setaffinity(0, self._cpus)
        return self

    def __exit__(self, *exc):
        if self._old:
            os.sched_setaffinity(0, self._old)
        return False


class HostPipeline:
    """End-to-end steps with host buffers: every step copies its input from pinned host memory to the device, runs
    ``fn`` on it (the public call) and copies the result back to pinned host memory. The three legs run on three
    streams with two input buffers, so step i's result leaves over PCIe while step i + 1's input arrives and its
    kernels run; every byte of every step still moves inside the timed region."""

    def __init__(self, torch, x_host, fn, out_host):
        self.torch, self.fn, self.x_host, self.out_host = torch, fn, x_host, out_host
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.x_dev = [torch.empty(x_host.shape, dtype=x_host.dtype, device="cuda") for _ in range(2)]
        self.x_free = [None, None]          # event after which x_dev[j] may be overwritten
        self.out_done = None
        self.i = 0

    def step(self, _):
        torch, j = self.torch, self.i % 2
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_in):
            if self.x_free[j] is not None:
                self.s_in.wait_event(self.x_free[j])
            self.x_dev[j].copy_(self.x_host, non_blocking=True)
            arrived = self.s_in.record_event()
        main.wait_event(arrived)
        y = self.fn(self.x_dev[j])
        computed = main.record_event()
        self.x_free[j] = computed
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(computed)
            self.out_host.copy_(y, non_blocking=True)
            y.record_stream(self.s_out)
            self.out_done = self.s_out.record_event()
        self.i += 1

    def finish(self):
        if self.out_done is not None:
            self.torch.cuda.current_stream().wait_event(self.out_done)


def base_line(args, d, metric, unit, value, ms_step, scaling, dtype, config):
    return {"metric": metric, "value": value, "unit": unit, "n_gpus": d.world if d else args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": config}


# ====================================================================================================== dense

DENSE_M, DENSE_N, DENSE_K = 8192, 28672, 4096


def dense_shape(args):
    if args.shape:
        return tuple(int(v) for v in args.shape.split(","))
    return DENSE_M, DENSE_N, DENSE_K


def dense_workload_name(m, n, k):
    if (m, n, k) == (DENSE_M, DENSE_N, DENSE_K):
        return f"llama3-8b gate_up linear: x bf16 [{m}, {k}] ~ N(0,1), w bf16 [{n}, {k}] ~ N(0,0.02) as MXFP8"
    return f"dense linear override: x bf16 [{m}, {k}], w bf16 [{n}, {k}] as MXFP8"


def dense_kernel_name(m, n_local):
    """The kernel the library's host picker sends this large-M shape to (csrc/gemm_host.cuh: use_pair_kernel)."""
    pair_tiles = ((m + 255) // 256) * (n_local // 256)
    blocks = (m + 127) // 128
    if (m > 64 and n_local % 256 == 0 and pair_tiles >= 148 // 2 and (blocks % 2 == 0 or blocks >= 15)
            and os.environ.get("FSO_B200_PAIR", "1")[:1] != "0"):
        return "gemm_mxf8_pair_kernel (cta_group::2, 256 x 256 per CTA pair)"
    return "gemm_mxf8_kernel<256, bf16>"


def dense_config(m, n, k, world):
    """The ``config`` object of the dense workload (the same in both arms)."""
    return {"workload": dense_workload_name(m, n, k), "M": m, "N": n, "K": k,
            "parallelism": f"column-parallel N-split x{world} (no collective)",
            "step": "quantize_activation + linear(xq, x_scale) == linear(x): 2 kernels",
            "l2": "operands and output of a step exceed the 126 MB L2 (x 64 MB, w 117 MB, y 470 MB at N=1)"}


def dense_inputs(torch, m, n, k, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(m, k, generator=g, dtype=torch.float32).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g, dtype=torch.float32)).to(torch.bfloat16)
    return x, w


def dense_cpu_runner(torch, m, n, k, budget_s: float, threads: int):
    """The oracle's dense path on host cores: quantize the activation rows (1x32 rule), dequantize, fp32 matmul
    against the dequantized MXFP8 weight. Returns (run(rows) -> (seconds, y), rows sized to about budget_s)."""
    from oracle import oracle as O

    O.build()
    torch.set_num_threads(threads)
    x, w = dense_inputs(torch, m, n, k)
    wq, ws = O.quantize_1x32(w)
    wd = torch.from_numpy(O.dequant(wq, ws))

    def run(rows):
        t0 = time.perf_counter()
        xq, xs = O.quantize_1x32(x[:rows])
        xd = torch.from_numpy(O.dequant(xq, xs))
        y = (xd @ wd.t()).to(torch.bfloat16)
        return time.perf_counter() - t0, y

    probe = min(32, m)
    dt_probe, _ = run(probe)
    rows = int(max(probe, min(m, probe * budget_s / max(dt_probe, 1e-6))))
    rows = max(probe, rows // 32 * 32) if rows >= 32 else rows
    return run, rows


def dense_reference(args):
    import torch

    if int(os.environ.get("RANK", "0")) != 0:
        return None
    m, n, k = dense_shape(args)
    threads = os.cpu_count() or 1
    budget = min(10.0, max(1.0, 60.0 / max(1, args.steps + args.warmup)))
    run, rows = dense_cpu_runner(torch, m, n, k, budget, threads)
    for _ in range(args.warmup):
        run(rows)
    dt = sum(run(rows)[0] for _ in range(args.steps)) / args.steps
    val = 2.0 * rows * n * k / dt / 1e12
    sample = f"first {rows} of {m} activation rows against the full [{n}, {k}] weight per step"
    line = base_line(args, None, "mxfp8_gemm_tflops", "TFLOP/s", val, dt * 1e3, "strong", "f32",
                     dense_config(m, n, k, int(os.environ.get("WORLD_SIZE", "1"))))
    line.update({"impl": "reference",
                 "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
                 "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                 "gpu_launches": 0})
    return line


def dense_ours(args):
    import torch

    import fish_scales_ops_b200 as fso
    from fish_scales_ops_b200 import _ops, parallel

    d = shared_dist(torch)
    m, n, k = dense_shape(args)
    r0, r1 = parallel.column_shard(n, d.world, d.rank)
    n_local = r1 - r0
    fso.build()
    x_cpu, w_cpu = dense_inputs(torch, m, n, k)
    weight = fso.dense.prepare_weight(w_cpu[r0:r1].cuda(), format="mxfp8")
    x = x_cpu.cuda()
    with NearGpu(torch, d.local) as near:
        x_host = x_cpu.pin_memory()
        y_host = torch.empty((m, n_local), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream()

    def step(ev):
        xq, sx = fso.dense.quantize_activation(x)
        if ev is not None:
            ev[0].record(stream)
        y = fso.dense.linear(xq, weight, x_scale=sx)
        if ev is not None:
            ev[1].record(stream)
        return y

    ms_total, clocks, pairs = timed_steps(torch, d, step, args.steps, args.warmup, per_step_events=True)
    gemm_ms = sum(a.elapsed_time(b) for a, b in pairs) / args.steps

    # end to end through the public call with host buffers: H2D of the activation, linear, D2H of the result, every
    # step; the copies of neighbouring steps overlap (PCIe is full duplex), the kernels of one step do not move
    pipe = HostPipeline(torch, x_host, lambda xd: fso.dense.linear(xd, weight), y_host)
    e_steps = max(3, min(args.steps, 20))
    e2e_ms, e2e_regions = timed_e2e(torch, d, pipe, e_steps)
    # sustained: back-to-back steps for at least two seconds (the timed K steps above are a burst of a few tens of
    # milliseconds; under the 1 kW cap the part settles at a lower clock)
    sus_steps = max(args.steps, int(2.2e3 / max(ms_total / args.steps, 1e-3)))
    sus_ms, sus_clocks, _ = timed_steps(torch, d, step, sus_steps, 0) if not args.no_sustained else (0.0, {}, None)
    ms_total, e2e_ms, gemm_ms, sus_ms = d.max_over_ranks([ms_total, e2e_ms, gemm_ms, sus_ms])
    status = _ops.device_status()
    if d.rank != 0:
        d.close()
        return None

    flops = 2.0 * m * n * k
    ms_step = ms_total / args.steps
    pk = peaks()
    fp8_peak = 2.0 * pk["bf16_burst"]
    gemm_tflops = 2.0 * m * n_local * k / (gemm_ms * 1e-3) / 1e12
    line = base_line(args, d, "mxfp8_gemm_tflops", "TFLOP/s", flops / (ms_step * 1e-3) / 1e12, ms_step, "strong",
                     "fp8_e4m3", dense_config(m, n, k, d.world))
    # DRAM traffic of one launch: the ncu captures of the two kernels on 8192 x 8192 x 4096 (203.4 MB of algorithmic
    # bytes) read + wrote 238.5 MB (pair kernel) and 193.4 MB (single-CTA kernel): operands fetched from HBM once or
    # twice, re-reads served by L2, the output written once. The kernel's traffic grows in proportion to its
    # algorithmic bytes, so the captured ratio is applied to this launch's bytes
    kernel_name = dense_kernel_name(m, n_local)
    captured_mb = 238.5 if "pair" in kernel_name else 193.4
    algo_bytes = (m * k + n_local * k) * (1 + 1 / 32) + 2.0 * m * n_local
    line["roofline"] = {
        "bound": "tensor", "kernel": kernel_name, "achieved": gemm_tflops, "peak": fp8_peak,
        "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak, "traffic": algo_bytes * (captured_mb / 203.4),
        "traffic_unit": "bytes per launch",
        "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture on 8192x8192x4096 "
                          f"({captured_mb} MB for 203.4 MB algorithmic), scaled by this launch's algorithmic bytes "
                          f"({algo_bytes / 1e6:.1f} MB)",
        "peak_source": f"2 x {pk['source']} bf16 burst ({pk['bf16_burst']} TF/s): an fp8 MMA does twice the bf16 "
                       f"work per cycle; nominal dense fp8 is 4500",
        "frac_of_nominal": gemm_tflops / 4500.0, "flops_per_launch": 2.0 * m * n_local * k, "ms_per_launch": gemm_ms}
    line["e2e"] = {"value": flops / (e2e_ms / e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                   "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * n_local * 2,
                   "ms_per_step": e2e_ms / e_steps, "regions_ms_per_step_and_device_allocs": e2e_regions,
                   "host_buffers": near.note}
    line["gpu_launches"] = 2 * args.steps
    line["clocks"] = clocks
    line["device_status"] = status
    if sus_ms > 0:
        sus_step = sus_ms / sus_steps
        mhz = sus_clocks.get("sm_mhz") or 0
        line["sustained"] = {"value": flops / (sus_step * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": sus_steps,
                             "seconds": sus_ms / 1e3, "ms_per_step": sus_step, "clocks": sus_clocks,
                             "ms_per_step_x_sm_mhz": sus_step * mhz,
                             "frac_of_2x_bf16_sustained": flops / (sus_step * 1e-3) / 1e12 / (2.0 * pk["bf16_sustained"])}
    if not args.no_cpu_baseline and d.world == 1:
        threads = os.cpu_count() or 1
        run, rows = dense_cpu_runner(torch, m, n, k, 10.0, threads)
        dt, y_cpu = run(rows)
        y_gpu = step(None)[:rows].float().cpu()
        line["cpu_baseline"] = {
            "value": 2.0 * rows * n * k / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"first {rows} of {m} activation rows against the full weight, one pass",
            "rel_frobenius_gpu_vs_cpu": float((y_gpu - y_cpu.float()).norm() / y_cpu.float().norm())}
    d.close()
    return line


# ====================================================================================================== MoE

def moe_inputs(torch, cfg, tokens, seed, device="cpu", skew=0.0):
    """hidden ~ N(0,1), router logits ~ N(0,1) -> softmax top-k (renormalised for the Mixtral config). ``skew`` > 0:
    the logits get the log of a Zipf(skew) popularity over a seeded ranking of the experts added (the skewed regime
    of BASELINE.json configs[3])."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    hidden = torch.randn(tokens, cfg["H"], generator=g, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn(tokens, cfg["E"], generator=g, dtype=torch.float32)
    if skew > 0:
        rank = torch.randperm(cfg["E"], generator=torch.Generator(device="cpu").manual_seed(4242)).to(torch.float32)
        logits = logits + torch.log((rank + 1.0) ** (-skew))
    p = torch.softmax(logits, dim=-1)
    w, ids = torch.topk(p, cfg["k"], dim=-1)
    if cfg["renorm"]:
        w = w / w.sum(dim=-1, keepdim=True)
    return hidden.to(device), ids.to(torch.int32).to(device), w.to(device)


def moe_expert_weights(torch, cfg, e0, e1, device):
    """bf16 ~ N(0, 0.02) experts [e0, e1), generated expert by expert on the device (seeded per expert, so every
    rank and the CPU arm see the same expert e whatever the sharding)."""
    n = e1 - e0
    w13 = torch.empty((n, 2 * cfg["I"], cfg["H"]), dtype=torch.bfloat16, device=device)
    w2 = torch.empty((n, cfg["H"], cfg["I"]), dtype=torch.bfloat16, device=device)
    for j, e in enumerate(range(e0, e1)):
        g = torch.Generator(device=device).manual_seed(1000 + e)
        w13[j] = (0.02 * torch.randn(2 * cfg["I"], cfg["H"], generator=g, device=device)).to(torch.bfloat16)
        w2[j] = (0.02 * torch.randn(cfg["H"], cfg["I"], generator=g, device=device)).to(torch.bfloat16)
    return w13, w2


def moe_cpu_runner(torch, cfg, sample_tokens, threads):
    """The oracle's MoE layer on host cores for a token sample, with only the experts that sample touches
    materialised (quantized weights prepared once, outside the timed call; the call dequantizes them, runs the fp32
    matmuls and requantizes the SwiGLU intermediate). Returns (run() -> (seconds, out), inputs)."""
    import numpy as np

    from oracle import oracle as O

    O.build()
    torch.set_num_threads(threads)
    hidden, ids, w = moe_inputs(torch, cfg, sample_tokens, 7)
    used = sorted(set(ids.reshape(-1).tolist()))
    remap = {e: j for j, e in enumerate(used)}
    ids_l = torch.tensor([[remap[int(v)] for v in row] for row in ids.tolist()], dtype=torch.int32)
    q13, s13, q2, s2 = [], [], [], []
    for e in used:
        w13, w2 = moe_expert_weights(torch, cfg, e, e + 1, "cpu")
        a, b = O.quantize_1x32(w13[0], interleave_i=cfg["I"])
        c, dd = O.quantize_1x32(w2[0])
        q13.append(a), s13.append(b), q2.append(c), s2.append(dd)
    q13, s13, q2, s2 = np.stack(q13), np.stack(s13), np.stack(q2), np.stack(s2)

    def run():
        t0 = time.perf_counter()
        out = O.moe_layer(hidden, q13, s13, q2, s2, ids_l, w, interleaved=True)
        return time.perf_counter() - t0, out

    return run, (hidden, ids, w)


def moe_cpu_check(torch, d, cfg, experts, e0, hidden_cpu, ids_cpu, w_cpu, out_gpu_rows, sample, threads):
    """The oracle's layer for the first ``sample`` tokens of rank 0, on the host cores, from the prepared experts'
    own bytes (the handle's bytes are pinned bit for bit against the oracle's quantizer by the tests). Under expert
    parallelism the touched experts' bytes travel to rank 0 from the ranks that own them. Every rank must call this;
    rank 0 gets (seconds, rel. Frobenius error, max |err| / max |ref|), the others None."""
    import numpy as np

    per = experts.num_experts
    used = torch.full((sample * cfg["k"],), -1, dtype=torch.int64, device="cuda")
    if d.rank == 0:
        u = sorted({int(v) for v in ids_cpu[:sample].reshape(-1).tolist()})
        used[:len(u)] = torch.tensor(u, device="cuda")
    if d.world > 1:
        d.dist.broadcast(used, src=0)
    used = [int(v) for v in used.tolist() if v >= 0]
    parts = []
    for g in used:
        owner, local = g // per, g % per
        if d.rank == owner:
            ts = [experts.w13[local].contiguous(), experts.sw13[local].contiguous(), experts.w2[local].contiguous(),
                  experts.sw2[local].contiguous()]
        else:
            ts = [torch.empty_like(experts.w13[0]), torch.empty_like(experts.sw13[0]), torch.empty_like(experts.w2[0]),
                  torch.empty_like(experts.sw2[0])]
        if d.world > 1:
            for t_ in ts:
                d.dist.broadcast(t_.view(torch.uint8) if t_.dtype != torch.int32 else t_, src=owner)
        if d.rank == 0:
            parts.append([ts[0].view(torch.uint8).cpu().numpy(), ts[1].cpu().numpy().view(np.uint32),
                          ts[2].view(torch.uint8).cpu().numpy(), ts[3].cpu().numpy().view(np.uint32)])
    if d.rank != 0:
        return None
    from oracle import oracle as O

    O.build()
    torch.set_num_threads(threads)
    remap = {g: j for j, g in enumerate(used)}
    ids_l = torch.tensor([[remap[int(v)] for v in row] for row in ids_cpu[:sample].tolist()], dtype=torch.int32)
    q13, s13, q2, s2 = (np.stack([p_[i] for p_ in parts]) for i in range(4))
    t0 = time.perf_counter()
    ref = O.moe_layer(hidden_cpu[:sample], q13, s13, q2, s2, ids_l, w_cpu[:sample], interleaved=True)
    dt = time.perf_counter() - t0
    got = out_gpu_rows.float().cpu()
    rel = float((got - ref).norm() / ref.norm())
    mx = float((got - ref).abs().max() / ref.abs().max())
    return dt, rel, mx


MOE_CPU_SAMPLE = {"dsv3": 4, "mixtral": 64, "dsv3_e64": 4}


def moe_reference(args):
    import torch

    if int(os.environ.get("RANK", "0")) != 0:
        return None
    cfg = MOE_CONFIGS[args.moe_config]
    threads = os.cpu_count() or 1
    sample = MOE_CPU_SAMPLE[args.moe_config]
    run, _ = moe_cpu_runner(torch, cfg, sample, threads)
    for _ in range(min(args.warmup, 1)):
        run()
    n = max(1, min(args.steps, 5))
    dt = sum(run()[0] for _ in range(n)) / n
    v = sample / dt
    note = f"{sample} tokens with their real routing; only the experts they touch are prepared (outside the timed call)"
    line = base_line(args, None, "moe_layer_tokens_per_s", "tokens/s", v, dt * 1e3, "weak", "f32",
                     {"workload": f"{args.moe_config} MoE layer", **{k_: cfg[k_] for k_ in ("E", "k", "H", "I")},
                      "sample": note})
    line.update({"impl": "reference",
                 "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": note},
                 "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                 "gpu_launches": 0})
    return line


def moe_ours(args):
    import torch

    import fish_scales_ops_b200 as fso
    from fish_scales_ops_b200 import _ops, parallel

    d = shared_dist(torch)
    cfg = MOE_CONFIGS[args.moe_config]
    if d.world > 1 and args.moe_config != "dsv3":
        raise SystemExit("the multi-GPU MoE workload is the DeepSeek-V3 config (expert parallel)")
    fso.build()
    e0, e1 = parallel.expert_shard(cfg["E"], d.world, d.rank)
    w13, w2 = moe_expert_weights(torch, cfg, e0, e1, "cuda")
    experts = fso.moe.prepare_experts(w13, w2, format="mxfp8")
    del w13, w2
    torch.cuda.empty_cache()
    tokens = args.moe_tokens or cfg["T"]
    skew = float(getattr(args, "skew", 0.0) or 0.0)
    hidden_cpu, ids_cpu, w_cpu = moe_inputs(torch, cfg, tokens, 100 + d.rank, skew=skew)
    hidden, ids, wts = hidden_cpu.cuda(), ids_cpu.cuda(), w_cpu.cuda()
    with NearGpu(torch, d.local) as near:
        hidden_host = hidden_cpu.pin_memory()
        out_host = torch.empty((tokens, cfg["H"]), dtype=torch.bfloat16).pin_memory()

    def run(h):
        if d.world == 1:
            return fso.moe.layer(h, experts, ids, wts)
        return parallel.expert_parallel_layer(h, experts, ids, wts, num_experts_global=cfg["E"])

    ms_total, clocks, _ = timed_steps(torch, d, lambda _: run(hidden), args.steps, args.warmup)

    pipe = HostPipeline(torch, hidden_host, run, out_host)
    e_steps = max(3, min(args.steps, 10))
    e2e_ms, e2e_regions = timed_e2e(torch, d, pipe, e_steps)
    # small batches are launch-bound when issued eagerly: the device time of one layer under CUDA-graph replay (the
    # reference's own protocol, bench/gemm/python/bench_moe_qwen3_30a3.py:748-811) is reported beside the eager step
    replay_us = None
    if d.world == 1 and tokens <= 1024:
        replay_us = graph_replay_us(torch, lambda i: run(hidden), 1, max(10, args.steps))
    stages = None
    if d.world == 1 and getattr(args, "stages", False):
        stages = moe_stage_times(torch, _ops, hidden, experts, ids, wts, max(5, min(args.steps, 20)))
    elif d.world > 1 and getattr(args, "stages", False) and ep_transport_is_peer():
        # phases of the expert-parallel step on this rank (CUDA events between the phases of the peer transport; the
        # host read shows up as the idle time its synchronisation leaves on the stream)
        sums, reps = {}, max(5, min(args.steps, 20))
        for _ in range(reps):
            parallel.PHASE_TRACE = []
            run(hidden)
            torch.cuda.synchronize()
            marks = parallel.PHASE_TRACE
            parallel.PHASE_TRACE = None
            for (_, ev_a), (name, ev_b) in zip(marks[:-1], marks[1:]):
                sums[name] = sums.get(name, 0.0) + ev_a.elapsed_time(ev_b)
        stages = {f"{name} (ms)": v / reps for name, v in sums.items()}
        stages["note"] = f"rank {d.rank}, {reps} steps, device time between phase boundaries of the peer transport"
    ms_total, e2e_ms = d.max_over_ranks([ms_total, e2e_ms])
    status = _ops.device_status()
    # correctness of what was timed: rank 0's first tokens against the CPU oracle (every N), and under expert
    # parallelism the two transports against each other, bit for bit, on this batch
    sample = min(4 if args.moe_config.startswith("dsv3") else 8, tokens)
    out_last = run(hidden)
    check = None
    if not getattr(args, "no_parity", False):
        check = moe_cpu_check(torch, d, cfg, experts, e0, hidden_cpu, ids_cpu, w_cpu, out_last[:sample], sample,
                              os.cpu_count() or 1)
    transports_equal = None
    if d.world > 1:
        a = parallel.expert_parallel_layer(hidden, experts, ids, wts, num_experts_global=cfg["E"], transport="peer")
        b = parallel.expert_parallel_layer(hidden, experts, ids, wts, num_experts_global=cfg["E"],
                                           transport="collective")
        eq = torch.tensor([1.0 if torch.equal(a, b) else 0.0], device="cuda")
        d.dist.all_reduce(eq, op=d.dist.ReduceOp.MIN)
        transports_equal = bool(eq.item() == 1.0)
    if d.rank != 0:
        d.close()
        return None
    ms_step = ms_total / args.steps
    total_tokens = tokens * d.world
    ep_transport = {"": "peer-memory stores", "peer": "peer-memory stores", "collective": "all-to-all-v"}.get(
        os.environ.get("FSO_B200_EP_TRANSPORT", ""), "peer-memory stores")
    pairs = total_tokens * cfg["k"]
    flops = 6.0 * pairs * cfg["H"] * cfg["I"]
    pk = peaks()
    fp8_peak = 2.0 * pk["bf16_burst"]
    weight_bytes = (e1 - e0) * 3 * cfg["H"] * cfg["I"] * (1 + 1 / 32)
    t_mem = weight_bytes / (pk["hbm_gbs"] * 1e9)
    t_cmp = flops / d.world / (fp8_peak * 1e12)
    line = base_line(args, d, "moe_layer_tokens_per_s", "tokens/s", total_tokens / (ms_step * 1e-3), ms_step, "weak",
                     "fp8_e4m3",
                     {"workload": f"{args.moe_config} MoE layer, {tokens} tokens per GPU, "
                                  + (f"Zipf({skew:g})-skewed" if skew > 0 else "uniform") + " softmax top-k routing",
                      **{k_: cfg[k_] for k_ in ("E", "k", "H", "I")},
                      "parallelism": f"expert parallel x{d.world} ({ep_transport} dispatch + combine)" if d.world > 1
                      else "single GPU", "l2": "expert weights of a step exceed L2"})
    line["roofline"] = {
        "bound": "hbm" if t_mem > t_cmp else "tensor", "kernel": "whole layer (route, gather, FC1, FC2, combine)",
        "achieved": flops / d.world / (ms_step * 1e-3) / 1e12, "peak": fp8_peak, "unit": "TFLOP/s",
        "frac": max(t_mem, t_cmp) / (ms_step * 1e-3), "traffic": None,
        "note": f"frac = max(weight bytes / measured HBM, 6*P*H*I / (2 x bf16 burst)) / step time per GPU; "
                f"weight stream {t_mem * 1e3:.3f} ms, tensor {t_cmp * 1e3:.3f} ms"}
    line["e2e"] = {"value": total_tokens / (e2e_ms / e_steps * 1e-3), "unit": "tokens/s",
                   "h2d_bytes_per_step": tokens * cfg["H"] * 2, "d2h_bytes_per_step": tokens * cfg["H"] * 2,
                   "ms_per_step": e2e_ms / e_steps, "regions_ms_per_step_and_device_allocs": e2e_regions,
                   "host_buffers": near.note}
    # own kernels per step: route (3, or 1 for small batches), gather, FC1, FC2, combine; under expert parallelism
    # also the two plan kernels, the quantizer, the dispatch kernel and the final reduction
    per_step = 7 if tokens * cfg["k"] > 1024 else 5
    if d.world == 1 and fso.moe._decode_band(tokens, cfg["k"], cfg["E"], cfg["I"])[0]:
        per_step += 1          # decode band: FC1 leaves fp32 accumulators, a row-wise SiLU(gate)*up requantizer follows
    if d.world > 1 and ep_transport.startswith("peer"):
        per_step += 5
    elif d.world > 1:
        per_step += 1
    line["gpu_launches"] = per_step * args.steps
    line["clocks"] = clocks
    line["device_status"] = status
    if check is not None:
        dt, rel, mx = check
        line["parity"] = {"rel_frobenius_gpu_vs_cpu": rel, "max_abs_err_over_max_ref": mx,
                          "within_tolerance": bool(rel <= 1e-2 and mx <= 2e-2), "tolerance": "1e-2 / 2e-2 (north_star)",
                          "sample": f"first {sample} tokens of rank 0 through the timed path at {d.world} GPU(s) against "
                                    f"the CPU oracle on the prepared experts' bytes"}
        line["cpu_baseline"] = {"value": sample / dt, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": f"{sample} tokens with their real routing, experts they touch already "
                                          f"quantized ({dt:.2f} s)"}
    if transports_equal is not None:
        line["transports_bit_equal"] = transports_equal
    if stages is not None:
        line["stages"] = stages
    if replay_us is not None:
        live = len({int(v) for v in ids_cpu.reshape(-1).tolist()})
        live_bytes = live * 3 * cfg["H"] * cfg["I"] * (1 + 1 / 32)
        line["graph_replay"] = {"us_per_layer": replay_us, "tokens_per_s": tokens / (replay_us * 1e-6),
                                "experts_in_use": live, "live_weight_bytes": live_bytes,
                                "frac_of_measured_hbm": live_bytes / (replay_us * 1e-6) / (pk["hbm_gbs"] * 1e9)}
    d.close()
    return line


def ep_transport_is_peer() -> bool:
    return os.environ.get("FSO_B200_EP_TRANSPORT", "") in ("", "peer")


def moe_stage_times(torch, _ops, hidden, experts, ids, wts, iters: int):
    """Device time of each kernel stage of the prefill route of one layer (route, gather + quantize, FC1 with the
    SwiGLU epilogue, FC2, combine), each captured into a CUDA graph of its own and replayed. A stage timed alone
    runs at a higher clock than inside the power-capped layer, so the stages need not add up to the layer."""
    t, h = int(hidden.shape[0]), int(hidden.shape[1])
    e, inter, k = experts.num_experts, experts.inter, int(ids.shape[1])
    plan = _ops.moe_plan(t, k, e)
    rows = int(plan.rows)
    _mm, blk0, slot, blk_expert = _ops.moe_route(ids, e, plan)
    fp8 = torch.float8_e4m3fn
    hq = torch.empty((rows, h), dtype=torch.uint8, device="cuda").view(fp8)
    sh = torch.empty((rows * h // 128,), dtype=torch.int32, device="cuda")
    dq = torch.empty((rows, inter), dtype=torch.uint8, device="cuda").view(fp8)
    sd = torch.empty((rows * inter // 128,), dtype=torch.int32, device="cuda")
    dn = torch.empty((rows, h), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    calls = {
        "route_us": lambda i: _ops.moe_route(ids, e, plan),
        "gather_quantize_us": lambda i: _ops.moe_gather_quant(hidden, slot, k, hq, sh),
        "fc1_swiglu_us": lambda i: _ops.moe_fc1_swiglu(hq, sh, experts.w13, experts.sw13, blk0, blk_expert, dq, sd),
        "fc2_us": lambda i: _ops.moe_fc2(dq, sd, experts.w2, experts.sw2, blk0, blk_expert, dn),
        "combine_us": lambda i: _ops.moe_combine(dn, slot, wts, None, None, out),
    }
    res = {name: graph_replay_us(torch, fn, 1, iters) for name, fn in calls.items()}
    res["blocks_in_use"] = int(blk0[-1].item())
    res["note"] = "prefill route, one stage per CUDA graph; 128-row blocks in use include each expert's padding"
    return res


# ====================================================================================================== decode / quantize

def graph_replay_us(torch, make_call, reps: int, iters: int):
    """Median device time per call of ``reps`` calls captured into one CUDA graph and replayed ``iters`` times."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(reps):
            make_call(i)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                make_call(i)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(5):
        e0.record()
        for _ in range(iters):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / iters / reps * 1e3)
    return sorted(times)[len(times) // 2]


def decode_ours(args):
    import torch

    import fish_scales_ops_b200 as fso
    from fish_scales_ops_b200 import _ops

    d = shared_dist(torch)
    fso.build()
    m = args.decode_m
    pk = peaks()
    cells = {}
    with ClockSampler(d.local) as clocks:
        for name, (n, k) in LLAMA.items():
            wbytes = n * k * (1 + 1 / 32)
            copies = int(2 * L2_BYTES / wbytes) + 1          # rotated copies: copies * bytes >= 2 x L2 (cold weights)
            weights = [fso.dense.prepare_weight(dense_inputs(torch, 1, n, k, seed=10 + c)[1].cuda(), format="mxfp8")
                       for c in range(copies)]
            x = dense_inputs(torch, m, n, k, seed=3)[0].cuda()
            xq, sx = fso.dense.quantize_activation(x)
            us_gemm = graph_replay_us(torch, lambda i: fso.dense.linear(xq, weights[i % copies], x_scale=sx), copies,
                                      max(5, args.steps // 5))
            us_lin = graph_replay_us(torch, lambda i: fso.dense.linear(x, weights[i % copies]), copies,
                                     max(5, args.steps // 5))
            nbytes = wbytes + m * k * (1 + 1 / 32) + 2 * m * n
            cells[name] = {"N": n, "K": k, "gemm_us": us_gemm, "linear_us": us_lin, "gemm_gbs": nbytes / us_gemm / 1e3,
                           "frac_of_measured_hbm": nbytes / us_gemm / 1e3 / pk["hbm_gbs"], "weight_copies": copies}
            del weights
    worst = min(cells.values(), key=lambda c: c["gemm_gbs"])
    total_us = sum(c["linear_us"] for c in cells.values())
    line = base_line(args, d, "dense_decode_weight_stream_gbs", "GB/s", worst["gemm_gbs"], total_us / 1e3, "strong",
                     "fp8_e4m3", {"workload": f"llama3-8b dense linears at M={m}, CUDA-graph replay, cold weights",
                                  "cells": cells, "l2": "rotated weight copies of at least 2 x L2 per shape"})
    line["roofline"] = {"bound": "hbm", "kernel": "gemm_mxf8_kernel<16, swapped> (split-K inside clusters)",
                        "achieved": worst["gemm_gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                        "frac": worst["gemm_gbs"] / pk["hbm_gbs"], "traffic": None,
                        "peak_source": f"{pk['source']} copy bandwidth"}
    line["gpu_launches"] = None
    line["clocks"] = clocks.summary()
    line["device_status"] = _ops.device_status()
    d.close()
    return line


def sweep_ours(args):
    """BASELINE.json configs[1] as one table: the four Llama-3-8B linears at M in {1, 16, 128, 1024, 8192}; per cell
    this library's GEMM, cuBLAS' MXFP8 GEMM on the same operands (torch._scaled_mm, the kernel the reference routes
    its wide-N calls to) and a bf16 torch.matmul, all under CUDA-graph replay over rotated weight copies (cold
    weights wherever a weight is smaller than twice L2). Compute-bound cells read as TFLOP/s, decode cells as GB/s."""
    import torch

    import fish_scales_ops_b200 as fso
    from fish_scales_ops_b200 import _ops

    d = shared_dist(torch)
    fso.build()
    pk = peaks()
    e8 = torch.float8_e8m0fnu
    cells = []
    with ClockSampler(d.local) as sampler:
        for name, (n, k) in LLAMA.items():
            wbytes = n * k * (1 + 1 / 32)
            copies = max(2, int(2 * L2_BYTES / wbytes) + 1)
            g = torch.Generator(device="cuda").manual_seed(77)
            masters = [(0.02 * torch.randn(n, k, generator=g, device="cuda")).to(torch.bfloat16) for _ in range(copies)]
            weights = [fso.dense.prepare_weight(w, format="mxfp8") for w in masters]
            for m in (1, 16, 128, 1024, 8192):
                x = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
                xq, sx = fso.dense.quantize_activation(x)
                iters = 20 if m <= 128 else 5
                us = graph_replay_us(torch, lambda i: fso.dense.linear(xq, weights[i % copies], x_scale=sx), copies, iters)
                us_lin = graph_replay_us(torch, lambda i: fso.dense.linear(x, weights[i % copies]), copies, iters)
                sa = sx.view(torch.uint8).view(e8)
                sbs = [w.scale.view(torch.uint8).view(e8) for w in weights]
                try:
                    us_cublas = graph_replay_us(torch, lambda i: torch._scaled_mm(
                        xq, weights[i % copies].weight.t(), scale_a=sa, scale_b=sbs[i % copies],
                        out_dtype=torch.bfloat16), copies, iters)
                    equal = bool(torch.equal(fso.dense.linear(xq, weights[0], x_scale=sx), torch._scaled_mm(
                        xq, weights[0].weight.t(), scale_a=sa, scale_b=sbs[0], out_dtype=torch.bfloat16)))
                except Exception:  # noqa: BLE001 - a torch build without this form: the column stays empty
                    us_cublas, equal = None, None
                us_bf16 = graph_replay_us(torch, lambda i: torch.matmul(x, masters[i % copies].t()), copies, iters)
                fl = 2.0 * m * n * k
                nbytes = wbytes + m * k * (1 + 1 / 32) + 2 * m * n
                cells.append({"shape": name, "M": m, "N": n, "K": k, "gemm_us": us, "linear_us": us_lin,
                              "tflops": fl / us / 1e6, "gbs": nbytes / us / 1e3,
                              "frac_of_2x_bf16_burst": fl / us / 1e6 / (2 * pk["bf16_burst"]),
                              "frac_of_measured_hbm": nbytes / us / 1e3 / pk["hbm_gbs"],
                              "cublas_mxfp8_us": us_cublas, "bit_equal_to_cublas": equal, "bf16_matmul_us": us_bf16})
            del weights, masters
            torch.cuda.empty_cache()
    head = next(c for c in cells if c["shape"] == "gate_up" and c["M"] == 8192)
    line = base_line(args, d, "mxfp8_gemm_tflops", "TFLOP/s", head["tflops"], head["gemm_us"] / 1e3, "strong",
                     "fp8_e4m3", {"workload": "llama3-8b dense linears, M in {1,16,128,1024,8192}, CUDA-graph replay "
                                              "over rotated weight copies", "cells": cells,
                                  "l2": "rotated weight copies of at least 2 x L2 per shape"})
    line["roofline"] = {"bound": "tensor", "kernel": "gemm_mxf8_kernel", "achieved": head["tflops"],
                        "peak": 2 * pk["bf16_burst"], "unit": "TFLOP/s", "frac": head["frac_of_2x_bf16_burst"],
                        "traffic": None}
    line["gpu_launches"] = None
    line["clocks"] = sampler.summary()
    line["device_status"] = _ops.device_status()
    d.close()
    return line


def quantize_ours(args):
    import torch

    import fish_scales_ops_b200 as fso
    from fish_scales_ops_b200 import _ops

    d = shared_dist(torch)
    fso.build()
    m, k = 8192, 4096
    x = dense_inputs(torch, m, 128, k)[0].cuda()
    copies = 4
    xs = [x.clone() for _ in range(copies)]
    # CUDA-graph replay: at 25 us per launch an eager loop would measure the host, not the kernel
    with ClockSampler(d.local) as sampler:
        us = graph_replay_us(torch, lambda i: fso.dense.quantize_activation(xs[i % copies]), copies,
                             max(5, args.steps // 4))
    clocks = sampler.summary()
    nbytes = m * k * (3 + 1 / 32)
    pk = peaks()
    line = base_line(args, d, "quantize_1x32_gbs", "GB/s", nbytes / us / 1e3, us / 1e3, "strong", "bf16->fp8_e4m3",
                     {"workload": f"1x32 MXFP8 activation quantizer on bf16 [{m}, {k}], {copies} rotated inputs",
                      "l2": "4 x 64 MB inputs + outputs exceed L2"})
    line["roofline"] = {"bound": "hbm", "kernel": "quantize_1x32_wide_kernel", "achieved": nbytes / us / 1e3,
                        "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": nbytes / us / 1e3 / pk["hbm_gbs"],
                        "traffic": None, "peak_source": f"{pk['source']} copy bandwidth"}
    line["gpu_launches"] = copies * args.steps
    line["clocks"] = clocks
    line["device_status"] = _ops.device_status()
    d.close()
    return line


def requant_ours(args):
    """Block-FP8 checkpoint -> MXFP8 at load (BASELINE.json configs[2], the largest shape N = 24576, K = 7168):
    the requantization kernel alone under CUDA-graph replay over rotated checkpoints. Algorithmic bytes per element:
    1 read + (1 + 1/32) written, + 4 per 128 x 128 tile."""
    import torch

    import fish_scales_ops_b200 as fso
    from fish_scales_ops_b200 import _ops

    d = shared_dist(torch)
    fso.build()
    n, k = 24576, 7168
    copies = 2
    g = torch.Generator(device="cuda").manual_seed(5)
    ws = [torch.randn(n, k, generator=g, device="cuda", dtype=torch.bfloat16).clamp_(-448, 448).to(torch.float8_e4m3fn)
          for _ in range(copies)]
    sc = torch.exp2(-8.0 + 4.0 * torch.rand(n // 128, k // 128, generator=g, device="cuda"))
    with ClockSampler(d.local) as sampler:
        us = graph_replay_us(torch, lambda i: _ops.requant_block_fp8(ws[i % copies], sc), copies, max(5, args.steps // 4))
    clocks = sampler.summary()
    nbytes = n * k * (2 + 1 / 32) + 4 * (n // 128) * (k // 128)
    pk = peaks()
    line = base_line(args, d, "requant_bs128_to_mxfp8_gbs", "GB/s", nbytes / us / 1e3, us / 1e3, "strong",
                     "fp8_e4m3 x f32 -> fp8_e4m3",
                     {"workload": f"block-FP8 (128x128 fp32 scales) -> MXFP8 requantization of [{n}, {k}], {copies} "
                                  f"rotated checkpoints", "l2": "2 x 176 MB inputs + outputs exceed L2"})
    line["roofline"] = {"bound": "hbm", "kernel": "requant_bs128_kernel", "achieved": nbytes / us / 1e3,
                        "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": nbytes / us / 1e3 / pk["hbm_gbs"],
                        "traffic": None, "peak_source": f"{pk['source']} copy bandwidth"}
    line["gpu_launches"] = copies * args.steps
    line["clocks"] = clocks
    line["device_status"] = _ops.device_status()
    d.close()
    return line


BSFP8_SHAPES = {"kv_b-like 7168x2048": (7168, 2048), "o-like 2048x7168": (2048, 7168), "wide 24576x7168": (24576, 7168)}


def bsfp8_ours(args):
    """BASELINE.json configs[2]: DeepSeek-V3 dense shapes stored as block-FP8 (one fp32 scale per 128 x 128 tile) are
    requantized to MXFP8 at load (``prepare_weight(format="bsfp8")``: the requantization kernel + the end-of-prepare
    fence) and then serve linears at M in {16, 512, 4096}. Per shape: the prepare time (eager calls, CUDA events) and
    its GB/s (1 byte read + 1 + 1/32 written per element), and per M the linear (activation quantizer + GEMM) under
    CUDA-graph replay."""
    import torch

    import fish_scales_ops_b200 as fso
    from fish_scales_ops_b200 import _ops

    d = shared_dist(torch)
    fso.build()
    pk = peaks()
    g = torch.Generator(device="cuda").manual_seed(9)
    cells = {}
    worst = None
    with ClockSampler(d.local) as sampler:
        for name, (n, k) in BSFP8_SHAPES.items():
            wq = torch.randn(n, k, generator=g, device="cuda", dtype=torch.bfloat16).clamp_(-448, 448).to(
                torch.float8_e4m3fn)
            sc = torch.exp2(-8.0 + 4.0 * torch.rand(n // 128, k // 128, generator=g, device="cuda"))
            for _ in range(3):
                fso.dense.prepare_weight(wq, format="bsfp8", scale=sc)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                fso.dense.prepare_weight(wq, format="bsfp8", scale=sc)
            e1.record()
            torch.cuda.synchronize()
            prep_us = e0.elapsed_time(e1) / 10 * 1e3            # eager calls: a load-time operation
            weight = fso.dense.prepare_weight(wq, format="bsfp8", scale=sc)
            nbytes = n * k * (2 + 1 / 32) + 4 * (n // 128) * (k // 128)
            cell = {"N": n, "K": k, "prepare_us": prep_us, "prepare_gbs": nbytes / prep_us / 1e3,
                    "prepare_frac_of_measured_hbm": nbytes / prep_us / 1e3 / pk["hbm_gbs"], "linear": {}}
            for m in (16, 512, 4096):
                x = torch.randn(m, k, generator=g, device="cuda", dtype=torch.bfloat16)
                us = graph_replay_us(torch, lambda i: fso.dense.linear(x, weight), 1, 20)
                cell["linear"][f"M={m}"] = {"us": us, "tflops": 2.0 * m * n * k / us / 1e6,
                                            "weight_stream_gbs": n * k * (1 + 1 / 32) / us / 1e3}
            cells[name] = cell
            worst = cell["prepare_gbs"]                    # the last (largest) shape: the one that streams from HBM
            del wq, sc, weight
            torch.cuda.empty_cache()
    line = base_line(args, d, "bsfp8_prepare_gbs", "GB/s", worst, max(c["prepare_us"] for c in cells.values()) / 1e3,
                     "strong", "fp8_e4m3 x f32 -> fp8_e4m3",
                     {"workload": "block-FP8 checkpoints (128x128 fp32 scales) requantized to MXFP8 at load, then "
                                  "linears at M in {16, 512, 4096}; value = the prepare of the 24576x7168 shape (the 15 MB shapes "
                                  "are bound by the eager call itself, about 50 us)",
                      "cells": cells, "l2": "the 7168x2048 / 2048x7168 weights (15 MB) fit in L2 under replay; the "
                                            "24576x7168 one (176 MB) does not"})
    line["roofline"] = {"bound": "hbm", "kernel": "requant_bs128_wide_kernel", "achieved": worst, "peak": pk["hbm_gbs"],
                        "unit": "GB/s", "frac": worst / pk["hbm_gbs"], "traffic": None,
                        "peak_source": f"{pk['source']} copy bandwidth"}
    line["gpu_launches"] = 3 * (2 * 13 + 3 * 2 * 20)
    line["clocks"] = sampler.summary()
    line["device_status"] = _ops.device_status()
    d.close()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense", choices=["dense", "moe", "decode", "quantize", "requant", "sweep", "bsfp8"])
    ap.add_argument("--skew", type=float, default=0.0, help="moe workload: Zipf exponent of the expert popularity")
    ap.add_argument("--stages", action="store_true",
                    help="moe workload: add the device time of each kernel stage of the layer (one GPU) or of each phase "
                         "of the expert-parallel step (several GPUs, rank 0)")
    ap.add_argument("--no-sustained", action="store_true", help="dense workload: skip the two-second sustained run")
    ap.add_argument("--no-extras", action="store_true",
                    help="dense workload at one GPU: do not attach the decode / quantize / requant / Mixtral objects")
    ap.add_argument("--moe-config", default="dsv3", choices=sorted(MOE_CONFIGS))
    ap.add_argument("--moe-tokens", type=int, default=0, help="moe workload: tokens per GPU override")
    ap.add_argument("--decode-m", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shape", default=None, help="dense workload: M,N,K override (profiling on a smaller case)")
    ap.add_argument("--no-moe", action="store_true",
                    help="dense workload: do not also measure the DeepSeek-V3 MoE layer (the line's \"moe\" object)")
    args = ap.parse_args()
    if args.impl == "reference":
        args.warmup = max(0, args.warmup)
        line = moe_reference(args) if args.workload == "moe" else dense_reference(args)
    else:
        args.warmup = max(3, args.warmup)
        both = args.workload == "dense" and not args.no_moe and args.shape is None
        if both:
            import torch

            shared_dist(torch).keep = True
        line = {"dense": dense_ours, "moe": moe_ours, "decode": decode_ours, "quantize": quantize_ours,
                "requant": requant_ours, "sweep": sweep_ours, "bsfp8": bsfp8_ours}[args.workload](args)
        if both:
            # BASELINE.json's metric has two halves: the GEMM (the line itself) and the MoE layer's tokens/s at
            # 1/2/4/8 GPUs, which rides along as the line's "moe" object (same timing rules, fewer steps)
            sub = argparse.Namespace(**vars(args))
            sub.steps, sub.warmup, sub.no_cpu_baseline, sub.moe_config, sub.moe_tokens = min(args.steps, 20), 3, True, \
                "dsv3", 0
            moe_line = moe_ours(sub)
            d = shared_dist(torch)
            keys = ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "scaling", "config",
                    "roofline", "e2e", "gpu_launches", "clocks", "device_status", "parity", "cpu_baseline",
                    "transports_bit_equal")
            if line is not None and moe_line is not None:
                line["moe"] = {k: moe_line[k] for k in keys if k in moe_line}
            if d.world == 1 and not args.no_extras and line is not None:
                # the rest of the measurement contract rides along at one GPU: decode-sized linears (HBM roofline),
                # the two quantizers, and the Mixtral layer in both routing regimes
                ex = argparse.Namespace(**vars(args))
                ex.steps, ex.warmup, ex.no_cpu_baseline, ex.no_parity = 20, 3, True, True
                short = ("metric", "value", "unit", "ms_per_step", "config", "roofline", "clocks", "device_status")
                for name, fn in (("decode", decode_ours), ("quantize", quantize_ours), ("requant", requant_ours),
                                 ("bsfp8", bsfp8_ours)):
                    sub_line = fn(ex)
                    line[name] = {k: sub_line[k] for k in short if k in sub_line}
                torch.cuda.empty_cache()
                ex.moe_config, ex.moe_tokens = "mixtral", 0
                for name, skew in (("moe_mixtral", 0.0), ("moe_mixtral_zipf", 1.2)):
                    ex.skew = skew
                    sub_line = moe_ours(ex)
                    line[name] = {k: sub_line[k] for k in keys if k in sub_line}
                    torch.cuda.empty_cache()
                # the decode band (BASELINE.json configs[3] at T in {1, 64}, and DeepSeek-V3 at 64 tokens): device time
                # of one layer under CUDA-graph replay against the stream of the live experts' weights
                ex.skew, ex.steps = 0.0, 30
                cells = {}
                for cfg_name, tok in (("mixtral", 1), ("mixtral", 64), ("dsv3", 64)):
                    ex.moe_config, ex.moe_tokens = cfg_name, tok
                    sub_line = moe_ours(ex)
                    cells[f"{cfg_name}_t{tok}"] = {"eager_ms_per_step": sub_line["ms_per_step"], **sub_line["graph_replay"]}
                    torch.cuda.empty_cache()
                line["moe_decode"] = {"metric": "moe_layer_graph_replay_us", "cells": cells,
                                      "note": "calls of at most 64 tokens; weights of the experts in use on MMA-M "
                                              "where the band rule picks the decode kernels"}
            d.keep = False
            d.close()
    if line is not None:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
