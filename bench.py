#!/usr/bin/env python
"""Headline benchmark: fp16 -> fp32 GEMM TFLOP/s on B200, C = A . B^T, 8192^3 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one launch of the sm_100a GEMM on one rank's operands.  With N GPUs
(one process per GPU, launched by torch.distributed.run) the problem is the
M-sharded configuration M = 8192*N, N = K = 8192: every rank owns an 8192-row
slab of A and C and a replica of B, nothing is exchanged while the clock runs
(weak scaling; at N = 8 this is the M = 65536 configuration).  Rank 0 prints ONE
JSON line.  `--impl reference` times the CPU restatement of the reference's CPU
GEMM (docs/nyc25.py:13-56) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fp16->fp32 GEMM TFLOP/s (8192^3 per GPU, M-sharded across GPUs)"
UNIT = "TFLOP/s"
M_PER_RANK = 8192
N_DIM = 8192
K_DIM = 8192
FLOPS_PER_STEP = 2.0 * M_PER_RANK * N_DIM * K_DIM
# algorithmic bytes of one launch: A + B read once, C written once
BYTES_PER_STEP = 2 * M_PER_RANK * K_DIM + 2 * N_DIM * K_DIM + 4 * M_PER_RANK * N_DIM
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel at this size, and the
# committed ncu summary the figure was read from
NCU_TRAFFIC_BYTES = 830.4e6 + 238.2e6
NCU_TRAFFIC_SOURCE = "profiles/gemm_wide_kernel_8192cubed.md"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", 0)),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def config_dict(world):
    return {"workload": f"M-sharded fp16 GEMM: M={M_PER_RANK * world} N={N_DIM} K={K_DIM}, "
                        f"{M_PER_RANK} rows of A and C per GPU, B replicated",
            "layout": "A MxK row-major fp16, B NxK row-major fp16, C MxN row-major fp32, fp32 accumulation",
            "values": "uniform [-1,1) from a position hash, seeds 20010106 / 19980724",
            "parallelism": f"m-shard x{world}, no collective in the timed region",
            "l2": "inputs exceed L2: A+B+C = 512 MiB per GPU against 126 MB of L2"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting",
               0x10: "sync_boost"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            self._nv = pynvml
            # The management library numbers the machine's GPUs, CUDA numbers the visible ones: look the
            # device up by its UUID so that the samples are of the GPU this process computes on.
            uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except TypeError:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def pin_to_gpu_numa_node(torch, dev):
    """Bind this process's threads to the cores of the NUMA node the GPU hangs off, so that the pinned host
    buffers allocated afterwards (first touch) and the copies' submitting threads are local to the GPU's
    host link.  Returns what was done, for the JSON line; does nothing where sysfs does not say."""
    try:
        props = torch.cuda.get_device_properties(dev)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return {"node": None, "note": "no NUMA affinity reported for the GPU"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"node": node, "note": "none of the node's cores is available to this process"}
        os.sched_setaffinity(0, allowed)
        return {"node": node, "cores": len(allowed)}
    except (OSError, ValueError, AttributeError) as e:
        return {"node": None, "note": f"not pinned: {type(e).__name__}"}


def host_link_ceiling(torch, dev, host_in, host_out, barrier, reps=4):
    """Pinned-memory copies of one step's bytes in both directions at once: what the host link alone allows.
    `host_in` (fp16 A, also standing for B, which has the same size) goes to the device twice, `host_out`
    comes back.  Returns GB/s per direction while both run and the seconds one step's bytes take."""
    d_in = torch.empty_like(host_in, device=dev)
    d_in2 = torch.empty_like(host_in, device=dev)
    d_out = torch.empty(host_out.shape, dtype=host_out.dtype, device=dev)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def both():
        with torch.cuda.stream(s_in):
            d_in.copy_(host_in, non_blocking=True)
            d_in2.copy_(host_in, non_blocking=True)
        with torch.cuda.stream(s_out):
            host_out.copy_(d_out, non_blocking=True)

    both()
    barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        both()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / reps
    h2d = 2 * host_in.numel() * host_in.element_size()
    d2h = host_out.numel() * host_out.element_size()
    return {"seconds_per_step": dt, "h2d_gbs": h2d / dt / 1e9, "d2h_gbs": d2h / dt / 1e9}


def cpu_sample(oracle, rows, a_rows=None, b=None):
    """Time the CPU oracle GEMM on `rows` rows of A against the full B; returns (TFLOP/s, seconds)."""
    if b is None:
        b = oracle.fill_f16(N_DIM, K_DIM, oracle.DATA_UNIFORM_PM1, oracle.SEED_B)
    if a_rows is None or a_rows.shape[0] != rows:
        a_rows = oracle.fill_f16(rows, K_DIM, oracle.DATA_UNIFORM_PM1, oracle.SEED_A)
    t0 = time.perf_counter()
    oracle.gemm_f16f32(a_rows, b)
    dt = time.perf_counter() - t0
    return 2.0 * rows * N_DIM * K_DIM / dt / 1e12, dt, a_rows, b


def other_configs(sp, torch, dev, peaks):
    """The remaining single-GPU configurations, measured briefly (25 launches, mean of the middle 13, the
    reference's protocol, gemm/gemm_test.cu:394-405): the skinny-N sweep in HBM GB/s and the attention forward."""

    def iqr_ms(fn, n=25):
        for _ in range(3):
            fn()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        ev[0].record()
        for i in range(n):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        ts = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(n))
        mid = ts[n // 4: n // 4 + (n + 1) // 2]
        return sum(mid) / len(mid)

    out = {}
    M, K = 16384, 8192
    # three copies of A used in rotation: a launch never finds rows in L2 that the previous one left there
    a_rot = []
    for i in range(3):
        a = torch.empty((M, K), dtype=torch.float16, device=dev)
        sp.init_test_data(a, sp.DATA_UNIFORM_PM1, sp.SEED_A)
        a_rot.append(a)
    for n in (64, 128, 256):
        b = torch.empty((n, K), dtype=torch.float16, device=dev)
        sp.init_test_data(b, sp.DATA_UNIFORM_PM1, sp.SEED_B, transpose_rule=True)
        c = torch.empty((M, n), dtype=torch.float32, device=dev)
        turn = [0]

        def launch():
            turn[0] = (turn[0] + 1) % 3
            sp.matmul_sm100(a_rot[turn[0]], b, c)

        ms = iqr_ms(launch)
        # the same launches with nothing between them (one event pair around 60): each sets itself up while
        # the previous one drains (programmatic dependent launch), which an event after every launch prevents
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(60):
            launch()
        e1.record()
        torch.cuda.synchronize()
        ms_b2b = e0.elapsed_time(e1) / 60
        nbytes = 2 * M * K + 2 * n * K + 4 * M * n
        out[f"gemm_M16384_N{n}_K8192"] = {"ms": ms, "tflops": 2.0 * M * n * K / ms / 1e9, "hbm_gbs": nbytes / ms / 1e6,
                                          "frac_of_measured_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                                          "back_to_back": {"ms": ms_b2b, "hbm_gbs": nbytes / ms_b2b / 1e6,
                                                           "frac_of_measured_hbm": nbytes / ms_b2b / 1e6 / peaks["hbm_gbs"]}}
    del a_rot, a
    BH, S, D = 256, 4096, 128
    qkv = []
    for seed in (101, 101 ^ 888, 101 ^ 1776):
        t = torch.empty((BH * S, D), dtype=torch.float16, device=dev)
        sp.init_test_data(t, sp.DATA_NORMAL_BM, seed)
        qkv.append(t.view(BH, S, D))
    o = torch.empty_like(qkv[0])
    ms = iqr_ms(lambda: sp.attn_fwd(qkv[0], qkv[1], qkv[2], o), n=15)
    flops = 4.0 * BH * S * S * D
    out["attention_B16_H16_S4096_D128"] = {"ms": ms, "tflops": flops / ms / 1e9,
                                            "frac_of_measured_bf16_burst": flops / ms / 1e9 / peaks["bf16_tflops"],
                                            "frac_of_nominal_2250": flops / ms / 1e9 / 2250.0}
    sp.status()
    return out


def run_attention(args, sp, torch, dist, dev, rank, world):
    """Attention forward, batch 16 x 16 heads, S = 4096, D = 128, the 256 (batch, head) slices dealt out in
    contiguous blocks over the ranks (strong scaling: the total problem is fixed).  One step = one launch on
    this rank's heads."""
    from spork_b200.sharding import head_slab

    BH_TOTAL, S, D = args.heads, 4096, args.head_dim
    slab = head_slab(BH_TOTAL, rank, world)
    qkv = []
    for seed in (101, 101 ^ 888, 101 ^ 1776):
        t = torch.empty((slab.count * S, D), dtype=torch.float16, device=dev)
        sp.init_test_data(t, sp.DATA_NORMAL_BM, seed, row0=slab.start * S)
        qkv.append(t.view(slab.count, S, D))
    o = torch.empty_like(qkv[0])
    causal = bool(args.causal)
    for _ in range(args.warmup):
        sp.attn_fwd(qkv[0], qkv[1], qkv[2], o, causal=causal)
    sp.status()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(dev.index) as clocks:
        events[0].record()
        for i in range(args.steps):
            sp.attn_fwd(qkv[0], qkv[1], qkv[2], o, causal=causal)
            events[i + 1].record()
        torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sp.status()
    t = torch.tensor([events[0].elapsed_time(events[-1])], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank != 0:
        return
    ms_per_step = float(t.item()) / args.steps
    flops = 4.0 * BH_TOTAL * S * S * D * (0.5 if causal else 1.0)
    value = flops / (ms_per_step * 1e-3) / 1e12
    peaks = measured_peaks()
    print(json.dumps({"metric": f"attention forward TFLOP/s (BH={BH_TOTAL} S=4096 D={D}, fp16, "
                                f"{'causal' if causal else 'non-causal'})", "value": value,
                      "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                      "dtype": "f16 in, f32 softmax, f16 out", "data": "synthetic",
                      "config": {"workload": f"attention forward BH={BH_TOTAL} S=4096 D={D}, heads sharded over ranks",
                                 "values": "N(0,1) by Box-Muller on a position hash, seeds 101, 101^888, 101^1776",
                                 "l2": "inputs exceed L2: Q,K,V,O = 1 GiB"},
                      "clocks": clocks.summary(), "gpu_launches": args.steps,
                      "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"],
                                   "unit": UNIT, "frac": value / world / peaks["bf16_tflops"], "traffic": None,
                                   "kernel": "spork::attn_sm100::attn_fwd_two_kernel<128>" if D == 128 else "spork::attn_sm100::attn_fwd_kernel<64>",
                                   "frac_of_nominal_2250": value / world / 2250.0}}), flush=True)


def run_shape(args, sp, torch, dev):
    """One single-GPU GEMM of a given shape through the default entry point, warm-up plus timed launches with
    one event pair each: the command profiler captures of the skinny-N configurations run."""
    M, N, K = (int(x) for x in args.shape.split(","))
    a = torch.empty((M, K), dtype=torch.float16, device=dev)
    b = torch.empty((N, K), dtype=torch.float16, device=dev)
    c = torch.empty((M, N), dtype=torch.float32, device=dev)
    sp.init_test_data(a, sp.DATA_UNIFORM_PM1, sp.SEED_A)
    sp.init_test_data(b, sp.DATA_UNIFORM_PM1, sp.SEED_B, transpose_rule=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2: written between launches
    for _ in range(args.warmup):
        sp.matmul_sm100(a, b, c)
    sp.status()
    times = []
    for _ in range(args.steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        sp.matmul_sm100(a, b, c)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    sp.status()
    ms = statistics.median(times)
    nbytes = 2 * M * K + 2 * N * K + 4 * M * N
    print(json.dumps({"kernel_only": True, "shape": [M, N, K], "ms_per_step": ms, "value": 2.0 * M * N * K / ms / 1e9,
                      "unit": UNIT, "hbm_gbs": nbytes / ms / 1e6, "l2": "flushed between launches"}), flush=True)


def run_reference(args, rank, world):
    """The reference arm: the reference's CPU GEMM (restated in oracle/) on this box's host cores."""
    if rank != 0:
        return
    from oracle import oracle

    threads = oracle.use_all_cores()
    # size a step so that the whole run takes a couple of minutes at most
    tf, dt, a_rows, b = cpu_sample(oracle, 64)
    step_target_s = min(2.0, 60.0 / (args.steps + args.warmup))  # the whole run stays near a minute
    rows = int(max(64, min(M_PER_RANK, (step_target_s / max(dt, 1e-6)) * 64)))
    rows -= rows % 64
    a_rows = None
    for _ in range(args.warmup):
        tf, dt, a_rows, b = cpu_sample(oracle, rows, a_rows, b)
    times = []
    for _ in range(args.steps):
        tf, dt, a_rows, b = cpu_sample(oracle, rows, a_rows, b)
        times.append(dt)
    step_s = sum(times) / len(times)
    value = 2.0 * rows * N_DIM * K_DIM / step_s / 1e12
    sample = f"{rows} of {M_PER_RANK} rows of A against the full B ({2.0 * rows * N_DIM * K_DIM / 1e9:.0f} GFLOP per step)"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": config_dict(args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=25,
                    help="timed launches; the default is the reference harness's 25 (gemm/gemm_test.cu:394-405)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU-baseline leg (N=1 runs it by default)")
    ap.add_argument("--workload", default="gemm", choices=["gemm", "attention"],
                    help="gemm = the headline line; attention = the companion forward kernel, heads sharded over ranks")
    ap.add_argument("--kernel-only", action="store_true",
                    help="profiling runs: only the warm-up and timed launches (no end-to-end, library or CPU legs)")
    ap.add_argument("--shape", default=None,
                    help="M,N,K of another single-GPU GEMM for --kernel-only runs (the skinny-N configurations)")
    ap.add_argument("--heads", type=int, default=256,
                    help="--workload attention: number of (batch, head) slices (256 is the configuration's; fewer "
                         "for a small profiler capture)")
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128])
    ap.add_argument("--causal", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch

    import spork_b200 as sp

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    if args.workload == "attention":
        run_attention(args, sp, torch, dist, dev, rank, world)
        if dist is not None:
            dist.destroy_process_group()
        return

    if args.shape is not None:
        run_shape(args, sp, torch, dev)
        return

    # ---- operands: this rank's slab of A, a replica of B (made on rank 0, broadcast over NVLink)
    a = torch.empty((M_PER_RANK, K_DIM), dtype=torch.float16, device=dev)
    b = torch.empty((N_DIM, K_DIM), dtype=torch.float16, device=dev)
    c = torch.empty((M_PER_RANK, N_DIM), dtype=torch.float32, device=dev)
    sp.init_test_data(a, sp.DATA_UNIFORM_PM1, sp.SEED_A, row0=rank * M_PER_RANK)
    if rank == 0:
        sp.init_test_data(b, sp.DATA_UNIFORM_PM1, sp.SEED_B, transpose_rule=True)
    if dist is not None:
        dist.broadcast(b, 0)
    torch.cuda.synchronize()

    def step():
        sp.matmul_sm100(a, b, c)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    if dist is not None:
        # every rank publishes whether its warm-up launches came back clean; a rank that failed (or never
        # reports) stops all of them here, before the timed region starts
        from spork_b200.multi_gpu import RankHealth, default_store

        RankHealth(default_store(), rank, world).guard("warmup", sp.status, timeout_s=120.0)
    else:
        sp.status()

    # ---- timed region: K launches, one CUDA event pair per launch on the launching stream
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    with ClockSampler(local_rank) as clocks:
        events[0].record()
        for i in range(args.steps):
            step()
            events[i + 1].record()
        torch.cuda.synchronize()
    barrier()
    sp.status()
    in_kernel_mhz = sp.last_clock_mhz()  # SM clock of the last timed launch, measured inside the kernel
    total_ms = events[0].elapsed_time(events[-1])
    launch_ms = [events[i].elapsed_time(events[i + 1]) for i in range(args.steps)]
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max = float(t.item())
    ms_per_step = total_ms_max / args.steps
    value = FLOPS_PER_STEP * world / (ms_per_step * 1e-3) / 1e12

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "ms_per_step": ms_per_step, "value": value, "unit": UNIT}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end to end through the host-buffer C-ABI entry: pinned host operands in, C back out, every step
    e2e_steps = max(3, min(args.steps, 10))
    all_cores = os.sched_getaffinity(0)
    numa = pin_to_gpu_numa_node(torch, dev)  # before the pinned buffers exist: their pages land on this node
    ha = a.cpu().pin_memory()
    hb = b.cpu().pin_memory()
    hc = torch.empty((M_PER_RANK, N_DIM), dtype=torch.float32).pin_memory()
    sp.matmul_sm100_htod(ha, hb, hc)  # allocates the staging buffers
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        sp.matmul_sm100_htod(ha, hb, hc)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = FLOPS_PER_STEP * world / float(t.item()) / 1e12
    e2e_ok = bool(torch.equal(hc.to(dev), c))
    # The ceiling the host link puts on that number: plain pinned copies of one step's bytes, host to device
    # and device to host at the same time, on every rank at once (one cudaMemcpyAsync per direction).
    link = host_link_ceiling(torch, dev, ha, hc, barrier)
    lt = torch.tensor([link["seconds_per_step"]], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    link_ceiling_tflops = FLOPS_PER_STEP * world / float(lt.item()) / 1e12
    os.sched_setaffinity(0, all_cores)  # the CPU-baseline leg below uses every core again

    # ---- context: the vendor library on the same operands, same protocol (not the product path)
    # fp16 in / fp32 out is the like-for-like figure (the call of gemm/gemm_test.cu:249-261 with fp16 operands);
    # fp16 out writes half the result bytes and is shown beside it.
    cublas_tflops = {"f16_in_f32_out": None, "f16_in_f16_out": None}
    if rank == 0:
        bt = b.t()
        n_lib = min(args.steps, 50)
        for key, call in (("f16_in_f32_out", lambda: torch.mm(a, bt, out_dtype=torch.float32)),
                          ("f16_in_f16_out", lambda: torch.mm(a, bt))):
            try:
                for _ in range(3):
                    call()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(n_lib):
                    call()
                e1.record()
                torch.cuda.synchronize()
                cublas_tflops[key] = FLOPS_PER_STEP / (e0.elapsed_time(e1) / n_lib * 1e-3) / 1e12
            except Exception:
                cublas_tflops[key] = None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    other = other_configs(sp, torch, dev, peaks) if world == 1 else None
    avg_launch_ms = sum(launch_ms) / len(launch_ms)
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    achieved = FLOPS_PER_STEP / (avg_launch_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_BYTES,
                "traffic_source": NCU_TRAFFIC_SOURCE,
                "peak_kind": f"{peaks['source']} cuBLAS bf16 burst (sustained {peaks['bf16_tflops_sustained']})",
                "frac_of_nominal_2250": achieved / 2250.0,
                "kernel": "spork::gemm_sm100::gemm_wide_kernel<false> (256 x 512 tiles per CTA pair)",
                "algorithmic_bytes": BYTES_PER_STEP,
                "avg_launch_ms": avg_launch_ms, "min_launch_ms": min(launch_ms),
                "sm_mhz_in_kernel": in_kernel_mhz,
                "frac_of_peak_at_that_clock": (FLOPS_PER_STEP / (launch_ms[-1] * 1e-3) / 1e12) /
                                              (sm_count * 8192 * in_kernel_mhz * 1e6 / 1e12) if in_kernel_mhz > 0 else None}

    # ---- the same launch repeated for a few hundred milliseconds: what the part sustains once the power cap
    # has pulled the clock down (reported beside the headline, not instead of it)
    sustained = None
    if world == 1:
        n_long = 300
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as long_clocks:   # a quarter of a second: enough samples to mean something
            e0.record()
            for _ in range(n_long):
                step()
            e1.record()
            torch.cuda.synchronize()
        sp.status()
        sustained = {"steps": n_long, "value": FLOPS_PER_STEP / (e0.elapsed_time(e1) / n_long * 1e-3) / 1e12,
                     "unit": UNIT, "sm_mhz_in_kernel": sp.last_clock_mhz(), "clocks": long_clocks.summary()}

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle import oracle

        oracle.use_all_cores()
        tf, dt, a_rows, b_host = cpu_sample(oracle, 64)
        rows = int(max(64, min(M_PER_RANK, (30.0 / max(dt, 1e-6)) * 64)))  # 10-15 s of CPU work (the 64-row probe runs slower per row)
        rows -= rows % 64
        tf, dt, _, _ = cpu_sample(oracle, rows, None, b_host)
        cpu_baseline = {"value": tf, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                        "sample": f"{rows} of {M_PER_RANK} rows of A against the full B, {dt:.1f} s"}

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic", "config": config_dict(world),
            "clocks": dict(clocks.summary(), sm_mhz_in_kernel=in_kernel_mhz),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 2 * M_PER_RANK * K_DIM + 2 * N_DIM * K_DIM,
                    "d2h_bytes_per_step": 4 * M_PER_RANK * N_DIM, "steps": e2e_steps, "result_matches_device_run": e2e_ok,
                    "link_ceiling_gbs": {"h2d": link["h2d_gbs"], "d2h": link["d2h_gbs"],
                                         "how": "rank 0's pinned copies of one step's bytes, both directions at once, "
                                                "while every rank does the same"},
                    "link_ceiling_tflops": link_ceiling_tflops, "frac_of_link": e2e_value / link_ceiling_tflops,
                    "host_numa": numa},
            "gpu_launches": args.steps, "roofline": roofline, "cpu_baseline": cpu_baseline, "sustained": sustained,
            "other_configs": other,
            "context": {"cublas_tflops_same_protocol": cublas_tflops,
                        "frac_of_nominal_fp16_peak": value / (2250.0 * world)}}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
