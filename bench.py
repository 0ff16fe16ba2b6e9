#!/usr/bin/env python
"""Benchmark of the MoE m-grouped FP8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|zipf|masked_gate_up|masked_down|tiny|
                                                                   registered|moe_task|layer|alpha|kgrouped]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # CPU arm: the oracle port of the reference simulator's arithmetic

Default workload (`gemm`): the DeepSeek-V3-shaped m-grouped contiguous FP8 GEMM, G=8 experts x 4096 rows, N=4096,
K=7168, per GPU.  With N GPUs every rank owns its own 8 experts (experts shard, no data-path collective): weak
scaling, value = total TFLOP/s over all ranks.  One step = one launch of the grouped GEMM over the whole batch.
Rank 0 prints ONE JSON line.  The default run continues with the expert-parallel MoE layer (object `moe_layer`) and, on
one GPU, with the four registered grouped-GEMM workloads (`registered`), the registered `moe` task's rows
(`moe_task`) and the decode-regime layer (`alpha_layer`).

After every timed region, outside it, the outputs the timed calls left behind are checked against the CPU oracle on a
sample (`parity_check`); a failed check makes the process exit non-zero.  On one GPU the kernels the reference scores
candidates against -- DeepGEMM's m-grouped FP8 GEMMs and flashinfer's TRT-LLM fused MoE, as installed in this image --
are timed on the same inputs with the same protocol (`comparators`); every speed-up quoted against them comes from the
two timed ALTERNATELY, call by call, so that both see the same SM clock of a power-capped GPU.  Every timed region is
preceded by about 30 ms of untimed calls of the same function (the clock needs that long to come back up after
host-side work).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DATASHEET_FP8_TFLOPS = 4500.0
DATASHEET_HBM_GBS = 8000.0

# DRAM bytes per launch of the dominant kernel (gg_fp8_mx_kernel on the `gemm` workload): dram__bytes_read.sum +
# dram__bytes_write.sum of the committed ncu capture of that kernel; not re-measured by this script.
NCU_TRAFFIC_BYTES = {"gemm": 781.5e6}

WORKLOADS = {
    # contiguous layout: G groups of m rows (or `sizes` rows each, padded to 128)
    "gemm": dict(G=8, m=4096, N=4096, K=7168,
                 desc="m-grouped contiguous FP8 GEMM, DeepSeek-V3 gate_up: G=8 x 4096 rows (M=32768), N=4096, K=7168"),
    "tiny": dict(G=2, m=128, N=512, K=512, desc="tiny contiguous FP8 GEMM G=2 x 128 rows, N=512, K=512"),
    "zipf": dict(G=64, zipf_rows=65536, N=7168, K=2048,
                 desc="load-imbalance stress, contiguous layout: G=64 experts, Zipf(s=1.2) token counts over 65536 "
                      "routed rows, each padded to a multiple of 128; N=7168, K=2048"),
    # masked layout (decode): G groups of max_m rows, masked_m ~ U{0..max_m}
    "masked_gate_up": dict(G=32, max_m=256, N=4096, K=7168, masked=True,
                           desc="masked-layout FP8 grouped GEMM (decode): G=32, max_m=256, masked_m~U[0,256], N=4096, K=7168"),
    "masked_down": dict(G=32, max_m=256, N=7168, K=2048, masked=True,
                        desc="masked-layout FP8 grouped GEMM (decode): G=32, max_m=256, masked_m~U[0,256], N=7168, K=2048"),
}

# the registered workload's four rows (G, expected rows per group, N, K, seed):
# evolution/benchmark/flashinfer_bench_evolve/tasks/grouped_gemm_fp8/workload.jsonl:1-4
REGISTERED = ((4, 8192, 6144, 7168, 1), (4, 8192, 4096, 4096, 3), (8, 4096, 7168, 3072, 6), (8, 4096, 4096, 2048, 8))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(bf16_burst=p.get("bf16_tflops"), bf16_sustained=p.get("bf16_tflops_sustained"),
                    hbm_gbs=p.get("hbm_gbs"), source="measured")
    return dict(bf16_burst=1590.0, bf16_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read only)."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._index = index
        self._period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self._period)

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
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_min_mhz": min(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------- timing helpers
class Timer:
    """CUDA-event timing on the current stream of one device; multi-rank results are the max over ranks."""

    def __init__(self, device, world, barrier):
        import torch
        self.torch, self.device, self.world, self.barrier = torch, device, world, barrier
        self._flush = None

    def _max_over_ranks(self, ms: float) -> float:
        if self.world == 1:
            return ms
        import torch.distributed as dist
        t = self.torch.tensor([ms], dtype=self.torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    SPIN_UP_MS = 30.0

    def spin_up(self, fn) -> None:
        """Untimed calls worth about SPIN_UP_MS of device time before a timed region: after host-side work (data
        generation, the oracle, a JIT build) the SM clock needs milliseconds under load to come back up, and a region
        timed during that ramp is slow by tens of percent.  The call count is the same on every rank."""
        torch = self.torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        fn()
        e1.record()
        e1.synchronize()
        per_call = max(e0.elapsed_time(e1) / 2.0, 1e-3)
        n = int(min(500, max(0, math.ceil(self.SPIN_UP_MS / per_call) - 2)))
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([n], dtype=torch.int64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            n = int(t.item())
        for _ in range(n):
            fn()
        torch.cuda.synchronize()

    def back_to_back(self, fn, steps: int, spin_up: bool = True) -> float:
        """ms per step of `steps` calls issued back to back, barrier + synchronize on both sides."""
        torch = self.torch
        if spin_up:
            self.spin_up(fn)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        return self._max_over_ranks(e0.elapsed_time(e1)) / steps

    def cold_l2_median(self, fn, iters: int = 30, warmup: int = 3) -> float:
        """The reference harness's protocol (benchmark_common.py:267-294 with cold_l2_cache=True): every iteration is
        timed by its own event pair after a write of 256 MB (twice the L2) outside the pair; median over iterations."""
        torch = self.torch
        if self._flush is None:
            self._flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)
        for _ in range(warmup):
            fn()
        self.spin_up(fn)
        ts = []
        for _ in range(iters):
            self._flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return self._max_over_ranks(statistics.median(ts))


def _interleaved_cold(timer, fn_a, fn_b, iters: int = 30):
    """Cold-L2 medians of two functions timed ALTERNATELY (flush, a, flush, b, ...): the SM clock of a power-capped
    GPU moves in steps that last tens of calls, so two series taken one after the other can differ by 20 % for that
    reason alone; taken alternately both see the same clock."""
    import torch
    if timer._flush is None:
        timer._flush = torch.empty(256 << 20, dtype=torch.uint8, device=timer.device)
    timer.spin_up(fn_a)
    ta, tb = [], []
    for _ in range(iters):
        for fn, ts in ((fn_a, ta), (fn_b, tb)):
            timer._flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
    return statistics.median(ta), statistics.median(tb)


def _group_sizes(cfg, seed=0):
    """Valid rows per group."""
    if cfg.get("masked"):
        import torch
        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, cfg["max_m"] + 1, (cfg["G"],), generator=g).tolist()
    if "zipf_rows" in cfg:
        from tirx_harness_b200.workloads import zipf_group_sizes
        return zipf_group_sizes(cfg["G"], cfg["zipf_rows"], 1.2)
    return [cfg["m"]] * cfg["G"]


def _device_case(cfg, seed, device):
    """Seeded synthetic operands generated on the device (same law as workloads.make_contiguous_case)."""
    import torch
    G, N, K = cfg["G"], cfg["N"], cfg["K"]
    sizes = _group_sizes(cfg, 0)
    masked = bool(cfg.get("masked"))
    if masked:
        rows_per = [cfg["max_m"]] * G
    else:
        rows_per = [(m + 127) // 128 * 128 for m in sizes]
    M = sum(rows_per)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    sfa = torch.exp2(torch.randint(-4, 1, (M, K // 128), generator=gen, device=device).float())
    sfb = torch.exp2(torch.randint(-4, 1, (G, (N + 127) // 128, K // 128), generator=gen, device=device).float())
    A = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=device)
    step = 4096
    for r0 in range(0, M, step):
        r1 = min(M, r0 + step)
        x = torch.randn((r1 - r0, K), generator=gen, device=device)
        A[r0:r1] = (x / sfa[r0:r1].repeat_interleave(128, 1)).clamp_(-448, 448).to(torch.float8_e4m3fn)
    B = torch.empty((G, N, K), dtype=torch.float8_e4m3fn, device=device)
    for g in range(G):
        x = torch.randn((N, K), generator=gen, device=device)
        full = sfb[g].repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)
        B[g] = (x / full).clamp_(-448, 448).to(torch.float8_e4m3fn)
    D = torch.zeros((M, N), dtype=torch.bfloat16, device=device)
    data = dict(A=A, B=B, SFA=sfa, SFB=sfb, D=D, G=G, M=M, N=N, K=K, sizes=sizes)
    if masked:
        data["masked_m"] = torch.tensor(sizes, dtype=torch.int32, device=device)
    else:
        gl = torch.full((M,), -1, dtype=torch.int32)
        r = 0
        for g, (m, mp) in enumerate(zip(sizes, rows_per)):
            gl[r:r + m] = g
            r += mp
        data["grouped_layout"] = gl.to(device)
    return data


def _bind(gg, cfg, data):
    if cfg.get("masked"):
        G, mm, N, K = cfg["G"], cfg["max_m"], cfg["N"], cfg["K"]
        return gg.bind_masked(data["A"].view(G, mm, K), data["SFA"].view(G, mm, K // 128), data["B"], data["SFB"],
                              data["D"].view(G, mm, N), data["masked_m"])
    return gg.setup(data, data["G"], data["M"], data["N"], data["K"])


def _algorithmic(cfg, sizes=None):
    """FLOPs and bytes over VALID rows only."""
    G, N, K = cfg["G"], cfg["N"], cfg["K"]
    rows = sum(sizes if sizes is not None else _group_sizes(cfg, 0))
    flops = 2.0 * rows * N * K
    bytes_ = rows * K + G * N * K + rows * N * 2 + rows * (K // 128) * 4 + G * ((N + 127) // 128) * (K // 128) * 4
    return flops, float(bytes_)


def _gemm_parity(cfg, data, rows=64):
    """Row sample of D as the timed launches left it, against the CPU oracle (simulator-order FMA chain)."""
    from oracle import checks
    if cfg.get("masked"):
        row_group = checks.masked_row_groups(data["masked_m"], cfg["max_m"])
    else:
        row_group = data["grouped_layout"]
    sfa = data.get("SFA_f32", data["SFA"])
    sfb = data.get("SFB_f32", data["SFB"])
    groups = None
    if data["G"] > 8:                 # bound the cost of decoding B: the first, the last and two middle groups with rows
        import torch
        have = torch.unique(row_group[row_group >= 0]).tolist()
        groups = sorted({have[0], have[len(have) // 3], have[2 * len(have) // 3], have[-1]}) if have else None
    return checks.grouped_gemm_rows(data["A"], sfa, data["B"], sfb, row_group, data["D"], target_rows=rows, groups=groups)


# ---------------------------------------------------------------------------------------------- comparators
def _comparator_env():
    """The installed comparator libraries build kernels on first use.  DeepGEMM's are quick (seconds per shape) and go
    to its cache folder; flashinfer's TRT-LLM MoE launcher takes minutes of host compilation, so a build of it made
    beforehand with the library's own JIT (on a machine without a GPU) may lie in the git-ignored baseline/_ref and is
    then offered to flashinfer as its ahead-of-time module folder."""
    dgc = os.path.join(ROOT, "baseline", "_ref", "deepgemm_cache")
    if os.path.isdir(dgc):
        os.environ.setdefault("DG_JIT_CACHE_DIR", dgc)
    aot = os.path.join(ROOT, "baseline", "_ref", "flashinfer_aot")
    if os.path.isdir(aot):
        import pathlib
        import flashinfer.jit.env as fenv
        fenv.FLASHINFER_AOT_DIR = pathlib.Path(aot)


def _guarded(name):
    """Comparator wrapper: an import, build or call failure is recorded once and never retried."""
    def deco(fn):
        def run(*a, **k):
            try:
                return fn(*a, **k)
            except BaseException as exc:      # noqa: BLE001 -- a comparator must not take the benchmark down
                if isinstance(exc, (KeyboardInterrupt, SystemExit)):
                    raise
                return {"library": name, "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        return run
    return deco


@_guarded("deep_gemm (vllm.third_party)")
def cmp_deepgemm(cfg, data, timer, iters, ours=None):
    """DeepGEMM m_grouped_fp8_gemm_nt_contiguous / _masked (what the grouped_gemm/fp8 task's baseline launches,
    tasks/grouped_gemm_fp8/baseline.py:30-42) on the same tensors, scales pre-converted to the layout it wants."""
    import torch
    _comparator_env()
    import vllm.third_party.deep_gemm as dg
    G, N, K = data["G"], data["N"], data["K"]
    sfa = data.get("SFA_f32", data["SFA"])
    sfb = data.get("SFB_f32", data["SFB"])
    d = torch.zeros_like(data["D"])
    if cfg.get("masked"):
        mm = cfg["max_m"]
        a3, d3 = data["A"].view(G, mm, K), d.view(G, mm, N)
        sfa_t = dg.transform_sf_into_required_layout(sfa.view(G, mm, K // 128), mm, K, (1, 128, 128), G, True, False)
        sfb_t = dg.transform_sf_into_required_layout(sfb, N, K, (1, 128, 128), G, False, False)
        expected_m = max(1, int(sum(data["sizes"]) / G))
        fn = lambda: dg.m_grouped_fp8_gemm_nt_masked((a3, sfa_t), (data["B"], sfb_t), d3, data["masked_m"], expected_m)
        name = "m_grouped_fp8_gemm_nt_masked"
    else:
        M = data["M"]
        sfa_t = dg.transform_sf_into_required_layout(sfa, M, K, (1, 128, 128), None, True, False)
        sfb_t = dg.transform_sf_into_required_layout(sfb, N, K, (1, 128, 128), G, False, False)
        fn = lambda: dg.m_grouped_fp8_gemm_nt_contiguous((data["A"], sfa_t), (data["B"], sfb_t), d, data["grouped_layout"])
        name = "m_grouped_fp8_gemm_nt_contiguous"
    t0 = time.perf_counter()
    fn()
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    ms_b2b = timer.back_to_back(fn, iters)
    ms_cold = timer.cold_l2_median(fn, iters)
    # same valid rows as ours?  (its padding rows are unspecified)
    if cfg.get("masked"):
        from oracle import checks
        valid = checks.masked_row_groups(data["masked_m"], cfg["max_m"]) >= 0
    else:
        valid = data["grouped_layout"] >= 0
    same = float((d[valid] == data["D"][valid]).float().mean().item()) if bool(valid.any()) else 1.0
    out = {"library": f"deep_gemm {dg.__version__} (vllm.third_party) {name}", "ms": ms_b2b, "ms_median_cold_l2": ms_cold,
           "first_call_s": round(build_s, 1), "outputs_identical_to_ours": round(same, 5)}
    if ours is not None:
        a, b = _interleaved_cold(timer, ours, fn, iters)
        out["interleaved_cold_l2"] = {"ours_ms": a, "ms": b, "speedup": b / a}
    return out


def _geomean(xs):
    xs = [x for x in xs if x and x > 0]
    return math.exp(sum(math.log(x) for x in xs) / len(xs)) if xs else None


def cpu_baseline(cfg, seed=0, rows_per_group=1024):
    """Times the CPU oracle (simulator-order FMA chain) on a bounded row sample of the workload, all host cores."""
    import numpy as np
    from oracle import oracle as orc
    G, N, K = cfg["G"], cfg["N"], cfg["K"]
    rows_per_group = max(1, min(rows_per_group, max(_group_sizes(cfg, 0)), 8192 // G))
    rng = np.random.default_rng(seed)
    M = G * rows_per_group
    A = rng.integers(0, 0x7F, size=(M, K), dtype=np.uint8)
    B = rng.integers(0, 0x7F, size=(G, N, K), dtype=np.uint8)
    sfa = np.exp2(rng.integers(-4, 1, size=(M, K // 128))).astype(np.float32)
    sfb = np.exp2(rng.integers(-4, 1, size=(G, (N + 127) // 128, K // 128))).astype(np.float32)
    gl = (np.arange(M) // rows_per_group).astype(np.int32)
    orc.lib()
    orc.set_num_threads(os.cpu_count() or 1)        # launchers export OMP_NUM_THREADS=1 to their ranks
    t0 = time.perf_counter()
    orc.gg_contiguous(A, B, sfa, sfb, gl, model=orc.SIM_CHAIN)
    dt = time.perf_counter() - t0
    flops = 2.0 * M * N * K
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"{rows_per_group} rows of each of the {G} groups (all N={N}, all K={K}; includes decoding "
                      f"each group's B once), {dt:.1f} s",
            "seconds": dt}


def _gemm_config(cfg, world, alg_bytes):
    return {"workload": cfg["desc"] + (f"; per GPU, {world} GPUs each own {cfg['G']} experts" if world > 1 else ""),
            "scales": "fp32, A 1x128 per row, B 128x128, 2^{-4..0}", "accumulate": "fp32", "out": "bf16",
            "l2": f"inputs ({alg_bytes / 1e6:.0f} MB per launch) larger than L2, no flush", "seed": 0,
            "timing": "CUDA events around K back-to-back launches, max over ranks"}


def run_reference(args):
    """--impl reference: the reference's CPU path (its simulator's arithmetic, restated in oracle/oracle.c; the
    simulator itself is Rust and cannot be built here).  Rank 0 only.  Every step times the same bounded row
    sample (1024 rows of each group); value = the sample's FLOPs over its time, ms_per_step = that time."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg = WORKLOADS[args.workload if args.workload in WORKLOADS else "gemm"]
    warm = max(0, args.warmup)
    for _ in range(warm):
        cpu_baseline(cfg, rows_per_group=8)           # short samples: page the library in, start the thread team
    steps = max(1, args.steps)
    vals, secs, r = [], [], None
    t_start = time.perf_counter()
    done = 0
    for s in range(steps):
        r = cpu_baseline(cfg, seed=s)
        vals.append(r["value"])
        secs.append(r["seconds"])
        done += 1
        if time.perf_counter() - t_start > 150.0:     # keep the arm inside a few minutes whatever --steps says
            break
    v = statistics.median(vals)
    flops, alg_bytes = _algorithmic(cfg)
    sample_ms = statistics.median(secs) * 1e3
    line = {
        "impl": "reference", "metric": "grouped_gemm_fp8_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": done, "warmup": warm, "ms_per_step": sample_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": _gemm_config(cfg, args.gpus, alg_bytes),
        "steps_requested": steps,
        "ms_per_step_full_workload_extrapolated": flops / (v * 1e12) * 1e3,
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU oracle port of the reference simulator's arithmetic on all host cores; a step = one bounded row "
                "sample of the workload (its time is ms_per_step)",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------- registered rows
def run_registered(args, device, timer):
    """The four rows of the registered grouped_gemm/fp8 workload in its own tensor contract (packed UE8M0 scales,
    MN-major, alignment 224, -1 padding) through `setup(data, G, M, N, K)`, with the DeepGEMM kernel the reference
    scores against on the same tensors.  score = comparator_ms / ours_ms per row and their geometric mean
    (evolution/tasks/grouped_gemm_fp8.yaml:8-13,30)."""
    import torch
    from tirx_harness_b200 import grouped_gemm as gg
    from tirx_harness_b200.workloads import make_registered_case
    rows = []
    iters = max(10, min(args.steps, 30))
    for (G, m, N, K, seed) in REGISTERED:
        data = make_registered_case(G, m, N, K, seed=seed, device=device)
        launch = gg.setup(data, data["G"], data["M"], data["N"], data["K"])
        for _ in range(3):
            launch()
        ms = timer.back_to_back(launch, iters)
        ms_cold = timer.cold_l2_median(launch, iters)
        cfg = dict(G=G, N=N, K=K)
        flops, alg_bytes = _algorithmic(cfg, data["actual_ms"])
        row = {"G": G, "expected_m": m, "N": N, "K": K, "M_padded": data["M"], "rows_valid": sum(data["actual_ms"]),
               "ms": ms, "ms_median_cold_l2": ms_cold, "tflops": flops / (ms_cold * 1e-3) / 1e12,
               "parity_check": _gemm_parity(cfg, data)}
        if not args.no_comparators:
            c = cmp_deepgemm(cfg, data, timer, iters, ours=launch)
            row["comparator"] = c
            if "interleaved_cold_l2" in c:
                row["speedup"] = c["interleaved_cold_l2"]["speedup"]
        rows.append(row)
        del data, launch
        torch.cuda.empty_cache()
    status = gg.device_status(device)
    return {"workload": "registered grouped_gemm/fp8 rows: packed UE8M0 scales (MN-major), alignment 224, -1 padding; rows per "
                        "group ~ U[0.7,1.3] x expected (the public DeepGEMM generator's law stands in for the un-vendored one)",
            "timing": "per-iteration CUDA events, 256 MB L2 flush before each, median (the reference's time_fn protocol); "
                      "ms = back-to-back mean beside it; speedup = comparator / ours from the two timed alternately "
                      "(comparator.interleaved_cold_l2), so that both see the same SM clock",
            "rows": rows, "geomean_speedup_vs_deepgemm": _geomean([r.get("speedup") for r in rows]),
            "parity_ok": all(r["parity_check"]["ok"] for r in rows), "device_status": status}


# ---------------------------------------------------------------------------------------------- moe task rows
MOE_TASK_ROWS = (1, 16, 80, 901, 14107)       # a spread of the registered workload's trace rows (tasks/moe/workload.jsonl)


def run_moe_task(args, device, timer):
    """The registered `moe` task (32 local of 256 experts, DeepSeek-V3 routing, fp32 128-block scales drawn
    uniform(0.01, 0.1)) through `setup(data, T)`, with flashinfer's trtllm_fp8_block_scale_moe called the way the task's
    baseline calls it (tasks/moe/baseline.py:17-51) on the same tensors."""
    import torch
    from tirx_harness_b200 import grouped_gemm as gg
    from tirx_harness_b200 import moe_layer
    H, I, E, El = 7168, 2048, 256, 32
    gen = torch.Generator(device=device).manual_seed(7)
    fp8 = lambda shape: torch.randn(shape, device=device, generator=gen).clamp_(-2.0, 2.0).to(torch.float8_e4m3fn)
    sc = lambda shape: torch.empty(shape, device=device).uniform_(0.01, 0.1, generator=gen)
    w1 = torch.empty((El, 2 * I, H), dtype=torch.float8_e4m3fn, device=device)
    w2 = torch.empty((El, H, I), dtype=torch.float8_e4m3fn, device=device)
    for e in range(El):
        w1[e], w2[e] = fp8((2 * I, H)), fp8((H, I))
    s1, s2 = sc((El, 2 * I // 128, H // 128)), sc((El, H // 128, I // 128))
    bias = (torch.randn(E, device=device, generator=gen) * 0.1).bfloat16()
    fi = None
    if not args.no_comparators:
        try:
            _comparator_env()
            from flashinfer.fused_moe import trtllm_fp8_block_scale_moe as fi
        except BaseException as exc:      # noqa: BLE001
            fi = f"unavailable: {type(exc).__name__}: {str(exc)[:200]}"
    rows = []
    fi_broken = None
    for T in (args.moe_rows or MOE_TASK_ROWS):
        iters = 10 if T > 4096 else 20
        data = dict(routing_logits=torch.randn((T, E), device=device, generator=gen), routing_bias=bias,
                    hidden_states=fp8((T, H)), hidden_states_scale=sc((H // 128, T)), gemm1_weights=w1,
                    gemm1_weights_scale=s1, gemm2_weights=w2, gemm2_weights_scale=s2, local_expert_offset=64,
                    routed_scaling_factor=2.5, output=torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=device))
        run = moe_layer.setup(data, T)
        for _ in range(3):
            run()
        ms = timer.back_to_back(run, iters)
        ms_cold = timer.cold_l2_median(run, iters)
        row = {"T": T, "ms": ms, "ms_median_cold_l2": ms_cold}
        if callable(fi) and fi_broken is None:
            try:
                call = lambda: fi(routing_logits=data["routing_logits"], routing_bias=bias, hidden_states=data["hidden_states"],
                                  hidden_states_scale=data["hidden_states_scale"], gemm1_weights=w1, gemm1_weights_scale=s1,
                                  gemm2_weights=w2, gemm2_weights_scale=s2, num_experts=E, top_k=8, n_group=8, topk_group=4,
                                  intermediate_size=I, local_expert_offset=64, local_num_experts=El,
                                  routed_scaling_factor=2.5, routing_method_type=2, use_shuffled_weight=False,
                                  tune_max_num_tokens=max(32768, T))
                ref = call()
                torch.cuda.synchronize()
                c_ms = timer.back_to_back(call, iters)
                c_cold = timer.cold_l2_median(call, iters)
                i_ours, i_cmp = _interleaved_cold(timer, run, call, iters)      # the two timed alternately: same SM clock
                o, r = data["output"].float(), ref.float()
                rms = float(((o - r).square().mean().sqrt() / (r.square().mean().sqrt() + 1e-8)).item())
                tok = (o - r).square().mean(-1).sqrt() / (r.square().mean(-1).sqrt() + 1e-8)
                row.update(comparator_ms=c_ms, comparator_ms_median_cold_l2=c_cold, speedup=i_cmp / i_ours,
                           interleaved_cold_l2={"ours_ms": i_ours, "ms": i_cmp},
                           rms_ratio_vs_comparator=rms, tokens_over_0p2=int((tok >= 0.2).sum().item()))
            except BaseException as exc:      # noqa: BLE001
                if isinstance(exc, (KeyboardInterrupt, SystemExit)):
                    raise
                fi_broken = f"unavailable: {type(exc).__name__}: {str(exc)[:200]}"
        rows.append(row)
        del data, run
    status = gg.device_status(device)
    lib = str(fi)
    if callable(fi):
        import flashinfer
        lib = f"flashinfer {getattr(flashinfer, '__version__', '?')} trtllm_fp8_block_scale_moe"
    return {"workload": "registered `moe` task: H=7168, I=2048, 32 local of 256 experts (offset 64), DeepSeek-V3 no-aux routing "
                        "top-8, fp32 block scales ~ U(0.01, 0.1), N(0,1) clamped to +-2 operands",
            "comparator": fi_broken or lib, "rows": rows,
            "geomean_speedup_vs_trtllm": _geomean([r.get("speedup") for r in rows]), "device_status": status}


LAYER = dict(T=16384, H=7168, I=2048, E=256, top_k=8,
             desc="MoE layer forward, expert parallel: 16384 tokens, hidden 7168, 256 experts x intermediate 2048, "
                  "softmax top-8; dispatch -> gate_up grouped GEMM -> SiLU*mul FP8 requant -> down grouped GEMM -> combine")


LAYER_SMALL = dict(LAYER, T=2048, E=32,
                   desc="one rank's share of the 8-GPU MoE layer run alone: 2048 tokens, 32 experts (small case for ncu)")


def _layer_case(world, rank, device, cfg=LAYER, seed=0):
    """This rank's token slice and experts (synthetic, generated on the device)."""
    import torch
    T, H, I, E = cfg["T"], cfg["H"], cfg["I"], cfg["E"]
    Tl, El = T // world, E // world
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000 + rank)
    hs = torch.randn((Tl, H), generator=gen, device=device).bfloat16()
    from tirx_harness_b200 import moe_ops
    xq, xs = moe_ops.quant_1x128(hs)

    def weights(n, k):
        nb, kb = n // 128, k // 128
        sc = torch.exp2(torch.randint(-4, 1, (El, nb, kb), generator=gen, device=device).float())
        w = torch.empty((El, n, k), dtype=torch.float8_e4m3fn, device=device)
        for e in range(El):
            x = torch.randn((n, k), generator=gen, device=device)
            w[e] = (x / sc[e].repeat_interleave(128, 0).repeat_interleave(128, 1)).clamp_(-448, 448).to(torch.float8_e4m3fn)
        return w, sc * (0.5 / k ** 0.5)       # keeps activations O(1) through the layer
    w13, s13 = weights(2 * I, H)
    w2, s2 = weights(H, I)
    logits = torch.randn((Tl, E), generator=gen, device=device)
    return dict(hidden_states=xq, hidden_states_scale=xs, routing_logits=logits, gemm1_weights=w13,
                gemm1_weights_scale=s13, gemm2_weights=w2, gemm2_weights_scale=s2,
                output=torch.zeros((Tl, H), dtype=torch.bfloat16, device=device))


def run_layer(args, world, rank, device, barrier, steps, warmup):
    """Times the expert-parallel MoE layer: strong scaling, T fixed, value = tokens/s of the whole job."""
    import torch
    import torch.distributed as dist
    from tirx_harness_b200 import ep_layer
    from tirx_harness_b200 import grouped_gemm as gg
    cfg = LAYER_SMALL if getattr(args, "layer_small", False) else LAYER
    data = _layer_case(world, rank, device, cfg)
    Tl = cfg["T"] // world
    layer = ep_layer.setup(data, Tl, top_k=cfg["top_k"], combine=args.combine, dispatch=args.dispatch, fuse_act=args.fuse_act)
    timer = Timer(device, world, barrier)
    for _ in range(max(warmup, 3)):
        layer()
    barrier()
    with ClockSampler(device.index) as clocks:
        ms = timer.back_to_back(layer, steps)
    status = gg.device_status(device)
    # ---- parity of what the timed steps left behind: every stage, every rank (outside the timed region)
    parity = None
    if not args.no_parity:
        from oracle import checks
        data["output"].fill_(float("nan"))
        layer()
        parity = checks.ep_layer_check(layer, data, world, rank)
        parity = {k: (v if not isinstance(v, dict) else {kk: (round(vv, 8) if isinstance(vv, float) else vv) for kk, vv in v.items()})
                  for k, v in parity.items()}
    # per-stage device times on this rank (events between the stages of one forward, a few extra steps)
    stages = layer.stage_times(5)
    barrier()
    counts = layer.counts_local.sum().item()
    # end to end with host buffers: tokens in (fp8 + scales + logits), output back
    hx = data["hidden_states"].view(torch.uint8).cpu().pin_memory()
    hs_ = data["hidden_states_scale"].cpu().pin_memory()
    hl = data["routing_logits"].cpu().pin_memory()
    ho = torch.empty(data["output"].shape, dtype=torch.bfloat16).pin_memory()
    dx8 = data["hidden_states"].view(torch.uint8)

    def e2e_step():
        dx8.copy_(hx, non_blocking=True)
        data["hidden_states_scale"].copy_(hs_, non_blocking=True)
        data["routing_logits"].copy_(hl, non_blocking=True)
        layer()
        ho.copy_(data["output"], non_blocking=True)

    # Pipelined form of the same step: the host copies go through device staging buffers on their own streams
    # (step i+1's inputs arrive while step i computes, step i's output leaves while step i+1 computes); the
    # compute stream only pays two device-to-device copies per step.
    sx, ss, sl = torch.empty_like(dx8), torch.empty_like(data["hidden_states_scale"]), torch.empty_like(data["routing_logits"])
    so = torch.empty_like(data["output"])
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    cur = torch.cuda.current_stream(device)
    ev_in, ev_taken, ev_staged, ev_out = (torch.cuda.Event() for _ in range(4))

    def stage_in(first):
        with torch.cuda.stream(s_in):
            if not first:
                s_in.wait_event(ev_taken)                   # the previous inputs have left the staging buffers
            sx.copy_(hx, non_blocking=True)
            ss.copy_(hs_, non_blocking=True)
            sl.copy_(hl, non_blocking=True)
            ev_in.record(s_in)

    def pipelined(n):
        stage_in(True)
        for i in range(n):
            cur.wait_event(ev_in)
            dx8.copy_(sx, non_blocking=True)
            data["hidden_states_scale"].copy_(ss, non_blocking=True)
            data["routing_logits"].copy_(sl, non_blocking=True)
            ev_taken.record(cur)
            if i + 1 < n:
                stage_in(False)
            layer()
            if i > 0:
                cur.wait_event(ev_out)                      # the previous output has left its staging buffer
            so.copy_(data["output"], non_blocking=True)
            ev_staged.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_staged)
                ho.copy_(so, non_blocking=True)
                ev_out.record(s_out)
        cur.wait_event(ev_out)
    e2e_steps = max(3, min(steps, 10))
    e2e_step()
    pipelined(2)
    serial_ms = timer.back_to_back(e2e_step, e2e_steps)
    e2e_ms = timer.back_to_back(lambda: pipelined(e2e_steps), 1) / e2e_steps
    H, I, k = cfg["H"], cfg["I"], cfg["top_k"]
    flops = 2.0 * cfg["T"] * k * (2 * I * H + H * I)
    h2d = hx.numel() + hs_.numel() * 4 + hl.numel() * 4
    d2h = ho.numel() * 2
    res = {
        "metric": "moe_layer_tokens_per_s", "value": cfg["T"] / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["desc"], "tokens_per_rank": Tl, "experts_per_rank": cfg["E"] // world,
                   "routing": "softmax top-8, ties to lowest index, weights renormalised",
                   "l2": "weights (1.4-11 GB per rank) larger than L2, no flush", "rows_this_rank": int(counts),
                   "combine": args.combine, "dispatch": args.dispatch, "fuse_act": bool(args.fuse_act)},
        "clocks": clocks.summary(),
        "e2e": {"value": cfg["T"] / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "serial_ms_per_step": serial_ms,
                "h2d_gbs_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
                "note": "per rank and step: fp8 tokens, scales, logits from pinned host memory, bf16 output back; copies on "
                        "their own streams overlap neighbouring steps; serial = one stream"},
        "gpu_launches": steps * 15,
        "tflops_grouped_gemms": flops / (ms * 1e-3) / 1e12,
        "stages_ms_rank0": {k: round(v, 4) for k, v in stages.items()},
        "parity_check": parity,
        "device_status": status,
    }
    layer.close()
    return res


ALPHA_ROWS = (1, 8, 16, 32, 64, 128)
ALPHA = dict(H=2048, I=128, E=512, top_k=10,
             desc="decode-regime MoE layer from bf16 activations and preselected routes (alphamoe contract): "
                  "K=2048, I=128, E=512, top-10, rows M in {1,8,16,32,64,128}")


def _alpha_comparator(data, M, timer_graph):
    """flashinfer trtllm_fp8_block_scale_routed_moe the way the alphamoe task's baseline runs it
    (tasks/alphamoe/baseline.py:60-156): [up; gate] weight order, 1x128 quantisation by an eager torch recipe inside
    the captured call, autotuned once, replayed as a CUDA graph."""
    import torch
    _comparator_env()
    from flashinfer import autotune
    from flashinfer.fused_moe import trtllm_fp8_block_scale_routed_moe
    hs, ids, wts = data["hidden_states"], data["topk_ids"], data["topk_weights"]
    w13, s13, w2, s2 = data["gemm1_weights"], data["gemm1_weights_scale"], data["gemm2_weights"], data["gemm2_weights_scale"]

    def swap(t):
        gate, up = t.chunk(2, dim=1)
        return torch.cat((up, gate), dim=1).contiguous()
    w13s, s13s = swap(w13), swap(s13)
    top_k = int(data["top_k"])

    def quant(x):
        rows, cols = x.shape
        g = x.float().reshape(rows, cols // 128, 128)
        sc = g.abs().amax(dim=-1).clamp_min(1.0e-8) / 448.0
        return (g / sc.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(rows, cols), sc

    def launch():
        xq, xs = quant(hs)
        # the installed flashinfer takes the routes packed: (expert id << 16) | bf16 bits of the weight
        packed = (ids << 16) | (wts.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF)
        return trtllm_fp8_block_scale_routed_moe(
            topk_ids=packed, routing_bias=None, hidden_states=xq, hidden_states_scale=xs.t().contiguous(),
            gemm1_weights=w13s, gemm1_weights_scale=s13s, gemm2_weights=w2, gemm2_weights_scale=s2,
            num_experts=w13.shape[0], top_k=top_k, n_group=None, topk_group=None, intermediate_size=w2.shape[2],
            local_expert_offset=0, local_num_experts=w13.shape[0], routed_scaling_factor=1.0, routing_method_type=5,
            use_shuffled_weight=False, tune_max_num_tokens=max(1, M))
    with autotune(tuning_buckets=(max(1, M),)):
        launch()
    side = torch.cuda.Stream(device=hs.device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = launch()
    torch.cuda.synchronize()
    us = timer_graph(graph.replay)
    o, r = data["output"].float(), out.float()
    rms = float(((o - r).square().mean().sqrt() / (r.square().mean().sqrt() + 1e-8)).item())
    return us, rms


def run_alpha(args, device):
    """Times the decode-regime layer on the six official row sizes of the alphamoe contract.  Per row: L2 is
    flushed (a 256 MB memset) before every timed call, each call is bracketed by its own CUDA events, the
    median is reported; the same with the call captured into a CUDA graph (how that task's baseline is timed).
    Roofline: the weights of the distinct experts touched must come from HBM once."""
    import torch
    from tirx_harness_b200 import alpha_moe
    from tirx_harness_b200 import grouped_gemm as gg
    cfg = ALPHA
    H, I, E, k = cfg["H"], cfg["I"], cfg["E"], cfg["top_k"]
    gen = torch.Generator(device=device).manual_seed(42)

    def qweights(rows, cols):          # e4m3 bytes + 128x128 scales of N(0, 0.125) weights, made on the device
        w = torch.randn((E, rows, cols), device=device, generator=gen) * 0.125
        blocks = w.view(E, rows // 128, 128, cols // 128, 128)
        sc = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-8) / 448.0
        q = (blocks / sc[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(E, rows, cols)
        return q, sc.float().contiguous()
    w13, s13 = qweights(2 * I, H)
    w2, s2 = qweights(H, I)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    peaks = _peaks()
    iters = max(10, min(args.steps, 50))
    rows = []
    cmp_note = None
    with ClockSampler(device.index) as clocks:
        for M in (args.alpha_rows or ALPHA_ROWS):
            hs = (torch.randn((M, H), device=device, generator=gen) * 0.25).bfloat16()
            scores = torch.randn((M, E), device=device, generator=gen)
            ids = torch.topk(scores, k, dim=-1).indices.to(torch.int32).contiguous()
            wts = torch.softmax(torch.randn((M, k), device=device, generator=gen), dim=-1).contiguous()
            data = dict(hidden_states=hs, topk_ids=ids, topk_weights=wts, gemm1_weights=w13, gemm1_weights_scale=s13,
                        gemm2_weights=w2, gemm2_weights_scale=s2, top_k=k, routed_scaling_factor=1.0,
                        output=torch.zeros((M, H), dtype=torch.bfloat16, device=device))
            op = alpha_moe.setup(data, M)
            for _ in range(max(args.warmup, 3)):
                op()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=device)
            with torch.cuda.stream(side):
                op()
                with torch.cuda.graph(graph, stream=side):
                    op()
            torch.cuda.synchronize()

            def timed(fn):
                ts = []
                for _ in range(iters):
                    flush.zero_()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    fn()
                    e1.record()
                    e1.synchronize()
                    ts.append(e0.elapsed_time(e1) * 1e3)
                ts.sort()
                return ts[len(ts) // 2]
            us = timed(op)
            us_graph = timed(graph.replay)
            distinct = int(torch.unique(ids).numel())
            alg = distinct * (2 * I * H + H * I + (2 * I // 128) * (H // 128) * 4 + (H // 128) * (I // 128) * 4) + 2 * M * H * 2
            row = {"M": M, "us": round(us, 2), "us_cuda_graph": round(us_graph, 2), "experts_touched": distinct,
                   "algorithmic_bytes": alg, "hbm_frac_graph": round(alg / (us_graph * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)}
            if not args.no_parity:
                from oracle import checks
                data["output"].fill_(float("nan"))
                graph.replay()
                torch.cuda.synchronize()
                row["parity_check"] = checks.alpha_layer_check(data)
            if not args.no_comparators and cmp_note is None:
                try:
                    c_us, rms = _alpha_comparator(data, M, timed)
                    row.update(comparator_us_cuda_graph=round(c_us, 2), speedup=round(c_us / us_graph, 3),
                               rms_ratio_vs_comparator=round(rms, 5))
                except BaseException as exc:      # noqa: BLE001
                    if isinstance(exc, (KeyboardInterrupt, SystemExit)):
                        raise
                    cmp_note = f"unavailable: {type(exc).__name__}: {str(exc)[:200]}"
            rows.append(row)
            del op, graph
    status = gg.device_status(device)
    total_graph = sum(r["us_cuda_graph"] for r in rows)
    big = rows[-1]
    return {
        "metric": "alphamoe_sum_latency_us", "value": total_graph, "unit": "us (sum over the six rows, CUDA-graph replay)",
        "n_gpus": 1, "steps": iters, "warmup": max(args.warmup, 3), "ms_per_step": total_graph * 1e-3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["desc"], "inputs": "N(0,0.25) bf16 tokens, N(0,0.125) weights quantised per 128x128, "
                   "top-10 of random scores, softmax weights (the task generator's distributions)",
                   "l2": "256 MB memset before every timed call", "timing": "CUDA events around each call, median"},
        "clocks": clocks.summary(), "e2e": None, "gpu_launches": iters * 2 * 6 * len(rows), "rows": rows,
        "comparator": cmp_note or "flashinfer trtllm_fp8_block_scale_routed_moe, autotuned, CUDA-graph replay",
        "geomean_speedup_vs_trtllm": _geomean([r.get("speedup") for r in rows]),
        "parity_ok": all(r.get("parity_check", {"ok": True})["ok"] for r in rows),
        "roofline": {"bound": "hbm", "achieved": big["algorithmic_bytes"] / (big["us_cuda_graph"] * 1e-6) / 1e9,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": big["hbm_frac_graph"], "traffic": None,
                     "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']}); row M={big['M']}"},
        "device_status": status,
    }


KGROUPED = dict(G=8, M=4096, N=7168, k=4096,
                desc="k-grouped FP8 GEMM (weight-gradient layout), fp32 accumulation onto D: G=8 groups x 4096 K rows, "
                     "M=4096, N=7168 (a [K_total,M], b [K_total,N] MN-major, packed UE8M0 scales per row and 128 K)")


def run_kgrouped(args, device):
    """d[g] += a[K rows of g].T @ b[K rows of g]: one block-scaled launch over all groups on the MN-major operands."""
    import torch
    from tirx_harness_b200 import grouped_gemm as gg
    cfg = KGROUPED
    G, M, N, k = cfg["G"], cfg["M"], cfg["N"], cfg["k"]
    K = G * k
    gen = torch.Generator(device=device).manual_seed(0)

    def fp8(rows, cols):          # random e4m3 bytes without the two NaN codes, magnitudes below 2
        b = torch.randint(0, 256, (rows, cols), dtype=torch.uint8, device=device, generator=gen) & 0xBF
        return b.view(torch.float8_e4m3fn)

    def words(rows, cols):        # four UE8M0 exponents per word, 2^{-4..0}
        e = torch.randint(123, 128, (rows, cols, 4), dtype=torch.int32, device=device, generator=gen)
        return (e[..., 0] | (e[..., 1] << 8) | (e[..., 2] << 16) | (e[..., 3] << 24)).contiguous()
    a, b = fp8(K, M), fp8(K, N)
    srows = G * ((k + 511) // 512)
    sfa, sfb = words(srows, M), words(srows, N)
    d = torch.zeros((G, M, N), dtype=torch.float32, device=device)
    launch = gg.bind_k_grouped(a, sfa, b, sfb, d, [k] * G)
    for _ in range(max(args.warmup, 3)):
        launch()
    torch.cuda.synchronize()
    steps = min(args.steps, 50)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(device.index) as clocks:
        e0.record()
        for _ in range(steps):
            launch()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    status = gg.device_status(device)
    flops = 2.0 * G * M * N * k
    alg_bytes = K * (M + N) + 2 * G * M * N * 4 + srows * (M + N) * 4
    peaks = _peaks()
    fp8_peak = 2.0 * (peaks["bf16_burst"] or peaks["bf16_sustained"])
    tf = flops / (ms * 1e-3) / 1e12
    return {
        "metric": "k_grouped_gemm_fp8_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["desc"], "l2": f"operands and D ({alg_bytes / 1e6:.0f} MB per call) larger than L2, no flush",
                   "timing": "CUDA events around back-to-back calls; a call = scale packing + one GEMM launch over all groups "
                             "(MN-major operands read as they are)"},
        "clocks": clocks.summary(), "e2e": None, "gpu_launches": steps * 2,
        "roofline": {"bound": "tensor", "achieved": tf, "peak": fp8_peak, "unit": "TFLOP/s", "frac": tf / fp8_peak,
                     "traffic": None, "peak_source": f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({peaks['source']})",
                     "algorithmic_gbs": alg_bytes / (ms * 1e-3) / 1e9},
        "device_status": status,
    }


def _round_floats(obj, nd=6):
    if isinstance(obj, float):
        return round(obj, nd) if math.isfinite(obj) else None
    if isinstance(obj, dict):
        return {k: _round_floats(v, nd) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_round_floats(v, nd) for v in obj]
    return obj


def run_ours(args):
    import torch
    import torch.distributed as dist
    from tirx_harness_b200 import grouped_gemm as gg

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    timer = Timer(device, world, barrier)
    single = {"kgrouped": lambda: run_kgrouped(args, device), "alpha": lambda: run_alpha(args, device),
              "registered": lambda: run_registered(args, device, timer), "moe_task": lambda: run_moe_task(args, device, timer)}
    if args.workload in single:
        if world > 1:
            raise SystemExit(f"the {args.workload} workload is a single-GPU measurement")
        res = single[args.workload]()
        print(json.dumps(_round_floats(res)), flush=True)
        if res.get("parity_ok") is False:
            raise SystemExit("parity check failed")
        return
    if args.workload == "layer":
        res = run_layer(args, world, rank, device, barrier, args.steps, args.warmup)
        if rank == 0:
            print(json.dumps(_round_floats(res)), flush=True)
        if world > 1:
            dist.destroy_process_group()
        if res["parity_check"] is not None and not res["parity_check"]["ok"]:
            raise SystemExit("parity check failed")
        return

    cfg = WORKLOADS[args.workload]
    data = _device_case(cfg, seed=rank, device=device)
    launch = _bind(gg, cfg, data)
    flops, alg_bytes = _algorithmic(cfg)
    layout_key = "masked_m" if cfg.get("masked") else "grouped_layout"

    for _ in range(max(args.warmup, 3)):
        launch()
    barrier()
    if gg.device_status(device) != 0:
        raise SystemExit("device status non-zero after warm-up")

    # ---- timed region: exactly K back-to-back launches, CUDA events on the launching stream, max over ranks; four
    # more regions of the same length follow so that the clock record covers a few hundred milliseconds
    trials = []
    with ClockSampler(local_rank) as clocks:
        ms_step = timer.back_to_back(launch, args.steps)
        for _ in range(4):
            trials.append(timer.back_to_back(launch, args.steps))
    status = gg.device_status(device)
    value = world * flops / (ms_step * 1e-3) / 1e12
    ms_cold = timer.cold_l2_median(launch, 30)
    # ---- parity: what the timed launches left in D, against the oracle (every rank checks its own)
    parity = None
    if not args.no_parity:
        data["D"].fill_(float("nan"))
        launch()
        torch.cuda.synchronize()
        parity = _gemm_parity(cfg, data)
        if world > 1:
            flag = torch.tensor([1 if parity["ok"] else 0], device=device, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            parity["ok_all_ranks"] = bool(flag.item())
    comparators = None
    if world == 1 and not args.no_comparators:
        comparators = {"deep_gemm": cmp_deepgemm(cfg, data, timer, max(10, min(args.steps, 30)), ours=launch)}
        c = comparators["deep_gemm"]
        if "ms_median_cold_l2" in c:
            c["speedup_ours_cold_l2"] = c["ms_median_cold_l2"] / ms_cold
            c["speedup_ours_back_to_back"] = c["ms"] / ms_step

    e2e = None
    if not args.no_e2e:
        # ---- end to end through the public call with HOST buffers: per step the activations (A, SFA,
        # grouped_layout) go host->device from pinned memory, the GEMM runs, D comes back device->host.
        # Weights (B, SFB) are resident model state.  Double-buffered the way a serving loop would run it: two
        # sets of activation/output buffers and three streams, so that the copy-in of step i+1 and the read-back
        # of step i-1 overlap the GEMM of step i (PCIe is full duplex).  Every step's copies are inside the timed
        # region; the serial figure (copy in, GEMM, copy out, one stream) is reported beside it.
        e2e_steps = max(4, min(args.steps, 12))
        hA = data["A"].view(torch.uint8).cpu().pin_memory()
        hS = data["SFA"].cpu().pin_memory()
        hL = data[layout_key].cpu().pin_memory()
        sets = []
        for k in range(2):
            dk = dict(data)
            if k == 1:
                for key in ("A", "SFA", layout_key, "D"):
                    dk[key] = data[key].clone()
            sets.append(dict(data=dk, launch=launch if k == 0 else _bind(gg, cfg, dk),
                             hD=torch.empty(data["D"].shape, dtype=torch.bfloat16).pin_memory(),
                             ev_in=torch.cuda.Event(), ev_comp=torch.cuda.Event(), ev_out=torch.cuda.Event()))
        s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
        cur = torch.cuda.current_stream(device)

        def serial_step():
            st = sets[0]
            st["data"]["A"].view(torch.uint8).copy_(hA, non_blocking=True)
            st["data"]["SFA"].copy_(hS, non_blocking=True)
            st["data"][layout_key].copy_(hL, non_blocking=True)
            st["launch"]()
            st["hD"].copy_(st["data"]["D"], non_blocking=True)

        def pipelined(n):
            for i in range(n):
                st = sets[i % 2]
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(st["ev_comp"])          # the GEMM that last read this input set is done
                    st["data"]["A"].view(torch.uint8).copy_(hA, non_blocking=True)
                    st["data"]["SFA"].copy_(hS, non_blocking=True)
                    st["data"][layout_key].copy_(hL, non_blocking=True)
                    st["ev_in"].record(s_in)
                cur.wait_event(st["ev_in"])
                if i >= 2:
                    cur.wait_event(st["ev_out"])                # this set's D has been read back
                st["launch"]()
                st["ev_comp"].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(st["ev_comp"])
                    st["hD"].copy_(st["data"]["D"], non_blocking=True)
                    st["ev_out"].record(s_out)
            for st in sets:
                cur.wait_event(st["ev_out"])

        serial_step()
        pipelined(2)
        serial_ms = timer.back_to_back(serial_step, e2e_steps)
        e2e_ms = timer.back_to_back(lambda: pipelined(e2e_steps), 1) / e2e_steps
        h2d = hA.numel() + hS.numel() * 4 + hL.numel() * 4
        d2h = sets[0]["hD"].numel() * 2
        e2e = {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps, "serial_ms_per_step": serial_ms,
               "h2d_gbs_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
               "note": "per rank and step: A, SFA, layout from pinned host memory, D back; weights resident; double-buffered "
                       "over three streams; serial = one stream.  Bound by the host link (all ranks share one host)"}
        del sets

    line = None
    if rank == 0:
        peaks = _peaks()
        burst = 2.0 * (peaks["bf16_burst"] or peaks["bf16_sustained"])
        sustained = 2.0 * (peaks["bf16_sustained"] or peaks["bf16_burst"])
        per_gpu = value / world
        traffic = NCU_TRAFFIC_BYTES.get(args.workload)
        ridge = burst * 1e12 / (peaks["hbm_gbs"] * 1e9)
        hbm_bound = flops / alg_bytes < ridge
        ck = clocks.summary()
        gbs = alg_bytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "grouped_gemm_fp8_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": _gemm_config(cfg, world, alg_bytes),
            "clocks": ck,
            "trials_ms_per_step": [ms_step] + trials,
            "ms_median_cold_l2": ms_cold,
            "ms_x_sm_ghz": ms_step * (ck["sm_mhz"] or 0) / 1e3,
            "e2e": e2e,
            "gpu_launches": args.steps * 3,      # per step: scale check+pack, block-scaled GEMM, promotion GEMM (exits at once when not needed)
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": "committed ncu capture" if traffic else None,
                         "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})", "tflops": per_gpu} if hbm_bound else
                        {"bound": "tensor", "achieved": per_gpu, "peak": burst, "unit": "TFLOP/s",
                         "frac": per_gpu / burst, "frac_of_sustained": per_gpu / sustained, "peak_sustained": sustained,
                         "traffic": traffic, "traffic_source": "committed ncu capture of this kernel and workload, not re-measured" if traffic else None,
                         "peak_source": f"2 x bf16_tflops (burst: the launches are timed alone) of MEASURED_PEAKS.json "
                                        f"({peaks['source']}); fp8 issues at twice the bf16 rate",
                         "frac_of_datasheet_4500": per_gpu / DATASHEET_FP8_TFLOPS,
                         "algorithmic_gbs": gbs, "hbm_peak_gbs": peaks["hbm_gbs"]},
            "parity_check": parity,
            "comparators": comparators,
            "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_baseline(cfg)
            cb.pop("seconds", None)
            line["cpu_baseline"] = cb
    extras = {}
    del data, launch
    torch.cuda.empty_cache()
    if args.with_layer:
        extras["moe_layer"] = run_layer(args, world, rank, device, barrier, min(args.steps, 20), args.warmup)
    if args.with_layer and world == 1 and args.workload == "gemm":
        torch.cuda.empty_cache()
        extras["registered"] = run_registered(args, device, timer)
        torch.cuda.empty_cache()
        extras["moe_task"] = run_moe_task(args, device, timer)
        torch.cuda.empty_cache()
        extras["alpha_layer"] = run_alpha(args, device)       # the decode-regime layer's six rows, a few seconds
    ok = True
    if rank == 0:
        line.update(extras)
        # flat summary at the END of the line (a truncated tail of the output still carries it)
        lay = extras.get("moe_layer")
        checks_ok = [line["parity_check"]["ok"] if line["parity_check"] else None]
        if world > 1 and line["parity_check"]:
            checks_ok.append(line["parity_check"].get("ok_all_ranks"))
        if lay and lay.get("parity_check"):
            checks_ok.append(lay["parity_check"]["ok"])
        for key in ("registered", "alpha_layer"):
            if key in extras:
                checks_ok.append(extras[key].get("parity_ok"))
        ok = all(c is not False for c in checks_ok)
        line["summary"] = {
            "gemm_tflops": value, "gemm_ms": ms_step, "gemm_frac_of_burst": line["roofline"].get("frac"),
            "layer_ms_per_step": lay["ms_per_step"] if lay else None,
            "layer_tokens_per_s": lay["value"] if lay else None,
            "layer_sm_mhz": lay["clocks"]["sm_mhz"] if lay else None,
            "layer_e2e_tokens_per_s": lay["e2e"]["value"] if lay else None,
            "registered_geomean_speedup_vs_deepgemm": extras["registered"]["geomean_speedup_vs_deepgemm"] if "registered" in extras else None,
            "moe_task_geomean_speedup_vs_trtllm": extras["moe_task"]["geomean_speedup_vs_trtllm"] if "moe_task" in extras else None,
            "alpha_geomean_speedup_vs_trtllm": extras["alpha_layer"]["geomean_speedup_vs_trtllm"] if "alpha_layer" in extras else None,
            "parity_ok": ok, "n_gpus": world,
        }
        print(json.dumps(_round_floats(line)), flush=True)
    if world > 1:
        flag = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity check failed")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["layer", "alpha", "kgrouped", "registered", "moe_task"],
                    default="gemm")
    ap.add_argument("--no-layer", dest="with_layer", action="store_false",
                    help="skip the measurements that follow the grouped-GEMM one (the expert-parallel MoE layer as "
                         "`moe_layer`; on one GPU also `registered`, `moe_task` and `alpha_layer`)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the post-timing checks against the CPU oracle")
    ap.add_argument("--no-comparators", action="store_true", help="do not time the installed DeepGEMM / flashinfer kernels")
    ap.add_argument("--combine", choices=["pull", "push"], default="push",
                    help="layer workload: how expert outputs travel back (see ep_layer.EpMoeLayer)")
    ap.add_argument("--dispatch", choices=["fused", "kernel"], default="fused",
                    help="layer workload: dispatch all-to-all inside the gate_up GEMM (default) or as its own kernel + barrier")
    ap.add_argument("--fuse-act", action="store_true", help="layer workload: SiLU*mul requant inside the gate_up GEMM's epilogue")
    ap.add_argument("--layer-small", action="store_true", help="layer workload at 2048 tokens / 32 experts (profiling)")
    ap.add_argument("--alpha-rows", type=int, nargs="*", default=None,
                    help="alpha workload: row sizes to run instead of the six official ones (profiling)")
    ap.add_argument("--moe-rows", type=int, nargs="*", default=None, help="moe_task workload: token counts to run")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
