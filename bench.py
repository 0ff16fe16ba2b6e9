#!/usr/bin/env python
"""Benchmark of the MoE m-grouped FP8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|masked|zipf|layer]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # CPU arm: the oracle port of the reference's simulator

Default workload (`gemm`): the DeepSeek-V3-shaped m-grouped contiguous FP8 GEMM, G=8 experts x 4096
rows, N=4096, K=7168, per GPU.  With N GPUs every rank owns its own 8 experts (experts shard, no
data-path collective): weak scaling, value = total TFLOP/s over all ranks.  One step = one launch
of the grouped GEMM over the whole batch.  Prints ONE JSON line on rank 0.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DATASHEET_FP8_TFLOPS = 4500.0
DATASHEET_HBM_GBS = 8000.0

# DRAM bytes per launch of the dominant kernel (gg_fp8_mx_kernel on the `gemm` workload) from the committed ncu
# capture (profiles/gg_fp8_mx_kernel_contiguous_c1.md): dram__bytes_read.sum + dram__bytes_write.sum.
NCU_TRAFFIC_BYTES = {"gemm": 799.4e6}

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


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(bf16_burst=p.get("bf16_tflops"), bf16_sustained=p.get("bf16_tflops_sustained"),
                    hbm_gbs=p.get("hbm_gbs"), source="measured")
    return dict(bf16_burst=1590.0, bf16_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read only)."""

    def __init__(self, index: int, period_s: float = 0.02):
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
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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


def _algorithmic(cfg):
    """FLOPs and bytes over VALID rows only."""
    G, N, K = cfg["G"], cfg["N"], cfg["K"]
    rows = sum(_group_sizes(cfg, 0))
    flops = 2.0 * rows * N * K
    bytes_ = rows * K + G * N * K + rows * N * 2 + rows * (K // 128) * 4 + G * ((N + 127) // 128) * (K // 128) * 4
    return flops, float(bytes_)


def cpu_baseline(cfg, seed=0, rows_per_group=1024):
    """Times the CPU oracle (simulator-order FMA chain) on a bounded row sample of the workload."""
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
    t0 = time.perf_counter()
    orc.gg_contiguous(A, B, sfa, sfb, gl, model=orc.SIM_CHAIN)
    dt = time.perf_counter() - t0
    flops = 2.0 * M * N * K
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"{rows_per_group} rows of each of the {G} groups (all N={N}, all K={K}; includes decoding "
                      f"each group's B once), {dt:.1f} s",
            "seconds": dt}


def run_reference(args):
    """--impl reference: the reference's CPU path (its simulator's arithmetic, restated in oracle/oracle.c;
    the simulator itself is Rust and cannot be built here).  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg = WORKLOADS[args.workload]
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_baseline(cfg, rows_per_group=4)
    steps = max(1, min(args.steps, 3))
    vals, secs = [], []
    for s in range(steps):
        r = cpu_baseline(cfg, seed=s)
        vals.append(r["value"])
        secs.append(r["seconds"])
    v = statistics.median(vals)
    flops, _ = _algorithmic(cfg)
    line = {
        "impl": "reference", "metric": "grouped_gemm_fp8_tflops", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": flops / (v * 1e12) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["desc"], "note": "CPU oracle port of the reference simulator's arithmetic; "
                   "each step times a bounded row sample and ms_per_step extrapolates to the full workload"},
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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
    layer = ep_layer.setup(data, Tl, top_k=cfg["top_k"], combine=args.combine)
    for _ in range(max(warmup, 3)):
        layer()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(device.index) as clocks:
        barrier()
        e0.record()
        for _ in range(steps):
            layer()
        e1.record()
        barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    status = gg.device_status(device)
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

    def timed(fn):
        barrier()
        e0.record()
        fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / e2e_steps
    e2e_step()
    pipelined(2)
    serial_ms = timed(lambda: [e2e_step() for _ in range(e2e_steps)])
    e2e_ms = timed(lambda: pipelined(e2e_steps))
    H, I, k = cfg["H"], cfg["I"], cfg["top_k"]
    flops = 2.0 * cfg["T"] * k * (2 * I * H + H * I)
    res = {
        "metric": "moe_layer_tokens_per_s", "value": cfg["T"] / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": cfg["desc"], "tokens_per_rank": Tl, "experts_per_rank": cfg["E"] // world,
                   "routing": "softmax top-8, ties to lowest index, weights renormalised",
                   "l2": "weights (1.4-11 GB per rank) larger than L2, no flush", "rows_this_rank": int(counts),
                   "combine": args.combine},
        "clocks": clocks.summary(),
        "e2e": {"value": cfg["T"] / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": hx.numel() + hs_.numel() * 4 + hl.numel() * 4, "d2h_bytes_per_step": ho.numel() * 2,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "serial_ms_per_step": serial_ms,
                "note": "per rank: fp8 tokens, scales and router logits copied from pinned host memory, bf16 output copied "
                        "back, every step; the host copies run on their own streams through device staging buffers and "
                        "overlap the neighbouring steps' compute; serial_ms_per_step = the same on one stream"},
        "gpu_launches": steps * 15,
        "tflops_grouped_gemms": flops / (ms * 1e-3) / 1e12,
        "stages_ms_rank0": {k: round(v, 4) for k, v in stages.items()},
        "device_status": status,
    }
    layer.close()
    return res


ALPHA_ROWS = (1, 8, 16, 32, 64, 128)
ALPHA = dict(H=2048, I=128, E=512, top_k=10,
             desc="decode-regime MoE layer from bf16 activations and preselected routes (alphamoe contract): "
                  "K=2048, I=128, E=512, top-10, rows M in {1,8,16,32,64,128}")


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
            rows.append({"M": M, "us": round(us, 2), "us_cuda_graph": round(us_graph, 2), "experts_touched": distinct,
                         "algorithmic_bytes": alg, "hbm_frac_graph": round(alg / (us_graph * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)})
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
        "roofline": {"bound": "hbm", "achieved": big["algorithmic_bytes"] / (big["us_cuda_graph"] * 1e-6) / 1e9,
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": big["hbm_frac_graph"], "traffic": None,
                     "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']}); row M=128"},
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
    fp8_peak = 2.0 * (peaks["bf16_sustained"] or peaks["bf16_burst"])
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
                     "traffic": None, "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']})",
                     "algorithmic_gbs": alg_bytes / (ms * 1e-3) / 1e9},
        "device_status": status,
    }


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

    if args.workload == "kgrouped":
        if world > 1:
            raise SystemExit("the kgrouped workload is a single-GPU measurement")
        print(json.dumps(run_kgrouped(args, device)), flush=True)
        return
    if args.workload == "alpha":
        if world > 1:
            raise SystemExit("the alpha workload is a single-GPU latency measurement")
        print(json.dumps(run_alpha(args, device)), flush=True)
        return
    if args.workload == "layer":
        res = run_layer(args, world, rank, device, barrier, args.steps, args.warmup)
        if rank == 0:
            print(json.dumps(res), flush=True)
        if world > 1:
            dist.destroy_process_group()
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

    # ---- timed region: K back-to-back launches, CUDA events on the launching stream
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for _ in range(args.steps):
            launch()
        e1.record()
        barrier()
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    status = gg.device_status(device)
    value = world * flops / (ms_step * 1e-3) / 1e12

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

        def timed(fn):
            barrier()
            e0.record()
            fn()
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) / e2e_steps
        serial_step()
        pipelined(2)
        serial_ms = timed(lambda: [serial_step() for _ in range(e2e_steps)])
        e2e_ms = timed(lambda: pipelined(e2e_steps))
        h2d = hA.numel() + hS.numel() * 4 + hL.numel() * 4
        d2h = sets[0]["hD"].numel() * 2
        e2e = {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps, "serial_ms_per_step": serial_ms,
               "note": "A, SFA, grouped_layout copied from pinned host memory and D copied back every step, weights "
                       "resident; double-buffered over three streams (copy-in of step i+1 and read-back of step i-1 "
                       "overlap the GEMM of step i); serial_ms_per_step = the same on one stream"}
        del sets

    if rank == 0:
        peaks = _peaks()
        fp8_peak = 2.0 * (peaks["bf16_sustained"] or peaks["bf16_burst"])
        per_gpu = value / world
        traffic = NCU_TRAFFIC_BYTES.get(args.workload)
        ridge = fp8_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)
        hbm_bound = flops / alg_bytes < ridge
        line = {
            "metric": "grouped_gemm_fp8_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": cfg["desc"] + (f"; per GPU, {world} GPUs each own {cfg['G']} experts" if world > 1 else ""),
                       "scales": "fp32, A 1x128 per row, B 128x128, 2^{-4..0}", "accumulate": "fp32", "out": "bf16",
                       "l2": f"inputs ({alg_bytes / 1e6:.0f} MB per launch) larger than L2, no flush", "seed": 0,
                       "timing": "CUDA events around K back-to-back launches, max over ranks"},
            "clocks": clocks.summary(),
            "e2e": e2e,
            "gpu_launches": args.steps * 3,      # per step: scale check+pack, block-scaled GEMM, promotion GEMM (exits at once when not needed)
            "roofline": {"bound": "hbm", "achieved": alg_bytes / (ms_step * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": alg_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         "traffic": traffic, "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})",
                         "tflops": per_gpu} if hbm_bound else
                        {"bound": "tensor", "achieved": per_gpu, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": per_gpu / fp8_peak, "traffic": traffic,
                         "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}); "
                                        "fp8 tensor rate is twice bf16",
                         "frac_of_datasheet_4500": per_gpu / DATASHEET_FP8_TFLOPS,
                         "algorithmic_gbs": alg_bytes / (ms_step * 1e-3) / 1e9,
                         "hbm_peak_gbs": peaks["hbm_gbs"]},
            "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_baseline(cfg)
            cb.pop("seconds", None)
            line["cpu_baseline"] = cb
    layer_res = None
    if args.with_layer:
        del data, launch
        torch.cuda.empty_cache()
        layer_res = run_layer(args, world, rank, device, barrier, min(args.steps, 20), args.warmup)
    alpha_res = None
    if args.with_layer and world == 1 and args.workload == "gemm":
        torch.cuda.empty_cache()
        alpha_res = run_alpha(args, device)       # the decode-regime layer's six rows, a few seconds
    if rank == 0:
        if layer_res is not None:
            line["moe_layer"] = layer_res
        if alpha_res is not None:
            line["alpha_layer"] = alpha_res
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["layer", "alpha", "kgrouped"], default="gemm")
    ap.add_argument("--no-layer", dest="with_layer", action="store_false",
                    help="skip the expert-parallel MoE layer measurement that follows the grouped-GEMM one "
                         "(it is reported as the extra object `moe_layer` of the same JSON line; on one GPU the "
                         "decode-regime layer's rows follow as `alpha_layer`)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--combine", choices=["pull", "push"], default="push",
                    help="layer workload: how expert outputs travel back (see ep_layer.EpMoeLayer)")
    ap.add_argument("--layer-small", action="store_true", help="layer workload at 2048 tokens / 32 experts (profiling)")
    ap.add_argument("--alpha-rows", type=int, nargs="*", default=None,
                    help="alpha workload: row sizes to run instead of the six official ones (profiling)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
