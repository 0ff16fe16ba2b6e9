import numpy as np
import torch


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def npf(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().float().numpy()


def rel_err(got_f32: np.ndarray, ref_f32: np.ndarray) -> float:
    """max |got-ref| / max(|ref|, 2^-7 * rms(ref)): the floor keeps near-zero outputs from dominating."""
    ref = ref_f32.astype(np.float64)
    if ref.size == 0:
        return 0.0
    floor = 2.0**-7 * np.sqrt((ref**2).mean())
    denom = np.maximum(np.abs(ref), max(floor, 1e-30))
    return float((np.abs(got_f32.astype(np.float64) - ref) / denom).max())


def bf16_ulp(ref_f32: np.ndarray) -> np.ndarray:
    """Spacing of bf16 values at |ref| (8 significand bits)."""
    a = np.abs(ref_f32.astype(np.float64))
    e = np.floor(np.log2(np.maximum(a, 2.0**-126)))
    return np.exp2(e - 7)


def assert_bf16_close(got_bits, ref_bits, min_exact=0.97):
    """bf16 outputs of two fp32-accurate computations can differ by one rounding step where the
    fp32 values straddle a rounding boundary: allow <= 1 bf16 ulp (taken at max(|ref|, 2^-7 rms(ref)),
    the same floor as rel_err, since sums that cancel to ~0 carry the absolute error of their
    terms), and require most outputs to be identical."""
    got = (got_bits.astype(np.uint32) << 16).view(np.float32)
    ref = (ref_bits.astype(np.uint32) << 16).view(np.float32)
    assert np.isfinite(got).all()
    if got.size == 0:
        return
    floor = 2.0**-7 * np.sqrt((ref.astype(np.float64) ** 2).mean())
    allowed = bf16_ulp(np.maximum(np.abs(ref), floor))
    assert (np.abs(got.astype(np.float64) - ref) <= allowed).all()
    if got.size:
        assert (got_bits == ref_bits).mean() >= min_exact


# ------------------------------------------------------------------------------------------------------------
# The reference's own correctness gates, restated (NumPy, float64 reductions) so that the parity tests apply
# exactly what the benchmark server applies.  Pinned by tests/test_gates_cpu.py against the threshold cases the
# reference's tests hold.

GG_DIFF_THRESHOLD = 1e-6      # evolution/benchmark/flashinfer_bench_evolve/tasks/grouped_gemm_fp8/benchmark.py:16


def calc_diff(got, ref) -> float:
    """1 - 2<x,y> / (<x,x> + <y,y>) in float64: the grouped-GEMM task's per-group error measure
    (tasks/grouped_gemm_fp8/benchmark.py:63-74 takes the maximum over the groups' valid-row views and requires
    it to be < 1e-6).  The function itself lives in the un-vendored tirx-kernels package, which re-exports the
    published DeepGEMM `calc_diff`; two all-zero tensors give 0."""
    x = np.asarray(got, np.float64)
    y = np.asarray(ref, np.float64)
    den = (x * x + y * y).sum()
    if den == 0:
        return 0.0
    return float(1.0 - 2.0 * (x * y).sum() / den)


def grouped_gemm_gate(got_views, ref_views):
    """compare_outputs of the grouped-GEMM task: every view finite and of the reference's shape, then
    max over groups of calc_diff < 1e-6.  -> (passed, max_diff)."""
    worst = 0.0
    for g, r in zip(got_views, ref_views, strict=True):
        g = np.asarray(g, np.float32)
        r = np.asarray(r, np.float32)
        if g.shape != r.shape or not np.isfinite(g).all():
            return False, float("inf")
        worst = max(worst, calc_diff(g, r))
    return worst < GG_DIFF_THRESHOLD, worst


MOE_ATOL, MOE_RTOL, MOE_MATCHED, MOE_RMS, MOE_TOKEN_MATCHED = 1.0, 0.3, 0.9, 0.2, 0.9999   # tasks/moe/benchmark.py:23-30


def moe_output_gate(got, ref, atol=MOE_ATOL, rtol=MOE_RTOL, matched=MOE_MATCHED, rms_limit=MOE_RMS,
                    token_matched=MOE_TOKEN_MATCHED):
    """compare_moe_outputs (tasks/moe/benchmark.py:185-211) on top of compare_outputs
    (benchmark_common.py:297-454) for one [T, H] output.  An element fails when its absolute error exceeds atol
    AND its relative error (|ref| + 1e-8 in the denominator) exceeds rtol; at least `matched` of the elements must
    pass; unless the largest absolute error is <= 1e-6 the error RMS over the reference RMS (+1e-8) must be
    strictly below `rms_limit`; and the share of tokens whose own RMS ratio is >= rms_limit (and whose largest
    error exceeds 1e-6) must leave at least `token_matched` of the tokens.  -> (passed, note, stats dict)."""
    x = np.asarray(got, np.float32).astype(np.float64)
    y = np.asarray(ref, np.float32).astype(np.float64)
    if x.shape != y.shape:
        return False, "wrong shape", {}
    if not np.isfinite(x).all():
        return False, "non-finite output", {}
    err = np.abs(x - y)
    rel = err / (np.abs(y) + 1e-8)
    bad = int(((err > atol) & (rel > rtol)).sum())
    ratio = 1.0 - bad / err.size if err.size else 1.0
    max_abs = float(err.max()) if err.size else 0.0
    rms_ratio = float(np.sqrt((err ** 2).mean()) / (np.sqrt((y ** 2).mean()) + 1e-8)) if err.size else 0.0
    stats = dict(max_abs=max_abs, matched=ratio, rms_ratio=rms_ratio)
    if ratio < matched:
        return False, f"elementwise matched ratio {ratio:.6g} < {matched:.6g}", stats
    if max_abs > 1e-6 and rms_ratio >= rms_limit:
        return False, f"output 0 normalized RMS ratio {rms_ratio:.6g} >= {rms_limit:.6g}", stats
    if err.size == 0:
        return True, "ok", stats
    tok = np.sqrt((err ** 2).mean(axis=-1)) / (np.sqrt((y ** 2).mean(axis=-1)) + 1e-8)
    bad_tok = (tok >= rms_limit) & (err.max(axis=-1) > 1e-6)
    tm = 1.0 - int(bad_tok.sum()) / bad_tok.size
    stats["token_matched"] = tm
    if tm < token_matched:
        return False, f"per-token normalized RMS matched ratio {tm:.6g} < {token_matched:.6g}", stats
    return True, "ok", stats


def moe_task_inputs(T: int, seed: int, local_expert_offset: int = 64, rsf: float = 2.5):
    """Seeded inputs of the registered `moe` task at its fixed geometry (hidden 7168, intermediate 2048, 256 experts,
    32 of them local), NumPy only so that the fixture generator and every test draw identical bytes on any machine.
    e4m3 operands are random codes with magnitude below 2 (the task clamps N(0,1) to +-2); scales are
    uniform(0.01, 0.1) like the task's; the bias holds bf16-representable values."""
    H, I, E, El = 7168, 2048, 256, 32
    rng = np.random.default_rng(seed)
    code = lambda shape: rng.integers(0, 256, size=shape, dtype=np.uint8) & np.uint8(0xBF)
    scale = lambda shape: (0.01 + 0.09 * rng.random(shape, dtype=np.float32)).astype(np.float32)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    bias32 = (0.1 * rng.standard_normal(E, dtype=np.float32)).astype(np.float32)
    bias = ((bias32.view(np.uint32) + np.uint32(0x8000)) & np.uint32(0xFFFF0000)).view(np.float32)
    return dict(routing_logits=logits, routing_bias=bias, hidden_states=code((T, H)),
                hidden_states_scale=scale((H // 128, T)), gemm1_weights=code((El, 2 * I, H)),
                gemm1_weights_scale=scale((El, 2 * I // 128, H // 128)), gemm2_weights=code((El, H, I)),
                gemm2_weights_scale=scale((El, H // 128, I // 128)), local_expert_offset=local_expert_offset,
                routed_scaling_factor=rsf)
