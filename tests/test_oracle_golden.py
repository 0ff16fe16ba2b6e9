"""Pins the CPU oracle against the reference's own golden vectors.

Sources of the expected values (paths inside mlc-ai/TIRx-harness):
  * tools/tests/numsim/corpus/test_fp8_blockwise_gemm_case.py:81-125 (typed in below)
  * tools/src/tirx_harness/numsim/engine-rs/src/runtime/tcgen_ops.rs:9104-9131 (FMA order)
  * tools/tests/numsim/integration/test_fp8_cta1_descriptor_layout.py:132-139 (ones -> 32)
  * tests/golden/*.npz, produced by tests/golden/make_golden.py from the reference's NumPy
    codecs, its B200 hardware cvt goldens and the alphamoe torch oracle.
"""
import os

import numpy as np
import pytest

from oracle import oracle as orc


def _g(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_e4m3_known_answers():
    bits = np.array([0x00, 0x01, 0x07, 0x08, 0x38, 0x3C, 0x7E, 0x80, 0xFE, 0x7F], np.uint8)
    dec = orc.e4m3_decode(bits)
    np.testing.assert_array_equal(
        dec[:-1], np.array([0.0, 2**-9, 7 * 2**-9, 2**-6, 1.0, 1.5, 448.0, -0.0, -448.0], np.float32))
    assert np.signbit(dec[7]) and np.isnan(dec[-1])
    vals = np.array([1.0625, 1.1875, 1000.0, -1000.0, np.nan], np.float32)
    np.testing.assert_array_equal(orc.e4m3_encode(vals),
                                  np.array([0x38, 0x3A, 0x7E, 0xFE, 0x7F], np.uint8))


def test_ue8m0_pack_known_answers():
    exps = np.array([[-1, 0, 1, 2], [3, -2, 4, -3]], np.int16)
    codes = (exps + 127).astype(np.uint8)
    packed = orc.ue8m0_pack(codes)
    assert packed.shape == (1, 2)
    assert int(packed[0, 0]) == 0x81807F7E and int(packed[0, 1]) == 0x7C837D82
    np.testing.assert_array_equal(orc.ue8m0_unpack(packed, 4), codes)
    np.testing.assert_array_equal(orc.ue8m0_decode(codes), np.exp2(exps).astype(np.float32))
    ends = orc.ue8m0_decode(np.array([0x00, 0x7F, 0xFE, 0xFF], np.uint8))
    np.testing.assert_array_equal(ends[:3], np.array([2.0**-127, 1.0, 2.0**127], np.float32))
    assert np.isnan(ends[3])


def test_codecs_match_reference_tables(golden_dir):
    g = _g(golden_dir, "codecs.npz")
    ours = orc.e4m3_decode(np.arange(256, dtype=np.uint8))
    np.testing.assert_array_equal(ours.view(np.uint32) & 0xFFBFFFFF,
                                  g["e4m3_all_decoded"].view(np.uint32) & 0xFFBFFFFF)
    np.testing.assert_array_equal(orc.e4m3_encode(g["e4m3_sweep"]), g["e4m3_sweep_bits"])
    e8 = orc.ue8m0_decode(np.arange(256, dtype=np.uint8))
    np.testing.assert_array_equal(e8[:255], g["e8m0_all_decoded"][:255])
    assert np.isnan(e8[255]) and np.isnan(g["e8m0_all_decoded"][255])
    np.testing.assert_array_equal(orc.bf16_rne(g["bf16_in"]), g["bf16_bits"])


def test_e4m3_encode_matches_b200_cvt_goldens(golden_dir):
    g = _g(golden_dir, "cvt_e4m3x2_f32.npz")
    src = g["f32_source"].view(np.float32)
    enc = orc.e4m3_encode(src).astype(np.uint16)
    got = (enc << 8) | np.roll(enc, -1)       # d = (cvt(a) << 8) | cvt(b), b = source[i+1]
    np.testing.assert_array_equal(got, g["e4m3x2_f32"])


def test_fma_chain_is_increasing_k_binary32():
    a = np.array([[1.0, 1.0, 1.0]], np.float32)
    b = np.array([[2.0**24, 1.0, -(2.0**24)]], np.float32)
    assert orc.fma_abt_increasing_k(a, b)[0, 0] == 0.0          # not 1.0: 2^24 + 1 rounds away
    d = np.array([[2.0 * 0.5]], np.float32)                       # D=2 with scale .5 as chain start
    assert orc.fma_abt_increasing_k(a, b, d)[0, 0] == 0.0
    ones = orc.e4m3_decode(np.full((64, 32), 0x38, np.uint8))
    np.testing.assert_array_equal(orc.fma_abt_increasing_k(ones, ones[:8]), np.full((64, 8), 32.0))


def test_one_scale_per_128_k(golden_dir):
    g = _g(golden_dir, "fp8_one_scale_per_128.npz")
    got = orc.fp8_blockwise_ue8m0(g["A"], g["B"], g["SFA"], g["SFB"])
    expected = np.float32(128 * (1 * 1 + 2 * 0.5 + 0.5 * 2 + 4 * 0.25))
    assert int(got[0, 0]) == int(np.asarray(expected).view(np.uint32) >> 16) == int(g["D"][0, 0])


@pytest.mark.parametrize("seed", [2800, 2801])
def test_fp8_blockwise_corpus_cases(golden_dir, seed):
    g = _g(golden_dir, f"fp8_blockwise_seed{seed}.npz")
    got = orc.fp8_blockwise_ue8m0(g["A"], g["B"], g["SFA"], g["SFB"])
    np.testing.assert_array_equal(got, g["D"])


@pytest.mark.parametrize("model", [orc.SIM_CHAIN, orc.BLOCK_PROMOTE])
def test_block128_scale_format_matches_reference_oracle(golden_dir, model):
    g = _g(golden_dir, "fp8_block128_seed2900.npz")
    A, B = g["A"], g["B"]
    M = A.shape[0]
    got = orc.gg_contiguous(A, B[None], g["sfa"], g["sfb"][None], np.zeros(M, np.int32), model=model)
    np.testing.assert_array_equal(got, g["D"])     # dyadic operands, 2^e scales: every order agrees


def test_grouped_protocol_case_zero_operands_padding_untouched():
    # tools/tests/numsim/corpus/kernels/gemm.py:449-522: zero operands, unit scales, -1 padding
    G, N, K = 4, 384, 512
    aligned = [256, 128, 384, 256]
    M = sum(aligned) + 64
    gl = np.full(M, -1, np.int32)
    s = 0
    for g, m in enumerate(aligned):
        gl[s:s + m - 16] = g
        s += m
    D = np.full((M, N), 0x7FC0, np.uint16)
    orc.gg_contiguous(np.zeros((M, K), np.uint8), np.zeros((G, N, K), np.uint8),
                      np.ones((M, K // 128), np.float32), np.ones((G, 3, K // 128), np.float32), gl, out=D)
    assert (D[gl >= 0] == 0).all() and (D[gl < 0] == 0x7FC0).all()


def test_masked_case_constant_operands():
    # gemm.py:705-795: A = 1.0 everywhere, B = 1.0 (g0) / 2.0 (g1); rows < masked_m[g] give K / 2K
    G, MAXM, N, K = 2, 32, 128, 128
    masked = np.array([13, 27], np.int32)
    A = np.full((G, MAXM, K), 0x38, np.uint8)
    B = np.full((G, N, K), 0x38, np.uint8)
    B[1] = 0x40
    D = orc.gg_masked(A, B, np.ones((G, MAXM, 1), np.float32), np.ones((G, 1, 1), np.float32), masked)
    f = orc.bf16_to_f32(D)
    assert (f[0, :13] == K).all() and (f[1, :27] == 2 * K).all()
    assert (D[0, 13:] == 0).all() and (D[1, 27:] == 0).all()


def test_models_agree_on_random_data_within_tolerance():
    rng = np.random.default_rng(0)
    M, N, K = 64, 256, 1024
    A = orc.e4m3_encode(rng.standard_normal((M, K)).astype(np.float32) * 64)
    B = orc.e4m3_encode(rng.standard_normal((1, N, K)).astype(np.float32) * 64)
    sfa = np.exp2(rng.uniform(-4, 0, (M, K // 128))).astype(np.float32)
    sfb = np.exp2(rng.uniform(-4, 0, (1, N // 128, K // 128))).astype(np.float32)
    gl = np.zeros(M, np.int32)
    d0 = orc.bf16_to_f32(orc.gg_contiguous(A, B, sfa, sfb, gl, model=orc.SIM_CHAIN))
    d1 = orc.bf16_to_f32(orc.gg_contiguous(A, B, sfa, sfb, gl, model=orc.BLOCK_PROMOTE))
    ref = (orc.e4m3_decode(A).astype(np.float64) * np.repeat(sfa, 128, 1)) @ \
          (orc.e4m3_decode(B[0]).astype(np.float64) * np.repeat(np.repeat(sfb[0], 128, 0), 128, 1)).T
    floor = 2.0**-7 * np.sqrt((ref**2).mean())
    for d in (d0, d1):
        assert (np.abs(d - ref) / np.maximum(np.abs(ref), floor)).max() < 2.0**-7
    # MN-major (transposed) scale storage gives identical bits
    sfa_t = np.ascontiguousarray(sfa.T).T
    np.testing.assert_array_equal(orc.gg_contiguous(A, B, sfa_t, sfb, gl), orc.bf16_rne(d0))


def test_quant_rule_matches_alphamoe_oracle(golden_dir):
    g = _g(golden_dir, "alphamoe_oracle.npz")
    q, s = orc.quant_1x128(g["quant_x"])
    np.testing.assert_array_equal(s, g["quant_s"])
    np.testing.assert_array_equal(q, g["quant_q"])
    q2, s2 = orc.quant_1x128(g["quant_x"], mn_major=True)
    np.testing.assert_array_equal(q2, q)
    np.testing.assert_array_equal(s2.T, s)


def test_silu_mul_requant_matches_alphamoe_oracle(golden_dir):
    g = _g(golden_dir, "alphamoe_oracle.npz")
    q, s = orc.silu_mul_requant(g["act_gate_up_bits"], gate_first=True)
    # torch evaluates silu as x*sigmoid(x); the device form is x/(1+exp2(-x*log2e)): last-ulp
    # differences in fp32 may move a value across an e4m3 rounding boundary
    np.testing.assert_allclose(s, g["act_s"], rtol=4e-7)
    dq, dr = orc.e4m3_decode(q), orc.e4m3_decode(g["act_q"])
    assert (q != g["act_q"]).mean() < 2e-3
    np.testing.assert_allclose(dq, dr, rtol=0.126, atol=2**-9)
    # the other operand order used by moe/definition.json
    gu = g["act_gate_up_bits"]
    inter = gu.shape[1] // 2
    swapped = np.concatenate([gu[:, inter:], gu[:, :inter]], axis=1)
    q3, s3 = orc.silu_mul_requant(swapped, gate_first=False)
    np.testing.assert_array_equal(q3, q)
    np.testing.assert_array_equal(s3, s)


def test_moe_layer_matches_alphamoe_oracle_within_its_bound(golden_dir):
    g = _g(golden_dir, "alphamoe_oracle.npz")
    T = g["layer_xq"].shape[0]
    res = orc.moe_layer(g["layer_xq"], g["layer_xs"], None, g["layer_w13"], g["layer_s13"],
                        g["layer_w2"], g["layer_s2"], top_k=2, gate_first=True,
                        routes=(g["layer_ids"], g["layer_w"]), fused_act=True)
    got = orc.bf16_to_f32(res["out"])
    ref = orc.bf16_to_f32(g["layer_out_bits"])
    # bound of alphamoe/definition.json reference_for_check_quantized, with atol=rtol=0.02
    bound = np.maximum(0.02 + 0.02 * np.abs(ref), 2.0 * g["layer_abs_sum"] * 2.0**-7)
    assert got.shape == (T, g["layer_w2"].shape[1])
    assert (np.abs(got - ref) <= bound).all()
    # integer artefacts: counts == bincount(routes), stable token order inside each expert
    plan = res["plan"]
    np.testing.assert_array_equal(plan["counts"], np.bincount(g["layer_ids"].reshape(-1), minlength=4))
    for e in range(4):
        rows = np.nonzero(plan["grouped_layout"] == e)[0]
        assert (np.diff(plan["src_pair"][rows]) > 0).all()
        assert rows.size == plan["counts"][e] and (plan["offsets"][e] % 128 == 0)


def test_alpha_moe_layer_matches_alphamoe_run_within_its_bound(golden_dir):
    """bf16 in, quantised inside, expert-order bf16 accumulation: against `run` of alphamoe/definition.json."""
    g = _g(golden_dir, "alphamoe_bf16_layer.npz")
    res = orc.alpha_moe_layer(g["hidden_bits"], g["ids"], g["w"], g["w13"], g["s13"], g["w2"], g["s2"],
                              routed_scaling_factor=float(g["rsf"]))
    # the in-call quantisation is integer work: bit-exact against the reference's eager Torch recipe
    np.testing.assert_array_equal(res["x_q"], g["xq"])
    np.testing.assert_array_equal(res["x_s"], g["xs"])
    np.testing.assert_array_equal(res["counts"], np.bincount(g["ids"].reshape(-1), minlength=g["w13"].shape[0]))
    got = orc.bf16_to_f32(res["out"])
    ref = orc.bf16_to_f32(g["out_bits"])
    bound = np.maximum(0.02 + 0.02 * np.abs(ref), 2.0 * g["abs_sum"] * 2.0**-7)      # the task's bound, atol=rtol=0.02
    assert (np.abs(got - ref) <= bound).all()
    assert (np.abs(got - ref) <= g["bound"]).all()                                   # and as published (0.1/0.1)
    # the accumulated contribution mass follows the same rounding rule: close to the reference's
    np.testing.assert_allclose(res["abs_sum"], g["abs_sum"], rtol=0.02, atol=0.02)
    # most elements agree to the bit: the differences are fp32 summation order inside the GEMMs
    assert (res["out"] == g["out_bits"]).mean() > 0.8


def test_route_softmax_topk_ties_and_weights():
    logits = np.zeros((3, 16), np.float32)
    logits[1, [5, 9, 2]] = [3.0, 3.0, 1.0]
    logits[2] = np.arange(16, dtype=np.float32)[::-1]
    ids, w = orc.route_softmax_topk(logits, 4)
    np.testing.assert_array_equal(ids[0], [0, 1, 2, 3])            # all tied: lowest indices
    np.testing.assert_array_equal(ids[1], [5, 9, 2, 0])
    np.testing.assert_array_equal(ids[2], [0, 1, 2, 3])
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-6)
    p = np.exp(logits[1] - logits[1].max())
    np.testing.assert_allclose(w[1], p[ids[1]] / p[ids[1]].sum(), rtol=1e-6)


def test_deepseek_routing_matches_reference_routing_block(golden_dir):
    g = _g(golden_dir, "moe_routing.npz")
    ids, w = orc.route_deepseek(g["logits"], g["bias"], routed_scaling_factor=float(g["rsf"]))
    np.testing.assert_array_equal(np.sort(ids, 1), g["topk_idx_sorted"])
    dense = np.zeros_like(g["weights_dense"])
    np.put_along_axis(dense, ids.astype(np.int64), w, 1)
    np.testing.assert_allclose(dense, g["weights_dense"], rtol=2e-6, atol=1e-7)


def test_k_grouped_oracle_matches_the_reference_case_expectation():
    """tools/tests/numsim/corpus/kernels/gemm.py:610-702: all-ones A, B = 1.0 for the first group's K rows and 2.0
    after, unit scales, D preset to 1.25 / -2.5: expected D[0] += k_0, D[1] += 2*k_1, compared with rtol=atol=0."""
    M = N = 128
    ks = [128, 256]
    K = sum(ks)
    A = np.full((K, M), 0x38, np.uint8)
    B = np.full((K, N), 0x38, np.uint8)
    B[ks[0]:] = 0x40
    rows = sum((k + 511) // 512 for k in ks)
    SFA = np.full((rows, M), 0x7F7F7F7F, np.uint32)
    SFB = np.full((rows, N), 0x7F7F7F7F, np.uint32)
    D = np.stack([np.full((M, N), 1.25, np.float32), np.full((M, N), -2.5, np.float32)])
    out = orc.kg_contiguous(A, B, SFA, SFB, ks, D)
    np.testing.assert_array_equal(out[0], np.float32(1.25 + ks[0]))
    np.testing.assert_array_equal(out[1], np.float32(-2.5 + 2 * ks[1]))


def test_moe_task_layer_against_the_reference_run(golden_dir):
    """The registered `moe` task's own operator (tasks/moe/definition.json `run`, executed by
    tests/golden/make_golden.py at the task's fixed geometry, T=16) against this repository's layer oracle on the
    same seeded inputs.  The reference keeps the intermediate in fp32 where the layer requantises it to e4m3, so
    the comparison is the task's own gate (compare_moe_outputs) plus the size of that requantisation noise."""
    from tests.util import moe_output_gate, moe_task_inputs
    g = np.load(os.path.join(golden_dir, "moe_task_layer.npz"))
    T = int(g["T"])
    x = moe_task_inputs(T, int(g["seed"]))
    rid, rw = orc.route_deepseek(x["routing_logits"], x["routing_bias"], routed_scaling_factor=x["routed_scaling_factor"])
    full = orc.moe_layer(x["hidden_states"], np.ascontiguousarray(x["hidden_states_scale"].T), None, x["gemm1_weights"],
                         x["gemm1_weights_scale"], x["gemm2_weights"], x["gemm2_weights_scale"], top_k=8,
                         e_lo=x["local_expert_offset"], routes=(rid, rw), model=orc.BLOCK_PROMOTE)
    got = orc.bf16_to_f32(full["out"])
    ref = orc.bf16_to_f32(g["out_bits"])
    assert full["plan"]["counts"].sum() > 0          # some routes are local
    ok, note, stats = moe_output_gate(got, ref)
    assert ok, note
    assert stats["rms_ratio"] < 0.05, stats          # e4m3 requantisation of the intermediate: a few percent
    assert stats["token_matched"] == 1.0
    # tokens without a local route are exactly zero in both
    local = ((rid >= x["local_expert_offset"]) & (rid < x["local_expert_offset"] + 32)).any(axis=1)
    assert (ref[~local] == 0).all() and (got[~local] == 0).all()
