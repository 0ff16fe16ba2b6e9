"""Parity of the CUDA grouped FP8 GEMM (through the C ABI) with the CPU oracle and golden fixtures.

Tolerance for floating-point values: max relative error <= 1e-3 against the simulator-order oracle,
asserted on the fp32 accumulator (the kernel's MOE_DTYPE_F32 output); the bf16 output must be the
round-to-nearest-even of that accumulator bit for bit, and within one bf16 rounding step (2^-8
relative, i.e. coarser than 1e-3) of the oracle's bf16.  Dyadic fixtures must match bit for bit.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tirx_harness_b200 import _lib
from tests.util import assert_bf16_close, bf16_bits, npf, rel_err, u8

pytestmark = pytest.mark.gpu

TOL = 1e-3


@pytest.fixture(scope="module")
def gg():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tirx_harness_b200 import grouped_gemm
    return grouped_gemm


def _oracle_contig(data, model=orc.SIM_CHAIN, out_f32=False):
    return orc.gg_contiguous(u8(data["A"]), u8(data["B"]), npf(data["SFA"]), npf(data["SFB"]),
                             data["grouped_layout"].cpu().numpy(), model=model, out_f32=out_f32)


def _check_contig(gg, data, tol=TOL, exact=False):
    from tirx_harness_b200 import workloads  # noqa: F401
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in data.items()}
    if data["SFA"].stride(0) == 1:      # keep an MN-major view MN-major on the device
        dev["SFA"] = data["SFA"].t().contiguous().cuda().t()
    dev["D"].fill_(float("nan"))
    launch = gg.setup(dev, data["G"], data["M"], data["N"], data["K"])
    launch()
    assert gg.device_status() == 0
    got_bits = bf16_bits(dev["D"])
    gl = data["grouped_layout"].numpy()
    valid = gl >= 0
    ref_bits = _oracle_contig(data)
    # padding rows keep the poison
    assert np.isnan(orc.bf16_to_f32(got_bits[~valid])).all()
    got, ref = orc.bf16_to_f32(got_bits[valid]), orc.bf16_to_f32(ref_bits[valid])
    assert np.isfinite(got).all()
    if exact:
        np.testing.assert_array_equal(got_bits[valid], ref_bits[valid])
    else:
        # fp32 accumulator against both oracle models
        d32 = torch.full(dev["D"].shape, float("nan"), dtype=torch.float32, device="cuda")
        gg.bind_contiguous(dev["A"], dev["SFA"], dev["B"], dev["SFB"], d32, dev["grouped_layout"])()
        assert gg.device_status() == 0
        got32 = d32.cpu().numpy()
        assert np.isnan(got32[~valid]).all()
        for model in (orc.SIM_CHAIN, orc.BLOCK_PROMOTE):
            assert rel_err(got32[valid], _oracle_contig(data, model, out_f32=True)[valid]) <= tol
        np.testing.assert_array_equal(got_bits[valid], orc.bf16_rne(got32[valid]))
        assert_bf16_close(got_bits[valid], ref_bits[valid])
    return dev, launch


def test_dyadic_block128_fixture_bit_exact(gg, golden_dir):
    g = np.load(os.path.join(golden_dir, "fp8_block128_seed2900.npz"))
    M, K = g["A"].shape
    N = g["B"].shape[0]
    A = torch.from_numpy(g["A"]).cuda().view(torch.float8_e4m3fn)
    B = torch.from_numpy(g["B"]).cuda().view(torch.float8_e4m3fn).view(1, N, K)
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    gl = torch.zeros(M, dtype=torch.int32, device="cuda")
    gg.m_grouped_fp8_gemm_nt_contiguous(A, torch.from_numpy(g["sfa"]).cuda(), B,
                                        torch.from_numpy(g["sfb"]).cuda().view(1, N // 128, K // 128), D, gl)
    assert gg.device_status() == 0
    np.testing.assert_array_equal(bf16_bits(D), g["D"])


def test_config0_tiny_contiguous(gg):
    from tirx_harness_b200.workloads import make_contiguous_case
    for law in ("pow2", "uniform_exp"):
        _check_contig(gg, make_contiguous_case(2, 128, 512, 512, seed=0, law=law))


def test_ragged_groups_padding_and_mn_major_scales(gg):
    from tirx_harness_b200.workloads import make_contiguous_case
    # group sizes not multiples of 128, -1 padding inside 128-row blocks, N not a multiple of 256
    data = make_contiguous_case(4, [200, 0, 77, 333], 384, 1024, seed=3, law="uniform_exp", alignment=32,
                                mn_major_sfa=True)
    _check_contig(gg, data)
    # the registered contract's alignment (224): 128-row blocks straddle two groups
    _check_contig(gg, make_contiguous_case(3, [224, 100, 448], 256, 512, seed=4, alignment=224))


def test_protocol_case_zero_operands(gg):
    from tirx_harness_b200.workloads import make_contiguous_case
    data = make_contiguous_case(4, [256, 250, 130, 256], 384, 512, seed=1)
    data["A"].view(torch.uint8).zero_()
    data["B"].view(torch.uint8).zero_()
    data["SFA"].fill_(1.0)
    data["SFB"].fill_(1.0)
    _check_contig(gg, data, exact=True)


def test_input_dependence_and_repeatability(gg):
    from tirx_harness_b200.workloads import make_contiguous_case
    data = make_contiguous_case(2, [128, 256], 512, 512, seed=7)
    dev, launch = _check_contig(gg, data)
    first = dev["D"].clone()
    dev["D"].fill_(float("nan"))
    launch()
    assert torch.equal(dev["D"][dev["grouped_layout"] >= 0], first[dev["grouped_layout"] >= 0])
    dev["SFA"].mul_(2.0)                       # in-place perturbation of a bound float input
    launch()
    torch.cuda.synchronize()
    v = dev["grouped_layout"] >= 0
    assert torch.equal(dev["D"][v].float(), first[v].float() * 2.0)


def test_empty_and_all_padding(gg):
    K, N = 256, 256
    A = torch.zeros((0, K), dtype=torch.float8_e4m3fn, device="cuda")
    B = torch.zeros((1, N, K), dtype=torch.float8_e4m3fn, device="cuda")
    D = torch.zeros((0, N), dtype=torch.bfloat16, device="cuda")
    gg.m_grouped_fp8_gemm_nt_contiguous(A, torch.zeros((0, 2), device="cuda"), B, torch.ones((1, 2, 2), device="cuda"),
                                        D, torch.zeros(0, dtype=torch.int32, device="cuda"))
    A = torch.zeros((128, K), dtype=torch.float8_e4m3fn, device="cuda")
    D = torch.full((128, N), 7.0, dtype=torch.bfloat16, device="cuda")
    gg.m_grouped_fp8_gemm_nt_contiguous(A, torch.ones((128, 2), device="cuda"), B, torch.ones((1, 2, 2), device="cuda"),
                                        D, torch.full((128,), -1, dtype=torch.int32, device="cuda"))
    assert gg.device_status() == 0
    assert (D == 7.0).all()


def test_bad_arguments_raise(gg):
    from tirx_harness_b200._lib import B200MoeError
    A = torch.zeros((128, 192), dtype=torch.float8_e4m3fn, device="cuda")
    B = torch.zeros((1, 256, 192), dtype=torch.float8_e4m3fn, device="cuda")
    with pytest.raises((ValueError, B200MoeError)):
        gg.m_grouped_fp8_gemm_nt_contiguous(A, torch.ones((128, 1), device="cuda"), B, torch.ones((1, 2, 1), device="cuda"),
                                            torch.zeros((128, 256), dtype=torch.bfloat16, device="cuda"),
                                            torch.zeros(128, dtype=torch.int32, device="cuda"))


def _check_masked(gg, data, tol=TOL):
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in data.items()}
    dev["D"].fill_(float("nan"))
    gg.m_grouped_fp8_gemm_nt_masked(dev["A"], dev["SFA"], dev["B"], dev["SFB"], dev["D"], dev["masked_m"])
    assert gg.device_status() == 0
    got_bits = bf16_bits(dev["D"])
    ref_bits = orc.gg_masked(u8(data["A"]), u8(data["B"]), npf(data["SFA"]), npf(data["SFB"]),
                             data["masked_m"].numpy())
    mm = data["masked_m"].numpy()
    rows = np.arange(data["max_m"])[None, :] < mm[:, None]
    assert np.isnan(orc.bf16_to_f32(got_bits[~rows])).all()        # masked-out rows untouched
    assert_bf16_close(got_bits[rows], ref_bits[rows])
    d32 = torch.full(dev["D"].shape, float("nan"), dtype=torch.float32, device="cuda")
    gg.m_grouped_fp8_gemm_nt_masked(dev["A"], dev["SFA"], dev["B"], dev["SFB"], d32, dev["masked_m"])
    assert gg.device_status() == 0
    got32 = d32.cpu().numpy()
    ref32 = orc.gg_masked(u8(data["A"]), u8(data["B"]), npf(data["SFA"]), npf(data["SFB"]), mm, out_f32=True)
    assert np.isnan(got32[~rows]).all()
    assert rel_err(got32[rows], ref32[rows]) <= tol
    np.testing.assert_array_equal(got_bits[rows], orc.bf16_rne(got32[rows]))


def test_masked_constant_case(gg):
    # corpus case: A = 1.0, B = 1.0 / 2.0, unit scales; rows < masked_m[g] equal K / 2K
    G, MAXM, N, K = 2, 32, 128, 128
    A = torch.full((G, MAXM, K), 0x38, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    Bb = torch.full((G, N, K), 0x38, dtype=torch.uint8, device="cuda")
    Bb[1] = 0x40
    D = torch.full((G, MAXM, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    mm = torch.tensor([13, 27], dtype=torch.int32, device="cuda")
    gg.m_grouped_fp8_gemm_nt_masked(A, torch.ones((G, MAXM, 1), device="cuda"), Bb.view(torch.float8_e4m3fn),
                                    torch.ones((G, 1, 1), device="cuda"), D, mm)
    assert gg.device_status() == 0
    assert (D[0, :13] == K).all() and (D[1, :27] == 2 * K).all()
    assert D[0, 13:].isnan().all() and D[1, 27:].isnan().all()


def test_masked_random_small(gg):
    from tirx_harness_b200.workloads import make_masked_case
    _check_masked(gg, make_masked_case(6, 256, 512, 512, seed=11, law="uniform_exp",
                                       masked_m=[0, 256, 1, 129, 128, 77]))
    _check_masked(gg, make_masked_case(5, 96, 384, 256, seed=12))       # max_m not a multiple of 128


def test_masked_decode_shapes_many_groups_few_rows(gg):
    """Decode regime: many groups with a handful of rows each.  Tiles with at most 16 valid rows fetch a 16-row box
    of A, the schedule comes from the shared-memory tables; checked for the promotion kernel (continuous scales,
    max_m not a multiple of 128) and the block-scaled single-CTA kernel (power-of-two scales, max_m = 128)."""
    from tirx_harness_b200.workloads import make_masked_case
    rng = np.random.default_rng(5)
    G = 96
    mm = rng.integers(0, 13, size=G)
    mm[[3, 40, 95]] = [40, 17, 16]                       # a full group, one just above and one at the small-box limit
    _check_masked(gg, make_masked_case(G, 40, 256, 512, seed=21, law="uniform_exp", masked_m=mm.tolist()))
    mm2 = rng.integers(0, 20, size=G)
    mm2[[0, 50]] = [128, 0]
    _check_masked(gg, make_masked_case(G, 128, 384, 512, seed=22, masked_m=mm2.tolist()))


def test_full_size_properties_config1(gg):
    """Full DeepSeek-V3 gate_up shape: checked through size-independent properties and a row sample."""
    from tirx_harness_b200.workloads import make_operand_b
    G, mpg, N, K = 8, 4096, 4096, 7168
    M = G * mpg
    gen = torch.Generator(device="cuda"); gen.manual_seed(0)
    sfa = torch.exp2(torch.randint(-4, 1, (M, K // 128), generator=gen, device="cuda").float())
    A = torch.empty((M, K), dtype=torch.float8_e4m3fn, device="cuda")
    for r0 in range(0, M, 4096):
        x = torch.randn((4096, K), generator=gen, device="cuda")
        A[r0:r0 + 4096] = (x / sfa[r0:r0 + 4096].repeat_interleave(128, 1)).clamp_(-448, 448).to(torch.float8_e4m3fn)
    cg = torch.Generator(); cg.manual_seed(1)
    Bc, sfbc = make_operand_b(G, N, K, cg)
    B, sfb = Bc.cuda(), sfbc.cuda()
    gl = torch.arange(M, device="cuda", dtype=torch.int32) // mpg
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    launch = gg.bind_contiguous(A, sfa, B, sfb, D, gl)
    launch()
    assert gg.device_status() == 0
    assert torch.isfinite(D).all()
    # (1) sampled rows against the oracle (every 509th row -> all groups, all row positions mod 128)
    step = 509
    ref = orc.gg_contiguous(u8(A), u8(B), npf(sfa), npf(sfb), gl.cpu().numpy(), row_step=step)
    rows = np.arange(0, M, step)
    assert_bf16_close(bf16_bits(D[::step]), ref[rows])
    # (2) linearity in the scales: doubling sfa doubles every output exactly (power of two)
    D1 = D.clone()
    sfa.mul_(2.0)
    launch()
    torch.cuda.synchronize()
    assert torch.equal(D.float(), D1.float() * 2.0)
    # (3) group independence: swapping two groups' rows and layout entries swaps their outputs
    sfa.mul_(0.5)
    A2 = A.clone(); A2[:mpg], A2[mpg:2 * mpg] = A[mpg:2 * mpg], A[:mpg]
    s2 = sfa.clone(); s2[:mpg], s2[mpg:2 * mpg] = sfa[mpg:2 * mpg], sfa[:mpg]
    gl2 = gl.clone(); gl2[:mpg], gl2[mpg:2 * mpg] = 1, 0
    D2 = torch.empty_like(D)
    gg.bind_contiguous(A2, s2, B, sfb, D2, gl2)()
    torch.cuda.synchronize()
    assert torch.equal(D2[:mpg], D1[mpg:2 * mpg]) and torch.equal(D2[mpg:2 * mpg], D1[:mpg])
    assert torch.equal(D2[2 * mpg:], D1[2 * mpg:])


def test_power_of_two_scale_path_equals_promotion_path(gg):
    """With 2^e scales the block-scaled-MMA path and the promotion path compute the same exact products in
    fp32; both must sit within tolerance of the oracle and agree with each other to fp32 rounding.  With one
    scale that is not a power of two the fast path must stand down (decided on the device, per call)."""
    from tirx_harness_b200.workloads import make_contiguous_case
    data = make_contiguous_case(3, [256, 130, 512], 768, 1024, seed=21, law="pow2")
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in data.items()}
    gl = data["grouped_layout"].numpy()
    valid = gl >= 0
    ref32 = _oracle_contig(data, orc.SIM_CHAIN, out_f32=True)
    outs = {}
    for name, ws in (("mx", True), ("promote", False)):
        d32 = torch.full(dev["D"].shape, float("nan"), dtype=torch.float32, device="cuda")
        gg.bind_contiguous(dev["A"], dev["SFA"], dev["B"], dev["SFB"], d32, dev["grouped_layout"], workspace=ws)()
        assert gg.device_status() == 0
        outs[name] = d32.cpu().numpy()
        assert np.isnan(outs[name][~valid]).all()
        assert rel_err(outs[name][valid], ref32[valid]) <= TOL
    assert rel_err(outs["mx"][valid], outs["promote"][valid]) <= 1e-4
    # MOE_OPT_GG_BLOCK_SCALED = 0 forces the promotion kernel even with workspace: bit-identical to the no-workspace run
    old = _lib.set_option(_lib.OPT_GG_BLOCK_SCALED, 0)
    d32 = torch.zeros(dev["D"].shape, dtype=torch.float32, device="cuda")
    launch = gg.bind_contiguous(dev["A"], dev["SFA"], dev["B"], dev["SFB"], d32, dev["grouped_layout"])
    launch()
    np.testing.assert_array_equal(d32.cpu().numpy()[valid], outs["promote"][valid])
    _lib.set_option(_lib.OPT_GG_BLOCK_SCALED, old)
    # one non-power-of-two scale: the same bound launch must now give the promotion result for the new scales
    dev["SFA"][5, 3] = 0.3
    launch()
    assert gg.device_status() == 0
    data["SFA"][5, 3] = 0.3
    ref_b = _oracle_contig(data, orc.BLOCK_PROMOTE, out_f32=True)
    got = d32.cpu().numpy()
    assert rel_err(got[valid], ref_b[valid]) <= 1e-4
    dev["SFA"][5, 3] = 0.25                      # back to a power of two: fast path again, still correct
    data["SFA"][5, 3] = 0.25
    launch()
    assert rel_err(d32.cpu().numpy()[valid], _oracle_contig(data, orc.SIM_CHAIN, out_f32=True)[valid]) <= TOL


def test_output_rows_off_the_32_byte_grid(gg):
    """N a multiple of 8 but not of 16: every other bf16 output row starts 16 bytes off a 32-byte boundary, so the
    epilogues must take their 16-byte stores there (and 32-byte sectors on the aligned rows); last column tile ragged.
    All three kernels: block-scaled pairs (2^e scales), promotion (other scales), single-CTA block-scaled (masked)."""
    from tirx_harness_b200.workloads import make_contiguous_case, make_masked_case
    for law in ("pow2", "uniform_exp"):
        _check_contig(gg, make_contiguous_case(2, [256, 77], 520, 512, seed=41, law=law))
        _check_contig(gg, make_contiguous_case(1, [130], 264, 256, seed=42, law=law))
    _check_masked(gg, make_masked_case(3, 128, 520, 512, seed=43, law="pow2", masked_m=[128, 5, 64]))
    _check_masked(gg, make_masked_case(2, 64, 264, 256, seed=44, law="uniform_exp", masked_m=[64, 33]))


def test_masked_power_of_two_path(gg):
    from tirx_harness_b200.workloads import make_masked_case
    _check_masked(gg, make_masked_case(5, 256, 512, 1024, seed=31, law="pow2", masked_m=[256, 0, 129, 77, 255]))
    _check_masked(gg, make_masked_case(3, 384, 384, 512, seed=32, law="pow2", masked_m=[384, 100, 257]))


def test_registered_contract_packed_ue8m0_scales_alignment_224(gg):
    """The registered grouped_gemm/fp8 layout: UE8M0 scales packed four per int32, stored MN-major
    (tools/tests/numsim/corpus/kernels/gemm.py:252-263 pins the packing), B scales per column, groups padded
    to 224 rows with -1 in grouped_layout."""
    from tirx_harness_b200.workloads import make_contiguous_case
    data = make_contiguous_case(3, [224, 300, 17], 512, 1024, seed=51, law="pow2", alignment=224)
    M, N, K, G = data["M"], data["N"], data["K"], data["G"]
    codes_a = (np.log2(data["SFA"].numpy()).astype(np.int32) + 127).astype(np.uint8)             # [M, K/128]
    sfa_words = orc.ue8m0_pack(codes_a)                                                            # [K/512, M]
    sfb_col = np.repeat(data["SFB"].numpy(), 128, axis=1)[:, :N]                                   # per column
    codes_b = (np.log2(sfb_col).astype(np.int32) + 127).astype(np.uint8)                           # [G, N, K/128]
    sfb_words = np.stack([orc.ue8m0_pack(codes_b[g]) for g in range(G)])                           # [G, K/512, N]
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in data.items()}
    dev["SFA"] = torch.from_numpy(sfa_words.view(np.int32)).cuda().t()                             # [M, K/512] MN-major
    dev["SFB"] = torch.from_numpy(sfb_words.view(np.int32)).cuda().permute(0, 2, 1)               # [G, N, K/512]
    dev["D"].fill_(float("nan"))
    gg.setup(dev, G, M, N, K)()
    assert gg.device_status() == 0
    gl = data["grouped_layout"].numpy()
    valid = gl >= 0
    got = bf16_bits(dev["D"])
    ref = _oracle_contig(data)
    assert np.isnan(orc.bf16_to_f32(got[~valid])).all()
    assert_bf16_close(got[valid], ref[valid])
    # identical to the fp32-scale entry on the same values
    d2 = torch.full_like(dev["D"], float("nan"))
    gg.bind_contiguous(dev["A"], data["SFA"].cuda(), dev["B"], data["SFB"].cuda(), d2, dev["grouped_layout"])()
    assert torch.equal(d2[dev["grouped_layout"] >= 0], dev["D"][dev["grouped_layout"] >= 0])
