"""k-grouped (weight-gradient layout) FP8 GEMM on the GPU, through the C ABI, against the CPU oracle and the
reference's own corpus case."""
import numpy as np
import pytest

import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _run(A, B, SFA, SFB, ks, D):
    from tirx_harness_b200 import grouped_gemm as gg
    dev = torch.device("cuda:0")
    a = torch.from_numpy(A).to(dev).view(torch.float8_e4m3fn)
    b = torch.from_numpy(B).to(dev).view(torch.float8_e4m3fn)
    sfa = torch.from_numpy(SFA.view(np.int32)).to(dev)
    sfb = torch.from_numpy(SFB.view(np.int32)).to(dev)
    d = torch.from_numpy(D.copy()).to(dev)
    launch = gg.bind_k_grouped(a, sfa, b, sfb, d, ks)
    launch()
    torch.cuda.synchronize()
    assert gg.device_status() == 0
    return launch, d


def test_reference_corpus_case_exact():
    """tools/tests/numsim/corpus/kernels/gemm.py:610-702 (G=2, M=N=128, unit scales, constant operands, preset D)."""
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
    _, d = _run(A, B, SFA, SFB, ks, D)
    got = d.cpu().numpy()
    np.testing.assert_array_equal(got[0], np.float32(1.25 + ks[0]))
    np.testing.assert_array_equal(got[1], np.float32(-2.5 + 2 * ks[1]))


def _random_case(M, N, ks, seed):
    rng = np.random.default_rng(seed)
    K = sum(ks)
    vals = np.arange(-2.0, 2.5, 0.5, dtype=np.float32)                 # the corpus's dyadic operand values
    A = orc.e4m3_encode(rng.choice(vals, size=(K, M)).astype(np.float32))
    B = orc.e4m3_encode(rng.choice(vals, size=(K, N)).astype(np.float32))
    rows = sum((k + 511) // 512 for k in ks)
    SFA = rng.integers(126, 129, size=(rows, M, 4), dtype=np.uint32)    # exponents {-1, 0, 1}
    SFB = rng.integers(126, 129, size=(rows, N, 4), dtype=np.uint32)
    pack = lambda c: (c[..., 0] | (c[..., 1] << 8) | (c[..., 2] << 16) | (c[..., 3] << 24)).astype(np.uint32)
    D = rng.standard_normal((len(ks), M, N)).astype(np.float32)
    return A, B, pack(SFA), pack(SFB), D


@pytest.mark.parametrize("mode", ["mn_major", "transposed", "per_group"])
@pytest.mark.parametrize("M,N,ks", [(128, 256, [128, 384]), (256, 208, [640, 0, 128, 1024]), (384, 512, [512, 512, 256])])
def test_k_grouped_matches_oracle(M, N, ks, mode, moe_option):
    """The three host strategies: MN-major operands fed to the tensor core as they are in one launch over all groups
    (default), K-major copies made by a transposing pre-pass, and one launch per group (more than 64 groups)."""
    from tirx_harness_b200 import _lib
    if mode == "transposed":
        moe_option(_lib.OPT_KG_MODE, _lib.KG_MODE_TRANSPOSE)
    elif mode == "per_group":
        moe_option(_lib.OPT_KG_MODE, _lib.KG_MODE_PER_GROUP)
    A, B, SFA, SFB, D = _random_case(M, N, ks, seed=M + N)
    want = orc.kg_contiguous(A, B, SFA, SFB, ks, D)
    launch, d = _run(A, B, SFA, SFB, ks, D)
    got = d.cpu().numpy()
    floor = 2.0**-7 * np.sqrt(np.mean(want.astype(np.float64) ** 2))
    err = np.abs(got - want) / np.maximum(np.abs(want), floor)
    assert err.max() <= 1e-3, err.max()
    # a group without K rows leaves its D untouched, bit for bit
    for g, k in enumerate(ks):
        if k == 0:
            np.testing.assert_array_equal(got[g], D[g])
    # accumulation: a second call adds the same products again
    launch()
    torch.cuda.synchronize()
    twice = d.cpu().numpy()
    np.testing.assert_allclose(twice - got, got - D, rtol=1e-3, atol=1e-3 * np.abs(want).max())


def test_k_grouped_rejects_bad_shapes():
    from tirx_harness_b200 import grouped_gemm as gg
    from tirx_harness_b200 import _lib
    A, B, SFA, SFB, D = _random_case(128, 128, [128, 128], seed=1)
    dev = torch.device("cuda:0")
    t = lambda x: torch.from_numpy(x).to(dev)
    with pytest.raises(_lib.B200MoeError):
        gg.bind_k_grouped(t(A).view(torch.float8_e4m3fn), t(SFA.view(np.int32)), t(B).view(torch.float8_e4m3fn),
                          t(SFB.view(np.int32)), t(D), [64, 192])()
