"""The reference's correctness gates as restated in tests/util.py, pinned by the threshold cases of the
reference's own tests (evolution/tests/test_moe_rms.py:57-116, evolution/tests/test_grouped_gemm_task.py:73-80)."""
import numpy as np
import pytest
import torch

from tests.util import calc_diff, grouped_gemm_gate, moe_output_gate


def _bf16(a):
    return torch.from_numpy(np.asarray(a, np.float32)).bfloat16().float().numpy()


@pytest.mark.parametrize("scale,passed", [(0.0, False), (0.1, False), (0.5, False), (1.0, True), (1.01, True)])
def test_low_amplitude_output(scale, passed):
    ref = _bf16(np.linspace(-0.25, 0.25, 128).reshape(4, 32))
    ok, note, stats = moe_output_gate(_bf16(ref * scale), ref)
    assert ok is passed
    assert stats["matched"] == 1.0                      # all errors are below atol: the elementwise rule cannot see them
    assert stats["rms_ratio"] == pytest.approx(abs(1.0 - scale), abs=0.003)
    if not passed:
        assert "output 0 normalized RMS ratio" in note


def test_genuine_zero_reference_passes():
    ref = np.zeros((1, 32), np.float32)
    ok, _, stats = moe_output_gate(ref.copy(), ref)
    assert ok and stats["rms_ratio"] == 0.0


@pytest.mark.parametrize("affected", [9, 1])
def test_sparse_missing_contribution_fails(affected):
    ref = np.full((100, 32), 0.125, np.float32)
    got = ref.copy()
    got[:affected] = 0
    ok, note, stats = moe_output_gate(got, ref)
    assert not ok
    assert stats["rms_ratio"] == pytest.approx((affected / 100) ** 0.5)
    if affected == 1:
        assert "per-token normalized RMS matched ratio" in note


@pytest.mark.parametrize("tokens,outliers,passed", [(9999, 1, False), (10000, 1, True), (10000, 2, False)])
def test_rare_token_outlier_budget(tokens, outliers, passed):
    ref = np.full((tokens, 32), 0.125, np.float32)
    got = ref.copy()
    got[:outliers] = 0
    ok, note, _ = moe_output_gate(got, ref)
    assert ok is passed
    if not passed:
        assert "per-token normalized RMS matched ratio" in note


def test_grouped_gemm_gate_valid_rows():
    """Equal views pass; a zeroed or non-finite group fails (test_grouped_gemm_task.py:73-80)."""
    views = [np.ones((2, 2), np.float32), np.ones((1, 2), np.float32)]
    ref = [v.copy() for v in views]
    assert grouped_gemm_gate(views, ref)[0]
    views[-1][:] = 0
    assert not grouped_gemm_gate(views, ref)[0]
    views[-1][:] = np.nan
    assert not grouped_gemm_gate(views, ref)[0]
    assert calc_diff(np.zeros(4), np.zeros(4)) == 0.0


def test_calc_diff_equals_the_installed_deepgemm_helper():
    """tirx-kernels re-exports DeepGEMM's calc_diff; where a DeepGEMM build is importable the restatement is
    checked against it on random bf16 data."""
    numeric = pytest.importorskip("vllm.third_party.deep_gemm.testing.numeric")
    rng = np.random.default_rng(3)
    x = _bf16(rng.standard_normal((64, 96)))
    y = _bf16(x + 1e-3 * rng.standard_normal(x.shape))
    want = float(numeric.calc_diff(torch.from_numpy(x), torch.from_numpy(y)))
    assert calc_diff(x, y) == pytest.approx(want, rel=1e-9, abs=1e-15)

