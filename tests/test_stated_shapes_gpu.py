"""Parity at the shapes the benchmark configurations state (not scaled-down stand-ins): the masked decode GEMMs
(G=32, max_m=256; N=4096,K=7168 and N=7168,K=2048), the Zipf-imbalanced contiguous GEMM (G=64, 65536 rows) and the
full MoE layer (16384 tokens, 256 experts) on one GPU."""
import numpy as np
import pytest
import torch

from oracle import checks
from oracle import oracle as orc
from tests.util import assert_bf16_close, bf16_bits, npf, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gg():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tirx_harness_b200 import grouped_gemm
    return grouped_gemm


@pytest.mark.parametrize("law", ["pow2", "uniform_exp"])
@pytest.mark.parametrize("N,K", [(4096, 7168), (7168, 2048)])
def test_masked_decode_shapes_full_compare(gg, N, K, law):
    """G=32 experts, max_m=256, masked_m ~ U{0..256}: every valid row against the oracle; rows at and past masked_m
    keep their NaN poison.  pow2 scales take the block-scaled kernel, continuous ones the promotion kernel."""
    from tirx_harness_b200.workloads import make_masked_case
    G, max_m = 32, 256
    data = make_masked_case(G, max_m, N, K, seed=N + K, law=law)
    mm = data["masked_m"].numpy()
    assert 0 < mm.sum() < G * max_m
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in data.items()}
    dev["D"].fill_(float("nan"))
    gg.bind_masked(dev["A"], dev["SFA"], dev["B"], dev["SFB"], dev["D"], dev["masked_m"])()
    assert gg.device_status() == 0
    ref = orc.gg_masked(u8(data["A"]), u8(data["B"]), npf(data["SFA"]), npf(data["SFB"]), mm)
    got = bf16_bits(dev["D"])
    valid = np.arange(max_m)[None, :] < mm[:, None]
    assert np.isnan(orc.bf16_to_f32(got[~valid])).all()
    assert_bf16_close(got[valid], ref[valid])
    # the reference task's own measure, per group
    from tests.util import grouped_gemm_gate
    views = [(orc.bf16_to_f32(got[g, :mm[g]]), orc.bf16_to_f32(ref[g, :mm[g]])) for g in range(G) if mm[g] > 0]
    ok, worst = grouped_gemm_gate([v[0] for v in views], [v[1] for v in views])
    assert ok, worst


def test_zipf_imbalanced_contiguous_shape(gg):
    """G=64 experts, Zipf(1.2) row counts over 65536 routed rows, each group padded to 128: padding rows keep their
    poison, every valid row is finite, and a row sample over the largest, two middle and the smallest group matches
    the oracle."""
    import bench
    cfg = bench.WORKLOADS["zipf"]
    data = bench._device_case(cfg, seed=0, device=torch.device("cuda", 0))
    sizes = data["sizes"]
    assert sum(sizes) == 65536 and len(sizes) == 64 and sizes[0] > 20 * sizes[-1]
    gl = data["grouped_layout"]
    # the layout itself: group g owns ceil(size/128)*128 consecutive rows, the first `size` of them valid
    want = np.full(data["M"], -1, np.int32)
    r = 0
    for g, m in enumerate(sizes):
        want[r:r + m] = g
        r += (m + 127) // 128 * 128
    np.testing.assert_array_equal(gl.cpu().numpy(), want)
    data["D"].fill_(float("nan"))
    gg.setup(data, data["G"], data["M"], data["N"], data["K"])()
    assert gg.device_status() == 0
    valid = gl >= 0
    assert bool(torch.isnan(data["D"][~valid].float()).all())
    assert bool(torch.isfinite(data["D"][valid].float()).all())
    res = bench._gemm_parity(cfg, data, rows=96)
    assert res["ok"] and res["rows"] >= 64 and res["groups"] == 4, res


def test_moe_layer_full_size_every_stage(gg):
    """16384 tokens, hidden 7168, 256 experts x intermediate 2048, top-8 on one GPU: routing, receive counts, every
    dispatched row, and sampled rows of both grouped GEMMs, the activation and the combine, against the oracle."""
    import bench
    from tirx_harness_b200 import ep_layer
    dev = torch.device("cuda", 0)
    cfg = bench.LAYER
    data = bench._layer_case(1, 0, dev, cfg)
    layer = ep_layer.setup(data, cfg["T"], top_k=cfg["top_k"])
    data["output"].fill_(float("nan"))
    layer()
    assert gg.device_status() == 0
    assert bool(torch.isfinite(data["output"].float()).all())
    res = checks.ep_layer_check(layer, data, 1, 0, tokens=96, rows=96, experts=4)
    layer.close()
    for stage in ("routing", "counts", "dispatch", "gate_up", "act", "down", "combine"):
        assert res[stage]["ok"], (stage, res[stage])
    assert res["dispatch"]["rows"] == cfg["T"] * cfg["top_k"]
    assert res["gate_up"]["rows"] >= 64 and res["down"]["rows"] >= 64
