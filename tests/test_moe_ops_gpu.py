"""Parity of the memory-bound MoE stages and of the single-GPU layer with the CPU oracle.

Integer artefacts (routing ids, counts, offsets, destination rows, grouped_layout) must be
bit-exact.  FP8 codes are compared exactly where the arithmetic is exactly specified (1x128
quantisation) and with a one-code-step allowance on a tiny fraction of elements where a
transcendental (exp2 in SiLU) may differ in the last ulp between libm and the GPU.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.util import assert_bf16_close, bf16_bits, npf, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tirx_harness_b200 import grouped_gemm, moe_ops
    moe_ops.status = grouped_gemm.device_status
    return moe_ops


def _codes_close(q, ref, max_mismatch=2e-3):
    assert q.shape == ref.shape
    if (q != ref).any():
        assert (q != ref).mean() <= max_mismatch
        dq, dr = orc.e4m3_decode(q), orc.e4m3_decode(ref)
        np.testing.assert_allclose(dq, dr, rtol=0.126, atol=2**-9)


def test_quant_1x128_bit_exact(ops):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn((96, 1024), generator=g) * torch.exp2(torch.randint(-8, 8, (96, 1), generator=g).float())).bfloat16()
    x[5, 256:384] = 0
    x[7, :128] = 1e-30
    for mn in (False, True):
        q, s = ops.quant_1x128(x.cuda(), mn_major=mn)
        rq, rs = orc.quant_1x128(x.float().numpy())
        assert ops.status() == 0
        np.testing.assert_array_equal(npf(s), rs)
        np.testing.assert_array_equal(u8(q), rq)


def test_silu_mul_requant_vs_oracle_and_golden(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "alphamoe_oracle.npz"))
    gu_bits = g["act_gate_up_bits"]
    gu = torch.from_numpy(gu_bits.view(np.int16)).view(torch.bfloat16).cuda()
    q, s = ops.silu_mul_requant(gu, gate_first=True)
    assert ops.status() == 0
    rq, rs = orc.silu_mul_requant(gu_bits, gate_first=True)
    np.testing.assert_allclose(npf(s), rs, rtol=1e-6)
    _codes_close(u8(q), rq)
    np.testing.assert_allclose(npf(s), g["act_s"], rtol=1e-6)      # the reference torch oracle's outputs
    _codes_close(u8(q), g["act_q"])
    # other operand order, MN-major scales, padding rows skipped
    gen = torch.Generator().manual_seed(9)
    gu2 = (torch.randn((300, 1024), generator=gen) * 4).bfloat16()
    layout = torch.randint(-1, 3, (300,), generator=gen).int()
    q2, s2 = ops.silu_mul_requant(gu2.cuda(), gate_first=False, layout=layout.cuda(), mn_major=True)
    rq2, rs2 = orc.silu_mul_requant(bf16_bits(gu2), gate_first=False, row_valid=(layout >= 0).numpy().astype(np.uint8))
    assert s2.stride(0) == 1
    np.testing.assert_allclose(npf(s2), rs2, rtol=1e-6)
    _codes_close(u8(q2), rq2)
    assert (u8(q2)[(layout < 0).numpy()] == 0).all()


def test_route_topk_ids_exact(ops):
    gen = torch.Generator().manual_seed(0)
    logits = torch.randn((777, 256), generator=gen)
    logits[3] = 0.0                       # all tied -> lowest indices
    logits[4, [200, 100]] = 9.0           # tie between two winners -> lower index first
    logits[5] = torch.arange(256).float().flip(0) * 0.01
    ids, w = ops.route_topk(logits.cuda(), 8)
    rid, rw = orc.route_softmax_topk(logits.numpy(), 8)
    assert ops.status() == 0
    np.testing.assert_array_equal(ids.cpu().numpy(), rid)
    np.testing.assert_allclose(npf(w), rw, rtol=2e-6)
    ids2, w2 = ops.route_topk(torch.randn((33, 48), generator=gen).cuda(), 5)
    assert ids2.shape == (33, 5) and torch.allclose(w2.sum(1), torch.ones(33, device="cuda"), rtol=1e-5)


@pytest.mark.parametrize("T,E_glob,e_lo,E_loc,top_k,align", [
    (1000, 64, 0, 64, 8, 128), (4099, 256, 32, 32, 8, 128), (5, 16, 0, 16, 2, 128), (300, 8, 2, 3, 2, 224),
    (2048, 256, 0, 256, 8, 128)])
def test_permute_plan_bit_exact(ops, T, E_glob, e_lo, E_loc, top_k, align):
    gen = torch.Generator().manual_seed(T)
    ids = torch.stack([torch.randperm(E_glob, generator=gen)[:top_k] for _ in range(T)]).int()
    if T > 100:
        ids[ids == e_lo + 1] = e_lo          # leave one local expert empty, skew another
    plan = ops.permute_plan(ids.cuda(), e_lo, E_loc, align)
    assert ops.status() == 0
    ref = orc.permute_plan(ids.numpy(), e_lo, E_loc, align, cap_rows=plan["cap_rows"])
    for k in ("counts", "offsets", "pos", "src_pair", "grouped_layout"):
        np.testing.assert_array_equal(plan[k].cpu().numpy(), ref[k], err_msg=k)
    local = (ids.numpy() >= e_lo) & (ids.numpy() < e_lo + E_loc)
    np.testing.assert_array_equal(ref["counts"], np.bincount(ids.numpy()[local] - e_lo, minlength=E_loc))


def test_permute_and_combine(ops):
    gen = torch.Generator().manual_seed(1)
    T, H, E, top_k = 200, 512, 8, 2
    x_q = torch.randint(0, 255, (T, H), generator=gen, dtype=torch.uint8)
    x_s = torch.rand((T, H // 128), generator=gen)
    ids = torch.stack([torch.randperm(E, generator=gen)[:top_k] for _ in range(T)]).int()
    plan = ops.permute_plan(ids.cuda(), 0, E, 128)
    a, s = ops.permute(x_q.cuda().view(torch.float8_e4m3fn), x_s.cuda(), plan["src_pair"], top_k)
    src = plan["src_pair"].cpu().numpy()
    valid = src >= 0
    np.testing.assert_array_equal(u8(a)[valid], x_q.numpy()[src[valid] // top_k])
    np.testing.assert_array_equal(npf(s)[valid], x_s.numpy()[src[valid] // top_k])
    assert (u8(a)[~valid] == 0).all()
    # scales given MN-major at the source as the moe workload stores them ([H/128, T])
    a2, s2 = ops.permute(x_q.cuda().view(torch.float8_e4m3fn), x_s.t().contiguous().cuda().t(), plan["src_pair"], top_k)
    assert torch.equal(s2, s) and torch.equal(a2.view(torch.uint8), a.view(torch.uint8))
    y = torch.randn((plan["cap_rows"], H), generator=gen).bfloat16()
    w = torch.rand((T, top_k), generator=gen)
    out = ops.combine(y.cuda(), plan["pos"], w.cuda())
    ref = orc.combine(bf16_bits(y), plan["pos"].cpu().numpy(), w.numpy())
    assert ops.status() == 0
    np.testing.assert_array_equal(bf16_bits(out), ref)


def _make_layer(T, H, I, E, top_k, seed, device="cuda"):
    from tirx_harness_b200.workloads import make_operand_b
    gen = torch.Generator().manual_seed(seed)
    hs = torch.randn((T, H), generator=gen).bfloat16()
    xq, xs = orc.quant_1x128(hs.float().numpy())
    w13, s13 = make_operand_b(E, 2 * I, H, gen, law="uniform_exp")
    w2, s2 = make_operand_b(E, H, I, gen, law="uniform_exp")
    s13, s2 = s13 * 0.05, s2 * 0.05
    logits = torch.randn((T, E), generator=gen)
    data = dict(hidden_states=torch.from_numpy(xq).view(torch.float8_e4m3fn), hidden_states_scale=torch.from_numpy(xs),
                routing_logits=logits, gemm1_weights=w13, gemm1_weights_scale=s13, gemm2_weights=w2,
                gemm2_weights_scale=s2, output=torch.zeros((T, H), dtype=torch.bfloat16))
    return {k: v.to(device) for k, v in data.items()}, data


def test_layer_stagewise_parity(ops):
    from tirx_harness_b200 import moe_layer
    T, H, I, E, top_k = 300, 512, 256, 8, 2
    dev, host = _make_layer(T, H, I, E, top_k, seed=21)
    layer = moe_layer.setup(dev, T, top_k=top_k, gate_first=False, fuse_act=False)
    dev["output"].fill_(float("nan"))
    layer()
    assert ops.status() == 0
    v = layer.view()
    # routing + plan: bit exact
    rid, rw = orc.route_softmax_topk(host["routing_logits"].numpy(), top_k)
    np.testing.assert_array_equal(v["ids"].cpu().numpy(), rid)
    np.testing.assert_allclose(npf(v["weights"]), rw, rtol=2e-6)
    plan = orc.permute_plan(rid, 0, E, 128, cap_rows=v["cap_rows"])
    for k in ("counts", "offsets", "pos", "src_pair", "grouped_layout"):
        np.testing.assert_array_equal(v[k].cpu().numpy(), plan[k], err_msg=k)
    gl, src = plan["grouped_layout"], plan["src_pair"]
    valid = gl >= 0
    xq, xs = u8(host["hidden_states"]), host["hidden_states_scale"].numpy()
    np.testing.assert_array_equal(u8(v["a1"])[valid], xq[src[valid] // top_k])
    np.testing.assert_array_equal(npf(v["s1"])[valid], xs[src[valid] // top_k])
    # each later stage against the oracle applied to the GPU's own previous stage
    a1 = np.where(valid[:, None], u8(v["a1"]), 0).astype(np.uint8)
    s1 = np.where(valid[:, None], npf(v["s1"]), 0).astype(np.float32)
    g1_ref = orc.gg_contiguous(a1, u8(host["gemm1_weights"]), s1, host["gemm1_weights_scale"].numpy(), gl)
    g1 = bf16_bits(v["g1"])
    assert_bf16_close(g1[valid], g1_ref[valid])
    rq, rs = orc.silu_mul_requant(g1, gate_first=False, row_valid=valid.astype(np.uint8))
    np.testing.assert_allclose(npf(v["s2"])[valid], rs[valid], rtol=1e-6)
    _codes_close(u8(v["a2"])[valid], rq[valid])
    a2 = np.where(valid[:, None], u8(v["a2"]), 0).astype(np.uint8)
    s2 = np.where(valid[:, None], npf(v["s2"]), 0).astype(np.float32)
    y_ref = orc.gg_contiguous(a2, u8(host["gemm2_weights"]), s2, host["gemm2_weights_scale"].numpy(), gl)
    y = bf16_bits(v["y"])
    assert_bf16_close(y[valid], y_ref[valid])
    out_ref = orc.combine(np.where(valid[:, None], y, 0).astype(np.uint16), plan["pos"], npf(v["weights"]))
    np.testing.assert_array_equal(bf16_bits(dev["output"]), out_ref)
    # end to end against the oracle's own pipeline: global normalised RMS error
    full = orc.moe_layer(xq, xs, host["routing_logits"].numpy(), u8(host["gemm1_weights"]),
                         host["gemm1_weights_scale"].numpy(), u8(host["gemm2_weights"]),
                         host["gemm2_weights_scale"].numpy(), top_k=top_k, gate_first=False)
    got, ref = dev["output"].float().cpu().numpy(), orc.bf16_to_f32(full["out"])
    assert np.sqrt(((got - ref) ** 2).mean()) <= 5e-3 * np.sqrt((ref**2).mean()) + 1e-30


def test_layer_with_given_routes_and_mn_major_input_scales(ops):
    from tirx_harness_b200 import moe_layer
    T, H, I, E, top_k = 130, 256, 128, 4, 2
    dev, host = _make_layer(T, H, I, E, top_k, seed=5)
    first = moe_layer.setup(dev, T, top_k=top_k)
    first()
    v = first.view()
    rid, _ = orc.route_softmax_topk(host["routing_logits"].numpy(), top_k)
    np.testing.assert_array_equal(v["ids"].cpu().numpy(), rid)
    dev2 = dict(dev)
    del dev2["routing_logits"]
    dev2["topk_ids"] = v["ids"].clone()                 # the routes the first run chose, passed explicitly
    dev2["topk_weights"] = v["weights"].clone()
    dev2["hidden_states_scale"] = dev["hidden_states_scale"].t().contiguous()      # [H/128, T]
    dev2["output"] = torch.zeros_like(dev["output"])
    moe_layer.setup(dev2, T, top_k=top_k)()
    assert ops.status() == 0
    assert torch.equal(dev["output"], dev2["output"])
    assert torch.isfinite(dev["output"]).all() and dev["output"].abs().max() > 0


@pytest.mark.parametrize("gate_first", [False, True])
def test_gate_up_gemm_with_fused_silu_requant(ops, gate_first):
    """The gate_up GEMM whose epilogue does SiLU*mul + requant, against the oracle that keeps gate_up in fp32."""
    from tirx_harness_b200 import grouped_gemm as gg
    from tirx_harness_b200.workloads import make_contiguous_case
    inter = 384
    data = make_contiguous_case(3, [200, 128, 77], 2 * inter, 512, seed=41, law="uniform_exp", mn_major_sfa=True)
    data["SFB"].mul_(0.05)
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in data.items()}
    dev["SFA"] = data["SFA"].t().contiguous().cuda().t()
    M = data["M"]
    act_q = torch.zeros((M, inter), dtype=torch.float8_e4m3fn, device="cuda")
    act_s = torch.zeros((inter // 128, M), dtype=torch.float32, device="cuda").t()
    gg.bind_gate_up_act(dev["A"], dev["SFA"], dev["B"], dev["SFB"], act_q, act_s, dev["grouped_layout"], gate_first)()
    assert ops.status() == 0
    gl = data["grouped_layout"].numpy()
    valid = gl >= 0
    g32 = orc.gg_contiguous(u8(data["A"]), u8(data["B"]), npf(data["SFA"]), npf(data["SFB"]), gl,
                            model=orc.BLOCK_PROMOTE, out_f32=True)
    rq, rs = orc.silu_mul_requant(g32, gate_first=gate_first, row_valid=valid.astype(np.uint8))
    np.testing.assert_allclose(npf(act_s)[valid], rs[valid], rtol=2e-5)
    _codes_close(u8(act_q)[valid], rq[valid], max_mismatch=5e-3)
    assert (u8(act_q)[~valid] == 0).all()                     # padding rows untouched


def test_layer_fused_activation_matches_oracle(ops):
    from tirx_harness_b200 import moe_layer
    T, H, I, E, top_k = 300, 512, 256, 8, 2
    dev, host = _make_layer(T, H, I, E, top_k, seed=22)
    layer = moe_layer.setup(dev, T, top_k=top_k, gate_first=False, fuse_act=True)
    dev["output"].fill_(float("nan"))
    layer()
    assert ops.status() == 0
    xq, xs = u8(host["hidden_states"]), host["hidden_states_scale"].numpy()
    full = orc.moe_layer(xq, xs, host["routing_logits"].numpy(), u8(host["gemm1_weights"]),
                         host["gemm1_weights_scale"].numpy(), u8(host["gemm2_weights"]),
                         host["gemm2_weights_scale"].numpy(), top_k=top_k, gate_first=False, fused_act=True)
    v = layer.view()
    n = full["a2"].shape[0]
    valid = full["plan"]["grouped_layout"][:n] >= 0
    np.testing.assert_allclose(npf(v["s2"])[:n][valid], full["s2"][valid], rtol=2e-5)
    _codes_close(u8(v["a2"])[:n][valid], full["a2"][valid], max_mismatch=5e-3)
    got, ref = dev["output"].float().cpu().numpy(), orc.bf16_to_f32(full["out"])
    assert np.isfinite(got).all()
    assert np.sqrt(((got - ref) ** 2).mean()) <= 5e-3 * np.sqrt((ref**2).mean()) + 1e-30


def test_deepseek_routing_ids_exact(ops, golden_dir):
    g = np.load(os.path.join(golden_dir, "moe_routing.npz"))
    logits = torch.from_numpy(g["logits"]).cuda()
    bias = torch.from_numpy(g["bias"]).bfloat16().cuda()
    ids, w = ops.route_deepseek(logits, bias, routed_scaling_factor=float(g["rsf"]))
    assert ops.status() == 0
    rid, rw = orc.route_deepseek(g["logits"], g["bias"], routed_scaling_factor=float(g["rsf"]))
    np.testing.assert_array_equal(ids.cpu().numpy(), rid)
    np.testing.assert_allclose(npf(w), rw, rtol=2e-6)
    np.testing.assert_array_equal(np.sort(ids.cpu().numpy(), 1), g["topk_idx_sorted"])      # the reference's own picks
    # ties everywhere: lowest groups, then lowest experts
    z = torch.zeros((3, 256), device="cuda")
    ids0, w0 = ops.route_deepseek(z, torch.zeros(256, dtype=torch.bfloat16, device="cuda"))
    np.testing.assert_array_equal(ids0.cpu().numpy()[0], [0, 1, 2, 3, 4, 5, 6, 7])
    np.testing.assert_allclose(npf(w0), 0.125, rtol=1e-6)


@pytest.mark.parametrize("T", [1, 7, 59, 200])          # the task's trace rows start at T = 1, 7, 14, 15, ...
def test_layer_with_registered_moe_task_keys(ops, T):
    """The `moe` task's data dict (DeepSeek routing, MN-major input scales, local_expert_offset): only the local
    experts' contributions are summed, as in tasks/moe/definition.json."""
    from tirx_harness_b200 import moe_layer
    H, I, E_loc, E_glob, top_k = 256, 128, 32, 256, 8
    dev, host = _make_layer(T, H, I, E_loc, top_k, seed=33)
    gen = torch.Generator().manual_seed(7)
    logits = torch.randn((T, E_glob), generator=gen) * 2
    bias = (torch.randn(E_glob, generator=gen) * 0.1).bfloat16()
    off, rsf = 64, 2.5
    data = dict(dev, routing_logits=logits.cuda(), routing_bias=bias.cuda(), local_expert_offset=off,
                routed_scaling_factor=rsf, hidden_states_scale=dev["hidden_states_scale"].t().contiguous())
    data["output"].fill_(float("nan"))
    layer = moe_layer.setup(data, T)
    layer()
    assert ops.status() == 0
    rid, rw = orc.route_deepseek(logits.numpy(), bias.float().numpy(), routed_scaling_factor=rsf)
    v = layer.view()
    np.testing.assert_array_equal(v["ids"].cpu().numpy(), rid)
    full = orc.moe_layer(u8(host["hidden_states"]), host["hidden_states_scale"].numpy(), None, u8(host["gemm1_weights"]),
                         host["gemm1_weights_scale"].numpy(), u8(host["gemm2_weights"]),
                         host["gemm2_weights_scale"].numpy(), top_k=top_k, e_lo=off, routes=(rid, rw))
    np.testing.assert_array_equal(v["counts"].cpu().numpy(), full["plan"]["counts"])
    got, ref = data["output"].float().cpu().numpy(), orc.bf16_to_f32(full["out"])
    assert np.isfinite(got).all()
    assert np.sqrt(((got - ref) ** 2).mean()) <= 5e-3 * np.sqrt((ref**2).mean()) + 1e-30
