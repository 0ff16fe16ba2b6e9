"""The committed candidates/<workload>/b200/solution.py files, loaded by path the way the reference's adapter loads a
candidate and driven through its protocol: poison the outputs, call, compare with the task's own gate, repeat and
require identical values, then change the inputs in place and require the next call to follow them."""
import os

import numpy as np
import pytest
import torch

from oracle import checks
from oracle import oracle as orc
from tests import harness_protocol as hp
from tests.util import grouped_gemm_gate, moe_output_gate, moe_task_inputs, npf, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _status():
    from tirx_harness_b200 import grouped_gemm
    return grouped_gemm.device_status()


def test_grouped_gemm_fp8_candidate_follows_the_protocol():
    from tirx_harness_b200.workloads import make_registered_case, output_views
    sol = hp.load_solution("grouped_gemm/fp8", "b200")
    assert sol.__name__ == "_tirx_grouped_gemm_fp8_b200.solution"
    host = make_registered_case(4, 300, 768, 1536, seed=9)                   # packed UE8M0, MN-major, alignment 224
    data = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in host.items()}
    inputs = {k: data[k] for k in ("A", "B", "SFA", "SFB", "D", "grouped_layout", "actual_ms", "aligned_ms", "alignment")}
    launch = sol.setup(inputs, host["G"], host["M"], host["N"], host["K"])
    views = output_views(data["D"], host["actual_ms"], host["aligned_ms"])
    gl = host["grouped_layout"].numpy()

    def reference():
        d = orc.gg_contiguous(u8(data["A"]), u8(data["B"]), npf(host["SFA_f32"]), npf(host["SFB_f32"]), gl)
        views, start = [], 0
        for actual, aligned in zip(host["actual_ms"], host["aligned_ms"]):
            views.append(orc.bf16_to_f32(d[start:start + actual]))
            start += aligned
        return views

    def compare(outs, ref=None):
        ok, worst = grouped_gemm_gate([v.float().cpu().numpy() for v in outs], ref or reference())
        assert ok, f"max group diff {worst:.3e}"
    data["D"].zero_()
    hp.checked_runs(launch, views, compare)
    assert _status() == 0
    assert not data["D"][torch.from_numpy(gl).cuda() < 0].any()              # padding rows are outside every view: untouched
    # inputs changed in place (the harness owns them): the same bound callable must follow
    a32 = data["A"].float()
    hp.perturb_inputs_([a32], seed=5)
    data["A"].copy_(a32.clamp_(-448, 448).to(torch.float8_e4m3fn))
    before = [v.clone() for v in views]
    hp.poison(views)
    launch()
    torch.cuda.synchronize()
    compare(views)
    assert any(not torch.equal(a, b) for a, b in zip(views, before))


def _small_moe_case(T, seed):
    """The `moe` task's keys at a reduced width (routing keeps the task's 256 experts in 8 groups)."""
    from tirx_harness_b200.workloads import make_operand_b
    H, I, E_loc, E_glob = 512, 256, 32, 256
    gen = torch.Generator().manual_seed(seed)
    hs = torch.randn((T, H), generator=gen).clamp_(-2, 2).to(torch.float8_e4m3fn)
    w13, s13 = make_operand_b(E_loc, 2 * I, H, gen, law="uniform_exp")
    w2, s2 = make_operand_b(E_loc, H, I, gen, law="uniform_exp")
    return dict(routing_logits=torch.randn((T, E_glob), generator=gen) * 2, routing_bias=(torch.randn(E_glob, generator=gen) * 0.1).bfloat16(),
                hidden_states=hs, hidden_states_scale=torch.empty((H // 128, T)).uniform_(0.01, 0.1, generator=gen),
                gemm1_weights=w13, gemm1_weights_scale=s13 * 0.05, gemm2_weights=w2, gemm2_weights_scale=s2 * 0.05,
                local_expert_offset=96, routed_scaling_factor=2.5)


def _moe_oracle(d):
    host = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in d.items()}
    rid, rw = orc.route_deepseek(host["routing_logits"].numpy(), host["routing_bias"].float().numpy(),
                                 routed_scaling_factor=host["routed_scaling_factor"])
    full = orc.moe_layer(u8(host["hidden_states"]), np.ascontiguousarray(host["hidden_states_scale"].numpy().T), None,
                         u8(host["gemm1_weights"]), host["gemm1_weights_scale"].numpy(), u8(host["gemm2_weights"]),
                         host["gemm2_weights_scale"].numpy(), top_k=8, e_lo=host["local_expert_offset"], routes=(rid, rw))
    return orc.bf16_to_f32(full["out"])


def test_moe_candidate_follows_the_protocol():
    sol = hp.load_solution("moe", "b200")
    T = 120
    data = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in _small_moe_case(T, seed=4).items()}
    data["output"] = torch.empty((T, 512), dtype=torch.bfloat16, device="cuda")
    run = sol.setup(data, T)

    def compare(out):
        ref = _moe_oracle(data)
        got = out.float().cpu().numpy()
        ok, note, stats = moe_output_gate(got, ref)                       # the task's gate ...
        assert ok, note
        assert stats["rms_ratio"] <= 5e-3, stats                          # ... and the layer's own, far tighter bound
    hp.checked_runs(run, data["output"], compare)
    assert _status() == 0
    before = data["output"].clone()
    floats = [data["routing_logits"], data["hidden_states_scale"], data["gemm1_weights_scale"], data["gemm2_weights_scale"]]
    hp.perturb_inputs_(floats, seed=11)
    for t in floats[1:]:
        t.abs_().clamp_min_(1e-3)                                       # scales stay positive
    hp.poison(data["output"])
    run()
    torch.cuda.synchronize()
    compare(data["output"])
    assert not torch.equal(before, data["output"])


def test_moe_candidate_matches_the_reference_run_fixture(golden_dir):
    """Full task geometry (7168 / 2048 / 32 of 256 experts), T=16: the candidate against what the reference's own
    `run` returned for the same seeded inputs (tests/golden/make_golden.py), under the task's gate; the e4m3
    requantisation of the intermediate is the only modelling difference (a few percent RMS)."""
    sol = hp.load_solution("moe", "b200")
    g = np.load(os.path.join(golden_dir, "moe_task_layer.npz"))
    T = int(g["T"])
    x = moe_task_inputs(T, int(g["seed"]))
    fp8 = lambda a: torch.from_numpy(a).cuda().view(torch.float8_e4m3fn)
    data = dict(routing_logits=torch.from_numpy(x["routing_logits"]).cuda(),
                routing_bias=torch.from_numpy(x["routing_bias"]).bfloat16().cuda(),
                hidden_states=fp8(x["hidden_states"]), hidden_states_scale=torch.from_numpy(x["hidden_states_scale"]).cuda(),
                gemm1_weights=fp8(x["gemm1_weights"]), gemm1_weights_scale=torch.from_numpy(x["gemm1_weights_scale"]).cuda(),
                gemm2_weights=fp8(x["gemm2_weights"]), gemm2_weights_scale=torch.from_numpy(x["gemm2_weights_scale"]).cuda(),
                local_expert_offset=x["local_expert_offset"], routed_scaling_factor=x["routed_scaling_factor"],
                output=torch.full((T, 7168), float("nan"), dtype=torch.bfloat16, device="cuda"))
    sol.setup(data, T)()
    assert _status() == 0
    ok, note, stats = moe_output_gate(data["output"].float().cpu().numpy(), orc.bf16_to_f32(g["out_bits"]))
    assert ok, note
    assert stats["rms_ratio"] < 0.05 and stats["token_matched"] == 1.0, stats


def test_alphamoe_candidate_follows_the_protocol():
    from tests.test_alpha_moe_gpu import _case
    sol = hp.load_solution("alphamoe", "b200")
    for M in (8, 48):
        c = _case(M, 512, 16, 4, seed=60 + M, rsf=2.5)
        dev = torch.device("cuda", 0)
        data = dict(hidden_states=c["hs"].to(dev), topk_ids=torch.from_numpy(c["ids"]).to(dev),
                    topk_weights=torch.from_numpy(c["w"]).to(dev),
                    gemm1_weights=torch.from_numpy(c["w13"]).to(dev).view(torch.float8_e4m3fn),
                    gemm1_weights_scale=torch.from_numpy(c["s13"]).to(dev),
                    gemm2_weights=torch.from_numpy(c["w2"]).to(dev).view(torch.float8_e4m3fn),
                    gemm2_weights_scale=torch.from_numpy(c["s2"]).to(dev), top_k=4, routed_scaling_factor=2.5,
                    output=torch.zeros((M, 512), dtype=torch.bfloat16, device=dev))
        run = sol.setup(data, M)

        def compare(out):
            res = checks.alpha_layer_check(data)
            assert res["ok"], res
        hp.checked_runs(run, data["output"], compare)
        assert _status() == 0
        before = data["output"].clone()
        hp.perturb_inputs_([data["hidden_states"], data["topk_weights"]], seed=3)
        hp.poison(data["output"])
        run()
        torch.cuda.synchronize()
        compare(data["output"])
        assert not torch.equal(before, data["output"])
