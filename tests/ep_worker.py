"""Worker for the multi-GPU expert-parallel tests and for the world-size-1 in-process check.

Run under torchrun (one rank per GPU):  python -m torch.distributed.run --nproc-per-node N tests/ep_worker.py
Every rank builds the same global problem from a seed, keeps its token slice and its experts, runs the
EP layer and compares its output slice (a) with the CPU oracle's single-rank pipeline fed with the GPU's
own routing and (b) bit for bit with the single-GPU MoeLayer over all tokens and all experts.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def build_global(T, H, I, E, seed):
    from oracle import oracle as orc
    from tirx_harness_b200.workloads import make_operand_b
    gen = torch.Generator().manual_seed(seed)
    hs = torch.randn((T, H), generator=gen).bfloat16()
    xq, xs = orc.quant_1x128(hs.float().numpy())
    w13, s13 = make_operand_b(E, 2 * I, H, gen, law="uniform_exp")
    w2, s2 = make_operand_b(E, H, I, gen, law="uniform_exp")
    logits = torch.randn((T, E), generator=gen)
    return dict(hidden_states=torch.from_numpy(xq).view(torch.float8_e4m3fn), hidden_states_scale=torch.from_numpy(xs),
                routing_logits=logits, gemm1_weights=w13, gemm1_weights_scale=s13 * 0.05, gemm2_weights=w2,
                gemm2_weights_scale=s2 * 0.05)


def run(T=512, H=512, I=256, E=16, top_k=4, seed=3, steps=3, combine="push", dispatch="fused"):
    import torch.distributed as dist
    from tirx_harness_b200 import ep_layer, grouped_gemm, moe_layer
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    g = build_global(T, H, I, E, seed)
    Tl, El = T // world, E // world
    tsl, esl = slice(rank * Tl, (rank + 1) * Tl), slice(rank * El, (rank + 1) * El)
    loc = dict(hidden_states=g["hidden_states"][tsl].cuda(), hidden_states_scale=g["hidden_states_scale"][tsl].cuda(),
               routing_logits=g["routing_logits"][tsl].contiguous().cuda(),
               gemm1_weights=g["gemm1_weights"][esl].cuda(), gemm1_weights_scale=g["gemm1_weights_scale"][esl].cuda(),
               gemm2_weights=g["gemm2_weights"][esl].cuda(), gemm2_weights_scale=g["gemm2_weights_scale"][esl].cuda(),
               output=torch.full((Tl, H), float("nan"), dtype=torch.bfloat16, device="cuda"))
    layer = ep_layer.setup(loc, Tl, top_k=top_k, combine=combine, dispatch=dispatch)
    for _ in range(steps):                      # repeated steps exercise the epoch logic and buffer reuse
        loc["output"].fill_(float("nan"))
        layer()
    assert grouped_gemm.device_status() == 0
    got = loc["output"].clone()
    # (b) single-GPU layer over everything, same kernels: must agree bit for bit
    full = {k: v.cuda() for k, v in g.items()}
    full["output"] = torch.zeros((T, H), dtype=torch.bfloat16, device="cuda")
    moe_layer.setup(full, T, top_k=top_k)()
    assert grouped_gemm.device_status() == 0
    assert torch.isfinite(got).all()
    assert torch.equal(got, full["output"][tsl]), f"rank {rank}: EP output differs from the single-GPU layer"
    # integer artefacts of the receive side: per-expert counts == bincount of the global routes
    from oracle import oracle as orc
    rid, rw = orc.route_softmax_topk(g["routing_logits"].numpy(), top_k)
    np.testing.assert_array_equal(layer.ids.cpu().numpy(), rid[tsl])
    cnt = np.bincount(rid.reshape(-1), minlength=E)
    np.testing.assert_array_equal(layer.counts_local.cpu().numpy(), cnt[esl])
    offs = np.concatenate([[0], np.cumsum((cnt[esl] + 127) // 128 * 128)])
    np.testing.assert_array_equal(layer.offsets.cpu().numpy(), offs)
    # (a) CPU oracle end to end (normalised RMS, the layer-level bound used for the single-GPU test)
    u8 = lambda t: t.contiguous().view(torch.uint8).numpy()
    ref = orc.moe_layer(u8(g["hidden_states"]), g["hidden_states_scale"].numpy(), g["routing_logits"].numpy(),
                        u8(g["gemm1_weights"]), g["gemm1_weights_scale"].numpy(), u8(g["gemm2_weights"]),
                        g["gemm2_weights_scale"].numpy(), top_k=top_k)
    r = orc.bf16_to_f32(ref["out"])[tsl]
    gf = got.float().cpu().numpy()
    rms = np.sqrt(((gf - r) ** 2).mean()) / np.sqrt((r**2).mean())
    assert rms <= 5e-3, rms
    # (c) the stage-by-stage check the benchmark runs after its timed region (collective over the ranks)
    from oracle import checks
    chk = checks.ep_layer_check(layer, loc, world, rank, tokens=32, rows=32, experts=2)
    assert chk["ok"] and chk["ok_this_rank"], chk
    layer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    print(f"rank {rank}/{world}: EP layer ok (rms {rms:.2e})", flush=True)


if __name__ == "__main__":
    run(combine=os.environ.get("EP_COMBINE", "push"), dispatch=os.environ.get("EP_DISPATCH", "fused"))
