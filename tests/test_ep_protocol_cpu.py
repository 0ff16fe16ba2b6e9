"""World-size-2 gloo ranks on CPU: the expert-parallel exchange protocol reproduces the single-rank
oracle layer, and its failure modes surface as errors on the host (no GPU involved)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.conftest import ROOT


def _problem(seed=4, T=64, H=256, I=128, E=8):
    from oracle import oracle as orc
    rng = np.random.default_rng(seed)
    xq, xs = orc.quant_1x128(rng.standard_normal((T, H)).astype(np.float32))
    w13 = orc.e4m3_encode(rng.standard_normal((E, 2 * I, H)).astype(np.float32) * 8)
    w2 = orc.e4m3_encode(rng.standard_normal((E, H, I)).astype(np.float32) * 8)
    s13 = np.exp2(rng.integers(-8, -4, (E, 2 * I // 128, H // 128))).astype(np.float32)
    s2 = np.exp2(rng.integers(-8, -4, (E, H // 128, I // 128))).astype(np.float32)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    return xq, xs, logits, w13, s13, w2, s2


def _worker(rank, world, port, mode, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from datetime import timedelta
    try:
        if mode == "absent" and rank == 1:
            q.put((rank, "absent"))
            return                                   # this rank never joins
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=8))
        from oracle import ep_model, oracle as orc
        xq, xs, logits, w13, s13, w2, s2 = _problem()
        T, E = logits.shape
        Tl, El = T // world, E // world
        ts, es = slice(rank * Tl, (rank + 1) * Tl), slice(rank * El, (rank + 1) * El)
        out, ids, counts = ep_model.ep_layer_rank(dist, rank, world, xq[ts], xs[ts], logits[ts], w13[es], s13[es],
                                                  w2[es], s2[es], top_k=2,
                                                  corrupt_counts=(mode == "corrupt" and rank == 0))
        full = orc.moe_layer(xq, xs, logits, w13, s13, w2, s2, top_k=2)
        ok = np.array_equal(out, full["out"][ts]) and np.array_equal(ids, full["ids"][ts]) and \
            np.array_equal(counts, full["plan"]["counts"][es])
        q.put((rank, "ok" if ok else "mismatch"))
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001 - the test inspects the failure text
        q.put((rank, f"error: {type(exc).__name__}: {exc}"))


def _run(mode, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    return res


def test_two_rank_protocol_matches_single_rank_oracle():
    assert _run("normal", 29641) == {0: "ok", 1: "ok"}


def test_wrong_published_counts_are_detected():
    res = _run("corrupt", 29642)
    assert any("protocol violation" in v for v in res.values()), res


def test_rank_that_never_joins_times_out_on_the_host():
    res = _run("absent", 29643)
    assert res[1] == "absent" and res[0].startswith("error"), res


def test_plan_from_counts_layout_rules():
    from oracle import ep_model
    counts_all = np.array([[3, 0, 130, 1], [5, 0, 0, 127]], np.int32)      # 2 ranks, 4 experts, 2 local each
    c0, o0, b0 = ep_model.plan_from_counts(counts_all, 0, 2, 128)
    c1, o1, b1 = ep_model.plan_from_counts(counts_all, 1, 2, 128)
    np.testing.assert_array_equal(c0, [8, 0]); np.testing.assert_array_equal(o0, [0, 128, 128])
    np.testing.assert_array_equal(c1, [130, 128]); np.testing.assert_array_equal(o1, [0, 256, 384])
    np.testing.assert_array_equal(b0, [0, 128, 0, 256])            # rank 0 writes first inside every expert
    np.testing.assert_array_equal(b1, [3, 128, 130, 257])          # rank 1 follows rank 0's rows
