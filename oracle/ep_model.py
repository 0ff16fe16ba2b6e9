"""NumPy model of the expert-parallel exchange protocol (TEST INFRASTRUCTURE ONLY).

Restates, for CPU ranks talking over a ``torch.distributed`` gloo group, what the CUDA kernels do over
peer memory: publish per-expert pair counts, derive receive offsets and send bases from the gathered
table, place rows (ordered by source rank, then pair order), run the per-rank expert pipeline with the
CPU oracle and pull-combine.  Used to check that the protocol reproduces the single-rank oracle layer
and to exercise failure handling (wrong counts, a rank that never joins) without any GPU.
"""
from __future__ import annotations

import numpy as np

from . import oracle as orc


def plan_from_counts(counts_all: np.ndarray, rank: int, e_local: int, align: int):
    """counts_all int [world, E_total] -> (counts_local, offsets[E_local+1], dst_base[E_total]).
    Same arithmetic as the device kernel that runs after the first barrier."""
    world, e_total = counts_all.shape
    total = counts_all.sum(0)
    start = np.zeros(e_total, np.int64)
    used = np.zeros(world, np.int64)
    for d in range(world):
        run = 0
        for j in range(e_local):
            e = d * e_local + j
            start[e] = run
            run += (total[e] + align - 1) // align * align
        used[d] = run
    before = counts_all[:rank].sum(0)
    dst_base = start + before
    mine = slice(rank * e_local, (rank + 1) * e_local)
    offsets = np.concatenate([start[mine], [used[rank]]])
    return total[mine].astype(np.int32), offsets.astype(np.int32), dst_base.astype(np.int32)


def ep_layer_rank(dist, rank, world, x_q, x_scale, logits, w13, s13, w2, s2, top_k, align=128, gate_first=False,
                  corrupt_counts=False):
    """One rank of the protocol over a process group `dist` (gloo).  Inputs are this rank's token slice
    and experts.  Returns (out bf16 bits [T_local, H], ids, counts_local)."""
    import torch
    T, H = x_q.shape
    e_local = w13.shape[0]
    e_total = e_local * world
    ids, w = orc.route_softmax_topk(logits, top_k)
    my_counts = np.bincount(ids.reshape(-1), minlength=e_total).astype(np.int32)
    if corrupt_counts:
        my_counts[0] += 1
    gathered = [torch.zeros(e_total, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(my_counts))                     # "publish counts" + barrier
    counts_all = np.stack([g.numpy() for g in gathered])
    counts_local, offsets, dst_base = plan_from_counts(counts_all, rank, e_local, align)
    # stable rank of every pair inside (this rank, expert)
    flat = ids.reshape(-1)
    seen = np.zeros(e_total, np.int64)
    pos = np.empty(flat.size, np.int64)
    for p, e in enumerate(flat):
        pos[p] = dst_base[e] + seen[e]
        seen[e] += 1
    owner = flat // e_local
    # dispatch: rows + scales + destination row, one message per destination rank
    send = []
    for d in range(world):
        sel = np.nonzero(owner == d)[0]
        tok = sel // top_k
        send.append((pos[sel], x_q[tok], x_scale[tok]))
    recv = [None] * world
    dist.all_to_all_object(recv, send) if hasattr(dist, "all_to_all_object") else _a2a_objects(dist, recv, send, world)
    cap = int(offsets[-1])
    a = np.zeros((cap, H), np.uint8)
    sa = np.zeros((cap, H // 128), np.float32)
    filled = np.zeros(cap, bool)
    for rows, q, s in recv:
        if (rows >= cap).any() or filled[rows].any():
            raise RuntimeError("dispatch protocol violation: row outside the receive layout or written twice")
        a[rows], sa[rows] = q, s
        filled[rows] = True
    layout = np.full(cap, -1, np.int32)
    for e in range(e_local):
        layout[offsets[e]:offsets[e] + counts_local[e]] = e
    if not np.array_equal(filled, layout >= 0):
        raise RuntimeError("dispatch protocol violation: received rows do not match the published counts")
    g1 = orc.gg_contiguous(a, w13, sa, s13, layout)
    a2, s2a = orc.silu_mul_requant(g1, gate_first=gate_first, row_valid=(layout >= 0).astype(np.uint8))
    y = orc.gg_contiguous(a2, w2, s2a, s2, layout)
    # combine: pull rows from the owners
    want = [pos[owner == d] for d in range(world)]
    asked = [None] * world
    _a2a_objects(dist, asked, want, world)
    reply = [y[r] for r in asked]
    got = [None] * world
    _a2a_objects(dist, got, reply, world)
    rows = np.zeros((flat.size, H), np.uint16)
    for d in range(world):
        rows[owner == d] = got[d]
    out = np.zeros((T, H), np.uint16)
    for t in range(T):
        acc = np.zeros(H, np.float32)
        for j in range(top_k):
            acc = acc + np.float32(w[t, j]) * orc.bf16_to_f32(rows[t * top_k + j])
        out[t] = orc.bf16_rne(acc)
    return out, ids, counts_local


def _a2a_objects(dist, out_list, in_list, world):
    """all-to-all of Python objects built from all_gather_object (gloo has no object all-to-all)."""
    gathered = [None] * world
    dist.all_gather_object(gathered, in_list)
    rank = dist.get_rank()
    for s in range(world):
        out_list[s] = gathered[s][rank]
