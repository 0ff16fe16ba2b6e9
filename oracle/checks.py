"""Sampled parity checks of device results against the CPU oracle.

TEST INFRASTRUCTURE ONLY, like the rest of this folder: used by ``tests/`` and by ``bench.py`` AFTER a timed
region, outside it, to show that the outputs the timed calls left behind are the right ones.  Nothing here
is on a product path; the checks read device tensors, copy a bounded sample to the host and compare it with
``oracle.py``.  Every function returns a plain dict that ends up in the benchmark's JSON line:
``{"ok": bool, "rows": n, "max_rel_err": x, ...}``.
"""
from __future__ import annotations

import numpy as np
import torch

from . import oracle as orc


def _u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.uint8).cpu().numpy()


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _bf16_ulp(ref: np.ndarray) -> np.ndarray:
    a = np.abs(ref.astype(np.float64))
    return np.exp2(np.floor(np.log2(np.maximum(a, 2.0 ** -126))) - 7)


def compare_bf16(got_bits: np.ndarray, ref_bits: np.ndarray) -> dict:
    """bf16 results of two fp32-accurate computations: identical except where the fp32 values straddle a rounding
    boundary.  ok = every element within one bf16 step (taken at max(|ref|, 2^-7 rms(ref))), at least 97 % identical,
    and the grouped-GEMM task's own measure 1 - 2<x,y>/(<x,x>+<y,y>) below its 1e-6 threshold."""
    got = orc.bf16_to_f32(got_bits).astype(np.float64)
    ref = orc.bf16_to_f32(ref_bits).astype(np.float64)
    if got.size == 0:
        return dict(ok=True, elements=0, max_rel_err=0.0, identical=1.0, calc_diff=0.0)
    finite = bool(np.isfinite(got).all())
    floor = 2.0 ** -7 * np.sqrt((ref ** 2).mean())
    denom = np.maximum(np.abs(ref), max(floor, 1e-30))
    err = np.abs(np.nan_to_num(got, nan=np.inf) - ref)
    step_ok = bool((err <= _bf16_ulp(np.maximum(np.abs(ref), floor))).all())
    identical = float((got_bits == ref_bits).mean())
    den = (got * got + ref * ref).sum()
    diff = float(1.0 - 2.0 * (got * ref).sum() / den) if den > 0 and finite else (0.0 if finite else float("inf"))
    return dict(ok=finite and step_ok and identical >= 0.97 and diff < 1e-6, elements=int(got.size),
                max_rel_err=float((err / denom).max()), identical=round(identical, 5), calc_diff=diff)


def sample_rows(valid_rows: torch.Tensor, target: int) -> torch.Tensor:
    """About `target` of the valid row indices, evenly spaced, always including the first and the last."""
    n = int(valid_rows.numel())
    if n <= target:
        return valid_rows
    pick = torch.linspace(0, n - 1, target, device=valid_rows.device).round().long().unique()
    return valid_rows[pick]


def grouped_gemm_rows(a, sfa, b, sfb, row_group, d, target_rows=64, model=None, groups=None) -> dict:
    """Row sample of an m-grouped FP8 GEMM result against the oracle.
    a e4m3 [R, K] (any row pitch), sfa f32 [R, K/128] (any strides), b e4m3 [G, N, K], sfb f32 [G, N/128, K/128],
    row_group int [R] (group of each row, negative = not computed), d bf16 [R, N] as the kernel left it.
    `groups`: restrict the sample to these groups (bounds the cost of decoding B)."""
    model = orc.SIM_CHAIN if model is None else model
    rg = row_group.to(torch.int64)
    present = torch.unique(rg[rg >= 0]).tolist()
    glist = [int(g) for g in (groups if groups is not None else present) if int(g) in set(present)]
    if not glist:
        return dict(ok=True, rows=0, groups=0, elements=0, max_rel_err=0.0, identical=1.0, calc_diff=0.0)
    per_group = max(1, -(-target_rows // len(glist)))
    idx = torch.cat([sample_rows(torch.nonzero(rg == g).flatten(), per_group) for g in glist])
    remap = {g: i for i, g in enumerate(glist)}
    gl = np.array([remap[int(g)] for g in rg[idx].tolist()], np.int32)
    gsel = torch.tensor(glist, device=b.device, dtype=torch.long)
    A = a.view(torch.uint8)[idx].cpu().numpy()
    SA = sfa[idx].float().cpu().numpy()
    B = b.view(torch.uint8).index_select(0, gsel).cpu().numpy()
    SB = sfb.index_select(0, gsel).float().cpu().numpy()
    ref = orc.gg_contiguous(A, B, SA, SB, gl, model=model)
    res = compare_bf16(_bits(d[idx]), ref)
    res["rows"] = int(idx.numel())
    res["groups"] = len(glist)
    return res


def masked_row_groups(masked_m: torch.Tensor, max_m: int) -> torch.Tensor:
    """Masked layout [G, max_m] flattened: group id for rows below masked_m[g], -1 for the rest."""
    G = masked_m.numel()
    r = torch.arange(max_m, device=masked_m.device).unsqueeze(0).expand(G, max_m)
    g = torch.arange(G, device=masked_m.device).unsqueeze(1).expand(G, max_m)
    return torch.where(r < masked_m.unsqueeze(1), g, torch.full_like(g, -1)).reshape(-1)


def silu_requant_rows(g1_bits_rows: np.ndarray, a2_rows: np.ndarray, s2_rows: np.ndarray, gate_first: bool) -> dict:
    """SiLU(gate)*up + 1x128 requantisation of sampled rows: the device's codes and scales against the oracle applied
    to the device's own bf16 gate_up rows.  Scales to 2e-5 relative; codes identical except where exp2 differs in
    the last place between libm and the GPU (at most one code step on at most 0.5 % of the elements)."""
    rq, rs = orc.silu_mul_requant(g1_bits_rows, gate_first=gate_first)
    scale_err = float(np.max(np.abs(s2_rows - rs) / np.maximum(np.abs(rs), 1e-30))) if rs.size else 0.0
    same = a2_rows == rq
    dec_g, dec_r = orc.e4m3_decode(a2_rows).astype(np.float64), orc.e4m3_decode(rq).astype(np.float64)
    # neighbouring e4m3 values differ by at most 1/8 of the larger one (2^-9 among the subnormals)
    within_one = bool((np.abs(dec_g - dec_r) <= 0.126 * np.abs(dec_r) + 2.0 ** -9).all())
    mismatch = float(1.0 - same.mean()) if same.size else 0.0
    return dict(ok=scale_err <= 2e-5 and within_one and mismatch <= 5e-3, rows=int(a2_rows.shape[0]),
                scale_rel_err=scale_err, code_mismatch=mismatch)


def _all_gather(t: torch.Tensor, world: int):
    if world == 1:
        return t.unsqueeze(0)
    import torch.distributed as dist
    # bytes on the wire: NCCL has no 16-bit integer type
    src = t.contiguous()
    out = torch.empty((world,) + tuple(src.shape), dtype=src.dtype, device=src.device)
    dist.all_gather_into_tensor(out.view(torch.uint8).reshape(world, -1), src.view(torch.uint8).reshape(-1))
    return out


def ep_layer_check(layer, data: dict, world: int, rank: int, tokens: int = 64, rows: int = 64, experts: int = 4) -> dict:
    """Stage-by-stage check of ONE forward of an expert-parallel layer (tirx_harness_b200.ep_layer.EpMoeLayer,
    combine="push") from the buffers that forward left behind; collective: every rank calls it.
      routing   sampled tokens: ids exact, weights to 2e-6, against the oracle's softmax top-k
      counts    per-expert receive counts = bincount of ALL ranks' routes, offsets = their aligned prefix (exact)
      dispatch  EVERY received row equals its source token's bytes and scales, and sits in the right expert (exact)
      gate_up   sampled rows of a few local experts against the oracle GEMM (bf16, one step)
      act       the same rows: SiLU*mul requant codes and scales against the oracle on the device's gate_up rows
      down      the same rows: oracle GEMM result against the slot of the token's home rank (exchanged over NCCL)
      combine   sampled tokens: output bits = fp32 weighted sum of the token's return slots in slot order (exact)
    Returns {"ok", stage results...}; "ok" is the AND over all ranks."""
    dev = layer.device
    T, H, I, k, El, Et = layer.T, layer.H, layer.I, layer.top_k, layer.E_local, layer.E_total
    w13, s13 = data["gemm1_weights"], data["gemm1_weights_scale"]
    w2, s2w = data["gemm2_weights"], data["gemm2_weights_scale"]
    torch.cuda.synchronize(dev)
    res: dict = {}
    # ---- routing
    tsel = sample_rows(torch.arange(T, device=dev), tokens)
    rid, rw = orc.route_softmax_topk(data["routing_logits"][tsel].float().cpu().numpy(), k)
    ids_s = layer.ids[tsel].cpu().numpy()
    w_s = layer.weights[tsel].cpu().numpy()
    res["routing"] = dict(ok=bool((ids_s == rid).all() and np.allclose(w_s, rw, rtol=2e-6, atol=0)), tokens=int(tsel.numel()))
    # ---- counts / offsets
    ids_all = _all_gather(layer.ids, world)                                   # [world, T, k]
    want = torch.bincount(ids_all.reshape(-1).long(), minlength=Et)[rank * El:(rank + 1) * El].to(torch.int32)
    aligned = (want + layer.align - 1) // layer.align * layer.align
    off = torch.zeros(El + 1, dtype=torch.int32, device=dev)
    off[1:] = torch.cumsum(aligned, 0)
    res["counts"] = dict(ok=bool(torch.equal(layer.counts_local, want) and torch.equal(layer.offsets, off)),
                         rows_received=int(want.sum().item()))
    # ---- dispatch: every received row
    used = int(off[El].item())
    lay = layer.layout[:used]
    vrows = torch.nonzero(lay >= 0).flatten()
    meta = layer.meta_t[:used][vrows].long()
    src, pair = meta >> 24, meta & 0xFFFFFF
    xq_all = _all_gather(layer.x_q.view(torch.uint8), world)                 # [world, T, H]
    xs_all = _all_gather(layer.xs.contiguous(), world)                       # [world, T, H/128]
    tok = pair // k
    same_bytes = True
    for c0 in range(0, int(vrows.numel()), 16384):                            # chunks bound the temporary to 117 MB
        sl = slice(c0, c0 + 16384)
        got = layer.a1_t.view(torch.uint8)[vrows[sl]]
        same_bytes &= bool(torch.equal(got, xq_all[src[sl], tok[sl]]))
        same_bytes &= bool(torch.equal(layer.s1_t[vrows[sl]], xs_all[src[sl], tok[sl]]))
    right_expert = bool(torch.equal(ids_all.reshape(world, -1)[src, pair] - rank * El, lay[vrows].to(ids_all.dtype)))
    res["dispatch"] = dict(ok=same_bytes and right_expert and int(vrows.numel()) == int(want.sum().item()),
                           rows=int(vrows.numel()))
    del xq_all, xs_all
    # ---- the two GEMMs and the activation on sampled rows of a few experts
    have = torch.nonzero(want > 0).flatten()
    pick = sample_rows(have, experts).tolist() if have.numel() else []
    lay_full = torch.full((layer.cap,), -1, dtype=torch.int32, device=dev)
    lay_full[:used] = lay
    fused = bool(layer.fuse_act)            # SiLU*mul requant inside the gate_up GEMM: no gate_up matrix in memory
    if not fused:
        res["gate_up"] = grouped_gemm_rows(layer.a1_t, layer.s1_t, w13, s13, lay_full, layer.g1, rows, groups=pick)
    keep = torch.zeros(layer.cap, dtype=torch.bool, device=dev)
    for g in pick:
        keep |= lay_full == int(g)
    R = sample_rows(torch.nonzero(keep).flatten(), rows)
    n = int(R.numel())
    if n:
        s2_rows = layer.s2.t()[R].float().cpu().numpy()
        a2_rows = layer.a2.view(torch.uint8)[R].cpu().numpy()
        used_g = torch.unique(lay_full[R]).tolist()
        remap = {int(g): i for i, g in enumerate(used_g)}
        gl = np.array([remap[int(g)] for g in lay_full[R].tolist()], np.int32)
        gsel = torch.tensor(used_g, device=dev, dtype=torch.long)
        if fused:
            # the epilogue requantises the fp32 accumulator: oracle gate_up kept in fp32 (per-K-block promotion model)
            g32 = orc.gg_contiguous(layer.a1_t.view(torch.uint8)[R].cpu().numpy(),
                                    w13.view(torch.uint8).index_select(0, gsel).cpu().numpy(),
                                    layer.s1_t[R].float().cpu().numpy(), s13.index_select(0, gsel).float().cpu().numpy(), gl,
                                    model=orc.BLOCK_PROMOTE, out_f32=True)
            res["gate_up+act"] = silu_requant_rows(g32, a2_rows, s2_rows, layer.gate_first)
        else:
            res["act"] = silu_requant_rows(_bits(layer.g1[R]), a2_rows, s2_rows, layer.gate_first)
        yref = orc.gg_contiguous(a2_rows, w2.view(torch.uint8).index_select(0, gsel).cpu().numpy(), s2_rows,
                                 s2w.index_select(0, gsel).float().cpu().numpy(), gl)          # bf16 bits [n, H]
    else:
        res["act"] = dict(ok=True, rows=0)
        yref = np.zeros((0, H), np.uint16)
    # exchange: (home rank, pair, reference row) of every sampled row, padded to `rows`
    send_meta = torch.full((rows, 2), -1, dtype=torch.int64, device=dev)
    send_y = torch.zeros((rows, H), dtype=torch.int16, device=dev)
    if n:
        m = layer.meta_t[R].long()
        send_meta[:n, 0], send_meta[:n, 1] = m >> 24, m & 0xFFFFFF
        send_y[:n] = torch.from_numpy(yref.view(np.int16)).to(dev)
    all_meta = _all_gather(send_meta, world).reshape(-1, 2)
    all_y = _all_gather(send_y, world).reshape(-1, H)
    mine = torch.nonzero(all_meta[:, 0] == rank).flatten()
    if layer.combine == "push" and mine.numel():
        got_bits = layer.y_t[all_meta[mine, 1]].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        res["down"] = compare_bf16(got_bits, all_y[mine].cpu().numpy().view(np.uint16))
        res["down"]["rows"] = int(mine.numel())
    elif layer.combine == "pull" and n:
        res["down"] = compare_bf16(_bits(layer.y_t[R]), yref)
        res["down"]["rows"] = n
    else:
        res["down"] = dict(ok=True, rows=0)
    # ---- combine on sampled tokens (push: the return slots of a token are local)
    if layer.combine == "push":
        slots = (tsel.unsqueeze(1) * k + torch.arange(k, device=dev).unsqueeze(0)).reshape(-1)
        y_rows = _bits(layer.y_t[slots])
        pos = np.arange(slots.numel(), dtype=np.int32).reshape(-1, k)
        want_out = orc.combine(y_rows, pos, w_s)
        res["combine"] = dict(ok=bool((want_out == _bits(layer.out[tsel])).all()), tokens=int(tsel.numel()))
    else:
        res["combine"] = dict(ok=True, tokens=0, note="not checked with combine=pull")
    ok = all(v["ok"] for v in res.values())
    flag = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    res["ok_this_rank"] = ok
    res["ok"] = bool(flag.item())
    return res


def alpha_layer_check(data: dict) -> dict:
    """All rows of one decode-regime layer call (the alphamoe contract) against the oracle restatement of the task's
    operator: every output element inside the task's bound max(0.02 + 0.02 |ref|, 2 * abs_sum * 2^-7)
    (evolution/tasks/alphamoe.yaml:48-57), and the share of bit-identical bf16 outputs."""
    hs, out = data["hidden_states"], data["output"]
    res = orc.alpha_moe_layer(_bits(hs), data["topk_ids"].cpu().numpy(), data["topk_weights"].float().cpu().numpy(),
                              _u8(data["gemm1_weights"]), data["gemm1_weights_scale"].float().cpu().numpy(),
                              _u8(data["gemm2_weights"]), data["gemm2_weights_scale"].float().cpu().numpy(),
                              routed_scaling_factor=float(data.get("routed_scaling_factor", 1.0)))
    got_bits = _bits(out)
    got, want = orc.bf16_to_f32(got_bits), orc.bf16_to_f32(res["out"])
    finite = bool(np.isfinite(got).all())
    bound = np.maximum(0.02 + 0.02 * np.abs(want), 2.0 * res["abs_sum"] * 2.0 ** -7)
    err = np.abs(np.nan_to_num(got, nan=np.inf) - want)
    identical = float((got_bits == res["out"]).mean())
    return dict(ok=finite and bool((err <= bound).all()) and identical > 0.9, rows=int(hs.shape[0]),
                max_err_over_bound=float((err / bound).max()), identical=round(identical, 5))
