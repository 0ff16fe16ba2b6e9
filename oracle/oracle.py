"""ctypes/NumPy front end of the CPU oracle (``oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The shipped
package never imports it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

SIM_CHAIN = 0       # scale every element, one FMA chain over all K (the simulator's model)
BLOCK_PROMOTE = 1   # chain per 128-K block, then acc = fma(partial, sfa*sfb, acc)

_c = ctypes
_i64 = _c.c_int64
_vp = _c.c_void_p


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` into ``liboracle.so`` next to it (gcc, OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_gg_contiguous.restype = _c.c_int
        _lib.orc_gg_masked.restype = _c.c_int
        _lib.orc_fp8_blockwise_ue8m0.restype = _c.c_int
        _lib.orc_permute_plan.restype = _i64
        _lib.orc_num_threads.restype = _c.c_int
    return _lib


def _p(a: np.ndarray):
    return _vp(a.ctypes.data)


def _c_arr(a, dtype):
    return np.ascontiguousarray(np.asarray(a, dtype=dtype))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Number of OpenMP threads of the following oracle calls (launchers export OMP_NUM_THREADS=1 to their ranks)."""
    lib().orc_set_num_threads(_c.c_int(int(n)))


# ---------------------------------------------------------------- codecs
def e4m3_decode(bits) -> np.ndarray:
    b = _c_arr(bits, np.uint8)
    out = np.empty(b.shape, np.float32)
    lib().orc_e4m3_decode(_p(b), _p(out), _i64(b.size))
    return out


def e4m3_encode(values) -> np.ndarray:
    v = _c_arr(values, np.float32)
    out = np.empty(v.shape, np.uint8)
    lib().orc_e4m3_encode(_p(v), _p(out), _i64(v.size))
    return out


def ue8m0_decode(bits) -> np.ndarray:
    b = _c_arr(bits, np.uint8)
    out = np.empty(b.shape, np.float32)
    lib().orc_ue8m0_decode(_p(b), _p(out), _i64(b.size))
    return out


def ue8m0_pack(codes) -> np.ndarray:
    c = _c_arr(codes, np.uint8)
    rows, blocks = c.shape
    assert blocks % 4 == 0
    out = np.empty((blocks // 4, rows), np.uint32)
    lib().orc_ue8m0_pack(_p(c), _p(out), _i64(rows), _i64(blocks))
    return out


def ue8m0_unpack(packed, blocks: int) -> np.ndarray:
    w = _c_arr(packed, np.uint32)
    assert w.shape[0] == blocks // 4
    rows = w.shape[1]
    out = np.empty((rows, blocks), np.uint8)
    lib().orc_ue8m0_unpack(_p(w), _p(out), _i64(rows), _i64(blocks))
    return out


def bf16_rne(values) -> np.ndarray:
    v = _c_arr(values, np.float32)
    out = np.empty(v.shape, np.uint16)
    lib().orc_bf16_rne(_p(v), _p(out), _i64(v.size))
    return out


def bf16_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ---------------------------------------------------------------- GEMM
def fma_abt_increasing_k(a, b, d_init=None) -> np.ndarray:
    a = _c_arr(a, np.float32)
    b = _c_arr(b, np.float32)
    M, K = a.shape
    N = b.shape[0]
    out = np.empty((M, N), np.float32)
    d = None if d_init is None else _c_arr(d_init, np.float32)
    lib().orc_fma_abt_increasing_k(_p(a), _p(b), _p(d) if d is not None else None, _p(out),
                                   _i64(M), _i64(N), _i64(K))
    return out


def _strides_elems(a: np.ndarray):
    return [s // a.itemsize for s in a.strides]


def gg_contiguous(A, B, sfa, sfb, grouped_layout, model=SIM_CHAIN, out=None, row_step=1,
                  out_f32=False):
    """A u8[M,K], B u8[G,N,K], sfa f32[M,K/128] (any strides), sfb f32[G,ceil(N/128),K/128],
    grouped_layout i32[M] -> D bf16 bits [M,N] (rows with negative layout untouched)."""
    A = _c_arr(A, np.uint8)
    B = _c_arr(B, np.uint8)
    sfa = np.asarray(sfa, np.float32)
    sfb = _c_arr(sfb, np.float32)
    gl = _c_arr(grouped_layout, np.int32)
    M, K = A.shape
    G, N, _ = B.shape
    assert sfa.shape == (M, K // 128) and sfb.shape == (G, (N + 127) // 128, K // 128)
    D = np.zeros((M, N), np.float32 if out_f32 else np.uint16) if out is None else out
    assert D.dtype == (np.float32 if out_f32 else np.uint16) and D.flags.c_contiguous
    sr, sk = _strides_elems(sfa)
    rc = lib().orc_gg_contiguous(_p(A), _p(B), _p(sfa), _i64(sr), _i64(sk), _p(sfb), _p(gl), _p(D),
                                 _i64(G), _i64(M), _i64(N), _i64(K), _c.c_int(model), _i64(row_step),
                                 _c.c_int(1 if out_f32 else 0))
    if rc != 0:
        raise ValueError(f"orc_gg_contiguous failed: {rc}")
    return D


def gg_masked(A, B, sfa, sfb, masked_m, model=SIM_CHAIN, out=None, out_f32=False):
    """A u8[G,max_m,K], B u8[G,N,K], sfa f32[G,max_m,K/128] (any strides), sfb f32[G,N/128,K/128],
    masked_m i32[G] -> D bf16 bits [G,max_m,N] (rows >= masked_m[g] untouched)."""
    A = _c_arr(A, np.uint8)
    B = _c_arr(B, np.uint8)
    sfa = np.asarray(sfa, np.float32)
    sfb = _c_arr(sfb, np.float32)
    mm = _c_arr(masked_m, np.int32)
    G, max_m, K = A.shape
    N = B.shape[1]
    assert sfa.shape == (G, max_m, K // 128)
    D = np.zeros((G, max_m, N), np.float32 if out_f32 else np.uint16) if out is None else out
    assert D.dtype == (np.float32 if out_f32 else np.uint16) and D.flags.c_contiguous
    sg, sr, sk = _strides_elems(sfa)
    rc = lib().orc_gg_masked(_p(A), _p(B), _p(sfa), _i64(sg), _i64(sr), _i64(sk), _p(sfb), _p(mm),
                             _p(D), _i64(G), _i64(max_m), _i64(N), _i64(K), _c.c_int(model),
                             _c.c_int(1 if out_f32 else 0))
    if rc != 0:
        raise ValueError(f"orc_gg_masked failed: {rc}")
    return D


def fp8_blockwise_ue8m0(A, B, SFA, SFB) -> np.ndarray:
    A = _c_arr(A, np.uint8)
    B = _c_arr(B, np.uint8)
    SFA = _c_arr(SFA, np.uint32)
    SFB = _c_arr(SFB, np.uint32)
    M, K = A.shape
    N = B.shape[0]
    D = np.empty((M, N), np.uint16)
    rc = lib().orc_fp8_blockwise_ue8m0(_p(A), _p(B), _p(SFA), _p(SFB), _p(D), _i64(M), _i64(N), _i64(K))
    if rc != 0:
        raise ValueError(f"orc_fp8_blockwise_ue8m0 failed: {rc}")
    return D


# ---------------------------------------------------------------- quantisation
def quant_1x128(x, mn_major=False):
    """x f32[rows,cols] -> (q u8[rows,cols], scales f32[rows,cols/128] (or [cols/128,rows]))."""
    x = _c_arr(x, np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), np.uint8)
    nb = cols // 128
    if mn_major:
        s = np.empty((nb, rows), np.float32)
        ss_r, ss_b = 1, rows
    else:
        s = np.empty((rows, nb), np.float32)
        ss_r, ss_b = nb, 1
    lib().orc_quant_1x128(_p(x), _p(q), _p(s), _i64(ss_r), _i64(ss_b), _i64(rows), _i64(cols))
    return q, s


def silu_mul_requant(gate_up_bits, gate_first=True, row_valid=None, mn_major=False):
    """gate_up [rows,2I] (uint16 = bf16 bits, or float32) -> (q u8[rows,I], scales f32[rows,I/128]
    or [I/128,rows])."""
    in_f32 = np.asarray(gate_up_bits).dtype == np.float32
    gu = _c_arr(gate_up_bits, np.float32 if in_f32 else np.uint16)
    rows, two_i = gu.shape
    inter = two_i // 2
    nb = inter // 128
    q = np.zeros((rows, inter), np.uint8)
    if mn_major:
        s = np.zeros((nb, rows), np.float32)
        ss_r, ss_b = 1, rows
    else:
        s = np.zeros((rows, nb), np.float32)
        ss_r, ss_b = nb, 1
    rv = None if row_valid is None else _c_arr(row_valid, np.uint8)
    lib().orc_silu_mul_requant(_p(gu), _c.c_int(1 if in_f32 else 0), _p(q), _p(s), _i64(ss_r), _i64(ss_b),
                               _p(rv) if rv is not None else None, _i64(rows), _i64(inter),
                               _c.c_int(1 if gate_first else 0))
    return q, s


# ---------------------------------------------------------------- routing / permutation / combine
def route_softmax_topk(logits, top_k: int):
    l = _c_arr(logits, np.float32)
    T, E = l.shape
    ids = np.empty((T, top_k), np.int32)
    w = np.empty((T, top_k), np.float32)
    lib().orc_route_softmax_topk(_p(l), _p(ids), _p(w), _i64(T), _i64(E), _i64(top_k))
    return ids, w


def route_deepseek(logits, bias, top_k=8, n_group=8, topk_group=4, routed_scaling_factor=1.0):
    """DeepSeek-V3 no-aux routing -> (ids int32 [T, top_k], weights f32 [T, top_k])."""
    l = _c_arr(logits, np.float32)
    b = _c_arr(bias, np.float32).reshape(-1)
    T, E = l.shape
    ids = np.empty((T, top_k), np.int32)
    w = np.empty((T, top_k), np.float32)
    lib().orc_route_deepseek(_p(l), _p(b), _p(ids), _p(w), _i64(T), _i64(E), _i64(n_group), _i64(topk_group),
                             _i64(top_k), _c.c_float(routed_scaling_factor))
    return ids, w


def permute_plan(ids, e_lo: int, e_local: int, align: int, cap_rows: int | None = None):
    """-> dict(counts, offsets, pos, grouped_layout, src_pair, total_rows)."""
    flat = _c_arr(ids, np.int32).reshape(-1)
    n = flat.size
    if cap_rows is None:
        cap_rows = ((n + align - 1) // align + e_local) * align
    counts = np.empty(e_local, np.int32)
    offsets = np.empty(e_local + 1, np.int32)
    pos = np.empty(n, np.int32)
    gl = np.empty(cap_rows, np.int32)
    src = np.empty(cap_rows, np.int32)
    total = lib().orc_permute_plan(_p(flat), _i64(n), _i64(e_lo), _i64(e_local), _i64(align),
                                   _p(counts), _p(offsets), _p(pos), _p(gl), _p(src), _i64(cap_rows))
    if total < 0:
        raise ValueError("permute_plan: cap_rows too small")
    return dict(counts=counts, offsets=offsets, pos=pos.reshape(np.asarray(ids).shape),
                grouped_layout=gl, src_pair=src, total_rows=int(total))


def combine(y_bits, pos, w) -> np.ndarray:
    y = _c_arr(y_bits, np.uint16)
    pos = _c_arr(pos, np.int32)
    w = _c_arr(w, np.float32)
    T, top_k = pos.shape
    H = y.shape[1]
    out = np.empty((T, H), np.uint16)
    lib().orc_combine(_p(y), _p(pos), _p(w), _p(out), _i64(T), _i64(top_k), _i64(H))
    return out


# ---------------------------------------------------------------- MoE layer (composition)
def moe_layer(x_q, x_scale, logits, w13, w13_scale, w2, w2_scale, top_k=8, e_lo=0, align=128,
              gate_first=False, model=SIM_CHAIN, routes=None, fused_act=False):
    """Single-rank MoE layer: route -> permute -> gate_up GEMM -> SiLU*mul requant -> down GEMM ->
    weighted combine.  x_q u8[T,H], x_scale f32[T,H/128]; w13 u8[E,2I,H], w2 u8[E,H,I].
    fused_act=True keeps gate_up in fp32 up to the requant (what a GEMM epilogue that applies
    SiLU*mul itself computes); False rounds it to bf16 first (separate kernels).
    Returns dict with every intermediate (bf16 bits for activations)."""
    T, H = x_q.shape
    E = w13.shape[0]
    inter = w2.shape[2]
    ids, w = route_softmax_topk(logits, top_k) if routes is None else routes
    plan = permute_plan(ids, e_lo, E, align)
    rows = plan["total_rows"]
    src = plan["src_pair"][:rows]
    gl = plan["grouped_layout"][:rows]
    valid = src >= 0
    tok = np.where(valid, src // top_k, 0)
    a1 = np.where(valid[:, None], x_q[tok], 0).astype(np.uint8)
    s1 = np.where(valid[:, None], x_scale[tok], 0).astype(np.float32)
    g1 = gg_contiguous(a1, w13, s1, w13_scale, gl, model=model, out_f32=fused_act)
    a2, s2 = silu_mul_requant(g1, gate_first=gate_first, row_valid=valid.astype(np.uint8))
    y = gg_contiguous(a2, w2, s2, w2_scale, gl, model=model)
    out = combine(y, plan["pos"], w)
    return dict(ids=ids, weights=w, plan=plan, a1=a1, s1=s1, g1=g1, a2=a2, s2=s2, y=y, out=out)


# ---------------------------------------------------------------- alpha-MoE (decode-regime layer)
def alpha_moe_layer(hidden_bits, ids, w, w13, w13_scale, w2, w2_scale, routed_scaling_factor=1.0,
                    model=SIM_CHAIN):
    """The `alphamoe` task operator, restated from its definition.json (`_quantize_inputs`,
    `_reference_quantized`): bf16 activations [M,H] (uint16 bits) are quantised per 1x128 inside; each
    route's expert computes gate_up (rows stacked [gate; up]) and SiLU(gate)*up in fp32, requantises
    per 128, multiplies by the down weights; the down contribution times
    fp32(weight * routed_scaling_factor) is rounded to bf16 and added to a zero bf16 accumulator with
    a bf16 rounding per update, experts in ascending id (the reference's `for expert in range(E)`).
    Intermediate size must be 128 (one down contribution per route), as in the task's rows.
    Returns dict(out=bf16 bits [M,H], abs_sum, x_q, x_s, counts, order, g1, a2, s2, d2)."""
    hidden_bits = _c_arr(hidden_bits, np.uint16)
    ids = _c_arr(ids, np.int32)
    w = _c_arr(w, np.float32)
    M, H = hidden_bits.shape
    top_k = ids.shape[1]
    E = w13.shape[0]
    inter = w2.shape[2]
    if inter != 128:
        raise ValueError("alpha_moe_layer models intermediate size 128 only")
    x_q, x_s = quant_1x128(bf16_to_f32(hidden_bits))
    expert = ids.reshape(-1)
    pair = np.arange(expert.size)
    keep = (expert >= 0) & (expert < E)
    order = pair[keep][np.lexsort((pair[keep], expert[keep]))]          # expert ascending, then pair index
    tok = order // top_k
    gl = expert[order].astype(np.int32)
    g1 = gg_contiguous(x_q[tok], w13, x_s[tok], w13_scale, gl, model=model, out_f32=True)
    a2, s2 = silu_mul_requant(g1, gate_first=True)
    d2 = gg_contiguous(a2, w2, s2, w2_scale, gl, model=model, out_f32=True)
    out = np.zeros((M, H), np.float32)
    abs_sum = np.zeros((M, H), np.float32)
    rsf = np.float32(routed_scaling_factor)
    for r, p in enumerate(order):
        t = p // top_k
        scale = np.float32(w.reshape(-1)[p] * rsf)
        c = bf16_to_f32(bf16_rne(d2[r] * scale))
        out[t] = bf16_to_f32(bf16_rne(out[t] + c))
        abs_sum[t] += np.abs(c)
    counts = np.bincount(expert[keep], minlength=E).astype(np.int32)
    return dict(out=bf16_rne(out), abs_sum=abs_sum, x_q=x_q, x_s=x_s, counts=counts, order=order.astype(np.int64),
                g1=g1, a2=a2, s2=s2, d2=d2)


# ---------------------------------------------------------------- k-grouped layout (weight-gradient shape)
def kg_contiguous(A, B, SFA, SFB, ks, D):
    """k-grouped FP8 GEMM with fp32 accumulation onto D, following the reference's corpus case
    (tools/tests/numsim/corpus/kernels/gemm.py:610-702: per-group K cursors, MN-major operands, D as the start of
    the fp32 chain).  A u8[K_total,M], B u8[K_total,N], SFA u32[sum(ceil(ks/512)),M], SFB u32[..,N] (UE8M0, byte j of
    a word = K block 4*word+j of its group), ks list of multiples of 128, D f32[G,M,N].  Returns the new D:
    D[g][m,n] = fma-chain over the group's k (increasing) of (a*sfa)*(b*sfb), starting from D[g][m,n]."""
    A = _c_arr(A, np.uint8)
    B = _c_arr(B, np.uint8)
    SFA = _c_arr(SFA, np.uint32)
    SFB = _c_arr(SFB, np.uint32)
    D = np.array(D, np.float32, copy=True)
    koff = srow = 0
    for g, k in enumerate(int(x) for x in ks):
        if k == 0:
            continue
        kb = k // 128
        words = (k + 511) // 512
        def scales(W):          # [words, rows] u32 -> f32 [rows, kb]
            b = np.stack([(W[srow:srow + words] >> np.uint32(8 * j)) & np.uint32(0xFF) for j in range(4)], axis=1)  # [words,4,rows]
            codes = b.reshape(words * 4, -1)[:kb].astype(np.uint8)
            return ue8m0_decode(codes).T.copy()
        sa, sb = scales(SFA), scales(SFB)
        a = e4m3_decode(A[koff:koff + k]).T * np.repeat(sa, 128, axis=1)       # [M, k], exact (powers of two)
        b = e4m3_decode(B[koff:koff + k]).T * np.repeat(sb, 128, axis=1)
        D[g] = fma_abt_increasing_k(a, b, d_init=D[g])
        koff += k
        srow += words
    return D
