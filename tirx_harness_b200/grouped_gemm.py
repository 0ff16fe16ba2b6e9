"""Host side of the m-grouped FP8 GEMM: PyTorch tensors in, one CUDA launch out.

Mirrors the reference's candidate interface for the registered workload ``grouped_gemm/fp8``
(mlc-ai/TIRx-harness: evolution/benchmark/flashinfer_bench_evolve/tasks/grouped_gemm_fp8/
benchmark.py:52-62 and evolution/tasks/grouped_gemm_fp8.yaml:15-25):

    launch = setup(data, G, M, N, K)     # untimed: validates, binds pointers
    launch()                             # timed: recomputes D in place from the current inputs

PyTorch is used for device memory and streams only; all arithmetic happens in the CUDA library
reached through the C ABI of include/b200moe.h.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _ptr(t: torch.Tensor) -> int:
    return t.data_ptr()


def _check_fp8(t: torch.Tensor, name: str, allow_pitch: bool = False) -> None:
    if t.dtype not in (torch.float8_e4m3fn, torch.uint8):
        raise TypeError(f"{name} must be float8_e4m3fn (or its uint8 bytes), got {t.dtype}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if allow_pitch and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1] and t.stride(0) % 16 == 0:
        return                      # rows with a trailer (pitch > K)
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _scale_strides(sfa: torch.Tensor, rows: int, kblocks: int, name: str):
    """Accepts [rows, K/128] in any stride order (row-major or MN-major/transposed view)."""
    if sfa.dtype != torch.float32 or not sfa.is_cuda:
        raise TypeError(f"{name} must be a float32 CUDA tensor")
    if tuple(sfa.shape) != (rows, kblocks):
        raise ValueError(f"{name} must have shape ({rows}, {kblocks}), got {tuple(sfa.shape)}")
    return sfa.stride(0), sfa.stride(1)


class _BoundGG:
    """A validated argument block; ``__call__`` launches on the current stream of the tensors' device."""

    def __init__(self, fn_name, a, b, sfa, sfa_strides, sfb, layout, d, G, M, N, K, rows_used=None,
                 workspace=True, scatter=None, mx_tile=0):
        rows_total = M if fn_name.endswith("contiguous") else G * M
        ws_bytes = _lib.lib().moe_gg_workspace_bytes(ctypes.c_int32(G), ctypes.c_int64(rows_total), ctypes.c_int32(N),
                                                    ctypes.c_int32(K)) if workspace else 0
        # scratch for the power-of-two-scale path, allocated once at bind time (set-up, untimed)
        self._ws = torch.empty(ws_bytes, dtype=torch.uint8, device=d.device) if ws_bytes else None
        self._keep = (a, b, sfa, sfb, layout, d, rows_used)
        self._fn = getattr(_lib.lib(), fn_name)
        self._device = d.device
        self._args = _lib.GGArgs(
            a=_ptr(a), b=_ptr(b), sfa=_ptr(sfa), sfa_stride_row=sfa_strides[0], sfa_stride_kblk=sfa_strides[1],
            sfb=_ptr(sfb), layout=_ptr(layout), d=_ptr(d), ldd=d.stride(-2), G=G, M=M, N=N, K=K,
            d_dtype=1 if d.dtype == torch.float32 else 0, lda=a.stride(-2) if a.dim() == 2 else 0,
            rows_used=_ptr(rows_used) if rows_used is not None else None,
            workspace=_ptr(self._ws) if self._ws is not None else None, workspace_bytes=ws_bytes, mx_tile=mx_tile)
        if scatter is not None:          # (meta int32[M] tensor, list of up to 8 base addresses)
            meta, bases = scatter
            self._keep = self._keep + (meta,)
            self._args.scatter_meta = _ptr(meta)
            self._args.scatter_meta_stride = meta.stride(0)
            for i, b_ in enumerate(bases):
                self._args.scatter_base[i] = b_
        self._argp = ctypes.byref(self._args)
        self.out = d

    def __call__(self):
        with torch.cuda.device(self._device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(self._fn(self._argp, ctypes.c_void_p(stream)))
        return self.out


def bind_contiguous(a, sfa, b, sfb, d, grouped_layout, rows_used=None, workspace=True, scatter=None,
                    mx_tile: int = 0) -> _BoundGG:
    """a fp8[M,K] (row pitch may exceed K), sfa f32[M,K/128] (any strides), b fp8[G,N,K], sfb
    f32[G,ceil(N/128),K/128], d bf16[M,N], grouped_layout int32[M] (group id per row, negative = padding row);
    rows_used: optional int32[1] device tensor with the number of leading rows in use; mx_tile: a
    ``_lib.MX_TILE_*`` value for this binding (0 = the process-wide option)."""
    _check_fp8(a, "a", allow_pitch=True); _check_fp8(b, "b")
    M, K = a.shape
    G, N, Kb = b.shape
    if Kb != K or K % 128:
        raise ValueError(f"K mismatch or not a multiple of 128: a K={K}, b K={Kb}")
    strides = _scale_strides(sfa, M, K // 128, "sfa")
    if sfb.dtype != torch.float32 or tuple(sfb.shape) != (G, (N + 127) // 128, K // 128) or not sfb.is_contiguous():
        raise ValueError(f"sfb must be contiguous float32 [{G}, {(N + 127) // 128}, {K // 128}]")
    if scatter is not None:
        if d.dtype != torch.bfloat16 or d.shape[1] != N or d.stride(1) != 1:
            raise ValueError("with scatter, d only supplies dtype (bf16) and row stride: shape [*, N]")
    elif d.dtype not in (torch.bfloat16, torch.float32) or tuple(d.shape) != (M, N) or d.stride(1) != 1:
        raise ValueError(f"d must be bfloat16 (or float32) [{M}, {N}] with unit column stride")
    if grouped_layout.dtype != torch.int32 or grouped_layout.numel() != M or not grouped_layout.is_contiguous():
        raise ValueError(f"grouped_layout must be contiguous int32 [{M}]")
    if rows_used is not None and (rows_used.dtype != torch.int32 or not rows_used.is_cuda):
        raise ValueError("rows_used must be an int32 CUDA tensor")
    return _BoundGG("moe_gg_fp8_contiguous", a, b, sfa, strides, sfb, grouped_layout, d, G, M, N, K, rows_used,
                    workspace and scatter is None, scatter, mx_tile)


def bind_masked(a, sfa, b, sfb, d, masked_m, workspace=True) -> _BoundGG:
    """a fp8[G,max_m,K], sfa f32[G,max_m,K/128] (contiguous, or MN-major: a [G*max_m, K/128] view of any
    strides), b fp8[G,N,K], sfb f32[G,ceil(N/128),K/128], d bf16[G,max_m,N], masked_m int32[G]."""
    _check_fp8(a, "a"); _check_fp8(b, "b")
    G, max_m, K = a.shape
    Gb, N, Kb = b.shape
    if Gb != G or Kb != K or K % 128:
        raise ValueError("a and b disagree on G or K, or K is not a multiple of 128")
    if sfa.dim() == 3:
        if not sfa.is_contiguous():
            raise ValueError("3-d sfa must be contiguous; pass a [G*max_m, K/128] view for other layouts")
        sfa2 = sfa.view(G * max_m, K // 128)
    else:
        sfa2 = sfa
    strides = _scale_strides(sfa2, G * max_m, K // 128, "sfa")
    if sfb.dtype != torch.float32 or tuple(sfb.shape) != (G, (N + 127) // 128, K // 128) or not sfb.is_contiguous():
        raise ValueError(f"sfb must be contiguous float32 [{G}, {(N + 127) // 128}, {K // 128}]")
    if d.dtype not in (torch.bfloat16, torch.float32) or tuple(d.shape) != (G, max_m, N) or not d.is_contiguous():
        raise ValueError(f"d must be contiguous bfloat16 (or float32) [{G}, {max_m}, {N}]")
    if masked_m.dtype != torch.int32 or masked_m.numel() != G or not masked_m.is_contiguous():
        raise ValueError(f"masked_m must be contiguous int32 [{G}]")
    return _BoundGG("moe_gg_fp8_masked", a, b, sfa2, strides, sfb, masked_m, d, G, max_m, N, K, None, workspace)


class _BoundGateUpAct:
    """gate_up grouped GEMM with SiLU*mul + 1x128 FP8 requant in the epilogue; ``__call__`` launches."""

    def __init__(self, a, sfa, sfa_strides, b, sfb, act_q, act_s, layout, gate_first, rows_used, G, M, N, K):
        self._keep = (a, sfa, b, sfb, act_q, act_s, layout, rows_used)
        self._device = a.device
        self._args = _lib.GGArgs(a=_ptr(a), b=_ptr(b), sfa=_ptr(sfa), sfa_stride_row=sfa_strides[0],
                                 sfa_stride_kblk=sfa_strides[1], sfb=_ptr(sfb), layout=_ptr(layout), d=None, ldd=0,
                                 G=G, M=M, N=N, K=K, d_dtype=0, lda=a.stride(0),
                                 rows_used=_ptr(rows_used) if rows_used is not None else None, workspace=None,
                                 workspace_bytes=0)
        self._act = (ctypes.c_void_p(_ptr(act_q)), ctypes.c_void_p(_ptr(act_s)), ctypes.c_int64(act_s.stride(0)),
                     ctypes.c_int64(act_s.stride(1)), ctypes.c_int32(1 if gate_first else 0))
        self.out = (act_q, act_s)

    def __call__(self):
        with torch.cuda.device(self._device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.lib().moe_gg_fp8_gate_up_act(ctypes.byref(self._args), *self._act, ctypes.c_void_p(stream)))
        return self.out


def bind_gate_up_act(a, sfa, b, sfb, act_q, act_s, grouped_layout, gate_first=False, rows_used=None):
    """a fp8[M,K], sfa f32[M,K/128], b fp8[G,2I,K], sfb f32[G,2I/128,K/128] -> act_q fp8[M,I], act_s f32[M,I/128]
    (any strides) = 1x128 requant of silu(gate)*up, computed from the fp32 accumulators inside the GEMM."""
    _check_fp8(a, "a", allow_pitch=True); _check_fp8(b, "b"); _check_fp8(act_q, "act_q")
    M, K = a.shape
    G, N, Kb = b.shape
    if Kb != K or K % 128 or N % 256:
        raise ValueError("K must match and be a multiple of 128; N = 2*I must be a multiple of 256")
    strides = _scale_strides(sfa, M, K // 128, "sfa")
    if sfb.dtype != torch.float32 or tuple(sfb.shape) != (G, N // 128, K // 128) or not sfb.is_contiguous():
        raise ValueError(f"sfb must be contiguous float32 [{G}, {N // 128}, {K // 128}]")
    if tuple(act_q.shape) != (M, N // 2) or tuple(act_s.shape) != (M, N // 256) or act_s.dtype != torch.float32:
        raise ValueError("act_q must be [M, I] and act_s float32 [M, I/128]")
    return _BoundGateUpAct(a, sfa, strides, b, sfb, act_q, act_s, grouped_layout, gate_first, rows_used, G, M, N, K)


def bind_contiguous_packed(a, sfa_words, b, sfb_words, d, grouped_layout, mx_tile: int = 0) -> _BoundGG:
    """The registered workload's own scale format: UE8M0 bytes packed four per int32.
    sfa_words int32 [M, ceil(K/512)] (any strides; DeepGEMM stores it MN-major), sfb_words int32
    [G, N, ceil(K/512)] (any strides).  Always runs the block-scaled-MMA kernel."""
    _check_fp8(a, "a"); _check_fp8(b, "b")
    M, K = a.shape
    G, N, _ = b.shape
    kq = (K // 128 + 3) // 4
    if sfa_words.dtype != torch.int32 or tuple(sfa_words.shape) != (M, kq):
        raise ValueError(f"packed SFA must be int32 [{M}, {kq}]")
    if sfb_words.dtype != torch.int32 or tuple(sfb_words.shape) != (G, N, kq):
        raise ValueError(f"packed SFB must be int32 [{G}, {N}, {kq}]")
    if d.dtype != torch.bfloat16 and d.dtype != torch.float32 or tuple(d.shape) != (M, N):
        raise ValueError(f"d must be [{M}, {N}] bf16 or f32")
    bound = _BoundGG("moe_gg_fp8_contiguous", a, b, sfa_words, (sfa_words.stride(0), sfa_words.stride(1)), sfb_words,
                     grouped_layout, d, G, M, N, K, None, True, None, mx_tile)
    bound._args.sf_format = 1
    for i in range(3):
        bound._args.sfb_stride[i] = sfb_words.stride(i)
    return bound


class _BoundKGrouped:
    """k-grouped (weight-gradient) GEMM bound to its tensors: ``d[g] += a[ks_g rows].T @ b[ks_g rows]``."""

    def __init__(self, a, sfa_words, b, sfb_words, d, ks):
        _check_fp8(a, "a"); _check_fp8(b, "b")
        K_total, M = a.shape
        N = b.shape[1]
        ks = [int(k) for k in ks]
        G = len(ks)
        scale_rows = sum((k + 511) // 512 for k in ks)
        if b.shape[0] != K_total or sum(ks) != K_total:
            raise ValueError("a is [K_total, M], b is [K_total, N] and sum(ks) must equal K_total")
        if sfa_words.dtype != torch.int32 or tuple(sfa_words.shape) != (scale_rows, M) or not sfa_words.is_contiguous():
            raise ValueError(f"packed SFA must be contiguous int32 [{scale_rows}, {M}]")
        if sfb_words.dtype != torch.int32 or tuple(sfb_words.shape) != (scale_rows, N) or not sfb_words.is_contiguous():
            raise ValueError(f"packed SFB must be contiguous int32 [{scale_rows}, {N}]")
        if d.dtype != torch.float32 or tuple(d.shape) != (G, M, N) or not d.is_contiguous():
            raise ValueError(f"d must be contiguous float32 [{G}, {M}, {N}]")
        L = _lib.lib()
        self.device = a.device
        ws_bytes = L.moe_kg_workspace_bytes(M, N, ctypes.c_int64(K_total))
        if ws_bytes == 0:
            raise ValueError("unsupported k-grouped shape (K_total must be a positive multiple of 128)")
        self._ws = torch.empty(ws_bytes, dtype=torch.uint8, device=self.device)
        self._ks = (ctypes.c_int32 * G)(*ks)
        self._keep = (a, sfa_words, b, sfb_words, d)
        self._args = _lib.KgArgs(a=a.data_ptr(), b=b.data_ptr(), sfa=sfa_words.data_ptr(), sfb=sfb_words.data_ptr(),
                                 d=d.data_ptr(), ks=self._ks, G=G, M=M, N=N, K_total=K_total,
                                 workspace=self._ws.data_ptr(), workspace_bytes=ws_bytes)
        self.d = d

    def __call__(self):
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.lib().moe_kg_fp8_contiguous(ctypes.byref(self._args), ctypes.c_void_p(stream)))
        return self.d


def bind_k_grouped(a, sfa_words, b, sfb_words, d, ks) -> _BoundKGrouped:
    """k-grouped FP8 GEMM with fp32 accumulation onto ``d`` (the weight-gradient layout of the reference's kernel
    family, tools/tests/numsim/corpus/kernels/gemm.py:610-702): ``a`` e4m3 [K_total, M] and ``b`` e4m3 [K_total, N]
    MN-major, group g owns ``ks[g]`` consecutive K rows (multiples of 128), packed UE8M0 scales int32
    [sum(ceil(ks/512)), M] / [.., N], ``d`` f32 [G, M, N].  Returns the zero-argument callable."""
    return _BoundKGrouped(a, sfa_words, b, sfb_words, d, ks)


def m_grouped_fp8_gemm_nt_contiguous(a, sfa, b, sfb, d, grouped_layout):
    """One-shot form (argument order of the kernel the reference baselines against: (a, sfa), (b, sfb), d, layout)."""
    return bind_contiguous(a, sfa, b, sfb, d, grouped_layout)()


def m_grouped_fp8_gemm_nt_masked(a, sfa, b, sfb, d, masked_m):
    return bind_masked(a, sfa, b, sfb, d, masked_m)()


def setup(data: dict, G: int, M: int, N: int, K: int):
    """Candidate entry of the registered workload: returns the zero-argument timed callable.

    ``data`` holds ``A`` fp8[M,K], ``B`` fp8[G,N,K], ``SFA`` f32[M,K/128] (any strides), ``SFB``
    f32[G,N/128,K/128] -- or the workload's packed UE8M0 form, ``SFA`` int32[M,K/512] and ``SFB``
    int32[G,N,K/512] with whatever strides they come with --, ``D`` bf16[M,N] (written in place) and
    ``grouped_layout`` int32[M];
    ``actual_ms`` / ``aligned_ms`` / ``alignment`` are accepted and not needed.
    """
    a, b, d = data["A"], data["B"], data["D"]
    if tuple(a.shape) != (M, K) or tuple(b.shape) != (G, N, K):
        raise ValueError(f"A/B shapes {tuple(a.shape)}/{tuple(b.shape)} do not match G={G} M={M} N={N} K={K}")
    if data["SFA"].dtype == torch.int32:          # the registered workload's packed UE8M0 scales
        return bind_contiguous_packed(a, data["SFA"], b, data["SFB"], d, data["grouped_layout"])
    bound = bind_contiguous(a, data["SFA"], b, data["SFB"], d, data["grouped_layout"])
    return bound


def device_status(device=None) -> int:
    """Synchronises and returns the device status word (0 = fine); raises if a kernel reported an error."""
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        out = ctypes.c_int32(0)
        _lib.check(_lib.lib().moe_device_status(ctypes.byref(out), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out.value
