"""Host wrappers of the memory-bound stages around the grouped GEMMs (PyTorch tensors -> C ABI)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_vp = ctypes.c_void_p
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64


def _stream(t: torch.Tensor):
    return _vp(torch.cuda.current_stream(t.device).cuda_stream)


def _scale_out(rows: int, nb: int, mn_major: bool, device):
    """Allocates a [rows, nb] scale tensor, physically [nb, rows] when mn_major."""
    if mn_major:
        return torch.empty((nb, rows), dtype=torch.float32, device=device).t()
    return torch.empty((rows, nb), dtype=torch.float32, device=device)


def quant_1x128(x: torch.Tensor, mn_major: bool = False, out=None):
    """bf16 [rows, cols] -> (e4m3 [rows, cols], f32 scales [rows, cols/128])."""
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous() and x.dim() == 2
    rows, cols = x.shape
    q, s = out if out is not None else (torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device),
                                        _scale_out(rows, cols // 128, mn_major, x.device))
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().moe_quant_1x128(_vp(x.data_ptr()), _vp(q.data_ptr()), _vp(s.data_ptr()),
                                              _i64(s.stride(0)), _i64(s.stride(1)), _i32(rows), _i32(cols), _stream(x)))
    return q, s


def silu_mul_requant(gate_up: torch.Tensor, gate_first: bool = True, layout=None, mn_major: bool = False, out=None):
    """bf16 [rows, 2I] -> (e4m3 [rows, I], f32 scales [rows, I/128]); rows with layout < 0 are skipped."""
    assert gate_up.dtype == torch.bfloat16 and gate_up.is_cuda and gate_up.is_contiguous()
    rows, two_i = gate_up.shape
    inter = two_i // 2
    q, s = out if out is not None else (torch.zeros((rows, inter), dtype=torch.float8_e4m3fn, device=gate_up.device),
                                        _scale_out(rows, inter // 128, mn_major, gate_up.device).zero_())
    with torch.cuda.device(gate_up.device):
        _lib.check(_lib.lib().moe_silu_mul_requant(
            _vp(gate_up.data_ptr()), _vp(q.data_ptr()), _vp(s.data_ptr()), _i64(s.stride(0)), _i64(s.stride(1)),
            _vp(layout.data_ptr()) if layout is not None else None, _i32(rows), _i32(inter),
            _i32(1 if gate_first else 0), _stream(gate_up)))
    return q, s


def route_topk(logits: torch.Tensor, top_k: int):
    """f32 [T, E] -> (ids int32 [T, top_k], weights f32 [T, top_k])."""
    assert logits.dtype == torch.float32 and logits.is_cuda and logits.is_contiguous()
    T, E = logits.shape
    ids = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().moe_route_topk(_vp(logits.data_ptr()), _vp(ids.data_ptr()), _vp(w.data_ptr()),
                                             _i32(T), _i32(E), _i32(top_k), _stream(logits)))
    return ids, w


def route_deepseek(logits: torch.Tensor, bias: torch.Tensor, top_k: int = 8, n_group: int = 8, topk_group: int = 4,
                   routed_scaling_factor: float = 1.0):
    """DeepSeek-V3 no-aux routing: f32 [T, E], bias bf16/f32 [E] -> (ids int32 [T, top_k], weights f32 [T, top_k])."""
    assert logits.dtype == torch.float32 and logits.is_cuda and logits.is_contiguous()
    assert bias.dtype in (torch.bfloat16, torch.float32) and bias.is_contiguous()
    T, E = logits.shape
    ids = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().moe_route_deepseek(_vp(logits.data_ptr()), _vp(bias.data_ptr()),
                                                 _i32(0 if bias.dtype == torch.bfloat16 else 1), _vp(ids.data_ptr()),
                                                 _vp(w.data_ptr()), _i32(T), _i32(E), _i32(n_group), _i32(topk_group),
                                                 _i32(top_k), ctypes.c_float(routed_scaling_factor), _stream(logits)))
    return ids, w


def plan_cap_rows(n_pairs: int, e_local: int, align: int) -> int:
    return (n_pairs + align - 1) // align * align + e_local * align


def permute_plan(ids: torch.Tensor, e_lo: int, e_local: int, align: int = 128, cap_rows: int | None = None):
    """ids int32 [T, top_k] (or flat) -> dict(counts, offsets, pos, src_pair, grouped_layout, cap_rows)."""
    assert ids.dtype == torch.int32 and ids.is_cuda and ids.is_contiguous()
    n = ids.numel()
    dev = ids.device
    cap = plan_cap_rows(n, e_local, align) if cap_rows is None else cap_rows
    counts = torch.empty(e_local, dtype=torch.int32, device=dev)
    offsets = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
    pos = torch.empty(ids.shape, dtype=torch.int32, device=dev)
    src = torch.empty(cap, dtype=torch.int32, device=dev)
    gl = torch.empty(cap, dtype=torch.int32, device=dev)
    L = _lib.lib()
    ws_bytes = L.moe_permute_workspace_bytes(_i64(n), _i32(e_local))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(L.moe_permute_plan(_vp(ids.data_ptr()), _i64(n), _i32(e_lo), _i32(e_local), _i32(align), _i32(cap),
                                      _vp(counts.data_ptr()), _vp(offsets.data_ptr()), _vp(pos.data_ptr()),
                                      _vp(src.data_ptr()), _vp(gl.data_ptr()), _vp(ws.data_ptr()),
                                      ctypes.c_size_t(ws_bytes), _stream(ids)))
    return dict(counts=counts, offsets=offsets, pos=pos, src_pair=src, grouped_layout=gl, cap_rows=cap)


def permute(x_q: torch.Tensor, x_scale: torch.Tensor, src_pair: torch.Tensor, top_k: int, mn_major: bool = True,
            out=None):
    """Gathers token rows into the grouped layout: -> (a e4m3 [rows, H], scales f32 [rows, H/128])."""
    T, H = x_q.shape
    rows = src_pair.numel()
    a, s = out if out is not None else (torch.zeros((rows, H), dtype=torch.float8_e4m3fn, device=x_q.device),
                                        _scale_out(rows, H // 128, mn_major, x_q.device).zero_())
    with torch.cuda.device(x_q.device):
        _lib.check(_lib.lib().moe_permute(_vp(x_q.data_ptr()), _vp(x_scale.data_ptr()), _i64(x_scale.stride(0)),
                                          _i64(x_scale.stride(1)), _vp(src_pair.data_ptr()), _i32(top_k),
                                          _vp(a.data_ptr()), _vp(s.data_ptr()), _i64(s.stride(0)), _i64(s.stride(1)),
                                          _i32(rows), _i32(H), _stream(x_q)))
    return a, s


def combine(y: torch.Tensor, pos: torch.Tensor, w: torch.Tensor, out=None):
    """y bf16 [rows, H], pos int32 [T, top_k], w f32 [T, top_k] -> bf16 [T, H]."""
    T, top_k = pos.shape
    H = y.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
    with torch.cuda.device(y.device):
        _lib.check(_lib.lib().moe_combine(_vp(y.data_ptr()), _vp(pos.data_ptr()), _vp(w.data_ptr()), _vp(out.data_ptr()),
                                          _i32(T), _i32(top_k), _i32(H), _stream(y)))
    return out
