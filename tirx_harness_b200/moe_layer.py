"""One MoE layer forward on one GPU: ``setup(data, T) -> callable``.

Mirrors the candidate contract of the reference's registered ``moe`` workload
(mlc-ai/TIRx-harness: evolution/benchmark/flashinfer_bench_evolve/tasks/moe/benchmark.py:143-182):
``setup`` may allocate scratch and bind pointers, the returned zero-argument callable redoes
routing, permutation, both grouped GEMMs, the SiLU*mul requant and the weighted combine from the
current inputs and writes the preallocated bf16 ``output`` in place.  Routing here is the
softmax top-k of the MoE-layer workload; ``topk_ids`` / ``topk_weights`` can be passed instead
of ``routing_logits`` (preselected routes, as in the alphamoe workload).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_vp = ctypes.c_void_p


def _p(t):
    return _vp(t.data_ptr()) if t is not None else None


class MoeLayer:
    """Binds one layer's tensors and workspace; ``__call__`` launches the whole pipeline."""

    def __init__(self, data: dict, T: int, top_k: int = 8, e_lo: int = 0, align: int = 128,
                 gate_first: bool = False, fuse_act: bool = False):
        x_q, xs = data["hidden_states"], data["hidden_states_scale"]
        w13, s13 = data["gemm1_weights"], data["gemm1_weights_scale"]
        w2, s2 = data["gemm2_weights"], data["gemm2_weights_scale"]
        out = data["output"]
        logits = data.get("routing_logits")
        ids, wts = data.get("topk_ids"), data.get("topk_weights")
        bias = data.get("routing_bias")               # present in the registered `moe` task: DeepSeek-V3 routing
        if bias is not None:
            if bias.dtype != torch.bfloat16 or not bias.is_contiguous():
                raise TypeError("routing_bias must be contiguous bfloat16")
            e_lo = int(data.get("local_expert_offset", e_lo))
        rsf = float(data.get("routed_scaling_factor", 1.0))
        H = x_q.shape[1]
        E, two_i, _ = w13.shape
        inter = two_i // 2
        if tuple(x_q.shape) != (T, H) or tuple(out.shape) != (T, H) or out.dtype != torch.bfloat16:
            raise ValueError("hidden_states / output must be [T, H]; output bf16")
        if tuple(xs.shape) == (H // 128, T) and T != H // 128:
            xs = xs.t()                      # MN-major [H/128, T] storage (the moe workload's layout)
        if tuple(xs.shape) != (T, H // 128) or xs.dtype != torch.float32:
            raise ValueError(f"hidden_states_scale must be f32 [T, H/128] (any strides), got {tuple(xs.shape)}")
        for name, t in (("gemm1_weights", w13), ("gemm2_weights", w2), ("hidden_states", x_q)):
            if t.dtype not in (torch.float8_e4m3fn, torch.uint8) or not t.is_contiguous():
                raise TypeError(f"{name} must be contiguous float8_e4m3fn")
        if tuple(w2.shape) != (E, H, inter):
            raise ValueError("gemm2_weights must be [E, H, I]")
        if tuple(s13.shape) != (E, two_i // 128, H // 128) or tuple(s2.shape) != (E, H // 128, inter // 128):
            raise ValueError("weight scale shapes do not match 128x128 blocks")
        self.device = x_q.device
        L = _lib.lib()
        self.ws_bytes = L.moe_workspace_bytes(T, H, inter, E, top_k, align)
        self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=self.device)
        e_global = logits.shape[1] if logits is not None else E
        self._keep = (x_q, xs, logits, ids, wts, w13, s13, w2, s2, out, bias)
        self.dims = dict(T=T, H=H, I=inter, E=E, top_k=top_k, align=align)
        self.args = _lib.LayerArgs(
            x_q=_p(x_q), x_scale=_p(xs), xs_stride_row=xs.stride(0), xs_stride_blk=xs.stride(1),
            logits=_p(logits), topk_ids=_p(ids), topk_weights=_p(wts), w13=_p(w13), w13_scale=_p(s13.contiguous()),
            w2=_p(w2), w2_scale=_p(s2.contiguous()), out=_p(out), workspace=_p(self.workspace),
            workspace_bytes=self.ws_bytes, T=T, H=H, I=inter, E=E, E_global=e_global, e_lo=e_lo, top_k=top_k,
            align=align, gate_first=1 if gate_first else 0, fuse_act=1 if fuse_act else 0,
            routing_bias=_p(bias), n_group=0, topk_group=0, routed_scaling_factor=rsf)
        self.out = out

    def __call__(self):
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.lib().moe_layer_forward(ctypes.byref(self.args), _vp(stream)))
        return self.out

    def view(self) -> dict:
        """Torch views of the intermediates inside the workspace (for tests and inspection)."""
        d = self.dims
        v = _lib.LayerView()
        _lib.check(_lib.lib().moe_layer_workspace_view(_p(self.workspace), d["T"], d["H"], d["I"], d["E"], d["top_k"],
                                                       d["align"], ctypes.byref(v)))
        base = self.workspace.data_ptr()
        cap = v.cap_rows
        n_pairs = d["T"] * d["top_k"]

        def sl(ptr, nbytes, dtype, shape):
            o = ptr - base
            return self.workspace[o:o + nbytes].view(dtype).view(shape)
        return dict(
            cap_rows=cap,
            ids=sl(v.ids, n_pairs * 4, torch.int32, (d["T"], d["top_k"])),
            weights=sl(v.weights, n_pairs * 4, torch.float32, (d["T"], d["top_k"])),
            counts=sl(v.counts, d["E"] * 4, torch.int32, (d["E"],)),
            offsets=sl(v.offsets, (d["E"] + 1) * 4, torch.int32, (d["E"] + 1,)),
            pos=sl(v.pos, n_pairs * 4, torch.int32, (d["T"], d["top_k"])),
            src_pair=sl(v.src_pair, cap * 4, torch.int32, (cap,)),
            grouped_layout=sl(v.grouped_layout, cap * 4, torch.int32, (cap,)),
            a1=sl(v.a1, cap * d["H"], torch.uint8, (cap, d["H"])),
            s1=sl(v.s1, cap * (d["H"] // 128) * 4, torch.float32, (d["H"] // 128, cap)).t(),
            g1=sl(v.g1, cap * 2 * d["I"] * 2, torch.bfloat16, (cap, 2 * d["I"])),
            a2=sl(v.a2, cap * d["I"], torch.uint8, (cap, d["I"])),
            s2=sl(v.s2, cap * (d["I"] // 128) * 4, torch.float32, (d["I"] // 128, cap)).t(),
            y=sl(v.y, cap * d["H"] * 2, torch.bfloat16, (cap, d["H"])),
        )


def setup(data: dict, T: int, **kw) -> MoeLayer:
    """``data``: hidden_states fp8 [T,H], hidden_states_scale f32 [T,H/128] or [H/128,T],
    routing_logits f32 [T,E] (or topk_ids/topk_weights), gemm1_weights fp8 [E,2I,H] (+_scale),
    gemm2_weights fp8 [E,H,I] (+_scale), output bf16 [T,H].  With the registered `moe` task's extra keys
    (routing_bias bf16 [E_global], local_expert_offset, routed_scaling_factor) the layer uses that task's
    DeepSeek-V3 routing and computes only the local experts' contributions."""
    return MoeLayer(data, T, **kw)
