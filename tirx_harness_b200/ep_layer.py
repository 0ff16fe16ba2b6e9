"""Expert-parallel MoE layer: one process per GPU, experts sharded, tokens sharded.

    layer = EpMoeLayer(data, T_local, top_k=8)      # collective: every rank of the group calls it
    layer()                                          # one forward on the current stream

Rank r owns experts [r*E_local, (r+1)*E_local) with their weights resident and T_local tokens.
Per forward: route -> publish per-expert counts to all peers -> barrier -> plan -> gate_up grouped GEMM that
carries the dispatch all-to-all itself (one warp of every CTA stores this rank's token records straight into the
owners' grouped-layout buffers over NVLink, first experts first; the GEMM's loaders start on an expert as soon as
its rows have all arrived, so the transfer hides behind the GEMM and needs no barrier; ``dispatch="kernel"`` runs
the older separate dispatch kernel + barrier instead) -> SiLU*mul requant -> down grouped GEMM whose epilogue sends every finished
output row straight to the slot of the rank that owns the token (256-byte bulk stores from a shared-memory
staging area, so the combine all-to-all rides on the GEMM and costs it nothing measurable) -> barrier ->
local weighted sum.  ``combine="pull"`` keeps the expert outputs local instead and lets the combine kernel
load them from the owners with 16-byte peer loads (2 GPUs: 0.78 ms for that stage against 0.23 ms).  The reference emulates this sharding on one GPU
with ``local_expert_offset`` (mlc-ai/TIRx-harness: evolution/benchmark/flashinfer_bench_evolve/tasks/
moe/definition.json); with world size 1 this class computes exactly what ``moe_layer.MoeLayer`` does.

torch.distributed is used only to exchange the 64-byte IPC handles at set-up; the data path is this
library's own kernels over peer-mapped memory, synchronised by a bounded flag barrier.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, grouped_gemm

_vp = ctypes.c_void_p
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64


def _a256(n: int) -> int:
    return (n + 255) // 256 * 256


class SymmetricBuffer:
    """One IPC-exportable allocation per rank, mapped by every other rank of the node."""

    def __init__(self, nbytes: int, group=None):
        import torch.distributed as dist
        self.L = _lib.lib()
        self.nbytes = nbytes
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        p = _vp()
        _lib.check(self.L.moe_ipc_alloc(ctypes.c_size_t(nbytes), ctypes.byref(p)))
        self.local = p.value
        self.ptrs = [None] * self.world
        self.ptrs[self.rank] = self.local
        self._opened = []
        if self.world > 1:
            handle = ctypes.create_string_buffer(64)
            _lib.check(self.L.moe_ipc_get_handle(_vp(self.local), handle))
            gathered = [None] * self.world
            dist.all_gather_object(gathered, bytes(handle.raw), group=group)
            for r, h in enumerate(gathered):
                if r == self.rank:
                    continue
                q = _vp()
                _lib.check(self.L.moe_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(q)))
                self.ptrs[r] = q.value
                self._opened.append(q.value)

    def close(self):
        torch.cuda.synchronize()
        for q in self._opened:
            self.L.moe_ipc_close(_vp(q))
        self._opened = []
        if self.local:
            self.L.moe_ipc_free(_vp(self.local))
            self.local = None


class EpMoeLayer:
    def __init__(self, data: dict, T_local: int, top_k: int = 8, align: int = 128, gate_first: bool = False,
                 group=None, fuse_act: bool = False, combine: str = "push", dispatch: str = "fused"):
        import torch.distributed as dist
        self.L = _lib.lib()
        x_q, xs = data["hidden_states"], data["hidden_states_scale"]
        self.logits = data["routing_logits"]
        w13, s13 = data["gemm1_weights"], data["gemm1_weights_scale"].contiguous()
        w2, s2 = data["gemm2_weights"], data["gemm2_weights_scale"].contiguous()
        self.out = data["output"]
        dev = x_q.device
        self.device = dev
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("at most 8 ranks (one NVLink domain)")
        H = x_q.shape[1]
        E_local, two_i, _ = w13.shape
        inter = two_i // 2
        E_total = self.logits.shape[1]
        if E_total != E_local * self.world:
            raise ValueError(f"router has {E_total} experts but {self.world} ranks x {E_local} local experts")
        if tuple(xs.shape) == (H // 128, T_local) and T_local != H // 128:
            xs = xs.t()
        if tuple(x_q.shape) != (T_local, H) or tuple(xs.shape) != (T_local, H // 128):
            raise ValueError("hidden_states must be [T_local, H] with scales [T_local, H/128]")
        self.x_q, self.xs, self.gate_first, self.fuse_act = x_q, xs, gate_first, fuse_act
        self.T, self.H, self.I, self.E_local, self.E_total, self.top_k, self.align = T_local, H, inter, E_local, E_total, top_k, align
        n_pairs = T_local * top_k
        self.n_pairs = n_pairs
        # worst case: every pair of every rank lands on this rank
        cap = (n_pairs * self.world + align - 1) // align * align + E_local * align
        self.cap = cap
        if combine not in ("push", "pull"):
            raise ValueError("combine must be 'push' or 'pull'")
        if dispatch not in ("fused", "kernel"):
            raise ValueError("dispatch must be 'fused' or 'kernel'")
        self.combine, self.dispatch = combine, dispatch
        # ---- symmetric region: a | sa | y (pull: [cap,H] expert outputs; push: [T_local*top_k,H] return slots)
        #      | counts | flags | meta
        y_rows = cap if combine == "pull" else n_pairs
        # one record per row: e4m3 bytes, its fp32 scales, and (fused dispatch) the row's return address
        pitch = (H + (H // 128) * 4 + 4 + 15) // 16 * 16
        self.pitch = pitch
        # flags: [0, world) barrier epochs, [64, 64 + E_local) arrival counters of the fused dispatch
        sizes = [cap * pitch, 0, y_rows * H * 2, self.world * E_total * 4, (64 + E_local) * 4, cap * 4]
        offs, o = [], 0
        for s in sizes:
            offs.append(o)
            o += _a256(s)
        with torch.cuda.device(dev):
            self.symm = SymmetricBuffer(o, group)
        self.peers = _lib.EpPeers()
        for r in range(self.world):
            base = self.symm.ptrs[r]
            self.peers.a[r], self.peers.sa[r], self.peers.y[r] = base + offs[0], base + offs[0] + H, base + offs[2]
            self.peers.counts[r], self.peers.flags[r] = base + offs[3], base + offs[4]
            self.peers.meta[r] = base + offs[5]
        self._local = dict(a=self.symm.local + offs[0], y=self.symm.local + offs[2])
        # ---- private scratch
        i32 = dict(dtype=torch.int32, device=dev)
        self.ids = torch.empty((T_local, top_k), **i32)
        self.weights = torch.empty((T_local, top_k), dtype=torch.float32, device=dev)
        self.pos = torch.empty((T_local, top_k), **i32)
        self.send_order = torch.empty(n_pairs, **i32)
        self.my_counts = torch.empty(E_total, **i32)
        self.dst_base = torch.empty(E_total, **i32)
        self.counts_local = torch.empty(E_local, **i32)
        self.offsets = torch.empty(E_local + 1, **i32)
        self.layout = torch.full((cap,), -1, **i32)
        self.ws_bytes = self.L.moe_ep_workspace_bytes(_i64(n_pairs), _i32(E_total))
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.g1 = torch.empty((cap if not fuse_act else 1, two_i), dtype=torch.bfloat16, device=dev)
        self.a2 = torch.empty((cap, inter), dtype=torch.float8_e4m3fn, device=dev)
        self.s2 = torch.empty((inter // 128, cap), dtype=torch.float32, device=dev)
        self._keep = (w13, s13, w2, s2)
        # the grouped GEMMs see the symmetric buffers as ordinary tensors of this process
        rec = self._wrap(self._local["a"], (cap, pitch), torch.uint8)
        self.a1_t = rec[:, :H].view(torch.float8_e4m3fn)                    # [cap, H], row pitch = record size
        self.s1_t = rec.view(torch.float32)[:, H // 4:H // 4 + H // 128]     # [cap, H/128], row stride = pitch/4
        self.y_t = self._wrap(self._local["y"], (y_rows, H), torch.bfloat16)
        if dispatch == "fused":      # return addresses travel inside the records: word (H + H/32) / 4 of every row
            self.meta_t = rec.view(torch.int32)[:, (H + H // 32) // 4]
        else:
            self.meta_t = self._wrap(self.symm.local + offs[5], (cap,), torch.int32)
        rows_used = self.offsets[E_local:E_local + 1]
        if fuse_act:
            self.gemm1 = grouped_gemm.bind_gate_up_act(self.a1_t, self.s1_t, w13, s13, self.a2, self.s2.t(), self.layout,
                                                       gate_first, rows_used)
        else:
            self.gemm1 = grouped_gemm.bind_contiguous(self.a1_t, self.s1_t, w13, s13, self.g1, self.layout, rows_used,
                                                      workspace=False)
        if combine == "push":
            bases = [self.peers.y[r] for r in range(self.world)]
            self.gemm2 = grouped_gemm.bind_contiguous(self.a2, self.s2.t(), w2, s2, self.y_t, self.layout, rows_used,
                                                      workspace=False, scatter=(self.meta_t, bases))
            self.slot_pos = torch.arange(n_pairs, dtype=torch.int32, device=dev).view(T_local, top_k)
        else:
            self.gemm2 = grouped_gemm.bind_contiguous(self.a2, self.s2.t(), w2, s2, self.y_t, self.layout, rows_used,
                                                      workspace=False)    # activation scales are amax/448, never 2^e
        if dispatch == "fused":
            self._send = _lib.EpSendArgs(
                peers=ctypes.pointer(self.peers), x_q=x_q.data_ptr(), x_scale=xs.data_ptr(), xs_row=xs.stride(0),
                xs_blk=xs.stride(1), ids=self.ids.data_ptr(), pos=self.pos.data_ptr(), send_order=self.send_order.data_ptr(),
                counts_local=self.counts_local.data_ptr(), n_pairs=n_pairs, pitch=pitch, top_k=top_k, E_local=E_local, H=H,
                cap_rows=cap, rank=self.rank, world=self.world)
        self.epoch = 0
        if self.world > 1:
            dist.barrier(group)

    def _wrap(self, ptr: int, shape, dtype):
        """A torch tensor over raw device memory (no copy, no ownership)."""
        n = 1
        for s in shape:
            n *= s
        itemsize = torch.empty((), dtype=dtype).element_size()

        class _Cai:
            __cuda_array_interface__ = {"shape": (n * itemsize,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        t = torch.as_tensor(_Cai(), device=self.device)
        return t.view(dtype).view(shape)

    def _barrier(self, st):
        self.epoch += 1
        _lib.check(self.L.moe_ep_barrier(ctypes.byref(self.peers), self.rank, self.world, self.epoch, st))

    def __call__(self, marks=None):
        """One forward.  ``marks``: optional list; a (name, cuda event) pair is appended after every stage
        (the benchmark's stage timing hook)."""
        L, P = self.L, ctypes.byref(self.peers)

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))
        with torch.cuda.device(self.device):
            st = _vp(torch.cuda.current_stream().cuda_stream)
            mark("start")
            _lib.check(L.moe_route_topk(_vp(self.logits.data_ptr()), _vp(self.ids.data_ptr()), _vp(self.weights.data_ptr()),
                                        _i32(self.T), _i32(self.E_total), _i32(self.top_k), st))
            mark("route")
            _lib.check(L.moe_ep_count_publish(P, _vp(self.ids.data_ptr()), _i64(self.n_pairs), self.rank, self.world,
                                              self.E_total, _vp(self.my_counts.data_ptr()), _vp(self.ws.data_ptr()),
                                              ctypes.c_size_t(self.ws_bytes), st))
            self._barrier(st)
            mark("counts+barrier")
            _lib.check(L.moe_ep_plan(P, _vp(self.ids.data_ptr()), _i64(self.n_pairs), self.rank, self.world, self.E_total,
                                     self.E_local, self.align, self.cap, _vp(self.counts_local.data_ptr()),
                                     _vp(self.offsets.data_ptr()), _vp(self.layout.data_ptr()), _vp(self.dst_base.data_ptr()),
                                     _vp(self.pos.data_ptr()),
                                     _vp(self.send_order.data_ptr()) if self.dispatch == "fused" else None,
                                     _vp(self.ws.data_ptr()), ctypes.c_size_t(self.ws_bytes), st))
            mark("plan")
            if self.dispatch == "fused":
                act = self.gemm1._act if self.fuse_act else (None, None, _i64(0), _i64(0), _i32(0))
                _lib.check(L.moe_ep_gate_up_dispatch(ctypes.byref(self.gemm1._args), ctypes.byref(self._send), *act, st))
                mark("dispatch+gate_up_gemm")
            else:
                _lib.check(L.moe_ep_dispatch(P, _vp(self.x_q.data_ptr()), _vp(self.xs.data_ptr()), _i64(self.xs.stride(0)),
                                             _i64(self.xs.stride(1)), _vp(self.ids.data_ptr()), _vp(self.pos.data_ptr()),
                                             _i64(self.n_pairs), self.top_k, self.E_local, self.H, self.cap,
                                             _i64(self.pitch), self.rank, self.world, st))
                self._barrier(st)
                mark("dispatch+barrier")
                self.gemm1()
                mark("gate_up_gemm")
            if not self.fuse_act:
                _lib.check(L.moe_silu_mul_requant(_vp(self.g1.data_ptr()), _vp(self.a2.data_ptr()), _vp(self.s2.data_ptr()),
                                                  _i64(1), _i64(self.cap), _vp(self.layout.data_ptr()), _i32(self.cap),
                                                  _i32(self.I), _i32(1 if self.gate_first else 0), st))
                mark("silu_mul_requant")
            self.gemm2()
            mark("down_gemm")
            self._barrier(st)
            if self.combine == "push":
                _lib.check(L.moe_combine(_vp(self.y_t.data_ptr()), _vp(self.slot_pos.data_ptr()),
                                         _vp(self.weights.data_ptr()), _vp(self.out.data_ptr()), _i32(self.T),
                                         _i32(self.top_k), _i32(self.H), st))
            else:
                _lib.check(L.moe_ep_combine(P, _vp(self.ids.data_ptr()), _vp(self.pos.data_ptr()),
                                            _vp(self.weights.data_ptr()), _vp(self.out.data_ptr()), self.T, self.top_k,
                                            self.E_local, self.H, self.world, st))
            mark("barrier+combine")
        return self.out

    def stage_times(self, steps: int = 5) -> dict:
        """Median device time of every stage in ms (CUDA events between the stages; collective: all ranks call)."""
        acc: dict = {}
        for _ in range(steps):
            marks: list = []
            self(marks)
            torch.cuda.synchronize(self.device)
            for (_, e0), (name, e1) in zip(marks[:-1], marks[1:]):
                acc.setdefault(name, []).append(e0.elapsed_time(e1))
        return {k: sorted(v)[len(v) // 2] for k, v in acc.items()}

    def close(self):
        self.symm.close()


def setup(data: dict, T_local: int, **kw) -> EpMoeLayer:
    return EpMoeLayer(data, T_local, **kw)
