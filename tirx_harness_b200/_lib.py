"""ctypes binding of the C ABI in ``include/b200moe.h``.

There is no fallback: if the CUDA library has not been built the import of any operator fails
with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200moe.so")

_c = ctypes


class GGArgs(_c.Structure):
    """``moe_gg_args`` of include/b200moe.h."""
    _fields_ = [
        ("a", _c.c_void_p), ("b", _c.c_void_p), ("sfa", _c.c_void_p),
        ("sfa_stride_row", _c.c_int64), ("sfa_stride_kblk", _c.c_int64),
        ("sfb", _c.c_void_p), ("layout", _c.c_void_p), ("d", _c.c_void_p), ("ldd", _c.c_int64),
        ("G", _c.c_int32), ("M", _c.c_int32), ("N", _c.c_int32), ("K", _c.c_int32),
        ("d_dtype", _c.c_int32), ("rows_used", _c.c_void_p),
        ("workspace", _c.c_void_p), ("workspace_bytes", _c.c_uint64),
        ("scatter_meta", _c.c_void_p), ("scatter_base", _c.c_void_p * 8),
        ("sf_format", _c.c_int32), ("sfb_stride", _c.c_int64 * 3), ("lda", _c.c_int64),
        ("ldb", _c.c_int64), ("accumulate", _c.c_int32), ("scatter_meta_stride", _c.c_int64),
        ("mx_tile", _c.c_int32),
    ]


class LayerArgs(_c.Structure):
    """``moe_layer_args`` of include/b200moe.h."""
    _fields_ = [
        ("x_q", _c.c_void_p), ("x_scale", _c.c_void_p), ("xs_stride_row", _c.c_int64), ("xs_stride_blk", _c.c_int64),
        ("logits", _c.c_void_p), ("topk_ids", _c.c_void_p), ("topk_weights", _c.c_void_p),
        ("w13", _c.c_void_p), ("w13_scale", _c.c_void_p), ("w2", _c.c_void_p), ("w2_scale", _c.c_void_p),
        ("out", _c.c_void_p), ("workspace", _c.c_void_p), ("workspace_bytes", _c.c_uint64),
        ("T", _c.c_int32), ("H", _c.c_int32), ("I", _c.c_int32), ("E", _c.c_int32), ("E_global", _c.c_int32),
        ("e_lo", _c.c_int32), ("top_k", _c.c_int32), ("align", _c.c_int32), ("gate_first", _c.c_int32),
        ("fuse_act", _c.c_int32), ("routing_bias", _c.c_void_p), ("n_group", _c.c_int32), ("topk_group", _c.c_int32),
        ("routed_scaling_factor", _c.c_float),
    ]


class LayerView(_c.Structure):
    """``moe_layer_view`` of include/b200moe.h."""
    _fields_ = [(n, _c.c_void_p) for n in ("ids", "counts", "offsets", "pos", "src_pair", "grouped_layout",
                                           "weights", "s1", "s2", "a1", "g1", "a2", "y")] + [("cap_rows", _c.c_int64)]


class KgArgs(_c.Structure):
    """``moe_kg_args`` of include/b200moe.h."""
    _fields_ = [
        ("a", _c.c_void_p), ("b", _c.c_void_p), ("sfa", _c.c_void_p), ("sfb", _c.c_void_p), ("d", _c.c_void_p),
        ("ks", _c.POINTER(_c.c_int32)), ("G", _c.c_int32), ("M", _c.c_int32), ("N", _c.c_int32), ("K_total", _c.c_int64),
        ("workspace", _c.c_void_p), ("workspace_bytes", _c.c_uint64),
    ]


class AlphaArgs(_c.Structure):
    """``moe_alpha_args`` of include/b200moe.h."""
    _fields_ = [
        ("hidden", _c.c_void_p), ("topk_ids", _c.c_void_p), ("topk_weights", _c.c_void_p),
        ("w13", _c.c_void_p), ("w13_scale", _c.c_void_p), ("w2", _c.c_void_p), ("w2_scale", _c.c_void_p),
        ("out", _c.c_void_p),
        ("M", _c.c_int32), ("H", _c.c_int32), ("I", _c.c_int32), ("E", _c.c_int32), ("top_k", _c.c_int32),
        ("routed_scaling_factor", _c.c_float), ("workspace", _c.c_void_p), ("workspace_bytes", _c.c_uint64),
    ]


class AlphaView(_c.Structure):
    """``moe_alpha_view`` of include/b200moe.h."""
    _fields_ = [(n, _c.c_void_p) for n in ("counts", "rowpos", "s1", "s2", "g1", "d2", "a1", "a2")] + [("max_m", _c.c_int64)]


class EpPeers(_c.Structure):
    """``moe_ep_peers`` of include/b200moe.h."""
    _fields_ = [("a", _c.c_void_p * 8), ("sa", _c.c_void_p * 8), ("y", _c.c_void_p * 8),
                ("counts", _c.c_void_p * 8), ("flags", _c.c_void_p * 8), ("meta", _c.c_void_p * 8)]


class EpSendArgs(_c.Structure):
    """``moe_ep_send_args`` of include/b200moe.h."""
    _fields_ = [("peers", _c.POINTER(EpPeers)), ("x_q", _c.c_void_p), ("x_scale", _c.c_void_p),
                ("xs_row", _c.c_int64), ("xs_blk", _c.c_int64), ("ids", _c.c_void_p), ("pos", _c.c_void_p),
                ("send_order", _c.c_void_p), ("counts_local", _c.c_void_p), ("n_pairs", _c.c_int64), ("pitch", _c.c_int64),
                ("top_k", _c.c_int32), ("E_local", _c.c_int32), ("H", _c.c_int32), ("cap_rows", _c.c_int32),
                ("rank", _c.c_int32), ("world", _c.c_int32)]


class B200MoeError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200MoeError(
                f"{LIB_PATH} is missing: build it with `python -m tirx_harness_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.moe_last_error.restype = _c.c_char_p
        _lib.moe_version.restype = _c.c_char_p
        for name in EXPORTS:
            fn = getattr(_lib, name)      # raises AttributeError if the symbol is absent
            if name in _SIZE_T_RETURN:
                fn.restype = _c.c_size_t
            elif name not in ("moe_last_error", "moe_version"):
                fn.restype = _c.c_int
    return _lib


# every symbol include/b200moe.h declares
EXPORTS = (
    "moe_gg_fp8_contiguous", "moe_gg_fp8_masked", "moe_gg_fp8_gate_up_act", "moe_gg_workspace_bytes", "moe_quant_1x128", "moe_silu_mul_requant",
    "moe_route_topk", "moe_route_deepseek", "moe_permute_workspace_bytes", "moe_permute_plan", "moe_permute_plan_static", "moe_permute",
    "moe_combine",
    "moe_workspace_bytes", "moe_layer_forward", "moe_layer_workspace_view", "moe_device_status",
    "moe_alpha_workspace_bytes", "moe_alpha_forward", "moe_alpha_workspace_view",
    "moe_kg_workspace_bytes", "moe_kg_fp8_contiguous",
    "moe_ipc_alloc", "moe_ipc_free", "moe_ipc_get_handle", "moe_ipc_open", "moe_ipc_close",
    "moe_ep_barrier", "moe_ep_workspace_bytes", "moe_ep_count_publish", "moe_ep_plan", "moe_ep_dispatch",
    "moe_ep_combine", "moe_ep_gate_up_dispatch", "moe_set_option", "moe_get_option",
    "moe_last_error", "moe_version",
)
_SIZE_T_RETURN = ("moe_gg_workspace_bytes", "moe_permute_workspace_bytes", "moe_workspace_bytes", "moe_ep_workspace_bytes",
                  "moe_alpha_workspace_bytes", "moe_kg_workspace_bytes")


# moe_set_option keys and values (include/b200moe.h)
OPT_GG_BLOCK_SCALED, OPT_MX_TILE, OPT_ALPHA_PATH, OPT_ALPHA_GEMV_MAX_ROUTES, OPT_KG_MODE, OPT_EP_WAIT_LIMIT_MS = range(6)
MX_TILE_AUTO, MX_TILE_PAIR, MX_TILE_SINGLE, MX_TILE_PAIR_240, MX_TILE_PAIR_224 = range(5)
ALPHA_PATH_AUTO, ALPHA_PATH_SWAP, ALPHA_PATH_MASKED, ALPHA_PATH_MIXED = range(4)
KG_MODE_MN_MAJOR, KG_MODE_TRANSPOSE, KG_MODE_PER_GROUP = range(3)


def set_option(option: int, value: int) -> int:
    """Sets a process-wide mode and returns the previous value (so a caller can restore it)."""
    old = ctypes.c_int32(0)
    check(lib().moe_get_option(ctypes.c_int32(option), ctypes.byref(old)))
    check(lib().moe_set_option(ctypes.c_int32(option), ctypes.c_int32(value)))
    return old.value


def check(rc: int) -> None:
    if rc != 0:
        raise B200MoeError(f"b200moe error {rc}: {lib().moe_last_error().decode()}")
