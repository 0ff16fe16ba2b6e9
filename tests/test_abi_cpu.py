"""The C-ABI library loads without a GPU and exports every symbol include/b200moe.h declares."""
import ctypes
import os
import re

from tests.conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"^(?:int|size_t|const char\*)\s+(moe_\w+)\s*\(", text, flags=re.M)))


def test_header_declares_the_hot_path_entry_points():
    names = _declared()
    for required in ("moe_gg_fp8_contiguous", "moe_gg_fp8_masked", "moe_silu_mul_requant", "moe_route_topk",
                     "moe_permute", "moe_combine", "moe_layer_forward", "moe_workspace_bytes", "moe_last_error"):
        assert required in names


def test_library_builds_loads_and_exports_all_declared_symbols():
    from tirx_harness_b200 import _lib, build
    build.build_library()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in b200moe.h but not exported"
    assert sorted(_lib.EXPORTS) == sorted(n for n in _declared() if n in _lib.EXPORTS)
    missing = [n for n in _declared() if n not in _lib.EXPORTS]
    assert not missing, f"declared but not bound in _lib.EXPORTS: {missing}"
    lib.moe_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.moe_version()


def test_struct_layouts_match_header_field_order():
    from tirx_harness_b200 import _lib
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    for cname, pystruct in (("moe_gg_args", _lib.GGArgs), ("moe_layer_args", _lib.LayerArgs),
                            ("moe_layer_view", _lib.LayerView), ("moe_ep_peers", _lib.EpPeers),
                            ("moe_alpha_args", _lib.AlphaArgs), ("moe_alpha_view", _lib.AlphaView),
                            ("moe_kg_args", _lib.KgArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = decl.split(None, 1)[1] if not decl.startswith("const") else decl.split(None, 2)[2]
            fields += [re.sub(r"\[\d+\]$", "", n.strip().lstrip("*").strip()) for n in names.split(",")]
        assert fields == [f[0] for f in pystruct._fields_], cname


def test_workspace_size_is_monotonic_and_cpu_callable():
    from tirx_harness_b200 import _lib
    L = _lib.lib()
    a = L.moe_workspace_bytes(128, 256, 256, 4, 2, 128)
    b = L.moe_workspace_bytes(256, 256, 256, 4, 2, 128)
    assert 0 < a < b
    assert L.moe_workspace_bytes(-1, 256, 256, 4, 2, 128) == 0
    assert L.moe_permute_workspace_bytes(ctypes.c_int64(4096), 32) >= 4 * 32 * 4
    # decode-regime layer: the workspace grows with the token count, not with it times the expert count squared
    small, big = L.moe_alpha_workspace_bytes(1, 2048, 128, 512, 10), L.moe_alpha_workspace_bytes(128, 2048, 128, 512, 10)
    assert 0 < small < big < (1 << 30)
    assert L.moe_alpha_workspace_bytes(8, 0, 128, 512, 10) == 0
    # k-grouped layout: K-major copies of both operands plus the scale tiles of the largest possible group
    kg = L.moe_kg_workspace_bytes(256, 384, ctypes.c_int64(1024))
    assert kg >= (256 + 384) * 1024
    assert L.moe_kg_workspace_bytes(256, 384, ctypes.c_int64(1000)) == 0          # K_total must be a multiple of 128
