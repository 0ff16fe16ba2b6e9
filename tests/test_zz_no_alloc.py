"""moe_permute_plan_static: the permutation plan for callers that cannot hand the library scratch memory.

A serving process that has given all of its GPU memory to its own pool has nothing left for this
library to allocate from.  This entry point keeps the plan's per-chunk counters in an array that is
part of the library itself, so the call allocates nothing.  The test drives it through the C ABI and
requires every integer output to equal what moe_permute_plan (caller-provided workspace) produces,
twice in a row with different routes, so that counters left in the built-in array by the first call
cannot leak into the second.  It runs last so that a failure here never hides another test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64


def _plan_static(L, ids, e_lo, e_local, align, cap, n_pairs=None):
    dev = ids.device
    n_pairs = ids.numel() if n_pairs is None else n_pairs
    out = dict(counts=torch.full((e_local,), -7, dtype=torch.int32, device=dev),
               offsets=torch.full((e_local + 1,), -7, dtype=torch.int32, device=dev),
               pos=torch.full((max(n_pairs, 1),), -7, dtype=torch.int32, device=dev).view(ids.shape if n_pairs else (1,)),
               src_pair=torch.full((cap,), -7, dtype=torch.int32, device=dev),
               grouped_layout=torch.full((cap,), -7, dtype=torch.int32, device=dev))
    rc = L.moe_permute_plan_static(_vp(ids.data_ptr()), _i64(n_pairs), _i32(e_lo), _i32(e_local), _i32(align),
                                   _i32(cap), _vp(out["counts"].data_ptr()), _vp(out["offsets"].data_ptr()),
                                   _vp(out["pos"].data_ptr()), _vp(out["src_pair"].data_ptr()),
                                   _vp(out["grouped_layout"].data_ptr()),
                                   _vp(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_static_plan_matches_workspace_plan_on_two_calls_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tirx_harness_b200 import _lib, grouped_gemm, moe_ops
    L = _lib.lib()
    gen = torch.Generator().manual_seed(123)
    cases = [(3000, 64, 0, 64, 8), (777, 256, 32, 32, 8)]          # second call: other sizes, other routes
    for T, e_glob, e_lo, e_loc, top_k in cases:
        ids = torch.stack([torch.randperm(e_glob, generator=gen)[:top_k] for _ in range(T)]).int().cuda()
        ref = moe_ops.permute_plan(ids, e_lo, e_loc, 128)
        rc, got = _plan_static(L, ids, e_lo, e_loc, 128, ref["cap_rows"])
        assert rc == 0, L.moe_last_error().decode()
        assert grouped_gemm.device_status() == 0
        for k in ("counts", "offsets", "pos", "src_pair", "grouped_layout"):
            assert torch.equal(got[k], ref[k]), k                  # integer outputs: exact
    # an empty batch right after a full one: the counters the earlier calls left in the built-in array are never read
    unused = torch.zeros((1, 8), dtype=torch.int32, device="cuda")           # a valid pointer; no pair is read
    rc, got = _plan_static(L, unused, 0, 16, 128, 16 * 128, n_pairs=0)
    assert rc == 0, L.moe_last_error().decode()
    assert grouped_gemm.device_status() == 0
    assert not got["counts"].any() and not got["offsets"].any()
    assert (got["grouped_layout"] == -1).all() and (got["src_pair"] == -1).all()


def test_static_plan_rejects_requests_beyond_its_built_in_scratch():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tirx_harness_b200 import _lib
    L = _lib.lib()
    T, top_k, e = 20000, 8, 256                                    # 157 chunks x 256 experts > 32768 counters
    ids = torch.randint(0, e, (T, top_k), dtype=torch.int32, device="cuda")
    rc, got = _plan_static(L, ids, 0, e, 128, T * top_k + e * 128)
    assert rc != 0 and b"exceeds the built-in scratch" in L.moe_last_error()
    assert (got["pos"] == -7).all()                                 # outputs untouched
