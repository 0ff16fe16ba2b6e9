"""Expert-parallel layer on GPUs: world size 1 in-process, world size 2 (and 4) as torchrun children."""
import os
import subprocess
import sys

import pytest
import torch

from tests.conftest import ROOT

pytestmark = pytest.mark.gpu


def test_ep_layer_world1_matches_single_gpu_layer():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from tests import ep_worker
    ep_worker.run(T=384, H=256, I=128, E=8, top_k=2, seed=11, steps=2, combine="push")
    ep_worker.run(T=384, H=256, I=128, E=8, top_k=2, seed=12, steps=2, combine="pull")
    ep_worker.run(T=384, H=256, I=128, E=8, top_k=2, seed=13, steps=2, combine="push", dispatch="kernel")
    ep_worker.run(T=1000, H=512, I=256, E=32, top_k=4, seed=14, steps=3, combine="push")      # many experts, ragged tail


@pytest.mark.parametrize("combine,dispatch", [("push", "fused"), ("pull", "fused"), ("push", "kernel")])
@pytest.mark.parametrize("world", [2, 4])
def test_ep_layer_multi_gpu(world, combine, dispatch):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", EP_COMBINE=combine, EP_DISPATCH=dispatch)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29511 + world), os.path.join(ROOT, "tests", "ep_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert r.stdout.count("EP layer ok") == world


def test_barrier_wait_runs_out_and_reports_instead_of_hanging():
    """A peer that never publishes its flag: with the wait limit set to a few milliseconds the barrier kernel
    returns, the device status word carries the peer-flag timeout bit, the status clears, and the device keeps
    working.  (The failing side is made on the host: rank 1's slot is a buffer of this process that nothing
    writes; no fault, no trap, no endless loop.)"""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ctypes
    import time
    from tirx_harness_b200 import _lib, grouped_gemm
    L = _lib.lib()
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")        # this rank's flag slots (slot 1 is never written)
    other = torch.zeros(64, dtype=torch.int32, device="cuda")       # stands in for the absent peer's buffer
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    peers = _lib.EpPeers()
    for r, flags in enumerate((mine, other)):
        peers.a[r] = peers.sa[r] = peers.y[r] = peers.counts[r] = peers.meta[r] = dummy.data_ptr()
        peers.flags[r] = flags.data_ptr()
    assert grouped_gemm.device_status() == 0
    old = _lib.set_option(_lib.OPT_EP_WAIT_LIMIT_MS, 5)
    try:
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        t0 = time.perf_counter()
        _lib.check(L.moe_ep_barrier(ctypes.byref(peers), 0, 2, 1, st))
        out = ctypes.c_int32(0)
        rc = L.moe_device_status(ctypes.byref(out), st)              # synchronises the stream
        waited = time.perf_counter() - t0
    finally:
        _lib.set_option(_lib.OPT_EP_WAIT_LIMIT_MS, old)
    assert rc == -3 and out.value == 1 << 4, (rc, out.value)          # MOE_ERR_DEVICE, STATUS_TIMEOUT_PEER_FLAG
    assert waited < 1.0, waited
    assert int(other[0].item()) == 1                                 # our own epoch was published before the wait
    assert grouped_gemm.device_status() == 0                         # read-and-clear: the word is clean again
    # the context is intact: a barrier of a world of one completes at once, and ordinary work runs
    _lib.check(L.moe_ep_barrier(ctypes.byref(peers), 0, 1, 2, st))
    assert grouped_gemm.device_status() == 0
    assert int((torch.arange(8, device="cuda") * 2).sum().item()) == 56
    with pytest.raises(_lib.B200MoeError):
        _lib.set_option(_lib.OPT_EP_WAIT_LIMIT_MS, 0)
