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


@pytest.mark.parametrize("combine", ["push", "pull"])
@pytest.mark.parametrize("world", [2, 4])
def test_ep_layer_multi_gpu(world, combine):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", EP_COMBINE=combine)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29511 + world), os.path.join(ROOT, "tests", "ep_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert r.stdout.count("EP layer ok") == world
