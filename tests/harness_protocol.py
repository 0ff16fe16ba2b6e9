"""The reference benchmark server's candidate protocol, restated for the tests (CUDA tensors, no reference import):
how a `solution.py` is loaded, how outputs are poisoned before every checked call, how repeatability is judged and
how inputs are perturbed in place after timing.  Follows mlc-ai/TIRx-harness evolution/benchmark/adapter.py:166-191
(`load_solution`) and evolution/benchmark/flashinfer_bench_evolve/benchmark_common.py:583-588 (`poison_outputs`),
:675-743 (`check_candidate_runs`), :796-865 (`perturb_inputs_`, `input_dependence_check`)."""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import torch

CANDIDATES_ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "candidates")


def load_solution(workload_dir: str, version: str):
    """Imports candidates/<workload_dir>/<version>/solution.py under the module name the adapter gives it
    (`_tirx_<workload with _ for />_<version>.solution`), without package marker files."""
    wdir = os.path.join(CANDIDATES_ROOT, workload_dir)
    path = os.path.join(wdir, version, "solution.py")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    stem = "_".join(part.replace("-", "_") for part in workload_dir.split("/"))
    package_name = f"_tirx_{stem}_{version}"
    module_name = f"{package_name}.solution"
    if package_name not in sys.modules:
        package = types.ModuleType(package_name)
        package.__path__ = [os.path.dirname(path)]
        sys.modules[package_name] = package
    spec = importlib.util.spec_from_file_location(module_name, path, submodule_search_locations=[os.path.dirname(path)])
    module = importlib.util.module_from_spec(spec)
    sys.modules[module_name] = module
    spec.loader.exec_module(module)
    return module


def poison(outputs) -> None:
    """NaN into every floating-point output tensor (views poison only the rows they cover)."""
    for t in ([outputs] if isinstance(outputs, torch.Tensor) else outputs):
        if t.is_floating_point():
            t.fill_(float("nan"))


def checked_runs(run, outputs, compare, runs: int = 3):
    """`runs` consecutive calls on one prepared candidate: poison, call, synchronise, compare; all calls must return
    exactly the same values.  `compare(outputs)` raises or returns False on a mismatch."""
    first = None
    for i in range(runs):
        poison(outputs)
        run()
        torch.cuda.synchronize()
        assert compare(outputs) is not False, f"run {i + 1}/{runs}"
        snap = [t.clone() for t in ([outputs] if isinstance(outputs, torch.Tensor) else outputs)]
        if first is None:
            first = snap
        else:
            for a, b in zip(snap, first, strict=True):
                assert torch.equal(a, b), f"run {i + 1}/{runs}: outputs are not repeatable across identical calls"


def perturb_inputs_(tensors, seed: int) -> None:
    """Noise of a quarter of each tensor's own spread (its magnitude if constant), added in place."""
    for index, tensor in enumerate(tensors):
        values = tensor.float()
        scale = values.std().item() or values.abs().mean().item() or 1.0
        gen = torch.Generator(device=tensor.device).manual_seed(seed + index)
        noise = torch.randn(values.shape, generator=gen, device=tensor.device, dtype=torch.float32)
        tensor.copy_((values + 0.25 * scale * noise).to(tensor.dtype))
