"""Candidate `b200` of the registered workload alphamoe (mlc-ai/TIRx-harness: evolution/tasks/alphamoe.yaml:17-47;
bound by evolution/benchmark/flashinfer_bench_evolve/tasks/alphamoe/benchmark.py `tirx_prepare`: nine inputs plus the
zero-initialised bf16 `output`).

    run = setup(data, M)      # untimed: allocates the workspace
    run()                     # timed and graph-capturable: 1x128 quantisation of the bf16 tokens, both projections, the
                              # activation and the bf16 accumulation chain of the task, from the current inputs

Everything runs in the CUDA library behind tirx_harness_b200.alpha_moe (C ABI `moe_alpha_forward`).
"""


def _module(name):
    """Imports tirx_harness_b200.<name>.  The benchmark server ships only the bytes of this file, so the package (with its
    built libb200moe.so) must already be on the worker: importable as is, under $B200MOE_ROOT, or in a parent
    folder of this file (a checkout that holds candidates/ beside tirx_harness_b200/)."""
    import importlib
    import os
    import sys
    try:
        return importlib.import_module("tirx_harness_b200." + name)
    except ImportError:
        pass
    roots = [os.environ.get("B200MOE_ROOT")]
    here = os.path.dirname(os.path.abspath(__file__))
    for _ in range(6):
        here = os.path.dirname(here)
        roots.append(here)
    for root in roots:
        if root and os.path.isdir(os.path.join(root, "tirx_harness_b200")):
            if root not in sys.path:
                sys.path.insert(0, root)
            return importlib.import_module("tirx_harness_b200." + name)
    raise ImportError("tirx_harness_b200 not found: set B200MOE_ROOT to the folder that holds it")


def setup(data, M):
    return _module("alpha_moe").setup(data, int(M))
