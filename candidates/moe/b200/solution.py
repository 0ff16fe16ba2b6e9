"""Candidate `b200` of the registered workload moe (mlc-ai/TIRx-harness: evolution/tasks/moe.yaml:29-42; bound by
evolution/benchmark/flashinfer_bench_evolve/tasks/moe/benchmark.py `tirx_prepare`: the ten inputs by name plus the
preallocated bf16 `output`).

    run = setup(data, seq_len)      # untimed: allocates the workspace, binds pointers
    run()                           # timed: DeepSeek-V3 routing, permutation, both grouped GEMMs, SiLU*mul FP8 requant
                                    # and the weighted combine of the local experts, from the current inputs

Everything runs in the CUDA library behind tirx_harness_b200.moe_layer (C ABI `moe_layer_forward`).
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


def setup(data, seq_len):
    return _module("moe_layer").setup(data, int(seq_len))
