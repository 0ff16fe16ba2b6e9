"""Candidate `b200` of the registered workload grouped_gemm/fp8 (mlc-ai/TIRx-harness:
evolution/tasks/grouped_gemm_fp8.yaml:15-25; loaded by evolution/benchmark/adapter.py `load_solution`, called by
evolution/benchmark/flashinfer_bench_evolve/tasks/grouped_gemm_fp8/benchmark.py `tirx_prepare`).

    launch = setup(inputs, G, M, N, K)      # untimed; inputs: A, B, SFA, SFB, D, grouped_layout, actual_ms, ...
    launch()                                # timed; recomputes D in place from the current inputs

The arithmetic runs in hand-written sm_100a CUDA (block-scaled tcgen05 MMA on CTA pairs) reached through the C ABI of
libb200moe.so; this file only binds the harness's tensors to it.
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


def setup(data, G, M, N, K):
    return _module("grouped_gemm").setup(data, int(G), int(M), int(N), int(K))
