"""Regenerates the golden fixtures in this folder from the reference checkout.

Run once on a machine that has a checkout of the reference; pass its path as the first argument
(or set TIRX_HARNESS_REF):

    python tests/golden/make_golden.py [REF]

It imports the reference's own Python oracles (NumPy codec helpers of
tools/tests/numsim/corpus/kernels/gemm.py, the hardware cvt goldens of
tools/tests/numsim/microtests/cases/ptx_cvt_fp8_goldens.py and the torch oracle
of the alphamoe task definition) and stores inputs together with the outputs
THEY produce.  The tests then compare this repository's CPU oracle (and through
it the CUDA kernels) against these files; nothing at test time reads the
reference checkout.
"""
from __future__ import annotations

import json
import os
import sys
import types

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TIRX_HARNESS_REF", "reference")
OUT = os.path.dirname(os.path.abspath(__file__))


def _load_gemm_helpers():
    """Execute the reference's corpus module with its third-party imports stubbed
    (tirx-kernels and the simulator bindings are absent; only plain NumPy helpers
    are used)."""
    class _Any:
        def __init__(self, *a, **k): pass
        def __getattr__(self, name): return _Any()
        def __call__(self, *a, **k): return _Any()
        def __getitem__(self, k): return _Any()
        def __iter__(self): return iter(())

    stubs = {
        "tests": types.ModuleType("tests"),
        "tests.numsim": types.ModuleType("tests.numsim"),
        "tests.numsim.support": types.ModuleType("tests.numsim.support"),
        "tests.numsim.support._tirx_kernels": types.ModuleType("tests.numsim.support._tirx_kernels"),
        "tirx_harness": types.ModuleType("tirx_harness"),
        "tirx_harness.numsim": types.ModuleType("tirx_harness.numsim"),
        "tirx_harness.numsim.cases": types.ModuleType("tirx_harness.numsim.cases"),
    }
    stubs["tests.numsim.support._tirx_kernels"].load_tirx_kernel = lambda name: _Any()
    for n in ("ComparisonRegion", "ComparisonSpec", "NumSimCase", "TensorMap"):
        setattr(stubs["tirx_harness.numsim.cases"], n, _Any)
    saved = {k: sys.modules.get(k) for k in stubs}
    sys.modules.update(stubs)
    try:
        path = os.path.join(REF, "tools/tests/numsim/corpus/kernels/gemm.py")
        mod = types.ModuleType("_ref_gemm")
        mod.__file__ = path
        exec(compile(open(path).read(), path, "exec"), mod.__dict__)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return mod


def cvt_goldens():
    sys.path.insert(0, os.path.join(REF, "tools/tests/numsim/microtests/cases"))
    import ptx_cvt_fp8_goldens as g
    np.savez_compressed(os.path.join(OUT, "cvt_e4m3x2_f32.npz"),
                        f32_source=g.F32_SOURCE.astype(np.uint32),
                        e4m3x2_f32=g.GOLDENS["e4m3x2.f32"].astype(np.uint16))


def codec_and_gemm(ref):
    # full decode table + encodes of a dense sweep, by the reference's codecs
    all_bits = np.arange(256, dtype=np.uint8)
    rng = np.random.default_rng(77)
    sweep = np.concatenate([
        np.linspace(-500, 500, 4001, dtype=np.float32),
        (rng.standard_normal(4096) * np.exp2(rng.integers(-12, 9, 4096))).astype(np.float32),
        np.array([0.0, -0.0, 2**-10, 2**-9, 3 * 2**-10, 448, 464, 465, 480, np.inf, -np.inf, np.nan],
                 dtype=np.float32),
    ])
    bf_in = (rng.standard_normal(4096) * np.exp2(rng.integers(-20, 20, 4096))).astype(np.float32)
    np.savez_compressed(
        os.path.join(OUT, "codecs.npz"),
        e4m3_all_decoded=ref._e4m3fn_bits_to_float32(all_bits),
        e4m3_sweep=sweep, e4m3_sweep_bits=ref._float32_to_e4m3fn_bits(sweep),
        e8m0_all_decoded=ref._e8m0_bits_to_float32(all_bits),
        bf16_in=bf_in, bf16_bits=ref._float32_to_bfloat16_bits(bf_in),
    )
    # the two FP8 block-scaled corpus cases (gemm.py:74-91, 407-446): inputs drawn exactly as
    # prepare_fp8_blockwise_case draws them, expectation by _fp8_blockwise_reference
    for (M, N, K, seed) in ((16, 256, 512, 2800), (512, 608, 512, 2801)):
        rng = np.random.default_rng(seed)
        operand_values = np.array([-2.0, -1.5, -1.0, -0.5, 0.0, 0.5, 1.0, 1.5, 2.0])
        codes = ref._float32_to_e4m3fn_bits(operand_values)
        A = rng.choice(codes, size=(M, K)).astype(np.uint8)
        B = rng.choice(codes, size=(N, K)).astype(np.uint8)
        kb = K // 128
        sfa_bits = ref._e8m0_bits_from_exponents(rng.integers(-1, 2, size=(M, kb), dtype=np.int16))
        sfb_bits = ref._e8m0_bits_from_exponents(rng.integers(-1, 2, size=(N, kb), dtype=np.int16))
        SFA, SFB = ref._pack_e8m0_scales(sfa_bits), ref._pack_e8m0_scales(sfb_bits)
        D = ref._fp8_blockwise_reference(A, B, SFA, SFB)
        np.savez_compressed(os.path.join(OUT, f"fp8_blockwise_seed{seed}.npz"),
                            A=A, B=B, SFA=SFA, SFB=SFB, D=D)
    # block-scale-per-128 known answer (test_fp8_blockwise_gemm_case.py:115-125)
    one = int(ref._float32_to_e4m3fn_bits(np.array([1.0], dtype=np.float32))[0])
    A = np.full((1, 512), one, np.uint8)
    SFA = ref._pack_e8m0_scales(ref._e8m0_bits_from_exponents([[0, 1, -1, 2]]))
    SFB = ref._pack_e8m0_scales(ref._e8m0_bits_from_exponents([[0, -1, 1, -2]]))
    np.savez_compressed(os.path.join(OUT, "fp8_one_scale_per_128.npz"), A=A, B=A.copy(), SFA=SFA,
                        SFB=SFB, D=ref._fp8_blockwise_reference(A, A, SFA, SFB))
    # a block-scaled case in THIS repo's scale format (A: 1x128 per row, B: 128x128 blocks) that the
    # reference oracle can still express: B's per-row scales are constant inside each 128-row block
    rng = np.random.default_rng(2900)
    M, N, K = 192, 384, 1024
    A = rng.choice(codes, size=(M, K)).astype(np.uint8)
    B = rng.choice(codes, size=(N, K)).astype(np.uint8)
    kb = K // 128
    ea = rng.integers(-4, 1, size=(M, kb), dtype=np.int16)
    eb_blk = rng.integers(-4, 1, size=(N // 128, kb), dtype=np.int16)
    eb = np.repeat(eb_blk, 128, axis=0)
    SFA = ref._pack_e8m0_scales(ref._e8m0_bits_from_exponents(ea))
    SFB = ref._pack_e8m0_scales(ref._e8m0_bits_from_exponents(eb))
    np.savez_compressed(os.path.join(OUT, "fp8_block128_seed2900.npz"), A=A, B=B,
                        sfa=np.exp2(ea).astype(np.float32), sfb=np.exp2(eb_blk).astype(np.float32),
                        D=ref._fp8_blockwise_reference(A, B, SFA, SFB))


def alphamoe_oracle():
    import torch
    d = json.load(open(os.path.join(
        REF, "evolution/benchmark/flashinfer_bench_evolve/tasks/alphamoe/definition.json")))
    ns: dict = {}
    exec(compile(d["reference"], "alphamoe/definition.json:reference", "exec"), ns)
    torch.manual_seed(5)
    # (1) per-token 1x128 quantisation rule
    x = (torch.randn(48, 512) * torch.exp2(torch.randint(-6, 6, (48, 1)).float())).float()
    x[3, 128:256] = 0.0            # an all-zero block hits the 1e-8 clamp
    q, s = ns["_quantize_per_token_group"](x)
    # (2) silu(gate)*up then requant, on bf16-representable gate_up
    gu = (torch.randn(40, 512) * 3).bfloat16()
    inter = 256
    act = torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()
    aq, asc = ns["_quantize_per_token_group"](act)
    # (3) a tiny routed layer through _reference_quantized
    T, H, I, E, top_k = 24, 128, 128, 4, 2
    hs = torch.randn(T, H).bfloat16()
    xq, xs = ns["_quantize_per_token_group"](hs)

    def qw(shape):
        w = torch.randn(*shape) * 0.5
        blocks = w.reshape(shape[0], shape[1] // 128, 128, shape[2] // 128, 128)
        sc = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-8) / 448.0
        wq = (blocks / sc[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
        return wq.reshape(shape), sc.float()
    w13, s13 = qw((E, 2 * I, H))
    w2, s2 = qw((E, H, I))
    ids = torch.stack([torch.randperm(E)[:top_k] for _ in range(T)]).int()
    tw = torch.rand(T, top_k).float()
    tw = tw / tw.sum(dim=1, keepdim=True)
    out, abs_sum = ns["_reference_quantized"](xq, xs, ids, tw, w13, s13, w2, s2, top_k, 1.0)
    u8 = lambda t: t.view(torch.uint8).numpy()
    np.savez_compressed(
        os.path.join(OUT, "alphamoe_oracle.npz"),
        quant_x=x.numpy(), quant_q=u8(q), quant_s=s.numpy(),
        act_gate_up_bits=gu.view(torch.int16).numpy().view(np.uint16), act_q=u8(aq), act_s=asc.numpy(),
        layer_xq=u8(xq), layer_xs=xs.numpy(), layer_ids=ids.numpy(), layer_w=tw.numpy(),
        layer_w13=u8(w13), layer_s13=s13.numpy(), layer_w2=u8(w2), layer_s2=s2.numpy(),
        layer_out_bits=out.view(torch.int16).numpy().view(np.uint16), layer_abs_sum=abs_sum.numpy(),
    )


def alphamoe_bf16_layer():
    """The alphamoe task's full operator (`run` of its definition.json: bf16 activations quantised inside,
    preselected routes, expert-order bf16 accumulation) on a small case with a non-trivial
    routed_scaling_factor; stores the inputs and what the reference returns."""
    import torch
    d = json.load(open(os.path.join(
        REF, "evolution/benchmark/flashinfer_bench_evolve/tasks/alphamoe/definition.json")))
    ns: dict = {}
    exec(compile(d["reference"], "alphamoe/definition.json:reference", "exec"), ns)
    torch.manual_seed(11)
    M, H, I, E, top_k, rsf = 12, 256, 128, 8, 3, 2.5
    hs = (torch.randn(M, H) * torch.exp2(torch.randint(-2, 3, (M, 1)).float())).bfloat16()

    def qw(shape):
        w = torch.randn(*shape) * 0.5
        blocks = w.reshape(shape[0], shape[1] // 128, 128, shape[2] // 128, 128)
        sc = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-8) / 448.0
        wq = (blocks / sc[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
        return wq.reshape(shape), sc.float()
    w13, s13 = qw((E, 2 * I, H))
    w2, s2 = qw((E, H, I))
    ids = torch.stack([torch.randperm(E)[:top_k] for _ in range(M)]).int()
    tw = torch.rand(M, top_k).float()
    tw = tw / tw.sum(dim=1, keepdim=True)
    out, bound = ns["reference_for_check"](hs, ids, tw, w13, s13, w2, s2, top_k, rsf)
    xq, xs = ns["_quantize_inputs"](hs)
    _, abs_sum = ns["_reference_quantized"](xq, xs, ids, tw, w13, s13, w2, s2, top_k, rsf)
    u8 = lambda t: t.view(torch.uint8).numpy()
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(
        os.path.join(OUT, "alphamoe_bf16_layer.npz"),
        hidden_bits=bits(hs), ids=ids.numpy(), w=tw.numpy(), w13=u8(w13), s13=s13.numpy(), w2=u8(w2), s2=s2.numpy(),
        rsf=np.float32(rsf), xq=u8(xq), xs=xs.numpy(), out_bits=bits(out), bound=bound.numpy(), abs_sum=abs_sum.numpy(),
    )


def moe_routing():
    """Runs the routing block of the reference's `moe` task oracle (definition.json, between the markers
    "# 2) No-aux routing" and "# 3) Local expert compute") on random logits and stores what it selects."""
    import torch
    d = json.load(open(os.path.join(
        REF, "evolution/benchmark/flashinfer_bench_evolve/tasks/moe/definition.json")))
    src = d["reference"]
    a = src.index("    # 2) No-aux routing")
    b = src.index("    # 3) Local expert compute")
    block = "\n".join(line[4:] if line.startswith("    ") else line for line in src[a:b].splitlines())
    torch.manual_seed(9)
    T, E = 96, 256
    ns = dict(torch=torch, routing_logits=torch.randn(T, E) * 2.0,
              routing_bias=(torch.randn(E) * 0.1).bfloat16(), T=T, E_global=E, N_GROUP=8, TOPK_GROUP=4, TOP_K=8,
              routed_scaling_factor=2.5)
    exec(compile(block, "moe/definition.json:routing", "exec"), ns)
    idx = torch.sort(ns["topk_idx"], dim=1).values.int().numpy()
    np.savez_compressed(os.path.join(OUT, "moe_routing.npz"), logits=ns["routing_logits"].numpy(),
                        bias=ns["routing_bias"].float().numpy(), topk_idx_sorted=idx,
                        weights_dense=ns["weights"].numpy(), rsf=np.float32(2.5))


def moe_task_layer():
    """Runs the registered `moe` task's own operator (`run` of tasks/moe/definition.json, fixed DeepSeek-V3 geometry)
    on the seeded inputs of tests/util.py:moe_task_inputs and stores what it returns; the inputs themselves (1.4 GB of
    weights) are regenerated from the seed by the tests."""
    import torch
    sys.path.insert(0, os.path.dirname(os.path.dirname(OUT)))
    from tests.util import moe_task_inputs
    d = json.load(open(os.path.join(
        REF, "evolution/benchmark/flashinfer_bench_evolve/tasks/moe/definition.json")))
    ns: dict = {}
    exec(compile(d["reference"], "moe/definition.json:reference", "exec"), ns)
    T, seed = 16, 2024
    x = moe_task_inputs(T, seed)
    fp8 = lambda a: torch.from_numpy(a).view(torch.float8_e4m3fn)
    out = ns["run"](torch.from_numpy(x["routing_logits"]), torch.from_numpy(x["routing_bias"]).bfloat16(),
                    fp8(x["hidden_states"]), torch.from_numpy(x["hidden_states_scale"]),
                    fp8(x["gemm1_weights"]), torch.from_numpy(x["gemm1_weights_scale"]),
                    fp8(x["gemm2_weights"]), torch.from_numpy(x["gemm2_weights_scale"]),
                    x["local_expert_offset"], x["routed_scaling_factor"])
    import hashlib
    digest = hashlib.sha256(b"".join(np.ascontiguousarray(x[k]).tobytes() for k in (
        "routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights_scale",
        "gemm2_weights_scale"))).hexdigest()
    np.savez_compressed(os.path.join(OUT, "moe_task_layer.npz"), T=np.int32(T), seed=np.int32(seed),
                        out_bits=out.view(torch.int16).numpy().view(np.uint16),
                        small_inputs_sha256=np.frombuffer(bytes.fromhex(digest), np.uint8))


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2] == "moe_task_layer":     # 20 GB of host memory, half a minute
        moe_task_layer()
        raise SystemExit
    ref = _load_gemm_helpers()
    moe_routing()
    cvt_goldens()
    codec_and_gemm(ref)
    alphamoe_oracle()
    alphamoe_bf16_layer()
    moe_task_layer()
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(OUT, f)))
