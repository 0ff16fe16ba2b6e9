"""Seeded synthetic inputs for the grouped FP8 GEMM workloads.

Stands in for the reference's input preparation (``prepare_m_grouped_contiguous`` of the un-vendored
tirx-kernels package, called from evolution/benchmark/flashinfer_bench_evolve/tasks/grouped_gemm_fp8/
baseline.py:6-18): operands x ~ N(0,1), one scale s = 2^e per block (A: 1x128 per row, B: 128x128),
stored byte = e4m3(clip(x / s, +-448)); ``grouped_layout`` holds the group id per row and -1 on padding.
Works on CPU or CUDA tensors; the same seed gives the same bytes on either.
"""
from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def draw_scales(shape, gen, law: str = "pow2") -> torch.Tensor:
    """2^U(-4,0): ``pow2`` draws integer exponents {-4..0} (exactly UE8M0-representable),
    ``uniform_exp`` draws real exponents in (-4, 0)."""
    if law == "pow2":
        e = torch.randint(-4, 1, shape, generator=gen).float()
    elif law == "uniform_exp":
        e = torch.rand(shape, generator=gen) * -4.0
    else:
        raise ValueError(law)
    return torch.exp2(e)


def quantize_with_scales(x: torch.Tensor, s_full: torch.Tensor) -> torch.Tensor:
    return (x / s_full).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)


def make_operand_a(rows: int, K: int, gen, law="pow2", chunk: int = 8192):
    kb = K // 128
    sfa = draw_scales((rows, kb), gen, law)
    a = torch.empty((rows, K), dtype=torch.float8_e4m3fn)
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        x = torch.randn((r1 - r0, K), generator=gen)
        a[r0:r1] = quantize_with_scales(x, sfa[r0:r1].repeat_interleave(128, dim=1))
    return a, sfa


def make_operand_b(G: int, N: int, K: int, gen, law="pow2"):
    nb, kb = (N + 127) // 128, K // 128
    sfb = draw_scales((G, nb, kb), gen, law)
    b = torch.empty((G, N, K), dtype=torch.float8_e4m3fn)
    for g in range(G):
        x = torch.randn((N, K), generator=gen)
        full = sfb[g].repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)
        b[g] = quantize_with_scales(x, full)
    return b, sfb


def contiguous_layout(actual_ms, alignment: int = 128):
    """-> (grouped_layout int32[M], aligned_ms, M): each group padded up to ``alignment`` rows, padding = -1."""
    aligned = [(m + alignment - 1) // alignment * alignment for m in actual_ms]
    M = sum(aligned)
    gl = torch.full((M,), -1, dtype=torch.int32)
    s = 0
    for g, (m, am) in enumerate(zip(actual_ms, aligned)):
        gl[s:s + m] = g
        s += am
    return gl, aligned, M


def make_contiguous_case(G, actual_ms, N, K, seed=0, law="pow2", alignment=128, device="cpu",
                         mn_major_sfa=False):
    """Dict with the registered workload's keys (A, B, SFA, SFB, D, grouped_layout, actual_ms,
    aligned_ms, alignment) plus G, M, N, K."""
    if isinstance(actual_ms, int):
        actual_ms = [actual_ms] * G
    gen = _gen(seed)
    gl, aligned, M = contiguous_layout(actual_ms, alignment)
    a, sfa = make_operand_a(M, K, gen, law)
    b, sfb = make_operand_b(G, N, K, gen, law)
    a.view(torch.uint8)[gl < 0] = 0
    data = dict(A=a, B=b, SFA=sfa, SFB=sfb, D=torch.zeros((M, N), dtype=torch.bfloat16),
                grouped_layout=gl)
    data = {k: v.to(device) for k, v in data.items()}
    if mn_major_sfa:
        data["SFA"] = data["SFA"].t().contiguous().t()
    data.update(actual_ms=tuple(actual_ms), aligned_ms=tuple(aligned), alignment=alignment, G=G, M=M, N=N, K=K)
    return data


def make_masked_case(G, max_m, N, K, seed=0, law="pow2", device="cpu", masked_m=None):
    gen = _gen(seed)
    if masked_m is None:
        masked_m = torch.randint(0, max_m + 1, (G,), generator=gen).to(torch.int32)
    else:
        masked_m = torch.as_tensor(masked_m, dtype=torch.int32)
    a, sfa = make_operand_a(G * max_m, K, gen, law)
    b, sfb = make_operand_b(G, N, K, gen, law)
    data = dict(A=a.view(G, max_m, K), B=b, SFA=sfa.view(G, max_m, K // 128), SFB=sfb,
                D=torch.zeros((G, max_m, N), dtype=torch.bfloat16), masked_m=masked_m)
    data = {k: v.to(device) for k, v in data.items()}
    data.update(G=G, max_m=max_m, N=N, K=K)
    return data


def zipf_group_sizes(G: int, total_rows: int, s: float = 1.2):
    """Per-group row counts proportional to rank^-s, summing to ``total_rows`` (largest remainder)."""
    w = [(r + 1) ** -s for r in range(G)]
    tot = sum(w)
    raw = [total_rows * x / tot for x in w]
    base = [int(x) for x in raw]
    rem = total_rows - sum(base)
    order = sorted(range(G), key=lambda i: raw[i] - base[i], reverse=True)
    for i in order[:rem]:
        base[i] += 1
    return base


def pack_ue8m0_words(scales: torch.Tensor) -> torch.Tensor:
    """Power-of-two fp32 scales [..., kb] -> int32 words [..., ceil(kb/4)]: byte j of word q is the biased exponent
    of K block 4q+j (the packing of tools/tests/numsim/corpus/kernels/gemm.py:252-263); missing blocks hold 2^0."""
    bits = scales.contiguous().view(torch.int32)
    if bool((bits & 0x807FFFFF).ne(0).any()):
        raise ValueError("scales must be positive powers of two")
    codes = (bits >> 23) & 0xFF
    pad = -codes.shape[-1] % 4
    if pad:
        codes = torch.nn.functional.pad(codes, (0, pad), value=127)
    c = codes.view(*codes.shape[:-1], -1, 4)
    return (c[..., 0] | (c[..., 1] << 8) | (c[..., 2] << 16) | (c[..., 3] << 24)).to(torch.int32)


def registered_actual_ms(G: int, expected_m: int, seed: int):
    """Rows per group of a registered grouped_gemm/fp8 row.  The reference draws them with `make_actual_ms` of the
    un-vendored tirx-kernels package; this stand-in uses the law of the public DeepGEMM generator it was ported
    from: uniform in [0.7, 1.3] x expected_m per group, seeded."""
    import random
    rng = random.Random(seed)
    return [int(expected_m * rng.uniform(0.7, 1.3)) for _ in range(G)]


def make_registered_case(G, expected_m, N, K, seed=0, alignment=224, device="cpu", actual_ms=None):
    """The registered workload's tensor contract (evolution/tasks/grouped_gemm_fp8.yaml:15-21): K-major A [M,K] and
    B [G,N,K] in e4m3, UE8M0 scales packed four per int32 and stored MN-major -- SFA [M, K/512] with strides (1, M),
    SFB [G, N, K/512] with strides (N*K/512, 1, N), one B scale per COLUMN (constant over each 128-column block) --
    groups padded to `alignment` rows with -1 in grouped_layout, D bf16 [M,N].  The fp32 form of the same scales
    comes along as SFA_f32 [M,K/128] / SFB_f32 [G,N/128,K/128] for oracles and comparators."""
    if actual_ms is None:
        actual_ms = registered_actual_ms(G, expected_m, seed)
    gl, aligned, M = contiguous_layout(actual_ms, alignment)
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    kb, nb = K // 128, (N + 127) // 128
    sfa = torch.exp2(torch.randint(-4, 1, (M, kb), generator=gen, device=dev).float())
    sfb = torch.exp2(torch.randint(-4, 1, (G, nb, kb), generator=gen, device=dev).float())
    a = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=dev)
    for r0 in range(0, M, 4096):
        r1 = min(M, r0 + 4096)
        x = torch.randn((r1 - r0, K), generator=gen, device=dev)
        a[r0:r1] = quantize_with_scales(x, sfa[r0:r1].repeat_interleave(128, dim=1))
    b = torch.empty((G, N, K), dtype=torch.float8_e4m3fn, device=dev)
    for g in range(G):
        x = torch.randn((N, K), generator=gen, device=dev)
        b[g] = quantize_with_scales(x, sfb[g].repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1))
    gl = gl.to(dev)
    a.view(torch.uint8)[gl < 0] = 0
    sfa_words = pack_ue8m0_words(sfa).t().contiguous().t()                              # [M, K/512], MN-major
    sfb_col = sfb.repeat_interleave(128, dim=1)[:, :N]                                    # [G, N, K/128]
    sfb_words = pack_ue8m0_words(sfb_col).permute(0, 2, 1).contiguous().permute(0, 2, 1)  # [G, N, K/512], N fastest
    return dict(A=a, B=b, SFA=sfa_words, SFB=sfb_words, D=torch.zeros((M, N), dtype=torch.bfloat16, device=dev),
                grouped_layout=gl, actual_ms=tuple(actual_ms), aligned_ms=tuple(aligned), alignment=alignment,
                SFA_f32=sfa, SFB_f32=sfb, G=G, M=M, N=N, K=K)


def output_views(d: torch.Tensor, actual_ms, aligned_ms):
    """Per-group views of the valid rows of D, as the reference's `output_views` forms them
    (tasks/grouped_gemm_fp8/baseline.py:21-27): padding rows are outside every view."""
    views, start = [], 0
    for actual, aligned in zip(actual_ms, aligned_ms):
        views.append(d.narrow(0, start, actual))
        start += aligned
    return tuple(views)
