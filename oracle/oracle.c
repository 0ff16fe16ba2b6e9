/*
 * CPU oracle for the MoE m-grouped FP8 block-scaled GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against (and the timed CPU baseline); nothing in the shipped library links,
 * imports or calls it.
 *
 * It restates, in plain C, the arithmetic contract of the reference's CPU
 * numerical simulator and of its NumPy / torch task oracles.  Each function
 * cites the reference file it follows (paths inside mlc-ai/TIRx-harness).
 *
 * Parity pinning: the codecs, the packed-scale layout, the increasing-K FMA
 * chain, the block-scaled GEMM cases, the SiLU-mul-requant rule and the MoE
 * layer rule are each checked against golden vectors taken from the
 * reference's own tests or produced by running the reference's Python oracles
 * (see tests/golden/ and its generator script).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Codecs                                                                   */
/* ------------------------------------------------------------------------ */

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* e4m3fn decode: tools/tests/numsim/corpus/kernels/gemm.py:154-163
 * (sign, 4-bit exponent bias 7, 3-bit mantissa; exponent 0 = subnormal with
 * step 2^-9; 0x7F / 0xFF = NaN; no infinities). */
static inline float e4m3_decode1(uint8_t b) {
    int e = (b >> 3) & 0xF, m = b & 7;
    float mag;
    if (e == 0xF && m == 7) return bits_f32(0x7FC00000u);
    if (e == 0) mag = ldexpf((float)m / 8.0f, -6);
    else mag = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (b & 0x80) ? -mag : mag;
}

/* e4m3fn encode, round-to-nearest-even, saturate to +-448, NaN -> 0x7F:
 * tools/tests/numsim/corpus/kernels/gemm.py:169-185; equals the hardware
 * cvt.rn.satfinite.e4m3x2.f32 result pinned by
 * tools/tests/numsim/microtests/cases/ptx_cvt_fp8_goldens.py (NaN there keeps
 * no sign: 0x7F). */
static inline uint8_t e4m3_encode1(float x) {
    uint32_t b = f32_bits(x);
    uint32_t sign = (b >> 24) & 0x80u;
    uint32_t a = b & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x7F;              /* NaN */
    float mag = bits_f32(a);
    if (mag >= 464.0f) return (uint8_t)(sign | 0x7E); /* above the 448/480 tie -> 448; inf too */
    /* scale so that one unit of the target grid is 1.0 and round to even */
    int e;
    (void)frexpf(mag, &e);        /* mag = f * 2^e, f in [0.5,1) ; exponent of mag is e-1 */
    int ue = e - 1;               /* unbiased exponent */
    if (mag == 0.0f) return (uint8_t)sign;
    if (ue < -6) ue = -6;         /* subnormal grid: step 2^-9 */
    float step = ldexpf(1.0f, ue - 3);
    float q = mag / step;         /* exact: power-of-two division */
    float r = nearbyintf(q);      /* default rounding mode = nearest even */
    float v = r * step;           /* rounded magnitude (may carry to the next binade) */
    if (v > 448.0f) v = 448.0f;
    if (v == 0.0f) return (uint8_t)sign;
    int e2;
    float f2 = frexpf(v, &e2);    /* v = f2 * 2^e2 */
    int ue2 = e2 - 1;
    uint32_t code;
    if (ue2 < -6) {
        code = (uint32_t)lrintf(ldexpf(v, 9));     /* subnormal: m = v / 2^-9 */
    } else {
        uint32_t m = (uint32_t)lrintf((f2 * 2.0f - 1.0f) * 8.0f);
        code = ((uint32_t)(ue2 + 7) << 3) | m;
    }
    return (uint8_t)(sign | code);
}

ORC_API void orc_e4m3_decode(const uint8_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = e4m3_decode1(in[i]);
}
ORC_API void orc_e4m3_encode(const float* in, uint8_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = e4m3_encode1(in[i]);
}

/* UE8M0 decode: gemm.py:238-242 (2^(b-127); 0xFF = NaN). */
static inline float ue8m0_decode1(uint8_t b) {
    if (b == 0xFF) return bits_f32(0x7FC00000u);
    return ldexpf(1.0f, (int)b - 127);
}
ORC_API void orc_ue8m0_decode(const uint8_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = ue8m0_decode1(in[i]);
}

/* Packed scale layout: gemm.py:252-272.  codes[rows][4*groups] -> words
 * [groups][rows]; byte j of a word is K-block 4*group+j (little endian). */
ORC_API void orc_ue8m0_pack(const uint8_t* codes, uint32_t* packed, int64_t rows, int64_t blocks) {
    int64_t groups = blocks / 4;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t g = 0; g < groups; ++g) {
            const uint8_t* c = codes + r * blocks + 4 * g;
            packed[g * rows + r] = (uint32_t)c[0] | ((uint32_t)c[1] << 8) | ((uint32_t)c[2] << 16) |
                                   ((uint32_t)c[3] << 24);
        }
}
ORC_API void orc_ue8m0_unpack(const uint32_t* packed, uint8_t* codes, int64_t rows, int64_t blocks) {
    int64_t groups = blocks / 4;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t g = 0; g < groups; ++g) {
            uint32_t w = packed[g * rows + r];
            for (int j = 0; j < 4; ++j) codes[r * blocks + 4 * g + j] = (uint8_t)(w >> (8 * j));
        }
}

/* bf16 round-to-nearest-even on the bit pattern: gemm.py:109-113
 * (bits + 0x7FFF + lsb) >> 16. */
static inline uint16_t bf16_rne1(float x) {
    uint32_t b = f32_bits(x);
    uint32_t bias = 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)((b + bias) >> 16);
}
static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
ORC_API void orc_bf16_rne(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = bf16_rne1(in[i]);
}

/* ------------------------------------------------------------------------ */
/* Increasing-K binary32 FMA chain                                          */
/* ------------------------------------------------------------------------ */

/* out[m,n] = fma-chain over k increasing of a[m,k]*b[n,k], starting from
 * d_init[m,n] (or 0).  This is the simulator's MMA arithmetic:
 * tools/src/tirx_harness/numsim/engine-rs/src/runtime/tcgen_ops.rs:4673-4733
 * and engine-rs/fp-env/src/lib.rs:352-386 (vectorised across N only, so the
 * per-element order is untouched). */
ORC_API void orc_fma_abt_increasing_k(const float* a, const float* b, const float* d_init,
                                      float* out, int64_t M, int64_t N, int64_t K) {
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float acc = d_init ? d_init[m * N + n] : 0.0f;
            for (int64_t k = 0; k < K; ++k) acc = fmaf(a[m * K + k], b[n * K + k], acc);
            out[m * N + n] = acc;
        }
}

/* ------------------------------------------------------------------------ */
/* Block-scaled grouped GEMM                                                */
/* ------------------------------------------------------------------------ */

enum { ORC_MODEL_SIM_CHAIN = 0, ORC_MODEL_BLOCK_PROMOTE = 1 };

#define RB 4   /* rows processed together (share one pass over B^T) */
#define NBLK 64

/* Core: rows [0,rows) of one group.  a8: [rows,K] e4m3; sfa row r, block kb at
 * sfa[r*sfa_sr + kb*sfa_sk]; bt: B^T decoded fp32 [K][N] (already scaled for
 * the sim-chain model, raw for block-promote); sfb: [N/128][K/128] fp32.
 *
 * model 0 (sim-chain): every decoded element is multiplied by its block scale
 *   first (tcgen_ops.rs:7630-7644), then one FMA chain runs over all of K
 *   (tcgen_ops.rs:4712-4733).
 * model 1 (block-promote): a chain over each 128-K block on raw values, then
 *   acc = fma(partial, sfa*sfb, acc) -- the arithmetic of a kernel that applies
 *   block scales while draining the accumulator.
 */
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
static void gemm_rows(const uint8_t* a8, const float* sfa, int64_t sfa_sr, int64_t sfa_sk,
                      const float* bt, const float* sfb, int64_t sfb_sn, int64_t sfb_sk,
                      const uint8_t* row_valid, void* d_out, int64_t ldd,
                      int64_t rows, int64_t N, int64_t K, int model, int out_f32) {
    uint16_t* d = (uint16_t*)d_out;
    float* df = (float*)d_out;
    const int64_t KB = K / 128;
#pragma omp parallel
    {
        float* arow = (float*)malloc(sizeof(float) * RB * K);
#pragma omp for schedule(dynamic, 1)
        for (int64_t r0 = 0; r0 < rows; r0 += RB) {
            int nr = (int)((rows - r0) < RB ? (rows - r0) : RB);
            int any = 0;
            for (int i = 0; i < nr; ++i) any |= row_valid ? row_valid[r0 + i] : 1;
            if (!any) continue;
            for (int i = 0; i < RB; ++i) {
                int64_t r = r0 + (i < nr ? i : 0);
                for (int64_t k = 0; k < K; ++k) {
                    float v = e4m3_decode1(a8[r * K + k]);
                    if (model == ORC_MODEL_SIM_CHAIN) v = v * sfa[r * sfa_sr + (k / 128) * sfa_sk];
                    arow[i * K + k] = v;
                }
            }
            for (int64_t n0 = 0; n0 < N; n0 += NBLK) {
                int nn = (int)((N - n0) < NBLK ? (N - n0) : NBLK);
                float acc[RB][NBLK];
                for (int i = 0; i < RB; ++i)
                    for (int j = 0; j < NBLK; ++j) acc[i][j] = 0.0f;
                if (model == ORC_MODEL_SIM_CHAIN) {
                    for (int64_t k = 0; k < K; ++k) {
                        const float* brow = bt + k * N + n0;
                        for (int i = 0; i < RB; ++i) {
                            float av = arow[i * K + k];
#pragma omp simd
                            for (int j = 0; j < NBLK; ++j)
                                if (j < nn) acc[i][j] = fmaf(av, brow[j], acc[i][j]);
                        }
                    }
                } else {
                    for (int64_t kb = 0; kb < KB; ++kb) {
                        float part[RB][NBLK];
                        for (int i = 0; i < RB; ++i)
                            for (int j = 0; j < NBLK; ++j) part[i][j] = 0.0f;
                        for (int64_t k = kb * 128; k < kb * 128 + 128; ++k) {
                            const float* brow = bt + k * N + n0;
                            for (int i = 0; i < RB; ++i) {
                                float av = arow[i * K + k];
#pragma omp simd
                                for (int j = 0; j < NBLK; ++j)
                                    if (j < nn) part[i][j] = fmaf(av, brow[j], part[i][j]);
                            }
                        }
                        for (int i = 0; i < RB; ++i) {
                            int64_t r = r0 + (i < nr ? i : 0);
                            float sa = sfa[r * sfa_sr + kb * sfa_sk];
                            for (int j = 0; j < nn; ++j) {
                                float s = sa * sfb[((n0 + j) / 128) * sfb_sn + kb * sfb_sk];
                                acc[i][j] = fmaf(part[i][j], s, acc[i][j]);
                            }
                        }
                    }
                }
                for (int i = 0; i < nr; ++i) {
                    if (row_valid && !row_valid[r0 + i]) continue;
                    if (out_f32)
                        for (int j = 0; j < nn; ++j) df[(r0 + i) * ldd + n0 + j] = acc[i][j];
                    else
                        for (int j = 0; j < nn; ++j) d[(r0 + i) * ldd + n0 + j] = bf16_rne1(acc[i][j]);
                }
            }
        }
        free(arow);
    }
}

/* Decode one group's B [N,K] e4m3 into B^T fp32 [K][N]; scaled by the 128x128
 * block scale when prescale != 0. */
static void decode_bt(const uint8_t* b8, const float* sfb, int64_t sfb_sn, int64_t sfb_sk,
                      float* bt, int64_t N, int64_t K, int prescale) {
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < K; ++k)
        for (int64_t n = 0; n < N; ++n) {
            float v = e4m3_decode1(b8[n * K + k]);
            if (prescale) v = v * sfb[(n / 128) * sfb_sn + (k / 128) * sfb_sk];
            bt[k * N + n] = v;
        }
}

/* m-grouped contiguous layout.  A [M,K] e4m3, B [G,N,K] e4m3, sfa fp32 with
 * element strides (row, K-block), sfb fp32 [G, ceil(N/128), K/128] row major,
 * grouped_layout int32[M]: group id per row, negative = padding row (left
 * untouched).  D [M,N] bf16 bits.  Layout contract:
 * evolution/tasks/grouped_gemm_fp8.yaml:15-21; math:
 * D_g = dequantize(A_g) @ dequantize(B_g)^T (same file :23-25).
 * row_step > 1 computes only rows r with r % row_step == 0 (bounded samples).
 * out_f32 != 0 writes the fp32 accumulator instead of bf16 bits (the value a
 * fused epilogue sees before any rounding). */
ORC_API int orc_gg_contiguous(const uint8_t* A, const uint8_t* B, const float* sfa,
                              int64_t sfa_sr, int64_t sfa_sk, const float* sfb,
                              const int32_t* grouped_layout, void* D, int64_t G, int64_t M,
                              int64_t N, int64_t K, int model, int64_t row_step, int out_f32) {
    if (K % 128 != 0) return -1;
    const int64_t KB = K / 128, NB = (N + 127) / 128;
    float* bt = (float*)malloc(sizeof(float) * (size_t)K * (size_t)N);
    uint8_t* valid = (uint8_t*)malloc((size_t)M);
    if (!bt || !valid) { free(bt); free(valid); return -2; }
    for (int64_t g = 0; g < G; ++g) {
        int any = 0;
        for (int64_t r = 0; r < M; ++r) {
            valid[r] = (grouped_layout[r] == (int32_t)g) && (row_step <= 1 || (r % row_step) == 0);
            any |= valid[r];
        }
        if (!any) continue;
        const float* sfb_g = sfb + g * NB * KB;
        decode_bt(B + g * N * K, sfb_g, KB, 1, bt, N, K, model == ORC_MODEL_SIM_CHAIN);
        /* restrict to the row span of this group to skip work */
        int64_t lo = 0, hi = M;
        while (lo < M && !valid[lo]) ++lo;
        while (hi > lo && !valid[hi - 1]) --hi;
        gemm_rows(A + lo * K, sfa + lo * sfa_sr, sfa_sr, sfa_sk, bt, sfb_g, KB, 1, valid + lo,
                  (char*)D + (size_t)lo * N * (out_f32 ? 4 : 2), N, hi - lo, N, K, model, out_f32);
    }
    free(bt); free(valid);
    return 0;
}

/* m-grouped masked layout.  A [G,max_m,K], B [G,N,K], D [G,max_m,N]; only rows
 * < masked_m[g] of each group are computed, the rest of D is left untouched
 * (tools/tests/numsim/corpus/kernels/gemm.py:705-795).  sfa indexed with
 * strides (group, row, K-block). */
ORC_API int orc_gg_masked(const uint8_t* A, const uint8_t* B, const float* sfa, int64_t sfa_sg,
                          int64_t sfa_sr, int64_t sfa_sk, const float* sfb,
                          const int32_t* masked_m, void* D, int64_t G, int64_t max_m,
                          int64_t N, int64_t K, int model, int out_f32) {
    if (K % 128 != 0) return -1;
    const int64_t KB = K / 128, NB = (N + 127) / 128;
    float* bt = (float*)malloc(sizeof(float) * (size_t)K * (size_t)N);
    if (!bt) return -2;
    for (int64_t g = 0; g < G; ++g) {
        int64_t rows = masked_m[g];
        if (rows <= 0) continue;
        if (rows > max_m) rows = max_m;
        const float* sfb_g = sfb + g * NB * KB;
        decode_bt(B + g * N * K, sfb_g, KB, 1, bt, N, K, model == ORC_MODEL_SIM_CHAIN);
        gemm_rows(A + g * max_m * K, sfa + g * sfa_sg, sfa_sr, sfa_sk, bt, sfb_g, KB, 1, NULL,
                  (char*)D + (size_t)g * max_m * N * (out_f32 ? 4 : 2), N, rows, N, K, model, out_f32);
    }
    free(bt);
    return 0;
}

/* Dense FP8 GEMM with per-row UE8M0 scales on BOTH operands, packed four to a
 * word: the reference corpus oracle _fp8_blockwise_reference (gemm.py:275-292).
 * A [M,K], B [N,K], SFA words [K/512][M], SFB words [K/512][N]; D bf16 bits.
 * Uses the sim-chain order; the corpus inputs are dyadic so any order agrees. */
ORC_API int orc_fp8_blockwise_ue8m0(const uint8_t* A, const uint8_t* B, const uint32_t* SFA,
                                    const uint32_t* SFB, uint16_t* D, int64_t M, int64_t N,
                                    int64_t K) {
    if (K % 512 != 0) return -1;
    const int64_t KB = K / 128;
    float* ad = (float*)malloc(sizeof(float) * (size_t)M * K);
    float* bd = (float*)malloc(sizeof(float) * (size_t)N * K);
    if (!ad || !bd) { free(ad); free(bd); return -2; }
    for (int64_t r = 0; r < M; ++r)
        for (int64_t k = 0; k < K; ++k) {
            int64_t kb = k / 128;
            uint8_t code = (uint8_t)(SFA[(kb / 4) * M + r] >> (8 * (kb % 4)));
            ad[r * K + k] = e4m3_decode1(A[r * K + k]) * ue8m0_decode1(code);
        }
    for (int64_t r = 0; r < N; ++r)
        for (int64_t k = 0; k < K; ++k) {
            int64_t kb = k / 128;
            uint8_t code = (uint8_t)(SFB[(kb / 4) * N + r] >> (8 * (kb % 4)));
            bd[r * K + k] = e4m3_decode1(B[r * K + k]) * ue8m0_decode1(code);
        }
    (void)KB;
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc = fmaf(ad[m * K + k], bd[n * K + k], acc);
            D[m * N + n] = bf16_rne1(acc);
        }
    free(ad); free(bd);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* Activation quantisation and SiLU-mul-requant                             */
/* ------------------------------------------------------------------------ */

/* Per-row 1x128 quantisation: s = max(amax,1e-8)/448; q = e4m3(clamp(x/s,+-448))
 * with true division -- alphamoe/definition.json `_quantize_per_token_group`
 * and alphamoe/baseline.py:14-26.  x fp32 [rows,cols]; q [rows,cols];
 * scales written at scales[r*ss_r + b*ss_b]. */
ORC_API void orc_quant_1x128(const float* x, uint8_t* q, float* scales, int64_t ss_r, int64_t ss_b,
                             int64_t rows, int64_t cols) {
    const int64_t nb = cols / 128;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t b = 0; b < nb; ++b) {
            const float* p = x + r * cols + b * 128;
            float amax = 0.0f;
            for (int j = 0; j < 128; ++j) { float a = fabsf(p[j]); if (a > amax) amax = a; }
            float s = (amax < 1.0e-8f ? 1.0e-8f : amax) / 448.0f;
            scales[r * ss_r + b * ss_b] = s;
            for (int j = 0; j < 128; ++j) {
                float v = p[j] / s;
                if (v > 448.0f) v = 448.0f;
                if (v < -448.0f) v = -448.0f;
                q[r * cols + b * 128 + j] = e4m3_encode1(v);
            }
        }
}

/* SiLU in fp32 as the corpus models the device form, x / (1 + exp2(-x*log2e)):
 * tools/tests/numsim/corpus/kernels/activation.py:34-38. */
static inline float silu_f32(float x) {
    return x / (1.0f + exp2f(-x * 1.4426950408889634f));
}

/* gate_up [rows, 2*I] (bf16 bits, or fp32 when in_f32 != 0) -> act = silu(gate)*up in fp32 -> 1x128 requant.
 * gate_first != 0: gate = columns [0,I), up = [I,2I)   (alphamoe/definition.json
 * `_reference_quantized`: silu(gate)*up with logical [gate; up]);
 * gate_first == 0: gate = columns [I,2I), up = [0,I)   (moe/definition.json:
 * silu(G1[:, I:]) * G1[:, :I]).
 * Rows with row_valid[r]==0 are skipped (outputs untouched). */
ORC_API void orc_silu_mul_requant(const void* gu_in, int in_f32, uint8_t* q, float* scales,
                                  int64_t ss_r, int64_t ss_b, const uint8_t* row_valid,
                                  int64_t rows, int64_t I, int gate_first) {
    const uint16_t* gu = (const uint16_t*)gu_in;
    const float* guf = (const float*)gu_in;
    const int64_t nb = I / 128;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        if (row_valid && !row_valid[r]) continue;
        const int64_t go = r * 2 * I + (gate_first ? 0 : I);
        const int64_t uo = r * 2 * I + (gate_first ? I : 0);
        for (int64_t b = 0; b < nb; ++b) {
            float act[128];
            float amax = 0.0f;
            for (int j = 0; j < 128; ++j) {
                float gv = in_f32 ? guf[go + b * 128 + j] : bf16_to_f32(gu[go + b * 128 + j]);
                float uv = in_f32 ? guf[uo + b * 128 + j] : bf16_to_f32(gu[uo + b * 128 + j]);
                float a = silu_f32(gv) * uv;
                act[j] = a;
                float aa = fabsf(a);
                if (aa > amax) amax = aa;
            }
            float s = (amax < 1.0e-8f ? 1.0e-8f : amax) / 448.0f;
            scales[r * ss_r + b * ss_b] = s;
            for (int j = 0; j < 128; ++j) {
                float v = act[j] / s;
                if (v > 448.0f) v = 448.0f;
                if (v < -448.0f) v = -448.0f;
                q[r * I + b * 128 + j] = e4m3_encode1(v);
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Routing, permutation plan, combine                                       */
/* ------------------------------------------------------------------------ */

/* Softmax over E logits, top-k by value with ties to the LOWEST expert index,
 * weights = selected probabilities renormalised to sum 1.  ids in descending
 * score order.  (Routing rule of the MoE-layer workload: softmax of N(0,1)
 * router logits, top-8.) */
ORC_API void orc_route_softmax_topk(const float* logits, int32_t* ids, float* w, int64_t T,
                                    int64_t E, int64_t top_k) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; ++t) {
        const float* l = logits + t * E;
        float mx = l[0];
        for (int64_t e = 1; e < E; ++e) if (l[e] > mx) mx = l[e];
        float sum = 0.0f;
        for (int64_t k = 0; k < top_k; ++k) {
            int64_t best = -1;
            for (int64_t e = 0; e < E; ++e) {
                int taken = 0;
                for (int64_t j = 0; j < k; ++j) if (ids[t * top_k + j] == e) taken = 1;
                if (taken) continue;
                if (best < 0 || l[e] > l[best]) best = e;
            }
            ids[t * top_k + k] = (int32_t)best;
            float p = expf(l[best] - mx);
            w[t * top_k + k] = p;
            sum += p;
        }
        for (int64_t k = 0; k < top_k; ++k) w[t * top_k + k] = w[t * top_k + k] / sum;
    }
}

/* Permutation plan for the contiguous grouped layout.
 * ids int32 [T*top_k] (pair p = t*top_k + j); experts [e_lo, e_lo+E_local) are
 * local, other pairs get pos = -1.  counts[e] = pairs routed to local expert e;
 * offsets[e] = start row of e (each expert padded up to a multiple of `align`),
 * offsets[E_local] = total rows; pos[p] = destination row, pairs keep their
 * order within an expert (stable, token order); grouped_layout[row] = local
 * expert id or -1 on padding; src_pair[row] = p or -1.
 * (Bit-exact artefacts: per-expert counts are checked like the reference checks
 * its receive counters against bincount(routes),
 * tools/tests/numsim/corpus/kernels/deepgemm.py:1444-1491.) */
ORC_API int64_t orc_permute_plan(const int32_t* ids, int64_t n_pairs, int64_t e_lo, int64_t E_local,
                                 int64_t align, int32_t* counts, int32_t* offsets, int32_t* pos,
                                 int32_t* grouped_layout, int32_t* src_pair, int64_t cap_rows) {
    for (int64_t e = 0; e < E_local; ++e) counts[e] = 0;
    for (int64_t p = 0; p < n_pairs; ++p) {
        int64_t e = (int64_t)ids[p] - e_lo;
        if (e >= 0 && e < E_local) counts[e]++;
    }
    int64_t total = 0;
    for (int64_t e = 0; e < E_local; ++e) {
        offsets[e] = (int32_t)total;
        total += ((int64_t)counts[e] + align - 1) / align * align;
    }
    offsets[E_local] = (int32_t)total;
    if (total > cap_rows) return -1;
    if (grouped_layout) for (int64_t r = 0; r < cap_rows; ++r) grouped_layout[r] = -1;
    if (src_pair) for (int64_t r = 0; r < cap_rows; ++r) src_pair[r] = -1;
    int32_t* fill = (int32_t*)calloc((size_t)E_local, sizeof(int32_t));
    for (int64_t p = 0; p < n_pairs; ++p) {
        int64_t e = (int64_t)ids[p] - e_lo;
        if (e >= 0 && e < E_local) {
            int64_t row = offsets[e] + fill[e]++;
            pos[p] = (int32_t)row;
            if (grouped_layout) grouped_layout[row] = (int32_t)e;
            if (src_pair) src_pair[row] = (int32_t)p;
        } else {
            pos[p] = -1;
        }
    }
    free(fill);
    return total;
}

/* Weighted combine: out[t,:] = bf16( sum_j w[t,j] * y[pos[t*top_k+j], :] ) with
 * fp32 accumulation (separate multiply and add, as torch does) in slot order
 * j = 0..top_k-1, skipping pos < 0 -- the fp32
 * weighted accumulation of moe/definition.json (`output.index_add_` of
 * O * w_tok, then .to(bfloat16)).  y bf16 bits [rows,H]. */
ORC_API void orc_combine(const uint16_t* y, const int32_t* pos, const float* w, uint16_t* out,
                         int64_t T, int64_t top_k, int64_t H) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; ++t)
        for (int64_t h = 0; h < H; ++h) {
            float acc = 0.0f;
            for (int64_t j = 0; j < top_k; ++j) {
                int32_t r = pos[t * top_k + j];
                if (r < 0) continue;
                acc = acc + w[t * top_k + j] * bf16_to_f32(y[(int64_t)r * H + h]);
            }
            out[t * H + h] = bf16_rne1(acc);
        }
}

/* Sets the number of OpenMP threads the following calls use (a launcher such as torchrun exports
 * OMP_NUM_THREADS=1 to its ranks, which would otherwise time a one-thread baseline). */
ORC_API void orc_set_num_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* DeepSeek-V3 "no-aux" routing of the registered `moe` workload
 * (evolution/benchmark/flashinfer_bench_evolve/tasks/moe/definition.json, block "2) No-aux routing"):
 *   s = sigmoid(logit); swb = s + bias; experts are split into n_group groups; a group's score is
 *   the sum of its two largest swb; the topk_group best groups are kept; among their experts the
 *   top_k largest swb are selected; weight = s / (sum of selected s + 1e-20) * routed_scaling_factor.
 * Ties go to the lowest index.  ids are written in descending swb order. */
ORC_API void orc_route_deepseek(const float* logits, const float* bias, int32_t* ids, float* w, int64_t T,
                                int64_t E, int64_t n_group, int64_t topk_group, int64_t top_k, float rsf) {
    const int64_t gs = E / n_group;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; ++t) {
        float s[1024], swb[1024], gscore[64];
        int keep[64];
        for (int64_t e = 0; e < E; ++e) {
            s[e] = 1.0f / (1.0f + expf(-logits[t * E + e]));
            swb[e] = s[e] + bias[e];
        }
        for (int64_t g = 0; g < n_group; ++g) {
            int64_t b1 = -1, b2 = -1;
            for (int64_t j = 0; j < gs; ++j) {
                int64_t e = g * gs + j;
                if (b1 < 0 || swb[e] > swb[b1]) { b2 = b1; b1 = e; }
                else if (b2 < 0 || swb[e] > swb[b2]) b2 = e;
            }
            gscore[g] = swb[b1] + swb[b2];
            keep[g] = 0;
        }
        for (int64_t k = 0; k < topk_group; ++k) {
            int64_t best = -1;
            for (int64_t g = 0; g < n_group; ++g)
                if (!keep[g] && (best < 0 || gscore[g] > gscore[best])) best = g;
            keep[best] = 1;
        }
        float sum = 0.0f;
        for (int64_t k = 0; k < top_k; ++k) {
            int64_t best = -1;
            for (int64_t e = 0; e < E; ++e) {
                if (!keep[e / gs]) continue;
                int taken = 0;
                for (int64_t j = 0; j < k; ++j) if (ids[t * top_k + j] == e) taken = 1;
                if (taken) continue;
                if (best < 0 || swb[e] > swb[best]) best = e;
            }
            ids[t * top_k + k] = (int32_t)best;
            sum += s[best];
        }
        for (int64_t k = 0; k < top_k; ++k) w[t * top_k + k] = s[ids[t * top_k + k]] / (sum + 1e-20f) * rsf;
    }
}
