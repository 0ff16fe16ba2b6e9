// Decode-regime MoE layer from bf16 activations and preselected routes (few tokens, hundreds of experts,
// intermediate size 128): the kernels around the two masked-layout grouped GEMMs.
//
//   alpha_plan_kernel          per-expert route counts and the slot of every route inside its expert
//   alpha_quant_scatter_kernel token row -> 1x128 FP8 quantisation -> the route's row of the masked A matrix
//   alpha_silu_requant_kernel  fp32 [gate; up] row -> SiLU(gate)*up -> 1x128 requant
//   alpha_combine_kernel       per token: contributions in ascending expert id, each rounded to bf16 and
//                              added to a bf16 accumulator with a rounding per update
//
// Every expert owns `max_m` consecutive rows of the intermediate matrices; only the first counts[e] are
// written or read, so the kernels touch (routes x row bytes) of memory whatever E is.
#pragma once

#include "moe_ops.cuh"

namespace b200 {

constexpr int ALPHA_PLAN_THREADS = 1024;
constexpr int STATUS_ALPHA_OVERFLOW = 1 << 12;      // an expert received more routes than max_m rows

// One CTA.  Deterministic: route p's slot is the number of earlier routes (smaller p) to the same expert.
// hist: [32 warps][E] in dynamic shared memory.  Warp w owns the contiguous routes [w*per, (w+1)*per).
__global__ void __launch_bounds__(ALPHA_PLAN_THREADS, 1)
alpha_plan_kernel(const int* __restrict__ ids, int n_pairs, int E, int max_m, int* __restrict__ counts,
                  int* __restrict__ rowpos, int* status) {
    extern __shared__ int hist[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < 32 * E; i += ALPHA_PLAN_THREADS) hist[i] = 0;
    pdl_wait();              // counts / rowpos may still be in use by the previous call's kernels
    __syncthreads();
    const int per = (((n_pairs + 31) / 32) + 31) & ~31;
    const int begin = warp * per;
    const int end = min(begin + per, n_pairs);
    for (int base = begin; base < end; base += 32) {
        const int p = base + lane;
        const int e = p < end ? __ldg(ids + p) : -1;
        const bool valid = e >= 0 && e < E;
        const unsigned mask = __match_any_sync(0xffffffffu, valid ? e : E + lane);
        if (valid && lane == __ffs(mask) - 1) hist[warp * E + e] += __popc(mask);
        __syncwarp();
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += ALPHA_PLAN_THREADS) {
        int run = 0;
        for (int w = 0; w < 32; ++w) {
            const int c = hist[w * E + e];
            hist[w * E + e] = run;
            run += c;
        }
        if (run > max_m) {
            atomicOr(status, STATUS_ALPHA_OVERFLOW);
            run = max_m;
        }
        counts[e] = run;
    }
    __syncthreads();
    for (int base = begin; base < end; base += 32) {
        const int p = base + lane;
        const int e = p < end ? __ldg(ids + p) : -1;
        const bool valid = e >= 0 && e < E;
        const unsigned mask = __match_any_sync(0xffffffffu, valid ? e : E + lane);
        const int leader = __ffs(mask) - 1;
        int first = 0;
        if (valid && lane == leader) {
            first = hist[warp * E + e];
            hist[warp * E + e] = first + __popc(mask);
        }
        first = __shfl_sync(0xffffffffu, first, leader);
        const int slot = first + __popc(mask & ((1u << lane) - 1u));
        if (p < end) rowpos[p] = (valid && slot < max_m) ? e * max_m + slot : -1;
        __syncwarp();
    }
}

// One warp per (route, 128-block).  x bf16 [M, H]; q e4m3 [rows_total, H]; scales MN-major: scale of
// (row, block b) at s[b * rows_total + row].
__global__ void alpha_quant_scatter_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rowpos,
                                           int n_pairs, int top_k, int H, long long rows_total,
                                           uint8_t* __restrict__ q, float* __restrict__ s) {
    const int nb = H >> 7;
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (w >= n_pairs * nb) return;
    const int p = w / nb, b = w - p * nb;
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + (long long)(p / top_k) * H + b * 128 + lane * 4));
    const int row = __ldg(rowpos + p);
    if (row < 0) return;
    float v[4], sc;
    bf16x4_to_float(raw, v);
    const uint32_t packed = quant_block_4(v, &sc);
    *reinterpret_cast<uint32_t*>(q + (long long)row * H + b * 128 + lane * 4) = packed;
    if (lane == 0) s[(long long)b * rows_total + row] = sc;
}

// Plan and quantisation in one launch, for the decode regime (a few thousand routes at most): one warp per
// (route, 128-block) finds its route's slot itself by scanning the route list (slot = number of earlier routes
// to the same expert; the route list is a few KB and stays in L1/L2) instead of waiting for a separate plan
// kernel; the warp of block 0 also publishes rowpos and, if no later route goes to the same expert, the
// expert's count.  `counts` must be zero on entry (experts without routes keep 0).  Same results as
// alpha_plan_kernel + alpha_quant_scatter_kernel, bit for bit.
__global__ void alpha_plan_quant_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, int n_pairs, int top_k,
                                        int E, int max_m, int H, long long rows_total, int* __restrict__ counts,
                                        int* __restrict__ rowpos, uint8_t* __restrict__ q, float* __restrict__ s, int* status) {
    const int nb = H >> 7;
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    if (w >= n_pairs * nb) return;
    const int p = w / nb, b = w - p * nb;
    // the token's values do not depend on the previous kernels of the stream: fetch them before waiting
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + (long long)(p / top_k) * H + b * 128 + lane * 4));
    const int e = __ldg(ids + p);
    int before = 0, after = 0;
    if (e >= 0 && e < E) {
        for (int base = 0; base < n_pairs; base += 32) {
            const int i = base + lane;
            const bool same = i < n_pairs && __ldg(ids + i) == e;
            before += same && i < p;
            after += same && i > p;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        before += __shfl_xor_sync(0xffffffffu, before, o);
        after += __shfl_xor_sync(0xffffffffu, after, o);
    }
    const bool valid = e >= 0 && e < E && before < max_m;
    const int row = valid ? e * max_m + before : -1;
    pdl_wait();              // counts / rowpos / a1 may still be in use by the previous call's kernels
    if (b == 0 && lane == 0) {
        rowpos[p] = row;
        if (e >= 0 && e < E && after == 0) {
            int c = before + 1;
            if (c > max_m) {
                atomicOr(status, STATUS_ALPHA_OVERFLOW);
                c = max_m;
            }
            counts[e] = c;
        }
    }
    if (!valid) return;
    float v[4], sc;
    bf16x4_to_float(raw, v);
    const uint32_t packed = quant_block_4(v, &sc);
    *reinterpret_cast<uint32_t*>(q + (long long)row * H + b * 128 + lane * 4) = packed;
    if (lane == 0) s[(long long)b * rows_total + row] = sc;
}

// One warp per route.  gu fp32 [rows_total, 2I] with gate = columns [0, I) when gate_first, else [I, 2I).
__global__ void alpha_silu_requant_kernel(const float* __restrict__ gu, const int* __restrict__ rowpos, int n_pairs,
                                          int inter, int gate_first, long long rows_total, uint8_t* __restrict__ q,
                                          float* __restrict__ s) {
    const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (p >= n_pairs) return;
    const int row = __ldg(rowpos + p);
    if (row < 0) return;
    const float* grow = gu + (long long)row * 2 * inter + (gate_first ? 0 : inter) + lane * 4;
    const float* urow = gu + (long long)row * 2 * inter + (gate_first ? inter : 0) + lane * 4;
    const int nb = inter >> 7;
    for (int b = 0; b < nb; ++b) {
        const float4 g = *reinterpret_cast<const float4*>(grow + b * 128);
        const float4 u = *reinterpret_cast<const float4*>(urow + b * 128);
        float a[4], sc;
        a[0] = __fmul_rn(silu_f32(g.x), u.x);
        a[1] = __fmul_rn(silu_f32(g.y), u.y);
        a[2] = __fmul_rn(silu_f32(g.z), u.z);
        a[3] = __fmul_rn(silu_f32(g.w), u.w);
        const uint32_t packed = quant_block_4(a, &sc);
        *reinterpret_cast<uint32_t*>(q + (long long)row * inter + b * 128 + lane * 4) = packed;
        if (lane == 0) s[(long long)b * rows_total + row] = sc;
    }
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// One CTA per token.  d fp32 [rows_total, H] holds the unweighted down projections.  The token's routes are
// ordered by expert id (ties by route index); out = bf16 chain: acc = bf16(acc + bf16(d * (w * rsf))).
__global__ void alpha_combine_kernel(const float* __restrict__ d, const int* __restrict__ ids,
                                     const float* __restrict__ w, const int* __restrict__ rowpos, float rsf, int top_k,
                                     int H, __nv_bfloat16* __restrict__ out) {
    __shared__ int s_row[32];
    __shared__ float s_scale[32];
    __shared__ int s_n;
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x < 32) {
        // lane j owns route j: its place in the order is the number of live routes with a smaller (expert, j)
        const int j = threadIdx.x;
        const bool have = j < top_k;
        const int rp = have ? __ldg(rowpos + t * top_k + j) : -1;
        const int e = have ? __ldg(ids + t * top_k + j) : 0;
        const float wt = have ? __ldg(w + t * top_k + j) : 0.0f;
        const bool live = rp >= 0;
        const unsigned live_mask = __ballot_sync(0xffffffffu, live);
        int rank = 0;
        for (int o = 0; o < top_k; ++o) {
            const int eo = __shfl_sync(0xffffffffu, e, o);
            if (((live_mask >> o) & 1u) && (eo < e || (eo == e && o < j))) ++rank;
        }
        if (live) {
            s_row[rank] = rp;
            s_scale[rank] = __fmul_rn(wt, rsf);
        }
        if (j == 0) s_n = __popc(live_mask);
    }
    __syncthreads();
    const int n = s_n;
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int k0 = 0; k0 < n; k0 += 8) {
            float4 v[8];                     // eight routes' loads in flight before the (ordered) bf16 chain
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (k0 + i < n) v[i] = __ldcs(reinterpret_cast<const float4*>(d + (long long)s_row[k0 + i] * H + c));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (k0 + i < n) {
                    const float sc = s_scale[k0 + i];
                    a0 = round_bf16(a0 + round_bf16(__fmul_rn(v[i].x, sc)));
                    a1 = round_bf16(a1 + round_bf16(__fmul_rn(v[i].y, sc)));
                    a2 = round_bf16(a2 + round_bf16(__fmul_rn(v[i].z, sc)));
                    a3 = round_bf16(a3 + round_bf16(__fmul_rn(v[i].w, sc)));
                }
            }
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1), hi = __floats2bfloat162_rn(a2, a3);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + (long long)t * H + c) = o;
    }
}

}  // namespace b200
