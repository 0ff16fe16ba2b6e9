// HBM-bound kernels either side of the grouped GEMMs: 1x128 activation quantisation, fused
// SiLU*mul + FP8 requantisation, softmax top-k routing, the stable permutation plan (counts,
// aligned group offsets, destination rows, grouped_layout), row gather and weighted combine.
// All are plain coalesced 16-byte-vector kernels; none uses tensor cores.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace b200 {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// four fp32 -> four e4m3 bytes (cvt.rn.satfinite.e4m3x2.f32), byte j = value j
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ float clamp448(float v) { return fminf(fmaxf(v, -448.0f), 448.0f); }

// Quantise one 128-wide block held as 4 values per lane: s = max(amax, 1e-8) / 448,
// q = e4m3(clamp(x / s)) with IEEE division.  Returns the packed bytes; *scale_out = s.
__device__ __forceinline__ uint32_t quant_block_4(const float (&x)[4], float* scale_out) {
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
    amax = warp_max(amax);
    const float s = __fdiv_rn(fmaxf(amax, 1.0e-8f), 448.0f);
    *scale_out = s;
    return pack4_e4m3(clamp448(__fdiv_rn(x[0], s)), clamp448(__fdiv_rn(x[1], s)),
                      clamp448(__fdiv_rn(x[2], s)), clamp448(__fdiv_rn(x[3], s)));
}

__device__ __forceinline__ void bf16x4_to_float(uint2 raw, float (&out)[4]) {
    out[0] = __uint_as_float(raw.x << 16);
    out[1] = __uint_as_float(raw.x & 0xFFFF0000u);
    out[2] = __uint_as_float(raw.y << 16);
    out[3] = __uint_as_float(raw.y & 0xFFFF0000u);
}

// x bf16 [rows, cols] -> q e4m3 [rows, cols], scales f32 at [r*ss_r + b*ss_b].  One warp per block.
__global__ void quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                   float* __restrict__ scales, long long ss_r, long long ss_b,
                                   int rows, int cols) {
    const int nb = cols >> 7;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)rows * nb) return;
    const int r = (int)(w / nb), b = (int)(w % nb);
    const long long off = (long long)r * cols + b * 128 + lane * 4;
    float v[4];
    bf16x4_to_float(__ldg(reinterpret_cast<const uint2*>(x + off)), v);
    float s;
    const uint32_t packed = quant_block_4(v, &s);
    *reinterpret_cast<uint32_t*>(q + off) = packed;
    if (lane == 0) scales[r * ss_r + b * ss_b] = s;
}

// SiLU in the device form the reference's corpus models: x / (1 + exp2(-x * log2(e))).
__device__ __forceinline__ float silu_f32(float x) {
    return __fdiv_rn(x, 1.0f + exp2f(-x * 1.4426950408889634f));
}

// gate_up bf16 [rows, 2I] -> act = silu(gate) * up (fp32) -> 1x128 requant: q e4m3 [rows, I],
// scales at [r*ss_r + b*ss_b].  gate_first: gate = columns [0, I), else gate = [I, 2I).
// Rows whose layout entry is negative (padding) are skipped.  One warp per row: all loads of up to four
// 128-blocks are issued before the first is consumed, so each lane keeps 64 bytes in flight.
__global__ void silu_mul_requant_kernel(const __nv_bfloat16* __restrict__ gu, uint8_t* __restrict__ q,
                                        float* __restrict__ scales, long long ss_r, long long ss_b,
                                        const int* __restrict__ layout, int rows, int inter,
                                        int gate_first) {
    const int nb = inter >> 7;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    if (layout != nullptr && __ldg(layout + r) < 0) return;
    const __nv_bfloat16* grow = gu + (long long)r * 2 * inter + (gate_first ? 0 : inter) + lane * 4;
    const __nv_bfloat16* urow = gu + (long long)r * 2 * inter + (gate_first ? inter : 0) + lane * 4;
    for (int b0 = 0; b0 < nb; b0 += 4) {
        uint2 graw[4], uraw[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (b0 + i < nb) {
                graw[i] = __ldcs(reinterpret_cast<const uint2*>(grow + (b0 + i) * 128));
                uraw[i] = __ldcs(reinterpret_cast<const uint2*>(urow + (b0 + i) * 128));
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (b0 + i < nb) {
                float g[4], u[4], a[4];
                bf16x4_to_float(graw[i], g);
                bf16x4_to_float(uraw[i], u);
#pragma unroll
                for (int j = 0; j < 4; ++j) a[j] = __fmul_rn(silu_f32(g[j]), u[j]);
                float s;
                const uint32_t packed = quant_block_4(a, &s);
                *reinterpret_cast<uint32_t*>(q + (long long)r * inter + (b0 + i) * 128 + lane * 4) = packed;
                if (lane == 0) scales[r * ss_r + (long long)(b0 + i) * ss_b] = s;
            }
        }
    }
}

// Softmax over E logits + top-k (ties -> lowest expert index), weights renormalised over the
// selected experts.  One warp per token; lane l holds experts l, l+32, ...  E <= 512, top_k <= 32.
constexpr int ROUTE_MAX_PER_LANE = 16;
__global__ void route_softmax_topk_kernel(const float* __restrict__ logits, int* __restrict__ ids,
                                          float* __restrict__ weights, int T, int E, int top_k) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    float v[ROUTE_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? __ldg(logits + (long long)t * E + e) : -INFINITY;
        mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    unsigned taken = 0;          // bit j: this lane's j-th expert already selected
    float my_w = 0.0f;           // lane k keeps the k-th selection
    int my_id = 0;
    float sum = 0.0f;
    for (int k = 0; k < top_k; ++k) {
        float best = -INFINITY;
        int best_e = 0x7FFFFFFF;
#pragma unroll
        for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
            const int e = lane + 32 * j;
            if (e < E && !((taken >> j) & 1u) && (v[j] > best || best_e == 0x7FFFFFFF)) {
                best = v[j];
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe != 0x7FFFFFFF && (best_e == 0x7FFFFFFF || ob > best || (ob == best && oe < best_e))) {
                best = ob;
                best_e = oe;
            }
        }
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        const float p = expf(best - mx);
        sum += p;
        if (lane == k) { my_w = p; my_id = best_e; }
    }
    if (lane < top_k) {
        ids[(long long)t * top_k + lane] = my_id;
        weights[(long long)t * top_k + lane] = __fdiv_rn(my_w, sum);
    }
}

// DeepSeek-V3 "no-aux" routing: s = sigmoid(logit), swb = s + bias; n_group groups of 32 experts (lane l of
// the warp holds expert g*32 + l of every group g); group score = sum of its two largest swb; the
// topk_group best groups are kept; among their experts the top_k largest swb win; weight =
// s / (sum of selected s + 1e-20) * rsf.  Ties -> lowest index.  One warp per token, n_group <= 16.
constexpr int DS_MAX_GROUPS = 16;
__device__ __forceinline__ float warp_max_f(float v) { return warp_max(v); }
__global__ void route_deepseek_kernel(const float* __restrict__ logits, const void* __restrict__ bias, int bias_is_bf16,
                                      int* __restrict__ ids, float* __restrict__ weights, int T, int n_group,
                                      int topk_group, int top_k, float rsf) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    const int E = n_group * 32;
    float s[DS_MAX_GROUPS], swb[DS_MAX_GROUPS], gscore[DS_MAX_GROUPS];
#pragma unroll
    for (int g = 0; g < DS_MAX_GROUPS; ++g) {
        if (g < n_group) {
            const int e = g * 32 + lane;
            const float b = bias_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[e])
                                         : reinterpret_cast<const float*>(bias)[e];
            s[g] = __fdiv_rn(1.0f, 1.0f + expf(-__ldg(logits + (long long)t * E + e)));
            swb[g] = s[g] + b;
            // two largest of the group: the maximum, then the maximum with its first holder removed
            const float m1 = warp_max(swb[g]);
            const unsigned holders = __ballot_sync(0xffffffffu, swb[g] == m1);
            const int first = __ffs(holders) - 1;
            const float m2 = warp_max(lane == first ? -INFINITY : swb[g]);
            gscore[g] = m1 + m2;
        } else {
            s[g] = 0.0f; swb[g] = -INFINITY; gscore[g] = -INFINITY;
        }
    }
    unsigned keep = 0;
    for (int k = 0; k < topk_group; ++k) {
        int best = -1;
        float bv = -INFINITY;
#pragma unroll
        for (int g = 0; g < DS_MAX_GROUPS; ++g)
            if (g < n_group && !((keep >> g) & 1u) && (best < 0 || gscore[g] > bv)) { best = g; bv = gscore[g]; }
        keep |= 1u << best;
    }
    unsigned taken = 0;
    float my_s = 0.0f, sum = 0.0f;
    int my_id = 0;
    for (int k = 0; k < top_k; ++k) {
        float best = -INFINITY;
        int best_e = 0x7FFFFFFF;
#pragma unroll
        for (int g = 0; g < DS_MAX_GROUPS; ++g) {
            if (g < n_group && ((keep >> g) & 1u) && !((taken >> g) & 1u) && (best_e == 0x7FFFFFFF || swb[g] > best)) {
                best = swb[g];
                best_e = g * 32 + lane;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe != 0x7FFFFFFF && (best_e == 0x7FFFFFFF || ob > best || (ob == best && oe < best_e))) {
                best = ob;
                best_e = oe;
            }
        }
        const int bg = best_e >> 5;
        float sel_s = 0.0f;
#pragma unroll
        for (int g = 0; g < DS_MAX_GROUPS; ++g) if (g == bg) sel_s = s[g];
        sel_s = __shfl_sync(0xffffffffu, sel_s, best_e & 31);
        if ((best_e & 31) == lane) taken |= 1u << bg;
        sum += sel_s;
        if (lane == k) { my_s = sel_s; my_id = best_e; }
    }
    if (lane < top_k) {
        ids[(long long)t * top_k + lane] = my_id;
        weights[(long long)t * top_k + lane] = __fdiv_rn(my_s, sum + 1e-20f) * rsf;
    }
}

// ------------------------------------------------------------------ permutation plan
// Pairs p = t*top_k + j are processed in chunks of 1024 (one block each, 32 warps in pair order).
// Step 1 (count):  chunk_counts[chunk][e] = pairs of the chunk routed to local expert e.
// Step 2 (scan):   per expert, exclusive scan over chunks (in place), counts[e], 128-aligned
//                  offsets[e], offsets[E] = total rows.
// Step 3 (place):  pos[p] = offsets[e] + chunk offset + rank inside the chunk (pair order kept ->
//                  the permutation is stable); src_pair[row] = p; grouped_layout[row] = e / -1.
constexpr int PLAN_CHUNK = 1024;

// per-warp histogram of the chunk into smem hist[32][E]; returns this pair's local expert (or -1)
// and its rank among equal experts inside the warp
__device__ __forceinline__ int plan_warp_hist(const int* __restrict__ ids, long long n_pairs, int e_lo,
                                              int E, int* hist, int* rank_in_warp) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const long long p = (long long)blockIdx.x * PLAN_CHUNK + threadIdx.x;
    int e = -1;
    if (p < n_pairs) {
        e = __ldg(ids + p) - e_lo;
        if (e < 0 || e >= E) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    *rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && *rank_in_warp == 0) hist[warp * E + e] = __popc(peers);
    __syncthreads();
    return e;
}

__global__ void plan_count_kernel(const int* __restrict__ ids, long long n_pairs, int e_lo, int E,
                                  int* __restrict__ chunk_counts) {
    extern __shared__ int hist[];
    int rank;
    plan_warp_hist(ids, n_pairs, e_lo, E, hist, &rank);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int s = 0;
#pragma unroll 8
        for (int w = 0; w < 32; ++w) s += hist[w * E + e];
        chunk_counts[(long long)blockIdx.x * E + e] = s;
    }
}

// one block; thread e scans its expert's column of chunk_counts, then thread 0.. build offsets
__global__ void plan_scan_kernel(int* __restrict__ chunk_counts, int n_chunks, int E, int align,
                                 int* __restrict__ counts, int* __restrict__ offsets) {
    extern __shared__ int cnt[];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int run = 0;
        for (int c = 0; c < n_chunks; ++c) {
            const int v = chunk_counts[(long long)c * E + e];
            chunk_counts[(long long)c * E + e] = run;
            run += v;
        }
        counts[e] = run;
        cnt[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = total;
            total += (cnt[e] + align - 1) / align * align;
        }
        offsets[E] = total;
    }
}

__global__ void plan_place_kernel(const int* __restrict__ ids, long long n_pairs, int e_lo, int E,
                                  const int* __restrict__ chunk_offsets, const int* __restrict__ counts,
                                  const int* __restrict__ offsets, int* __restrict__ pos,
                                  int* __restrict__ src_pair, int* __restrict__ grouped_layout,
                                  int cap_rows, const int* __restrict__ offsets2 = nullptr,
                                  int* __restrict__ order2 = nullptr) {
    // offsets2 / order2 (optional): a second stable ordering of the same pairs, order2[offsets2[e] + rank of the
    // pair among the pairs of expert e] = pair; dense (no padding rows)
    extern __shared__ int hist[];
    int rank;
    const int e = plan_warp_hist(ids, n_pairs, e_lo, E, hist, &rank);
    // exclusive scan over the 32 warps, per expert
    for (int x = threadIdx.x; x < E; x += blockDim.x) {
        int run = 0;
        for (int w = 0; w < 32; ++w) {
            const int v = hist[w * E + x];
            hist[w * E + x] = run;
            run += v;
        }
    }
    __syncthreads();
    const long long p = (long long)blockIdx.x * PLAN_CHUNK + threadIdx.x;
    if (p < n_pairs) {
        int row = -1;
        if (e >= 0) {
            const int within = chunk_offsets[(long long)blockIdx.x * E + e] + hist[(threadIdx.x >> 5) * E + e] + rank;
            if (order2 != nullptr) order2[offsets2[e] + within] = (int)p;
            row = offsets[e] + within;
            if (row >= cap_rows) row = -1;
            else if (src_pair != nullptr) src_pair[row] = (int)p;
        }
        pos[p] = row;
    }
    // grouped_layout / src_pair of padding rows: grid-stride over all capacity rows
    if (grouped_layout == nullptr) return;
    const int total = offsets[E];
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < cap_rows;
         r += (long long)gridDim.x * blockDim.x) {
        int g = -1;
        if (r < total) {
            int lo = 0, hi = E;                 // offsets[lo] <= r < offsets[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (offsets[mid] <= r) lo = mid; else hi = mid;
            }
            if (r - offsets[lo] < counts[lo]) g = lo;
        }
        grouped_layout[r] = g;
        if (g < 0 && src_pair != nullptr) src_pair[r] = -1;
    }
}

// Row gather into the contiguous grouped layout: for every row with src_pair >= 0 copy the token's
// e4m3 row (H bytes, 16-byte vectors) and its H/128 scales.  One warp per destination row.
// Source scales at [t*xs_r + b*xs_b]; destination scales at [row*ds_r + b*ds_b].
__global__ void gather_rows_kernel(const uint8_t* __restrict__ x, const float* __restrict__ xs,
                                   long long xs_r, long long xs_b, const int* __restrict__ src_pair,
                                   int top_k, uint8_t* __restrict__ a, float* __restrict__ as_,
                                   long long ds_r, long long ds_b, int rows, int H) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    const int p = __ldg(src_pair + r);
    if (p < 0) return;
    const int t = p / top_k;
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * H);
    uint4* dst = reinterpret_cast<uint4*>(a + (long long)r * H);
    for (int i = lane; i < (H >> 4); i += 32) dst[i] = __ldg(src + i);
    for (int b = lane; b < (H >> 7); b += 32) as_[r * ds_r + b * ds_b] = __ldg(xs + t * xs_r + b * xs_b);
}

// out[t, :] = bf16( sum_j w[t,j] * y[pos[t,j], :] ), fp32 multiply then add in slot order, pos < 0
// skipped.  One block per token, 8 bf16 (16 bytes) per thread per step.
__global__ void combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                               const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T,
                               int top_k, int H) {
    const int t = blockIdx.x;
    if (t >= T) return;
    __shared__ int s_pos[32];
    __shared__ float s_w[32];
    if (threadIdx.x < top_k) {
        s_pos[threadIdx.x] = pos[(long long)t * top_k + threadIdx.x];
        s_w[threadIdx.x] = w[(long long)t * top_k + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < (H >> 3); c += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int j = 0; j < top_k; ++j) {
            const int r = s_pos[j];
            if (r < 0) continue;
            const float wj = s_w[j];
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(y + (long long)r * H) + c);
            const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] = __fadd_rn(acc[2 * i], __fmul_rn(wj, __uint_as_float(u[i] << 16)));
                acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __fmul_rn(wj, __uint_as_float(u[i] & 0xFFFF0000u)));
            }
        }
        uint4 o;
        __nv_bfloat162 h;
        h = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
        reinterpret_cast<uint4*>(out + (long long)t * H)[c] = o;
    }
}

}  // namespace b200

// ====================================================================== expert parallelism
// One process per GPU.  Every rank owns E_local consecutive experts and a slice of the tokens.
// Receive buffers live in peer-mapped ("symmetric") memory: a rank's dispatch kernel STORES token
// rows straight into the owner rank's grouped-layout A buffer over NVLink, and the combine kernel
// LOADS the expert outputs it needs from the owners' Y buffers while it forms the weighted sum.
// No TMA touches peer memory; all peer traffic is plain 16-byte loads/stores.
namespace b200 {

constexpr int EP_MAX_WORLD = 8;

struct EpPeers {
    uint8_t* a[EP_MAX_WORLD];            // receive buffer of each rank: cap_rows records of `pitch` bytes,
                                         // each = H e4m3 bytes followed by H/128 fp32 scales
    float* sa[EP_MAX_WORLD];             // = a + H: the scales of row r at sa + r*pitch/4
    const __nv_bfloat16* y[EP_MAX_WORLD];// bf16 [cap_rows, H] expert outputs of each rank
    int* counts[EP_MAX_WORLD];           // int32 [world, E_total]: row s = pairs rank s routes to each expert
    int* flags[EP_MAX_WORLD];            // int32 [world]: barrier epochs written by each peer
    int* meta[EP_MAX_WORLD];             // int32 [cap_rows]: (source rank << 24) | source pair index of each row (written
                                         // by ep_dispatch_kernel; the dispatching GEMM keeps it inside the record instead)
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void red_relaxed_sys_add(int* p, int v) {
    asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Arrival counters live behind the barrier flags of each rank's symmetric region: flags[EP_ARRIVE_OFFSET + j] counts
// the rows that have landed for local expert j in the current forward.
constexpr int EP_ARRIVE_OFFSET = 64;
constexpr int EP_SEND_BUFFERS = 3;                 // token records in flight per sending warp
constexpr int EP_SEND_INFLIGHT = 6;                // bulk stores of a sending warp that may be on their way at once
constexpr int EP_SEND_BATCH = 24;                  // complete rows reported per system-scope fence
constexpr int EP_SEND_RING = 64;                   // arrival counters remembered until their rows are counted in (> INFLIGHT + BATCH + 2)
constexpr int EP_SEND_RECORD_MAX = 7424;           // bytes: H + H/32 + 4 for H <= 7168, rounded up to 128

// What the gate_up GEMM needs to carry the dispatch all-to-all itself (one sending warp per CTA): this rank's
// tokens and routes, where every pair goes (pos, from the exchange plan), the order to send them in (local
// expert index first, so that every rank's first expert is complete first), and both sides' arrival counters.
struct EpSend {
    uint8_t* a[EP_MAX_WORLD];            // receive buffers of all ranks (records of `pitch` bytes: row, scales, return address)
    int* arrive[EP_MAX_WORLD];           // arrival counters of all ranks, [E_local] each
    const uint8_t* x;                    // this rank's tokens, e4m3 [T, H]
    const float* xs;                     // their scales at [t * xs_r + b * xs_b]
    long long xs_r, xs_b, pitch;
    const int* ids;                      // [n_pairs] global expert of every pair
    const int* pos;                      // [n_pairs] destination row inside the owner's buffer
    const int* order;                    // [n_pairs] pairs in sending order
    const int* expected;                 // [E_local] rows this rank receives per local expert
    int n_pairs, top_k, E_local, H, cap_rows, rank;
};

// Cross-GPU barrier: thread s publishes `epoch` into peer s's flag slot for this rank, then waits
// (bounded: `limit_ns` of wall time, 2 s unless the host set another limit) until peer s's epoch shows up
// in the local slot; a wait that runs out ORs STATUS_TIMEOUT_PEER_FLAG into the status word and returns.
// Launched after the kernel whose peer stores must be visible; __threadfence_system orders them before the flag.
__global__ void ep_barrier_kernel(EpPeers peers, int rank, int world, int epoch, unsigned long long limit_ns,
                                  int* status) {
    const int s = threadIdx.x;
    if (s >= world) return;
    __threadfence_system();
    st_release_sys(peers.flags[s] + rank, epoch);
    const int* mine = peers.flags[rank] + s;
    const uint64_t t0 = globaltimer_ns();
    while (ld_acquire_sys(mine) < epoch) {
        if (globaltimer_ns() - t0 > limit_ns) {
            atomicOr(status, STATUS_TIMEOUT_PEER_FLAG);
            break;
        }
    }
}

// Publishes this rank's per-expert pair counts (E_total ints) into row `rank` of every peer's table, and clears this
// rank's arrival counters for the forward that begins: no peer can send a row of it before the barrier that follows
// this kernel, and every row of the previous forward was counted before that forward's gate_up GEMM finished.
__global__ void ep_publish_counts_kernel(EpPeers peers, const int* __restrict__ my_counts, int rank,
                                         int world, int E_total) {
    for (int j = threadIdx.x; j < E_total / world; j += blockDim.x) peers.flags[rank][EP_ARRIVE_OFFSET + j] = 0;
    for (int i = threadIdx.x; i < world * E_total; i += blockDim.x) {
        const int d = i / E_total, e = i % E_total;
        peers.counts[d][rank * E_total + e] = my_counts[e];
    }
}

// From the gathered table counts_all[world][E_total] (local copy) derive, in one block:
//   recv side: offsets[E_local+1] of this rank's experts (each padded to `align` rows)
//   send side: dst_base[E_total] = first destination row, in the owner's buffer, of this rank's
//              pairs for expert e (owner's expert start + rows of lower-ranked senders)
// If the rows this rank is about to receive (aligned) exceed its capacity, STATUS_CAPACITY is raised: the
// dispatch kernels of the senders drop the rows that do not fit.
__global__ void ep_plan_kernel(const int* __restrict__ counts_all, int rank, int world, int E_total,
                               int E_local, int align, int cap_rows, int* __restrict__ counts_local,
                               int* __restrict__ offsets, int* __restrict__ dst_base, int* __restrict__ send_base,
                               int* status) {
    extern __shared__ int sh[];           // total[E_total], start[E_total]
    int* total = sh;
    int* start = sh + E_total;
    for (int e = threadIdx.x; e < E_total; e += blockDim.x) {
        int t = 0;
        for (int s = 0; s < world; ++s) t += counts_all[s * E_total + e];
        total[e] = t;
    }
    __syncthreads();
    // per owner rank: exclusive scan of aligned totals over its E_local experts
    for (int d = threadIdx.x; d < world; d += blockDim.x) {
        int run = 0;
        for (int j = 0; j < E_local; ++j) {
            const int e = d * E_local + j;
            start[e] = run;
            run += (total[e] + align - 1) / align * align;
        }
        if (d == rank) {
            offsets[E_local] = run;
            if (run > cap_rows) atomicOr(status, STATUS_CAPACITY);
        }
    }
    __syncthreads();
    // sending order of this rank's pairs: local expert index first, destination rank second, so that expert 0 of
    // every rank is complete first; send_base[e] = first slot of the pairs for global expert e (may be NULL)
    if (send_base != nullptr && threadIdx.x == 0) {
        int run = 0;
        for (int j = 0; j < E_local; ++j)
            for (int d = 0; d < world; ++d) {
                const int e = d * E_local + j;
                send_base[e] = run;
                run += counts_all[rank * E_total + e];
            }
    }
    for (int e = threadIdx.x; e < E_total; e += blockDim.x) {
        int before = 0;
        for (int s = 0; s < rank; ++s) before += counts_all[s * E_total + e];
        dst_base[e] = start[e] + before;
        if (e / E_local == rank) {
            offsets[e - rank * E_local] = start[e];
            counts_local[e - rank * E_local] = total[e];
        }
    }
}

// grouped_layout of the receive buffer: row r belongs to local expert e iff
// offsets[e] <= r < offsets[e] + counts_local[e]; everything else is padding (-1).
__global__ void ep_layout_kernel(const int* __restrict__ offsets, const int* __restrict__ counts_local,
                                 int E_local, int* __restrict__ grouped_layout, int cap_rows) {
    const int total = offsets[E_local];
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < cap_rows;
         r += (long long)gridDim.x * blockDim.x) {
        int g = -1;
        if (r < total) {
            int lo = 0, hi = E_local;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (offsets[mid] <= r) lo = mid; else hi = mid;
            }
            if (r - offsets[lo] < counts_local[lo]) g = lo;
        }
        grouped_layout[r] = g;
    }
}

// Dispatch: pair p = t*top_k + j goes to row pos[p] of the rank that owns expert ids[p].
// Receive rows are `pitch` bytes apart and hold the H e4m3 bytes followed by the H/128 fp32 scales, so one
// token -> one contiguous record.  One warp per token: the record is assembled once in shared memory (bulk
// load of the e4m3 row + the scales) and leaves as ONE bulk store of H + H/32 bytes per destination, issued
// by lane j for destination j.  NVLink then carries large packets instead of 16-byte stores.
constexpr int DISPATCH_WARPS = 4;
constexpr int EP_DISPATCH_MAX_SMEM = 64 * 1024;
__global__ void ep_dispatch_kernel(EpPeers peers, const uint8_t* __restrict__ x, const float* __restrict__ xs,
                                   long long xs_r, long long xs_b, const int* __restrict__ ids,
                                   const int* __restrict__ pos, long long n_pairs, int top_k, int E_local,
                                   int H, int cap_rows, int rank, long long pitch, int* status) {
    extern __shared__ __align__(128) uint8_t dsm[];
    __shared__ uint64_t bars[DISPATCH_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * DISPATCH_WARPS + warp;
    const int rec = (H + (H >> 5) + 15) & ~15;         // record bytes: row + scales, rounded up to 16
    uint8_t* buf = dsm + (long long)warp * rec;
    const uint32_t bar = smem_u32(&bars[warp]);
    if (lane == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncwarp();
    if (t * top_k >= n_pairs) return;
    if (lane == 0) {
        mbar_arrive_expect_tx(bar, (uint32_t)H);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(buf)), "l"(x + t * H), "r"(H), "r"(bar) : "memory");
    }
    float* sbuf = reinterpret_cast<float*>(buf + H);
    for (int b = lane; b < (H >> 7); b += 32) sbuf[b] = __ldg(xs + t * xs_r + (long long)b * xs_b);
    // bounded wait for the row (2 s), then make the generic-proxy scale writes visible to the bulk engine
    {
        bool ok = mbar_try_wait(bar, 0);
        const uint64_t t0 = globaltimer_ns();
        while (!ok) {
            ok = mbar_try_wait(bar, 0);
            if (!ok && globaltimer_ns() - t0 > kWaitLimitNs) { atomicOr(status, STATUS_TIMEOUT_SMEM_FULL); break; }
        }
        if (!__all_sync(0xffffffffu, ok)) return;
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane < top_k) {
        const long long p = t * top_k + lane;
        const int row = __ldg(pos + p);
        if (row >= cap_rows) atomicOr(status, STATUS_CAPACITY);       // the owner's buffer is too small: row dropped
        if (row >= 0 && row < cap_rows) {
            const int d = __ldg(ids + p) / E_local;
            uint8_t* dst = peers.a[d] + (long long)row * pitch;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(dst), "r"(smem_u32(buf)), "r"(rec) : "memory");
            // where this row's result has to go back to: lets the owner's down GEMM send it straight to our slot
            peers.meta[d][row] = (rank << 24) | (int)p;
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}

// Combine: out[t,:] = bf16( sum_j w[t,j] * Y_owner(ids[t,j])[pos[t,j], :] ), rows fetched from the
// owners' buffers with 16-byte peer loads; fp32 multiply then add in slot order.
__global__ void ep_combine_kernel(EpPeers peers, const int* __restrict__ ids, const int* __restrict__ pos,
                                  const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T, int top_k,
                                  int E_local, int H) {
    const int t = blockIdx.x;
    if (t >= T) return;
    __shared__ const __nv_bfloat16* s_row[32];
    __shared__ float s_w[32];
    if (threadIdx.x < top_k) {
        const int r = pos[(long long)t * top_k + threadIdx.x];
        const int d = ids[(long long)t * top_k + threadIdx.x] / E_local;
        s_row[threadIdx.x] = r < 0 ? nullptr : peers.y[d] + (long long)r * H;
        s_w[threadIdx.x] = w[(long long)t * top_k + threadIdx.x];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < (H >> 3); c += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        // peer loads take microseconds: issue a batch of eight before the first is consumed
        for (int j0 = 0; j0 < top_k; j0 += 8) {
            uint4 raw[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const __nv_bfloat16* rp = (j0 + jj < top_k) ? s_row[j0 + jj] : nullptr;
                raw[jj] = rp != nullptr ? *(reinterpret_cast<const uint4*>(rp) + c) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                if (j0 + jj < top_k && s_row[j0 + jj] != nullptr) {
                    const float wj = s_w[j0 + jj];
                    const uint32_t u[4] = {raw[jj].x, raw[jj].y, raw[jj].z, raw[jj].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[2 * i] = __fadd_rn(acc[2 * i], __fmul_rn(wj, __uint_as_float(u[i] << 16)));
                        acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __fmul_rn(wj, __uint_as_float(u[i] & 0xFFFF0000u)));
                    }
                }
            }
        }
        uint4 o;
        __nv_bfloat162 h;
        h = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
        reinterpret_cast<uint4*>(out + (long long)t * H)[c] = o;
    }
}

}  // namespace b200
