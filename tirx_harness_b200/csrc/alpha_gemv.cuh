// Decode-regime MoE layer for a handful of tokens (a few dozen routes): two CUDA-core kernels that stream each
// routed expert's weights once, spread over all SMs.  With 1-16 tokens a 128-row tensor-core tile is all padding
// and a launch costs more than the weights take to read, so this path has no plan, no gather and no separate
// reduction: five launches become two.
//
//   alpha_gemv_gate_up_kernel   CTA = (route, slice of 16 gate + 16 up features).  Quantises the token's bf16 row
//                               itself (1x128, the task's rule), then per feature: exact e4m3 products summed in
//                               fp32 per 128-K block, promoted with sfa[kb]*sfb[block,kb] in increasing kb (the
//                               block-promote model of the tensor-core path), SiLU(gate)*up in fp32 -> act[route].
//   alpha_gemv_down_kernel      CTA = (token, 32 output features).  Orders the token's routes by expert id, and per
//                               route requantises act (1x128), multiplies by the expert's W2 rows, promotes, scales by
//                               fp32(weight*rsf), rounds to bf16 and adds to a bf16 accumulator with a rounding per
//                               update: the task's reduction, fused.
#pragma once

#include <cuda_fp16.h>

#include "alpha_moe.cuh"
#include "moe_ops.cuh"

namespace b200 {

// 16 e4m3 bytes (one uint4) -> 16 floats
__device__ __forceinline__ void e4m3x16_to_float(const uint4& raw, float (&out)[16]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xFFFFu), __NV_E4M3);
        const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
        out[4 * i + 0] = a.x; out[4 * i + 1] = a.y; out[4 * i + 2] = b.x; out[4 * i + 3] = b.y;
    }
}

__device__ __forceinline__ float e4m3_round_trip(float v) {      // decode(e4m3(v)), v already clamped
    const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    const __half_raw h = __nv_cvt_fp8_to_halfraw(q, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}

constexpr int AGV_SLICES = 8;          // CTAs per route in the gate_up kernel: 16 gate + 16 up features each
constexpr int AGV_MAX_H = 4096;        // the token row is held in shared memory as floats

// x bf16 [M, H]; w13 e4m3 [E, 256, H] rows [gate; up]; s13 f32 [E, 2, H/128]; act f32 [n_pairs, 128];
// g1 f32 [n_pairs, 256] (gate_up, kept for inspection).  256 threads.
__global__ void __launch_bounds__(256)
alpha_gemv_gate_up_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, const uint8_t* __restrict__ w13,
                          const float* __restrict__ s13, int top_k, int E, int H, float* __restrict__ act,
                          float* __restrict__ g1) {
    __shared__ float xq[AGV_MAX_H];            // dequantised-to-code values: decode(e4m3(x/s)), exact small floats
    __shared__ float xs[AGV_MAX_H / 128];      // the row's block scales
    const int p = blockIdx.x / AGV_SLICES, slice = blockIdx.x % AGV_SLICES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = H >> 7;
    // First kernel of a call: its inputs (ids, the token rows) may be the output of whatever ran before it in
    // the stream -- the previous call's `out`, a router or norm kernel -- so nothing is read before the wait.
    // Dependents are released only after it: the second kernel reads ids and weights ahead of its own wait,
    // which is safe exactly because it cannot start before everything older than this kernel has completed.
    pdl_wait();
    pdl_launch_dependents();
    const int e = __ldg(ids + p);
    const bool live = e >= 0 && e < E;
    // warp w: activation features i0, i0+1 of this slice -> 4 rows of W13 (gate i0, up i0, gate i0+1, up i0+1).
    // A 128-K block is 8 consecutive 16-byte chunks = 8 consecutive lanes; 32 lanes cover 4 blocks per round; the
    // 16 loads of four rounds of the four rows, and the expert's block scales, are requested before anything else
    // (the kernel is a chain of HBM round trips otherwise): they travel while the token row is quantised.
    const int chunks = H >> 4;
    const int i0 = slice * 16 + warp * 2;
    const uint4* wrow[4];
    uint4 raw[4][4];
    float sreg[2] = {0.0f, 0.0f};              // lane (half * 16 + kb % 16), register kb / 16: scale of (half, kb)
    if (live) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int half = r & 1, i = i0 + (r >> 1);
            wrow[r] = reinterpret_cast<const uint4*>(w13 + ((long long)e * 256 + half * 128 + i) * H);
        }
#pragma unroll
        for (int rd = 0; rd < 4; ++rd) {
            const int c = rd * 32 + lane;
#pragma unroll
            for (int r = 0; r < 4; ++r) raw[rd][r] = c < chunks ? __ldg(wrow[r] + c) : make_uint4(0, 0, 0, 0);
        }
        const float* sbase = s13 + ((long long)e * 2 + (lane >> 4)) * KB;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int kb = (lane & 15) + 16 * j;
            if (kb < KB) sreg[j] = __ldg(sbase + kb);
        }
    }
    // 1x128 quantisation of the token's row
    const __nv_bfloat16* xrow = x + (long long)(p / top_k) * H;
    for (int b = warp; b < KB; b += 8) {
        float v[4], sc;
        bf16x4_to_float(__ldg(reinterpret_cast<const uint2*>(xrow + b * 128 + lane * 4)), v);
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = warp_max(amax);
        sc = __fdiv_rn(fmaxf(amax, 1.0e-8f), 448.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) xq[b * 128 + lane * 4 + i] = e4m3_round_trip(clamp448(__fdiv_rn(v[i], sc)));
        if (lane == 0) xs[b] = sc;
    }
    __syncthreads();
    if (!live) return;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int c0 = 0; c0 < chunks; c0 += 128) {
        if (c0 > 0) {
#pragma unroll
            for (int rd = 0; rd < 4; ++rd) {
                const int c = c0 + rd * 32 + lane;
#pragma unroll
                for (int r = 0; r < 4; ++r) raw[rd][r] = c < chunks ? __ldg(wrow[r] + c) : make_uint4(0, 0, 0, 0);
            }
        }
        const float sv = c0 == 0 ? sreg[0] : sreg[1];          // 128 chunks = 16 K blocks per pass
#pragma unroll
        for (int rd = 0; rd < 4; ++rd) {
            const int c = c0 + rd * 32 + lane;
            const float* xv = xq + (c < chunks ? c : 0) * 16;
            float part[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                float wv[16];
                e4m3x16_to_float(raw[rd][r], wv);
                float pr = 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) pr = fmaf(xv[j], wv[j], pr);
                pr += __shfl_xor_sync(0xffffffffu, pr, 1);
                pr += __shfl_xor_sync(0xffffffffu, pr, 2);
                pr += __shfl_xor_sync(0xffffffffu, pr, 4);
                part[r] = pr;
            }
            // promotion in increasing kb: the four blocks of this round, one after the other
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int kb = ((c0 + rd * 32) >> 3) + g;
                if (kb < KB) {                                   // warp-uniform
                    const float sx = xs[kb];
                    const float sw_gate = __shfl_sync(0xffffffffu, sv, kb & 15);
                    const float sw_up = __shfl_sync(0xffffffffu, sv, 16 + (kb & 15));
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        acc[r] = fmaf(__shfl_sync(0xffffffffu, part[r], g * 8), __fmul_rn(sx, (r & 1) ? sw_up : sw_gate), acc[r]);
                }
            }
        }
    }
    if (lane < 2) {
        const int i = i0 + lane;
        const float g = lane == 0 ? acc[0] : acc[2], u = lane == 0 ? acc[1] : acc[3];
        g1[(long long)p * 256 + i] = g;
        g1[(long long)p * 256 + 128 + i] = u;
        act[(long long)p * 128 + i] = __fmul_rn(silu_f32(g), u);
    }
}

// act f32 [n_pairs, 128]; w2 e4m3 [E, H, 128]; s2w f32 [E, H/128, 1]; out bf16 [M, H].
// CTA = (token, 32 output features), 4 warps x 8 features.
__global__ void __launch_bounds__(128)
alpha_gemv_down_kernel(const float* __restrict__ act, const int* __restrict__ ids, const float* __restrict__ wts,
                       const uint8_t* __restrict__ w2, const float* __restrict__ s2w, float rsf, int top_k, int E, int H,
                       __nv_bfloat16* __restrict__ out) {
    __shared__ int s_pair[32], s_exp[32];
    __shared__ float s_scale[32], s_wsc[32];
    __shared__ int s_n;
    const int tiles = H >> 5;
    const int t = blockIdx.x / tiles, h0 = (blockIdx.x % tiles) * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    // ids / weights are read before the wait below: the gate_up kernel in front of this one releases its dependents
    // only after everything older in the stream has completed, so they are final by the time this CTA exists.
    if (warp == 0) {
        // lane j owns route j: its place in the order is the number of live routes with a smaller (expert, j)
        const bool have = lane < top_k;
        const int e = have ? __ldg(ids + t * top_k + lane) : -1;
        const float wt = have ? __ldg(wts + t * top_k + lane) : 0.0f;
        const bool live = have && e >= 0 && e < E;
        const float wsc = live ? __ldg(s2w + (long long)e * (H >> 7) + (h0 >> 7)) : 0.0f;    // this tile's W2 block scale
        const unsigned live_mask = __ballot_sync(0xffffffffu, live);
        int rank = 0;
        for (int o = 0; o < top_k; ++o) {
            const int eo = __shfl_sync(0xffffffffu, e, o);
            if (((live_mask >> o) & 1u) && (eo < e || (eo == e && o < lane))) ++rank;
        }
        if (live) {
            s_pair[rank] = t * top_k + lane;
            s_exp[rank] = e;
            s_scale[rank] = __fmul_rn(wt, rsf);
            s_wsc[rank] = wsc;
        }
        if (lane == 0) s_n = __popc(live_mask);
    }
    __syncthreads();
    const int n = s_n;
    const int hw = h0 + warp * 8;
    constexpr int R = 10;          // routes in flight per pass: the task's top-10 in one
    float accv[8];
#pragma unroll
    for (int f = 0; f < 8; ++f) accv[f] = 0.0f;
    for (int k0 = 0; k0 < n; k0 += R) {
        // W2 rows of all routes of the pass are requested before the wait (weights do not depend on the kernel in
        // front), the activations right after it: one HBM round trip per pass instead of one per four routes
        uint32_t wraw[R][8];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int k = k0 + r < n ? k0 + r : n - 1;
            const uint8_t* wbase = w2 + ((long long)s_exp[k] * H + hw) * 128;
#pragma unroll
            for (int f = 0; f < 8; ++f) wraw[r][f] = __ldg(reinterpret_cast<const uint32_t*>(wbase + f * 128) + lane);
        }
        if (k0 == 0) pdl_wait();                                 // act is written by the gate_up kernel just before this one
        float4 a[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int k = k0 + r < n ? k0 + r : n - 1;
            a[r] = __ldcg(reinterpret_cast<const float4*>(act + (long long)s_pair[k] * 128) + lane);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (k0 + r < n) {                                   // warp-uniform
                const int k = k0 + r;
                // requantise the route's 128 activations (lane holds 4): s = max(amax,1e-8)/448, code = e4m3(clamp(a/s))
                float amax = warp_max(fmaxf(fmaxf(fabsf(a[r].x), fabsf(a[r].y)), fmaxf(fabsf(a[r].z), fabsf(a[r].w))));
                const float sc = __fdiv_rn(fmaxf(amax, 1.0e-8f), 448.0f);
                const float q0 = e4m3_round_trip(clamp448(__fdiv_rn(a[r].x, sc)));
                const float q1 = e4m3_round_trip(clamp448(__fdiv_rn(a[r].y, sc)));
                const float q2 = e4m3_round_trip(clamp448(__fdiv_rn(a[r].z, sc)));
                const float q3 = e4m3_round_trip(clamp448(__fdiv_rn(a[r].w, sc)));
                const float sab = __fmul_rn(sc, s_wsc[k]);
                const float ws = s_scale[k];
#pragma unroll
                for (int f = 0; f < 8; ++f) {
                    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wraw[r][f] & 0xFFFFu), __NV_E4M3);
                    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wraw[r][f] >> 16), __NV_E4M3);
                    const float2 w01 = __half22float2(*reinterpret_cast<const __half2*>(&lo));
                    const float2 w23 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
                    float part = fmaf(q3, w23.y, fmaf(q2, w23.x, fmaf(q1, w01.y, __fmul_rn(q0, w01.x))));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                    const float d = fmaf(part, sab, 0.0f);
                    accv[f] = round_bf16(accv[f] + round_bf16(__fmul_rn(d, ws)));
                }
            }
        }
    }
    if (n == 0) pdl_wait();
    if (lane < 8) {
        float v = accv[0];
#pragma unroll
        for (int f = 1; f < 8; ++f) v = lane == f ? accv[f] : v;
        out[(long long)t * H + h0 + warp * 8 + lane] = __float2bfloat16_rn(v);
    }
}

}  // namespace b200
