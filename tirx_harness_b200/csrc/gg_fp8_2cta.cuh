// m-grouped FP8 block-scaled GEMM, CTA-pair version (tcgen05 cta_group::2).
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 output tile:
//   CTA r loads A rows [128 r, 128 r + 128) of the tile and B rows (= output columns) [128 r, 128 r + 128);
//   the leader (r = 0) issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32): the tensor cores of both
//   SMs read A from their own shared memory and B from both, and each SM's TMEM receives its 128 rows
//   x 256 columns.  Per SM the operand traffic drops from 48 KB to 32 KB per 128-K block, which is what
//   lets six stages cover the load latency.  No load is multicast: each CTA fetches what it stages.
// Roles per CTA (384 threads): warp 0 TMA producer, warp 1 MMA issuer (leader only; allocates TMEM in
// both), warp 2 block-scale loader, warps 4..11 promotion + epilogue of this CTA's 128 rows.
// Barriers: operand `full` lives in the leader (both producers arrive on it, CTA 1 remotely); `empty`
// and `tmem_full` are per CTA and are signalled by a multicast tcgen05.commit; `tmem_empty` lives in
// the leader and collects the 16 epilogue warps of the pair.  Every wait is bounded.
#pragma once

#include "gg_fp8.cuh"

namespace b200 {

namespace gg2 {
constexpr int BM = 128;               // rows per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BK = 128;
constexpr int STAGES = 6;
constexpr int ACC_STAGES = 2;
constexpr int THREADS = 384;
constexpr int A_STAGE_BYTES = BM * BK;          // 16 KB
constexpr int B_STAGE_BYTES = (BN / 2) * BK;    // 16 KB: this CTA's half of the B tile
constexpr int TMEM_COLS = 512;
constexpr int SMEM_TILE_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int SF_SLOTS = 8;
constexpr int SF_SLOT_FLOATS = 132;
constexpr int OFF_BARS = SMEM_TILE_BYTES;
constexpr int OFF_SF = OFF_BARS + 512;
constexpr int OFF_PREFIX = OFF_SF + SF_SLOTS * SF_SLOT_FLOATS * 4;
constexpr int SMEM_BYTES = OFF_PREFIX + (gg::MAX_MASKED_GROUPS + 1) * 4 + 12 + 1024;
}  // namespace gg2

// ------------------------------------------------------------------ cluster helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;"
                 ::"r"(cluster_bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// No memory ordering attached: for signals that only hand back TMEM (ordered by tcgen05 fences).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load whose completion may be signalled on the peer CTA's mbarrier (cta_group::2 form, no multicast)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* tmap, uint32_t cluster_bar,
                                                 int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(tmap), "r"(cluster_bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result_addr, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_result_addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f8f6f4_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on the mbarrier at the same shared-memory offset in every CTA of `mask` once all earlier
// tcgen05 operations of this thread are complete
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask) : "memory");
}

// Static persistent schedule over CLUSTERS.  Both CTAs of a pair and all their warps walk the same
// sequence.  A tile = (256-row block, column block, group); tile.m0 is THIS CTA's first row.  In the
// contiguous layout the block's 256 layout entries (8 per lane) are fetched one tile ahead.
template <bool MASKED>
struct PairScheduler {
    const GGParams& p;
    const int* prefix;   // masked: prefix of 256-row blocks per group
    int t, lane, prev_g, total, stride, rank;
    int vals[8];

    __device__ __forceinline__ void fetch() {
        if (t < total) {
            const int m0 = (t / p.num_n_blocks) * 256;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = m0 + lane * 8 + j;
                vals[j] = r < p.M ? __ldg(p.layout + r) : -1;
            }
        }
    }
    __device__ __forceinline__ int next_group(int after) const {
        int best = INT_MAX;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (vals[j] > after && vals[j] < p.G && vals[j] < best) best = vals[j];
        return __reduce_min_sync(0xffffffffu, best);
    }

    __device__ __forceinline__ PairScheduler(const GGParams& p_, const int* prefix_, int lane_, int rank_)
        : p(p_), prefix(prefix_), t(blockIdx.x >> 1), lane(lane_), prev_g(-1), stride(gridDim.x >> 1), rank(rank_) {
        if (MASKED) {
            total = prefix_[p_.G] * p_.num_n_blocks;
        } else {
            int rows = p_.M;
            if (p_.rows_used != nullptr) {
                int used = __ldg(p_.rows_used);
                rows = used < 0 ? 0 : (used > p_.M ? p_.M : used);
            }
            total = ((rows + 255) / 256) * p_.num_n_blocks;
            fetch();
        }
    }

    __device__ __forceinline__ bool next(Tile& tile) {
        if (MASKED) {
            if (t >= total) return false;
            int mbg = t / p.num_n_blocks;
            int lo = 0, hi = p.G;
            while (hi - lo > 1) {
                int mid = (lo + hi) >> 1;
                if (prefix[mid] <= mbg) lo = mid; else hi = mid;
            }
            int mb = mbg - prefix[lo];
            tile.g = lo;
            tile.n_blk = t % p.num_n_blocks;
            const int row0 = mb * 256 + rank * gg2::BM;          // first row of this CTA inside the group
            tile.m0 = lo * p.M + row0;
            int mm = __ldg(p.layout + lo);
            if (mm > p.M) mm = p.M;
            int left = mm - row0;
            tile.rows = left < 0 ? 0 : (left < gg2::BM ? left : gg2::BM);
            t += stride;
            return true;
        } else {
            while (t < total) {
                const int g = next_group(prev_g);
                if (g == INT_MAX) {
                    t += stride;
                    prev_g = -1;
                    fetch();
                    continue;
                }
                tile.m0 = (t / p.num_n_blocks) * 256 + rank * gg2::BM;
                tile.n_blk = t % p.num_n_blocks;
                tile.g = g;
                tile.rows = gg2::BM;
                prev_g = g;
                if (next_group(g) == INT_MAX) {
                    t += stride;
                    prev_g = -1;
                    fetch();
                }
                return true;
            }
            return false;
        }
    }
};

template <bool MASKED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gg2::THREADS, 1)
gg_fp8_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const GGParams p, int* status) {
    using namespace gg2;
    if (p.mode_flag != nullptr && *p.mode_flag == 0) return;
    extern __shared__ uint8_t smem_raw[];
    // the dynamic shared window starts at the same offset in both CTAs, so aligned offsets match too
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
    // [0,S) full (leader's is used), [S,2S) empty, then 2 tmem_full, 2 tmem_empty (leader's is used),
    // then SF_SLOTS scale-full and SF_SLOTS scale-empty
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC_STAGES + 2 * SF_SLOTS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    float* sf_ring = reinterpret_cast<float*>(smem + OFF_SF);
    int* prefix = reinterpret_cast<int*>(smem + OFF_PREFIX);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();

    const uint32_t full_bar = smem_u32(bars);
    const uint32_t empty_bar = smem_u32(bars + STAGES);
    const uint32_t tfull_bar = smem_u32(bars + 2 * STAGES);
    const uint32_t tempty_bar = smem_u32(bars + 2 * STAGES + ACC_STAGES);
    const uint32_t sffull_bar = smem_u32(bars + 2 * STAGES + 2 * ACC_STAGES);
    const uint32_t sfempty_bar = smem_u32(bars + 2 * STAGES + 2 * ACC_STAGES + SF_SLOTS);
    // the leader's copies, as shared::cluster addresses usable from either CTA
    const uint32_t leader_full_bar = map_to_cta(full_bar, 0);
    const uint32_t leader_tempty_bar = map_to_cta(tempty_bar, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);        // the leader's producer arrives; both CTAs' copies complete_tx here
            mbar_init(empty_bar + 8 * s, 1);       // multicast commit
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(tfull_bar + 8 * s, 1);       // multicast commit
            mbar_init(tempty_bar + 8 * s, 16);     // 8 epilogue warps in each CTA
        }
        for (int s = 0; s < SF_SLOTS; ++s) {
            mbar_init(sffull_bar + 8 * s, 32);
            mbar_init(sfempty_bar + 8 * s, 8);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (MASKED) {
        if (warp == 3) {
            int running = 0;
            for (int base = 0; base < p.G; base += 32) {
                int g = base + lane;
                int mm = 0;
                if (g < p.G) {
                    mm = __ldg(p.layout + g);
                    mm = mm < 0 ? 0 : (mm > p.M ? p.M : mm);
                }
                int blocks = (mm + 255) / 256;
                int incl = blocks;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += v;
                }
                if (g < p.G) prefix[g] = running + incl - blocks;
                running += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) prefix[p.G] = running;
        }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_base_slot), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // both CTAs' barriers are initialised before anyone signals the peer
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const int KB = p.num_k_blocks;

    if (warp < 4) {
        setmaxnreg_dec<88>();
        if (warp == 0) {
            // ------------------------------------------------ TMA producer (both CTAs)
            PairScheduler<MASKED> sched(p, prefix, lane, rank);
            Tile tile;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            while (ok && sched.next(tile)) {
                const int b_row = tile.g * p.N + tile.n_blk * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < KB; ++kb) {
                    ok = mbar_wait_warp(empty_bar + 8 * stage, phase ^ 1, abort_flag, status,
                                        STATUS_TIMEOUT_SMEM_EMPTY);
                    if (!ok) break;
                    if (lane == 0) {
                        const uint32_t fb = leader_full_bar + 8 * stage;
                        if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * stage, 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
                        tma_load_2d_pair(smem_u32(smem_a + stage * A_STAGE_BYTES), &tmap_a, fb, kb * BK, tile.m0);
                        tma_load_2d_pair(smem_u32(smem_b + stage * B_STAGE_BYTES), &tmap_b, fb, kb * BK, b_row);
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        } else if (warp == 1 && rank == 0) {
            // ------------------------------------------------ MMA issuer (leader CTA only)
            PairScheduler<MASKED> sched(p, prefix, lane, rank);
            Tile tile;
            constexpr uint32_t idesc = make_idesc_e4m3_f32(2 * BM, BN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            while (ok && sched.next(tile)) {
                for (int kb = 0; kb < KB; ++kb) {
                    ok = mbar_wait_warp(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, status,
                                        STATUS_TIMEOUT_TMEM_EMPTY);
                    if (!ok) break;
                    ok = mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, status,
                                        STATUS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        const uint64_t adesc = make_smem_desc_sw128(smem_u32(smem_a + stage * A_STAGE_BYTES));
                        const uint64_t bdesc = make_smem_desc_sw128(smem_u32(smem_b + stage * B_STAGE_BYTES));
                        const uint32_t tmem_d = tmem_base + acc * BN;
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k)
                            umma_f8f6f4_pair(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
                        umma_commit_pair(empty_bar + 8 * stage, 3);    // both producers may refill the stage
                        umma_commit_pair(tfull_bar + 8 * acc, 3);      // both epilogues may drain the block
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
                }
            }
        } else if (warp == 2) {
            // ------------------------------------------------ scale loader (both CTAs, own rows)
            PairScheduler<MASKED> sched(p, prefix, lane, rank);
            Tile tile;
            uint32_t slot = 0, sphase = 0;
            bool ok = true;
            while (ok && sched.next(tile)) {
                const float* rp[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int r = tile.m0 + lane + 32 * j;
                    if (r >= p.rows_total) r = p.rows_total - 1;
                    rp[j] = p.sfa + (long long)r * p.sfa_sr;
                }
                int nb = ((tile.n_blk * BN) >> 7) + (lane & 1);
                if (nb >= p.nb128) nb = p.nb128 - 1;
                const float* bp = p.sfb + ((long long)tile.g * p.nb128 + nb) * KB;
                for (int kb0 = 0; kb0 < KB && ok; kb0 += 4) {
                    float v[4][4], b[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (kb0 + u < KB) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) v[u][j] = __ldg(rp[j] + (long long)(kb0 + u) * p.sfa_sk);
                            b[u] = __ldg(bp + kb0 + u);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (ok && kb0 + u < KB) {
                            ok = mbar_wait_warp(sfempty_bar + 8 * slot, sphase ^ 1, abort_flag, status,
                                                STATUS_TIMEOUT_SF_EMPTY);
                            if (ok) {
                                float* dst = sf_ring + slot * SF_SLOT_FLOATS;
#pragma unroll
                                for (int j = 0; j < 4; ++j) dst[lane + 32 * j] = v[u][j];
                                if (lane < 2) dst[128 + lane] = b[u];
                                mbar_arrive(sffull_bar + 8 * slot);
                                if (++slot == SF_SLOTS) { slot = 0; sphase ^= 1; }
                            }
                        }
                    }
                }
            }
        }
    } else {
        // ---------------------------------------------------- promotion + epilogue (both CTAs)
        setmaxnreg_inc<208>();
        const int ew = warp - 4;
        const int quarter = warp & 3;
        const int half = ew >> 2;
        const int row_in_tile = quarter * 32 + lane;
        PairScheduler<MASKED> sched(p, prefix, lane, rank);
        Tile tile;
        uint32_t acc = 0, acc_phase = 0, slot = 0, sphase = 0;
        bool ok = true;
        while (ok && sched.next(tile)) {
            const int n0 = tile.n_blk * BN + half * 128;
            const int row = tile.m0 + row_in_tile;
            bool row_valid;
            if (MASKED) row_valid = row_in_tile < tile.rows;
            else row_valid = (row < p.M) && (__ldg(p.layout + row) == tile.g);

            unsigned long long accr[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) accr[j] = 0ull;

            for (int kb = 0; kb < KB; ++kb) {
                ok = mbar_wait_warp(sffull_bar + 8 * slot, sphase, abort_flag, status, STATUS_TIMEOUT_SF_FULL);
                if (!ok) break;
                const float* sfp = sf_ring + slot * SF_SLOT_FLOATS;
                const float s = sfp[row_in_tile] * sfp[128 + half];
                __syncwarp();
                if (lane == 0) mbar_arrive(sfempty_bar + 8 * slot);
                if (++slot == SF_SLOTS) { slot = 0; sphase ^= 1; }
                const unsigned long long s2 = pack_f32x2(s, s);

                ok = mbar_wait_warp(tfull_bar + 8 * acc, acc_phase, abort_flag, status,
                                    STATUS_TIMEOUT_TMEM_FULL);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN + half * 128;
                uint32_t v0[16], v1[16];
                tmem_ld_32x32b_x16(taddr, v0);
#pragma unroll
                for (int c = 0; c < 8; c += 2) {
                    tmem_ld_wait(v0);
                    tmem_ld_32x32b_x16(taddr + (c + 1) * 16, v1);
#pragma unroll
                    for (int j = 0; j < 8; ++j) fma_f32x2(accr[c * 8 + j], v0[2 * j], v0[2 * j + 1], s2);
                    tmem_ld_wait(v1);
                    if (c + 2 < 8) {
                        tmem_ld_32x32b_x16(taddr + (c + 2) * 16, v0);
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        // a release at cluster scope here cost 0.65 ms per launch: the hand-back only
                        // orders TMEM reads, which the tcgen05 fence above already covers
                        if (lane == 0) {
                            if (rank == 0) mbar_arrive(tempty_bar + 8 * acc);
                            else mbar_arrive_cluster_relaxed(leader_tempty_bar + 8 * acc);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) fma_f32x2(accr[(c + 1) * 8 + j], v1[2 * j], v1[2 * j + 1], s2);
                }
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
            if (!ok) break;
            if (row_valid && p.d_f32) {
                float* drow = reinterpret_cast<float*>(p.d) + (long long)row * p.ldd + n0;
#pragma unroll
                for (int j = 0; j < 128; j += 4) {
                    if (n0 + j + 4 <= p.N) {
                        float4 o;
                        unpack_f32x2(accr[j / 2], o.x, o.y);
                        unpack_f32x2(accr[j / 2 + 1], o.z, o.w);
                        *reinterpret_cast<float4*>(drow + j) = o;
                    }
                }
            } else if (row_valid) {
                __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.d) + (long long)row * p.ldd + n0;
#pragma unroll
                for (int j = 0; j < 128; j += 8) {
                    if (n0 + j + 8 <= p.N) {
                        uint4 out;
                        out.x = cvt_bf16x2(accr[j / 2 + 0]);
                        out.y = cvt_bf16x2(accr[j / 2 + 1]);
                        out.z = cvt_bf16x2(accr[j / 2 + 2]);
                        out.w = cvt_bf16x2(accr[j / 2 + 3]);
                        *reinterpret_cast<uint4*>(drow + j) = out;
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------- teardown
    // No CTA may leave while its partner can still signal its barriers or read its shared memory.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

}  // namespace b200
