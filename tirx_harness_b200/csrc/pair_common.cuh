// Helpers shared by the CTA-pair kernels (tcgen05 cta_group::2): cluster addressing, the pair forms of TMA
// load, TMEM allocation, MMA commit, and the persistent tile schedule over clusters of two CTAs.
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 output tile: CTA r loads A rows
// [128 r, 128 r + 128) of the tile and B rows (= output columns) [128 r, 128 r + 128); the leader (r = 0) issues
// tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32): the tensor cores of both SMs read A from their own shared
// memory and B from both, and each SM's TMEM receives its 128 rows x 256 columns.  Per SM the operand traffic
// drops from 48 KB to 32 KB per 128-K block.  No load is multicast: each CTA fetches what it stages.
#pragma once

#include "gg_fp8.cuh"

namespace b200 {

constexpr int PAIR_BM = 128;          // rows per CTA of a pair (256 per pair)

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
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
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
            const int row0 = mb * 256 + rank * PAIR_BM;          // first row of this CTA inside the group
            tile.m0 = lo * p.M + row0;
            int mm = __ldg(p.layout + lo);
            if (mm > p.M) mm = p.M;
            int left = mm - row0;
            tile.rows = left < 0 ? 0 : (left < PAIR_BM ? left : PAIR_BM);
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
                tile.m0 = (t / p.num_n_blocks) * 256 + rank * PAIR_BM;
                tile.n_blk = t % p.num_n_blocks;
                tile.g = g;
                tile.rows = PAIR_BM;
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

}  // namespace b200
