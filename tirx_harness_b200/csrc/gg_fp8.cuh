// m-grouped FP8 block-scaled GEMM for sm_100a (contiguous and masked layouts).
//
//   D_g[rows, N] (bf16) = sum over 128-wide K blocks kb of
//        (A_g[rows, kb] . B_g[N, kb]^T  in e4m3 x e4m3 -> fp32 on tcgen05)  *  sfa[row, kb] * sfb[g, n/128, kb]
//
// One persistent CTA per SM, 640 threads (20 warps), four roles:
//   warp 0        TMA producer: A tile 128 x 128 B and B tile 256 x 128 B per K block into a
//                 4-stage shared-memory ring (SWIZZLE_128B), completion on mbarriers
//   warp 1        MMA issuer: four tcgen05.mma (128 x 256 x 32) per K block into one of two
//                 256-column TMEM accumulators; tcgen05.commit releases the smem stage and
//                 publishes the accumulator
//   warp 2        scale loader: per K block the 128 row scales of the tile and the two 128x128
//                 block scales go from global memory into an 8-slot shared-memory ring, several
//                 blocks ahead of their use, so the promotion never waits on L2 latency
//   warps 4..19   sixteen promotion/epilogue warps = four column groups (64 columns each) x the four
//                 TMEM lane quarters: per K block they drain the TMEM accumulator (tcgen05.ld),
//                 apply the block scales acc += partial * (sfa * sfb) in registers, hand the TMEM
//                 buffer back, and after the last K block convert to bf16 and store the valid rows.
//                 The drain is the step that bounds this kernel (128 KB of TMEM per K block against
//                 512 tensor-pipe cycles); sixteen warps keep twice as many TMEM loads in flight as
//                 eight and halve each thread's share.
// The MMA of K block i+1 runs while block i is being promoted (double-buffered TMEM).
// FUSE_ACT (gate_up GEMM of a MoE layer): a tile's 256 columns are [up 32 | gate 32] for each of the four
// column groups, so every epilogue thread ends up holding matching gate/up values; it forms silu(gate)*up
// in fp32, the four groups exchange their 32-column amax through shared memory, and the 128-wide block
// is requantised to e4m3 with its scale and stored -- the gate_up matrix itself is never written.
// Every wait is bounded (see mbar_wait_warp); on expiry the CTA unwinds and the host sees a status.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <limits.h>

#include "ptx.cuh"
#include "moe_ops.cuh"

namespace b200 {

namespace gg {
constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;              // bytes == elements (fp8)
constexpr int STAGES = 4;
constexpr int ACC_STAGES = 2;
constexpr int EPI_WARPS = 16;                      // promotion / epilogue warps: 4 column groups x 4 TMEM lane quarters
constexpr int EPI_WARP0 = 4;                       // first of them (warps 0..2: TMA, MMA, scale loader; warp 3 idles)
constexpr int COL_GROUPS = 4;
constexpr int GROUP_COLS = BN / COL_GROUPS;        // 64 accumulator columns per epilogue thread
constexpr int THREADS = 32 * (EPI_WARP0 + EPI_WARPS);   // 640
constexpr int A_STAGE_BYTES = BM * BK;             // 16 KB
constexpr int B_STAGE_BYTES = BN * BK;             // 32 KB
constexpr int TMEM_COLS = 512;
constexpr int MAX_MASKED_GROUPS = 1024;
constexpr int SMALL_A_ROWS = 16;                   // masked layout: A box for tiles with at most this many valid rows
constexpr int SCATTER_STAGES = 3;                  // scattered-output variant: one stage fewer ...
constexpr int STAGING_ROW_BYTES = 528;             // ... and 128 staging rows of 512 B + 16 B pad (bank-conflict free)
constexpr int FUSE_B_BOX_ROWS = 32;                // fused activation: B arrives as eight 32-row boxes [up 32 | gate 32] x 4
constexpr int STAGING_BYTES = 128 * STAGING_ROW_BYTES;
constexpr int SMEM_TILE_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int SF_SLOTS = 8;                        // scale ring: per slot 128 row scales + 2 block scales
constexpr int SF_SLOT_FLOATS = 132;
constexpr int OFF_BARS = SMEM_TILE_BYTES;          // mbarriers, TMEM base, abort flag
constexpr int OFF_SF = OFF_BARS + 512;
constexpr int OFF_AMAX = OFF_SF + SF_SLOTS * SF_SLOT_FLOATS * 4;     // fused activation: float [2 parity][4 groups][128]
constexpr int OFF_PREFIX = OFF_AMAX + 2 * COL_GROUPS * 128 * 4;
// + masked-layout prefix table + slack for 1024-byte alignment
constexpr int SMEM_BYTES = OFF_PREFIX + (MAX_MASKED_GROUPS + 1) * 4 + 12 + 1024;
// masked layout: after prefix[G+1] come the clamped masked_m[G] and a direct (group, row block) table of the
// first MASKED_LIST_CAP row blocks, so that the per-tile schedule lookup is one shared-memory load
constexpr int MASKED_LIST_CAP = 2048;
constexpr int MASKED_TABLE_INTS = (MAX_MASKED_GROUPS + 1) + MAX_MASKED_GROUPS + MASKED_LIST_CAP;
constexpr int SMEM_BYTES_MASKED = OFF_PREFIX + MASKED_TABLE_INTS * 4 + 12 + 1024;
constexpr int SMEM_BYTES_SCATTER = SMEM_BYTES - (A_STAGE_BYTES + B_STAGE_BYTES) + STAGING_BYTES;
// dispatching variant (contiguous layout: no prefix table): the sending warp's record buffers take that place
constexpr int SMEM_BYTES_DISPATCH = OFF_PREFIX + EP_SEND_BUFFERS * EP_SEND_RECORD_MAX + EP_SEND_RING * 8 + 1024;
}  // namespace gg

struct GGParams {
    const float* sfa;
    long long sfa_sr, sfa_sk;
    const float* sfb;            // [G][nb128][KB]
    const int* layout;           // grouped_layout[M] or masked_m[G]
    const int* rows_used;        // contiguous, optional: device count of leading rows in use (<= M)
    const int* mode_flag;        // optional: this kernel runs only if *mode_flag == mode_gen (see gg_fp8_mx.cuh)
    int mode_gen;                // generation number of the call (block-scaled path)
    // scattered output (expert-parallel down GEMM): row r is stored at scatter_base[meta >> 24] + (meta & 0xFFFFFF) * ldd
    // with meta = scatter_meta[r]; the bases may be other GPUs' memory (plain stores only)
    const int* scatter_meta;     // meta of row r at scatter_meta[r * scatter_meta_stride]
    long long scatter_meta_stride;
    __nv_bfloat16* scatter_base[8];
    // fused SiLU*mul requant (FUSE_ACT kernels): N = 2*inter, outputs replace d
    uint8_t* act_q;              // e4m3 [M, inter]
    float* act_s;                // scale of (row r, 128-block b) at act_s[r*act_ss_r + b*act_ss_b]
    long long act_ss_r, act_ss_b;
    int inter, gate_first;
    void* d;                     // bf16 (or fp32 when d_f32 != 0)
    long long ldd;
    int d_f32;
    int d_accumulate;            // fp32 output only: add to d instead of overwriting it
    long long* trace;            // developer aid: per-CTA wait-cycle counters [grid][8], or nullptr
    EpSend ep;                   // DISPATCH kernels only: the all-to-all this GEMM carries (moe_ops.cuh)
    int G, M, N, K;              // M: total rows (contiguous) / rows per group (masked)
    int rows_total;              // rows of the flattened A / D (M or G*M)
    int num_n_blocks;            // ceil(N / BN)
    int num_k_blocks;            // K / 128
    int nb128;                   // ceil(N / 128)
    int num_m_blocks;            // contiguous: ceil(M / BM)
    // block-scaled kernels: column tiles of balanced width, in units of 16 columns: the first nt_rem tiles are
    // nt_base + 1 units wide, the others nt_base (all of them 224 or 240 columns where N allows it)
    int nt_base, nt_rem;
    // block-scaled pair kernel launched with programmatic stream serialization behind the kernel that re-tiles packed
    // scales: only the packed scale tiles come from that kernel, so the prologue and the first operand loads run
    // beside it and the producer waits (griddepcontrol.wait) right before its first scale load
    int pdl_scales;
};

// first column and width of column tile nt of a block-scaled kernel
__host__ __device__ __forceinline__ int mx_tile_col0(int nt_base, int nt_rem, int nt) {
    return 16 * (nt * nt_base + (nt < nt_rem ? nt : nt_rem));
}
__host__ __device__ __forceinline__ int mx_tile_width(int nt_base, int nt_rem, int nt) {
    return 16 * (nt_base + (nt < nt_rem ? 1 : 0));
}

struct Tile {
    int m0;          // first row of the tile in the flattened A / D
    int n_blk;       // column block (BN wide)
    int g;           // group
    int rows;        // masked: number of valid rows in this tile (<= BM); contiguous: BM
};

// Masked layout tables in shared memory (all threads of the CTA call this before the first __syncthreads that
// precedes any Scheduler use): tables[0..G] = prefix of 128-row blocks, then masked_m clamped to [0, M], then
// the (group << 16 | row block) of each of the first MASKED_LIST_CAP row blocks.  The masked_m loads are
// issued by all threads at once: one global round trip instead of one per 32 groups.
__device__ __forceinline__ void build_masked_tables(const GGParams& p, int* tables, int scan_warp) {
    int* prefix = tables;
    int* mm_s = tables + gg::MAX_MASKED_GROUPS + 1;
    int* list = mm_s + gg::MAX_MASKED_GROUPS;
    for (int g = threadIdx.x; g < p.G; g += blockDim.x) {
        int mm = __ldg(p.layout + g);
        mm_s[g] = mm < 0 ? 0 : (mm > p.M ? p.M : mm);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == scan_warp) {
        int running = 0;
        for (int base = 0; base < p.G; base += 32) {
            const int g = base + lane;
            const int blocks = g < p.G ? (mm_s[g] + gg::BM - 1) / gg::BM : 0;
            int incl = blocks;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int first = running + incl - blocks;
            if (g < p.G) {
                prefix[g] = first;
                for (int mb = 0; mb < blocks && first + mb < gg::MASKED_LIST_CAP; ++mb) list[first + mb] = (g << 16) | mb;
            }
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) prefix[p.G] = running;
    }
}

// Static persistent schedule.  All warps of a CTA walk the same sequence.
//  contiguous: tile index t -> (128-row block, column block); a row block is visited once per
//              distinct non-negative group id found in it (one when groups are 128-aligned).  The
//              block's 128 layout entries (4 per lane) are fetched one tile AHEAD: as soon as a tile has
//              been handed out and its block holds no further group, the loads for the next candidate
//              are issued, so their latency is hidden behind the tile's K loop.
//  masked:     compact enumeration of (group, row block < ceil(masked_m/128), column block)
//              through a prefix table in shared memory.
template <bool MASKED>
struct Scheduler {
    const GGParams& p;
    const int* prefix;   // masked: smem prefix of row blocks per group, [G+1]
    int t, lane, prev_g, total;
    int vals[4];         // contiguous: layout entries of the row block of tile t held by this lane

    __device__ __forceinline__ void fetch() {
        if (t < total) {
            const int m0 = (t / p.num_n_blocks) * gg::BM;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = m0 + lane * 4 + j;
                vals[j] = r < p.M ? __ldg(p.layout + r) : -1;
            }
        }
    }
    // smallest group id > after in the fetched block, INT_MAX if none.  Warp-collective.
    __device__ __forceinline__ int next_group(int after) const {
        int best = INT_MAX;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (vals[j] > after && vals[j] < p.G && vals[j] < best) best = vals[j];
        return __reduce_min_sync(0xffffffffu, best);
    }

    __device__ __forceinline__ Scheduler(const GGParams& p_, const int* prefix_, int lane_)
        : p(p_), prefix(prefix_), t(blockIdx.x), lane(lane_), prev_g(-1) {
        if (MASKED) {
            total = prefix_[p_.G] * p_.num_n_blocks;
        } else {
            int m_blocks = p_.num_m_blocks;
            if (p_.rows_used != nullptr) {       // only the leading rows hold data: skip the rest outright
                int used = __ldg(p_.rows_used);
                used = used < 0 ? 0 : (used > p_.M ? p_.M : used);
                m_blocks = (used + gg::BM - 1) / gg::BM;
            }
            total = m_blocks * p_.num_n_blocks;
            fetch();
        }
    }

    __device__ __forceinline__ bool next(Tile& tile) {
        if (MASKED) {
            if (t >= total) return false;
            const int mbg = t / p.num_n_blocks;
            const int* mm_s = prefix + gg::MAX_MASKED_GROUPS + 1;
            int lo, mb;
            if (mbg < gg::MASKED_LIST_CAP) {
                const int e = mm_s[gg::MAX_MASKED_GROUPS + mbg];
                lo = e >> 16;
                mb = e & 0xFFFF;
            } else {
                lo = 0;
                int hi = p.G;                // find g with prefix[g] <= mbg < prefix[g+1]
                while (hi - lo > 1) {
                    int mid = (lo + hi) >> 1;
                    if (prefix[mid] <= mbg) lo = mid; else hi = mid;
                }
                mb = mbg - prefix[lo];
            }
            tile.g = lo;
            tile.n_blk = t % p.num_n_blocks;
            tile.m0 = lo * p.M + mb * gg::BM;
            const int left = mm_s[lo] - mb * gg::BM;
            tile.rows = left < gg::BM ? left : gg::BM;
            t += gridDim.x;
            return true;
        } else {
            while (t < total) {
                const int g = next_group(prev_g);
                if (g == INT_MAX) {             // block exhausted (or all padding): next candidate
                    t += gridDim.x;
                    prev_g = -1;
                    fetch();
                    continue;
                }
                tile.m0 = (t / p.num_n_blocks) * gg::BM;
                tile.n_blk = t % p.num_n_blocks;
                tile.g = g;
                tile.rows = gg::BM;
                prev_g = g;
                if (next_group(g) == INT_MAX) { // nothing else in this block: start fetching the next one now
                    t += gridDim.x;
                    prev_g = -1;
                    fetch();
                }
                return true;
            }
            return false;
        }
    }
};

// Bounded wait (2 s) of one warp until every row of local expert g has arrived in this rank's receive buffer:
// lane 0 polls the arrival counter with acquire semantics at system scope (the rows were stored by other GPUs).
__device__ __forceinline__ bool wait_expert_arrived(const EpSend& ep, int g, volatile int* abort_flag, int* status) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        const int want = __ldg(ep.expected + g);
        const int* ctr = ep.arrive[ep.rank] + g;
        if (ld_acquire_sys(ctr) < want) {
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (ld_acquire_sys(ctr) < want) {
                if ((++spins & 63u) == 0) {
                    if (*abort_flag) { ok = false; break; }
                    if (globaltimer_ns() - t0 > kWaitLimitNs) {
                        *abort_flag = 1;
                        atomicOr(status, STATUS_TIMEOUT_PEER_FLAG);
                        ok = false;
                        break;
                    }
                }
            }
        }
    }
    return __all_sync(0xffffffffu, ok);
}

// DISPATCH: the gate_up GEMM of an expert-parallel layer that carries the dispatch all-to-all itself.  Warp 3 of
// every CTA sends this rank's token records (e4m3 row + scales) straight into the owners' receive buffers, local
// expert 0 of every rank first; the TMA producer and the scale loader wait, per expert, until that expert's rows
// have all arrived (arrival counters incremented by the senders after their stores completed).  The transfer thus
// overlaps the GEMM tile by tile and needs no barrier of its own.  Senders never wait for anything remote, and
// every CTA of the grid is resident (persistent grid <= SM count), so the waits cannot form a cycle.
template <bool MASKED, bool FUSE_ACT = false, bool SCATTER = false, bool DISPATCH = false>
__global__ void __launch_bounds__(gg::THREADS, 1)
gg_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              const __grid_constant__ CUtensorMap tmap_a_small, const GGParams p, int* status) {
    static_assert(!(MASKED && FUSE_ACT), "the fused activation epilogue exists for the contiguous layout only");
    static_assert(!(SCATTER && (MASKED || FUSE_ACT)), "scattered output exists for the plain contiguous GEMM only");
    static_assert(!(DISPATCH && (MASKED || SCATTER)), "the dispatching variant is a contiguous-layout gate_up GEMM");
    using namespace gg;
    // SCATTER trades one pipeline stage for a 128 x 528-byte staging area from which finished rows leave
    // as 512-byte bulk stores (possibly to another GPU) without holding up the promotion warps.
    constexpr int NSTAGES = SCATTER ? gg::SCATTER_STAGES : gg::STAGES;
    constexpr int TILES_END = NSTAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
    constexpr int BARS_AT = TILES_END + (SCATTER ? gg::STAGING_BYTES : 0);
    constexpr int SF_AT = BARS_AT + 512;
    constexpr int AMAX_AT = SF_AT + SF_SLOTS * SF_SLOT_FLOATS * 4;
    constexpr int PREFIX_AT = AMAX_AT + 2 * COL_GROUPS * 128 * 4;
    if (p.mode_flag != nullptr && *p.mode_flag != p.mode_gen) return;   // the power-of-two-scale path took this call
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle atoms the MMA descriptors address
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + NSTAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BARS_AT);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty,
    // then SF_SLOTS scale-full and SF_SLOTS scale-empty barriers
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * NSTAGES + 2 * ACC_STAGES + 2 * SF_SLOTS + 1 + 8 + EP_SEND_BUFFERS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    float* sf_ring = reinterpret_cast<float*>(smem + SF_AT);
    int* prefix = reinterpret_cast<int*>(smem + PREFIX_AT);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);       // a value the compiler knows to be warp-uniform
    const int lane = threadIdx.x & 31;

    const uint32_t full_bar = smem_u32(bars);
    const uint32_t empty_bar = smem_u32(bars + NSTAGES);
    const uint32_t tfull_bar = smem_u32(bars + 2 * NSTAGES);
    const uint32_t tempty_bar = smem_u32(bars + 2 * NSTAGES + ACC_STAGES);
    const uint32_t sffull_bar = smem_u32(bars + 2 * NSTAGES + 2 * ACC_STAGES);
    const uint32_t sfempty_bar = smem_u32(bars + 2 * NSTAGES + 2 * ACC_STAGES + SF_SLOTS);
    const uint32_t amax_bar = smem_u32(bars + 2 * NSTAGES + 2 * ACC_STAGES + 2 * SF_SLOTS);
    const uint32_t stg_bar = amax_bar + 8;            // SCATTER: 4 "row free" + 4 "row filled" barriers, one pair per lane quarter
    const uint32_t send_bar = stg_bar + 64;           // DISPATCH: one "record loaded" barrier per send buffer
    float* amax_x = reinterpret_cast<float*>(smem + AMAX_AT);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int s = 0; s < ACC_STAGES; ++s) {
            mbar_init(tfull_bar + 8 * s, 1);
            mbar_init(tempty_bar + 8 * s, EPI_WARPS);     // one arrival per epilogue warp
        }
        for (int s = 0; s < SF_SLOTS; ++s) {
            mbar_init(sffull_bar + 8 * s, 32);            // every lane of the loader warp arrives
            mbar_init(sfempty_bar + 8 * s, EPI_WARPS);    // one arrival per epilogue warp
        }
        mbar_init(amax_bar, EPI_WARPS * 32);              // every epilogue thread, once per tile
        for (int q = 0; q < 4; ++q) {
            mbar_init(stg_bar + 8 * q, 1);                // the group-0 warp of the quarter
            mbar_init(stg_bar + 8 * (4 + q), COL_GROUPS); // one arrival per column group of the quarter
        }
        for (int b = 0; b < EP_SEND_BUFFERS; ++b) mbar_init(send_bar + 8 * b, 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (MASKED) build_masked_tables(p, prefix, 3);
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    const int KB = p.num_k_blocks;

    // Register budget.  Warps sit on the SM's four sub-partitions by warp index modulo 4: each holds one of warps
    // 0..3 and four epilogue warps.  The launch gives every warp 96 registers per thread (5 x 96 = 480 per lane and
    // sub-partition); 64 + 4 x 104 = 480 re-divides exactly that, so setmaxnreg.inc never waits for registers
    // that cannot come.
    if (warp < EPI_WARP0) {
        setmaxnreg_dec<64>();
        if (warp == 0) {
            // ------------------------------------------------ TMA producer
            Scheduler<MASKED> sched(p, prefix, lane);
            Tile tile;
            uint32_t stage = 0, phase = 0;
            uint32_t issued = 0, issued_parity = 0;   // per-stage: a load was issued / its phase parity
            bool ok = true;
            int arrived_g = -1;
            while (ok && sched.next(tile)) {
                const int b_row = tile.g * p.N + tile.n_blk * BN;
                if (DISPATCH && tile.g != arrived_g) {
                    ok = wait_expert_arrived(p.ep, tile.g, abort_flag, status);
                    if (!ok) break;
                    arrived_g = tile.g;
                    // the rows were written through NVLink; the TMA loads below read them through the async proxy
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                }
                for (int kb = 0; kb < KB; ++kb) {
                    ok = mbar_wait_warp(empty_bar + 8 * stage, phase ^ 1, abort_flag, status,
                                        STATUS_TIMEOUT_SMEM_EMPTY);
                    if (!ok) break;
                    if (elect_one_sync()) {
                        const uint32_t fb = full_bar + 8 * stage;
                        // masked tiles with few valid rows (decode) fetch a SMALL_A_ROWS-row box of A only: the
                        // other rows of the stage keep stale bytes whose products land in rows nobody stores
                        const bool small_a = MASKED && tile.rows <= gg::SMALL_A_ROWS;
                        mbar_arrive_expect_tx(fb, (small_a ? gg::SMALL_A_ROWS * BK : A_STAGE_BYTES) + B_STAGE_BYTES);
                        tma_load_2d(smem_u32(smem_a + stage * A_STAGE_BYTES), small_a ? &tmap_a_small : &tmap_a, fb, kb * BK,
                                    tile.m0);
                        if (FUSE_ACT) {
                            // tmap_b has a 32-row box here: [up 32 | gate 32] for each of the four column groups
                            const int up0 = tile.g * p.N + (p.gate_first ? p.inter : 0) + tile.n_blk * 128;
                            const int gate0 = tile.g * p.N + (p.gate_first ? 0 : p.inter) + tile.n_blk * 128;
                            const uint32_t sb = smem_u32(smem_b + stage * B_STAGE_BYTES);
#pragma unroll
                            for (int cg = 0; cg < COL_GROUPS; ++cg) {
                                tma_load_2d(sb + (2 * cg) * FUSE_B_BOX_ROWS * BK, &tmap_b, fb, kb * BK, up0 + cg * FUSE_B_BOX_ROWS);
                                tma_load_2d(sb + (2 * cg + 1) * FUSE_B_BOX_ROWS * BK, &tmap_b, fb, kb * BK, gate0 + cg * FUSE_B_BOX_ROWS);
                            }
                        } else {
                            tma_load_2d(smem_u32(smem_b + stage * B_STAGE_BYTES), &tmap_b, fb, kb * BK, b_row);
                        }
                    }
                    issued |= 1u << stage;
                    issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == NSTAGES) { stage = 0; phase ^= 1; }
                }
            }
            // Unwinding after a failed wait: give every copy this warp issued a bounded chance to
            // land before the CTA exits (on the normal path the MMA warp has consumed them all).
            if (!ok && lane == 0) {
                for (int s = 0; s < NSTAGES; ++s) {
                    if (!((issued >> s) & 1u)) continue;
                    const uint32_t par = (issued_parity >> s) & 1u;
                    for (int it = 0; it < (1 << 20); ++it)
                        if (mbar_try_wait(full_bar + 8 * s, par)) break;
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ MMA issuer
            // Warp-uniform loop, one elected lane issues: stage, phase and descriptors stay in uniform registers, which
            // is what the tcgen05 instructions take.  (A single diverged lane needed more issue time per K block
            // than the tensor pipe needs to multiply it.)
            Scheduler<MASKED> sched(p, prefix, lane);
            Tile tile;
            constexpr uint32_t idesc = make_idesc_e4m3_f32(BM, BN);
            const uint64_t adesc0 = make_smem_desc_sw128(smem_u32(smem_a));
            const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(smem_b));
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            while (ok && sched.next(tile)) {
                for (int kb = 0; kb < KB; ++kb) {
                    ok = mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, status, STATUS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    ok = mbar_wait_warp(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_TMEM_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one_sync()) {
                        const uint64_t adesc = adesc0 + stage * (A_STAGE_BYTES >> 4);
                        const uint64_t bdesc = bdesc0 + stage * (B_STAGE_BYTES >> 4);
                        const uint32_t tmem_d = tmem_base + acc * BN;
                        // advance 32 bytes of K inside the 128-byte swizzled row: +2 in 16-byte units
                        umma_f8f6f4(tmem_d, adesc, bdesc, idesc, 0u);
                        umma_f8f6f4(tmem_d, adesc + 2, bdesc + 2, idesc, 1u);
                        umma_f8f6f4(tmem_d, adesc + 4, bdesc + 4, idesc, 1u);
                        umma_f8f6f4(tmem_d, adesc + 6, bdesc + 6, idesc, 1u);
                        umma_commit(empty_bar + 8 * stage);   // stage reusable once the MMAs have read it
                        umma_commit(tfull_bar + 8 * acc);     // accumulator of this K block complete
                    }
                    if (++stage == NSTAGES) { stage = 0; phase ^= 1; }
                    if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
                }
            }
        } else if (warp == 2) {
            // ------------------------------------------------ scale loader
            Scheduler<MASKED> sched(p, prefix, lane);
            Tile tile;
            uint32_t slot = 0, sphase = 0;
            bool ok = true;
            int arrived_g = -1;
            while (ok && sched.next(tile)) {
                if (DISPATCH && tile.g != arrived_g) {      // the row scales travel inside the records
                    ok = wait_expert_arrived(p.ep, tile.g, abort_flag, status);
                    if (!ok) break;
                    arrived_g = tile.g;
                }
                const float* rp[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int r = tile.m0 + lane + 32 * j;
                    if (r >= p.rows_total) r = p.rows_total - 1;
                    rp[j] = p.sfa + (long long)r * p.sfa_sr;
                }
                int nb = ((tile.n_blk * BN) >> 7) + (lane & 1);
                if (FUSE_ACT)      // slot word 128 = up block, 129 = gate block of this tile's 128 activation columns
                    nb = tile.n_blk + ((((lane & 1) != 0) != (p.gate_first != 0)) ? (p.inter >> 7) : 0);
                if (nb >= p.nb128) nb = p.nb128 - 1;
                const float* bp = p.sfb + ((long long)tile.g * p.nb128 + nb) * KB;
                // asynchronous 4-byte copies straight into the ring slot; the slot's `full` barrier gets one
                // deferred arrival per lane.  Up to SF_SLOTS K blocks are in flight, across tile borders, so
                // short-K tiles (one K block each) do not expose a global-load latency per tile.
                for (int kb = 0; kb < KB; ++kb) {
                    ok = mbar_wait_warp(sfempty_bar + 8 * slot, sphase ^ 1, abort_flag, status, STATUS_TIMEOUT_SF_EMPTY);
                    if (!ok) break;
                    const uint32_t dst = smem_u32(sf_ring + slot * SF_SLOT_FLOATS);
#pragma unroll
                    for (int j = 0; j < 4; ++j) cp_async_4(dst + (lane + 32 * j) * 4, rp[j] + (long long)kb * p.sfa_sk);
                    if (lane < 2) cp_async_4(dst + (128 + lane) * 4, bp + kb);
                    cp_async_mbar_arrive_noinc(sffull_bar + 8 * slot);
                    if (++slot == SF_SLOTS) { slot = 0; sphase ^= 1; }
                }
            }
            cp_async_wait_all();      // nothing may still be writing this CTA's shared memory at exit
        } else if (DISPATCH) {
            // ------------------------------------------------ sender of the dispatch all-to-all (warp 3)
            // This warp owns pairs order[blockIdx.x + i * gridDim.x].  Per pair the token's record -- e4m3 row (bulk
            // load), its scales and the row's return address (written by the lanes) -- is assembled in one of
            // EP_SEND_BUFFERS shared-memory buffers and leaves as ONE bulk store into the owner's receive buffer.
            // Software pipeline: the load of pair i is in flight while pair i-1 is stored.  Lane 0 issues every bulk
            // operation and commits exactly one bulk group per pair, so group numbers are pair numbers.  A buffer is
            // refilled as soon as its last store has READ it (wait_group.read); a row is counted as arrived only when
            // its store is COMPLETE (wait_group), up to EP_SEND_INFLIGHT stores later, so the round trip of a store over
            // NVLink is not part of a row's issue time.  Counting = one fence at system scope for EP_SEND_BATCH complete
            // rows, then a relaxed add per counter (a fence per row cost more than sending the row).  A row's scales are
            // requested one step ahead.
            // Routing data of 32 pairs is fetched at once, one pair per lane.
            const EpSend& ep = p.ep;
            uint8_t* stage_base = smem + PREFIX_AT;
            const int meta_off = ep.H + (ep.H >> 5);
            const int rec = (meta_off + 4 + 15) & ~15;
            const int stride = gridDim.x;
            const int my_rows = ep.n_pairs > (int)blockIdx.x ? (ep.n_pairs - 1 - (int)blockIdx.x) / stride + 1 : 0;
            // arrival counter of every stored row until it has been counted in (lane 0 only)
            int** ring = reinterpret_cast<int**>(stage_base + EP_SEND_BUFFERS * EP_SEND_RECORD_MAX);
            int counted = 0;                             // rows [0, counted) have been counted in
            // Counts rows [counted, upto) in: ONE fence at system scope (the expensive part: it also waits for what
            // the rest of the SM has in flight), then one relaxed add per run of rows with the same counter.
            auto count_rows = [&](int upto) {            // lane 0 only
                if (upto <= counted) return;
                asm volatile("fence.acq_rel.sys;" ::: "memory");
                int* cur = nullptr;
                int n = 0;
                for (; counted < upto; ++counted) {
                    int* c = ring[counted % EP_SEND_RING];
                    if (c != cur) {
                        if (cur != nullptr && n > 0) red_relaxed_sys_add(cur, n);
                        cur = c;
                        n = 0;
                    }
                    ++n;
                }
                if (cur != nullptr && n > 0) red_relaxed_sys_add(cur, n);
            };
            const int nblk = ep.H >> 7;                  // scales per row (at most 64: two per lane)
            auto load_scales = [&](long long t, float& s0, float& s1) {
                s0 = lane < nblk ? __ldg(ep.xs + t * ep.xs_r + (long long)lane * ep.xs_b) : 0.0f;
                s1 = lane + 32 < nblk ? __ldg(ep.xs + t * ep.xs_r + (long long)(lane + 32) * ep.xs_b) : 0.0f;
            };
            bool ok = true;
            // state of the pair whose load is in flight (finished one step later)
            int started = -1;                            // last pair whose record load was issued
            int prev_row = -1, prev_d = 0;
            int* prev_ctr = nullptr;
            long long tr_load = 0, tr_read = 0, tr_done = 0;
            const long long tr_s0 = B200_TRACE(p.trace) ? clock64() : 0;
            auto finish = [&](int it_prev) {             // store pair it_prev (its load was started one step earlier)
                const int b = it_prev % EP_SEND_BUFFERS;
                const long long c0 = B200_TRACE(p.trace) ? clock64() : 0;
                ok = mbar_wait_warp(send_bar + 8 * b, (uint32_t)(it_prev / EP_SEND_BUFFERS) & 1u, abort_flag, status,
                                    STATUS_TIMEOUT_SMEM_FULL);
                if (B200_TRACE(p.trace)) tr_load += clock64() - c0;
                if (lane == 0) {
                    if (ok)
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                     ::"l"(ep.a[prev_d] + (long long)prev_row * ep.pitch),
                                       "r"(smem_u32(stage_base + b * EP_SEND_RECORD_MAX)), "r"(rec) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");       // group number = pair number
                    ring[it_prev % EP_SEND_RING] = ok ? prev_ctr : nullptr;
                }
            };
            float sc0 = 0.0f, sc1 = 0.0f;
            bool have_sc = false;
            for (int base = 0; ok && base < my_rows; base += 32) {
                int m_pr = 0, m_row = -1, m_e = 0;
                if (base + lane < my_rows) {
                    m_pr = __ldg(ep.order + blockIdx.x + (long long)(base + lane) * stride);
                    m_row = __ldg(ep.pos + m_pr);
                    m_e = __ldg(ep.ids + m_pr);
                }
                const int cnt = my_rows - base < 32 ? my_rows - base : 32;
                for (int i = 0; ok && i < cnt; ++i) {
                    const int it = base + i;
                    const int b = it % EP_SEND_BUFFERS;
                    const int pr = __shfl_sync(0xffffffffu, m_pr, i);
                    const int row = __shfl_sync(0xffffffffu, m_row, i);
                    const int e = __shfl_sync(0xffffffffu, m_e, i);
                    const int pr_next = __shfl_sync(0xffffffffu, m_pr, (i + 1) & 31);
                    if (row < 0 || row >= ep.cap_rows) {            // the owner's buffer is too small: give up, report
                        if (lane == 0) atomicOr(status, STATUS_CAPACITY);
                        ok = false;
                        break;
                    }
                    // (1) Groups 0 .. it-2 have been committed.  Buffer b was last read by the store of pair it-3: "all
                    // but the latest group have been read" frees it.  Rows whose stores are COMPLETE (all but the latest
                    // EP_SEND_INFLIGHT groups) are counted in; this also bounds the stores in flight.
                    if (lane == 0) {
                        const long long c0 = B200_TRACE(p.trace) ? clock64() : 0;
                        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        const long long c1 = B200_TRACE(p.trace) ? clock64() : 0;
                        asm volatile("cp.async.bulk.wait_group %0;" ::"n"(EP_SEND_INFLIGHT) : "memory");
                        if (B200_TRACE(p.trace)) { tr_read += c1 - c0; tr_done += clock64() - c1; }
                        // complete rows are reported EP_SEND_BATCH at a time (the first few in small batches: the
                        // receivers' first experts are waiting for them)
                        const int batch = counted < 2 * EP_SEND_BATCH ? 4 : EP_SEND_BATCH;
                        if (it - 1 - EP_SEND_INFLIGHT - counted >= batch) count_rows(it - 1 - EP_SEND_INFLIGHT);
                    }
                    __syncwarp();
                    // (2) start assembling pair `it` in buffer b
                    const long long t = pr / ep.top_k;
                    uint8_t* buf = stage_base + b * EP_SEND_RECORD_MAX;
                    if (lane == 0) {
                        mbar_arrive_expect_tx(send_bar + 8 * b, (uint32_t)ep.H);
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(smem_u32(buf)), "l"(ep.x + t * ep.H), "r"(ep.H), "r"(send_bar + 8 * b) : "memory");
                        *reinterpret_cast<int*>(buf + meta_off) = (ep.rank << 24) | pr;     // where the result goes back to
                    }
                    if (!have_sc) load_scales(t, sc0, sc1);
                    float* sbuf = reinterpret_cast<float*>(buf + ep.H);
                    if (lane < nblk) sbuf[lane] = sc0;
                    if (lane + 32 < nblk) sbuf[lane + 32] = sc1;
                    fence_proxy_async_smem();
                    __syncwarp();
                    started = it;
                    // the next pair's scales are requested now and used one step later (their latency overlaps the wait below)
                    have_sc = i + 1 < cnt;
                    if (have_sc) load_scales(pr_next / ep.top_k, sc0, sc1);
                    // (3) store the pair started one step ago
                    if (it > 0) finish(it - 1);
                    prev_row = row;
                    prev_d = e / ep.E_local;
                    prev_ctr = ep.arrive[prev_d] + (e - prev_d * ep.E_local);
                }
            }
            if (ok && my_rows > 0) finish(my_rows - 1);
            // Unwinding after a failed wait: a record load that was started but never stored gets a bounded chance
            // to land before the CTA exits.
            if (!ok && started >= 0 && lane == 0) {
                const uint32_t bar = send_bar + 8 * (started % EP_SEND_BUFFERS);
                const uint32_t par = (uint32_t)(started / EP_SEND_BUFFERS) & 1u;
                for (int spin = 0; spin < (1 << 20); ++spin)
                    if (mbar_try_wait(bar, par)) break;
            }
            if (B200_TRACE(p.trace) && lane == 0) {
                p.trace[blockIdx.x * 8 + 0] = clock64() - tr_s0;
                p.trace[blockIdx.x * 8 + 1] = tr_load;
                p.trace[blockIdx.x * 8 + 2] = tr_read;
                p.trace[blockIdx.x * 8 + 3] = tr_done;
                p.trace[blockIdx.x * 8 + 4] = my_rows;
            }
            // drain: every store complete (also on the failure path), then the rows not yet counted are counted in
            if (lane == 0) {
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                const int stored = ok ? my_rows : (started < 0 ? 0 : started);     // pairs whose ring entry was written
                if (counted < stored - EP_SEND_RING) counted = stored - EP_SEND_RING;
                count_rows(stored);
            }
        }
    } else {
        // ---------------------------------------------------- promotion + epilogue
        setmaxnreg_inc<104>();
        const int quarter = warp & 3;                       // TMEM lanes this warp may touch: [32 quarter, +32)
        const int cg = (warp - EPI_WARP0) >> 2;             // which 64 columns of the 256-wide tile
        const int row_in_tile = quarter * 32 + lane;
        Scheduler<MASKED> sched(p, prefix, lane);
        Tile tile;
        uint32_t acc = 0, acc_phase = 0, slot = 0, sphase = 0, act_phase = 0, stg_phase = 0;
        bool ok = true;
        while (ok && sched.next(tile)) {
            const int n0 = tile.n_blk * BN + cg * GROUP_COLS;
            const int row = tile.m0 + row_in_tile;
            bool row_valid;
            if (MASKED) row_valid = row_in_tile < tile.rows;
            else row_valid = (row < p.M) && (__ldg(p.layout + row) == tile.g);
            unsigned long long accr[GROUP_COLS / 2];      // 64 fp32 accumulators as f32x2 pairs
#pragma unroll
            for (int j = 0; j < GROUP_COLS / 2; ++j) accr[j] = 0ull;

            for (int kb = 0; kb < KB; ++kb) {
                ok = mbar_wait_warp(sffull_bar + 8 * slot, sphase, abort_flag, status, STATUS_TIMEOUT_SF_FULL);
                if (!ok) break;
                const float* sfp = sf_ring + slot * SF_SLOT_FLOATS;
                const float sa_row = sfp[row_in_tile];
                // plain: columns [64 cg, +64) lie in 128-column block cg / 2.  fused: first half up, second half gate.
                const float s = sa_row * sfp[128 + (FUSE_ACT ? 0 : (cg >> 1))];
                const float sg = FUSE_ACT ? sa_row * sfp[129] : s;
                __syncwarp();
                if (lane == 0) mbar_arrive(sfempty_bar + 8 * slot);
                if (++slot == SF_SLOTS) { slot = 0; sphase ^= 1; }
                const unsigned long long s2 = pack_f32x2(s, s);
                const unsigned long long s2g = pack_f32x2(sg, sg);     // columns 32..63 (gate) when fused

                ok = mbar_wait_warp(tfull_bar + 8 * acc, acc_phase, abort_flag, status,
                                    STATUS_TIMEOUT_TMEM_FULL);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN + cg * GROUP_COLS;
                // four 16-column chunks, double-buffered: chunk c+1 is in flight while chunk c is
                // multiplied in (two fp32 FMAs per instruction)
                uint32_t v0[16], v1[16];
                tmem_ld_32x32b_x16(taddr, v0);
#pragma unroll
                for (int c = 0; c < 4; c += 2) {
                    tmem_ld_wait(v0);
                    tmem_ld_32x32b_x16(taddr + (c + 1) * 16, v1);
#pragma unroll
                    for (int j = 0; j < 8; ++j) fma_f32x2(accr[c * 8 + j], v0[2 * j], v0[2 * j + 1], c < 2 ? s2 : s2g);
                    tmem_ld_wait(v1);
                    if (c + 2 < 4) {
                        tmem_ld_32x32b_x16(taddr + (c + 2) * 16, v0);
                    } else {
                        // all loads have landed: hand the accumulator back to the MMA warp
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) fma_f32x2(accr[(c + 1) * 8 + j], v1[2 * j], v1[2 * j + 1], c + 1 < 2 ? s2 : s2g);
                }
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
            if (!ok) break;
            if (FUSE_ACT) {
                // accr[0..16) = up columns, accr[16..32) = gate columns of this group's 32 activations
                float amax = 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float u0, u1, g0, g1;
                    unpack_f32x2(accr[j], u0, u1);
                    unpack_f32x2(accr[16 + j], g0, g1);
                    const float a0 = __fmul_rn(silu_f32(g0), u0), a1 = __fmul_rn(silu_f32(g1), u1);
                    amax = fmaxf(amax, fmaxf(fabsf(a0), fabsf(a1)));
                    accr[j] = pack_f32x2(a0, a1);
                }
                // the 128-wide quantisation block spans the four column groups: exchange the 32-column maxima
                amax_x[(act_phase * COL_GROUPS + cg) * 128 + row_in_tile] = amax;
                mbar_arrive(amax_bar);
                ok = mbar_wait_warp(amax_bar, act_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
                if (!ok) break;
#pragma unroll
                for (int o = 0; o < COL_GROUPS; ++o) amax = fmaxf(amax, amax_x[(act_phase * COL_GROUPS + o) * 128 + row_in_tile]);
                act_phase ^= 1;
                const float sc = __fdiv_rn(fmaxf(amax, 1.0e-8f), 448.0f);
                if (row_valid) {
                    uint8_t* qrow = p.act_q + (long long)row * p.inter + tile.n_blk * 128 + cg * 32;
#pragma unroll
                    for (int j = 0; j < 16; j += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float a0, a1, a2, a3;
                            unpack_f32x2(accr[j + 2 * i], a0, a1);
                            unpack_f32x2(accr[j + 2 * i + 1], a2, a3);
                            w[i] = pack4_e4m3(clamp448(__fdiv_rn(a0, sc)), clamp448(__fdiv_rn(a1, sc)),
                                              clamp448(__fdiv_rn(a2, sc)), clamp448(__fdiv_rn(a3, sc)));
                        }
                        *reinterpret_cast<uint4*>(qrow + j * 2) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    if (cg == 0) p.act_s[(long long)row * p.act_ss_r + (long long)tile.n_blk * p.act_ss_b] = sc;
                }
            } else
            if (row_valid && p.d_f32) {
                float* drow = reinterpret_cast<float*>(p.d) + (long long)row * p.ldd + n0;
#pragma unroll
                for (int j = 0; j < GROUP_COLS; j += 4) {
                    if (n0 + j + 4 <= p.N) {
                        float4 o;
                        unpack_f32x2(accr[j / 2], o.x, o.y);
                        unpack_f32x2(accr[j / 2 + 1], o.z, o.w);
                        *reinterpret_cast<float4*>(drow + j) = o;
                    }
                }
            } else if (SCATTER) {
                // The four column groups of a lane quarter fill one 512-byte staging row per output row (128 bytes
                // each); the group-0 warp then sends every row with one bulk store.  Two mbarriers per quarter order
                // "previous store has read the row" -> fill -> send; their waits are bounded like every other.
                uint8_t* stg_row = smem + TILES_END + row_in_tile * gg::STAGING_ROW_BYTES;
                const uint32_t free_bar = stg_bar + 8 * quarter, filled_bar = stg_bar + 8 * (4 + quarter);
                if (cg == 0) {
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // previous tile's store has read it
                    __syncwarp();
                    if (lane == 0) mbar_arrive(free_bar);
                } else {
                    ok = mbar_wait_warp(free_bar, stg_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
                    if (!ok) break;
                }
#pragma unroll
                for (int j = 0; j < GROUP_COLS; j += 8) {
                    uint4 out;
                    out.x = cvt_bf16x2(accr[j / 2 + 0]);
                    out.y = cvt_bf16x2(accr[j / 2 + 1]);
                    out.z = cvt_bf16x2(accr[j / 2 + 2]);
                    out.w = cvt_bf16x2(accr[j / 2 + 3]);
                    *reinterpret_cast<uint4*>(stg_row + cg * (GROUP_COLS * 2) + j * 2) = out;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(filled_bar);
                if (cg == 0) {
                    ok = mbar_wait_warp(filled_bar, stg_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
                    if (!ok) break;
                    if (row_valid) {
                        const int meta = __ldg(p.scatter_meta + (long long)row * p.scatter_meta_stride);
                        __nv_bfloat16* drow = p.scatter_base[(meta >> 24) & 7] + (long long)(meta & 0xFFFFFF) * p.ldd + tile.n_blk * BN;
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 512;"
                                     ::"l"(drow), "r"(smem_u32(stg_row)) : "memory");
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                stg_phase ^= 1;
            } else if (row_valid) {
                __nv_bfloat16* drow;
                if (p.scatter_meta != nullptr) {
                    const int meta = __ldg(p.scatter_meta + (long long)row * p.scatter_meta_stride);
                    drow = p.scatter_base[(meta >> 24) & 7] + (long long)(meta & 0xFFFFFF) * p.ldd + n0;
                } else {
                    drow = reinterpret_cast<__nv_bfloat16*>(p.d) + (long long)row * p.ldd + n0;
                }
                // one 32-byte sector per thread and store where the row is 32-byte aligned, else 16-byte stores
                const bool wide = (reinterpret_cast<uintptr_t>(drow) & 31u) == 0;
#pragma unroll
                for (int j = 0; j < GROUP_COLS; j += 16) {
                    if (n0 + j < p.N) {
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = cvt_bf16x2(accr[j / 2 + i]);
                        if (wide && n0 + j + 16 <= p.N) {
                            st_global_v8(drow + j, o);
                        } else {
                            if (n0 + j + 8 <= p.N) *reinterpret_cast<uint4*>(drow + j) = make_uint4(o[0], o[1], o[2], o[3]);
                            if (n0 + j + 16 <= p.N) *reinterpret_cast<uint4*>(drow + j + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------- teardown
    if (SCATTER) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // this thread's bulk stores are complete
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace b200
