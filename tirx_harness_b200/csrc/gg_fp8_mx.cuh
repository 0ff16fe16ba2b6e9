// m-grouped FP8 GEMM, power-of-two-scale fast path: block scales applied INSIDE the tensor core.
//
// When every block scale is an exact power of two in [2^-126, 2^127] (the UE8M0 scale format of the
// registered grouped_gemm/fp8 workload, and the 2^{-4..0} law of the benchmark configurations), the
// product a*sfa and b*sfb can be formed by tcgen05.mma.kind::mxf8f6f4.block_scale itself: the scales
// are staged into TMEM as UE8M0 bytes and the accumulator simply runs over all of K.  No per-K-block
// promotion is needed, so the tensor pipe is never waiting on the CUDA cores.  The result is the same
// sum of exactly-scaled e4m3 products accumulated in fp32.
//
//   mx_prep_kernel     checks every scale and writes the UE8M0 bytes, four K blocks per 32-bit word,
//                      in the 32x16-byte tile order tcgen05.cp expects; stores the call's generation number
//                      into a flag if any scale is not a power of two (then this path stands down and the
//                      promotion kernel runs instead)
//   gg_fp8_mx_kernel   CTA pairs (cta_group::2), 256-row tiles of at most 240 columns (column tiles balanced in
//                      units of 16), 6-stage TMA ring; the scale words of four K blocks travel with the first
//                      of their stages; the leader's issuing warp runs tcgen05.cp (smem -> TMEM) and 16
//                      block-scaled MMAs per group of four K blocks.  Two accumulators in TMEM: the 8 epilogue
//                      warps of each CTA drain tile i while tile i+1 is multiplied (the first warpgroup the tile's
//                      first 128 columns, the second the rest); every thread stores its row as 32-byte sectors
//                      (st.global.v8: 32 full sectors per warp instruction, no staging, no wait).  Staging rows in
//                      shared memory for 128-byte bulk stores took 6400 cycles per tile, most of it waiting for the
//                      previous store to have read the staging slot: more than a K=2048 tile's MMAs.  256-column tiles
//                      with one accumulator (MOE_OPT_MX_TILE) are kept for measurement: the serialised drain
//                      costs them 4 to 25 % (most on short K).
//                      The producer and the MMA issuer are warp-uniform loops in which ONE ELECTED LANE issues:
//                      a single diverged lane has every TMA / tcgen05 operand moved from vector registers and
//                      needed about 880 cycles per K block where the tensor pipe needs 512.
#pragma once

#include "pair_common.cuh"

namespace b200 {

namespace mx {
constexpr int BM = 128, BK = 128;
constexpr int BN = 256;                               // widest column tile of the pair kernel (one accumulator)
constexpr int BN_WIDE = 256;
constexpr int STAGES = 6;
constexpr int THREADS = 384;
constexpr int A_STAGE_BYTES = BM * BK;
constexpr int B_STAGE_BYTES = (BN_WIDE / 2) * BK;     // sized for the wider tile; the 240-column tile uses 120 rows of it
constexpr int SMEM_TILE_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int SFQ_SLOTS = 4;                          // ring of scale tiles, one per group of 4 K blocks
constexpr int SFQ_SLOT_BYTES = 512 + 2 * 512;         // SFA (this CTA's 128 rows) + SFB (the tile's columns, 2 x 128 entries)
constexpr int OFF_SFQ = SMEM_TILE_BYTES;
constexpr int OFF_BARS = OFF_SFQ + SFQ_SLOTS * SFQ_SLOT_BYTES;
constexpr int OFF_PREFIX = OFF_BARS + 256;
constexpr int SMEM_BYTES = OFF_PREFIX + (gg::MAX_MASKED_GROUPS + 1) * 4 + 12 + 1024;
constexpr int TMEM_COLS = 512;
constexpr int TMEM_SF_STRIDE = 12;                    // per scale buffer: 4 columns SFA + 8 columns SFB
}  // namespace mx

// Packed scale tiles in the workspace (units of 128 words = one tcgen05.cp tile of 512 bytes):
//   SFA  [row block of 128][quad]                      word r = the four K-block bytes of row 128*block + r
//   SFB  [group][column tile][quad][2]                 word i of half h = those of column (tile's first) + 128*h + i
// so a kernel finds the scales of its column tile at entry 0 whatever the tile's first column and width are.
struct MxWorkspace {
    int* flag;                 // == gen after mx_prep_kernel: some scale of THIS call is not a power of two
    int gen;                   // the call's generation number (host counter): no memset between calls, a value left
                               // by an earlier call can never equal it
    uint32_t* sfa_packed;      // [row_blocks128][quads][128]
    uint32_t* sfb_packed;      // [G][n_tiles][quads][2][128]
    int row_blocks, quads;
    int n_tiles, nt_base, nt_rem;   // column tiles of the consuming kernel (mx_tile_col0 / mx_tile_width)
};

// position of row r (0..127) inside a 128-row scale tile: 32 rows of 16 bytes, word r/32 of row r%32
__device__ __forceinline__ int sf_tile_index(int r) { return (r & 31) * 4 + (r >> 5); }

__device__ __forceinline__ uint32_t ue8m0_of(float s, int* bad) {
    const uint32_t bits = __float_as_uint(s);
    const uint32_t e = bits >> 23;                    // sign must be 0, so this is the biased exponent
    if ((bits & 0x807FFFFFu) != 0u || e == 0u || e == 255u) *bad = 1;
    return e & 0xFFu;
}

// grid.x covers rows_total rounded up to 128, grid.y = quads (SFA); the tail blocks of grid.x beyond
// that handle SFB.  One thread per (row, quad).  Rows whose output is never stored -- padding rows
// (negative layout entry), rows past *rows_used, masked-out rows (row >= masked_m[g]) -- usually hold
// uninitialised scales in real callers: they get the neutral byte and cannot veto the fast path.
__global__ void mx_prep_kernel(const float* __restrict__ sfa, long long sfa_sr, long long sfa_sk,
                               const float* __restrict__ sfb, int rows_total, int KB, int G, int nb128,
                               MxWorkspace ws, const int* __restrict__ layout, int masked_max_m,
                               const int* __restrict__ rows_used) {
    int bad = 0;
    const int q = blockIdx.y;
    if ((int)blockIdx.x < ws.row_blocks) {
        const int r = blockIdx.x * 128 + threadIdx.x;
        uint32_t word = 0x7F7F7F7Fu;
        bool live = r < rows_total;
        if (live) {
            if (masked_max_m > 0) live = (r % masked_max_m) < __ldg(layout + r / masked_max_m);
            else {
                const int g = __ldg(layout + r);
                live = g >= 0 && g < G && (rows_used == nullptr || r < __ldg(rows_used));
            }
        }
        if (live) {
            word = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kb = 4 * q + i;
                const uint32_t b = kb < KB ? ue8m0_of(__ldg(sfa + (long long)r * sfa_sr + (long long)kb * sfa_sk), &bad) : 0x7Fu;
                word |= b << (8 * i);
            }
        }
        ws.sfa_packed[((long long)blockIdx.x * ws.quads + q) * 128 + sf_tile_index(threadIdx.x)] = word;
    } else {
        const int idx = blockIdx.x - ws.row_blocks;       // (group, column tile, half)
        if (idx < G * ws.n_tiles * 2) {
            const int h = idx & 1, gt = idx >> 1, g = gt / ws.n_tiles, nt = gt - g * ws.n_tiles;
            const int col = mx_tile_col0(ws.nt_base, ws.nt_rem, nt) + 128 * h + threadIdx.x;
            uint32_t word = 0x7F7F7F7Fu;
            if (col < nb128 * 128) {
                word = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int kb = 4 * q + i;
                    const uint32_t b = kb < KB ? ue8m0_of(__ldg(sfb + ((long long)g * nb128 + (col >> 7)) * KB + kb), &bad) : 0x7Fu;
                    word |= b << (8 * i);
                }
            }
            ws.sfb_packed[(((long long)gt * ws.quads + q) * 2 + h) * 128 + sf_tile_index(threadIdx.x)] = word;
        }
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) *reinterpret_cast<volatile int*>(ws.flag) = ws.gen;
}

// Same outputs from scales that already ARE UE8M0 bytes packed four to an int32 (the registered
// grouped_gemm/fp8 contract): word (row m, word q) of A at sfa[m*a_sr + q*a_sq]; word (g, column n, q) of B
// at sfb[g*b_sg + n*b_sn + q*b_sq] -- B scales are per column here.  Nothing to check: every byte is 2^e.
__global__ void mx_prep_packed_kernel(const uint32_t* __restrict__ sfa, long long a_sr, long long a_sq,
                                      const uint32_t* __restrict__ sfb, long long b_sg, long long b_sn, long long b_sq,
                                      int rows_total, int N, int G, MxWorkspace ws) {
    pdl_launch_dependents();      // a GEMM launched with programmatic serialization may start its prologue now
    const int q = blockIdx.y;
    if ((int)blockIdx.x < ws.row_blocks) {
        const int r = blockIdx.x * 128 + threadIdx.x;
        const uint32_t word = r < rows_total ? __ldg(sfa + (long long)r * a_sr + (long long)q * a_sq) : 0x7F7F7F7Fu;
        ws.sfa_packed[((long long)blockIdx.x * ws.quads + q) * 128 + sf_tile_index(threadIdx.x)] = word;
    } else {
        const int idx = blockIdx.x - ws.row_blocks;       // (group, column tile, half)
        if (idx < G * ws.n_tiles * 2) {
            const int h = idx & 1, gt = idx >> 1, g = gt / ws.n_tiles, nt = gt - g * ws.n_tiles;
            const int n = mx_tile_col0(ws.nt_base, ws.nt_rem, nt) + 128 * h + threadIdx.x;
            const uint32_t word = n < N ? __ldg(sfb + (long long)g * b_sg + (long long)n * b_sn + (long long)q * b_sq) : 0x7F7F7F7Fu;
            ws.sfb_packed[(((long long)gt * ws.quads + q) * 2 + h) * 128 + sf_tile_index(threadIdx.x)] = word;
        }
    }
}

// ------------------------------------------------------------------ PTX for this path
__device__ __forceinline__ void tma_load_1d_pair(uint32_t smem_dst, const void* tmap, uint32_t cluster_bar, int32_t c0) {
    asm volatile(
        "cp.async.bulk.tensor.1d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3}], [%2];"
        ::"r"(smem_dst), "l"(tmap), "r"(cluster_bar), "r"(c0)
        : "memory");
}
// shared-memory descriptor of one 128-row scale tile: 8-row groups of 16-byte rows, 128 bytes apart, no swizzle
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}
// 32 rows x 128 bits from shared memory, broadcast to the four 32-lane quarters of TMEM, in both CTAs
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
// block-scaled instruction descriptor: e4m3 x e4m3, UE8M0 scales, K-major operands; sf_id = which byte
// of the 32-bit scale word (= which of the four K blocks) this instruction uses
__device__ __forceinline__ uint32_t make_idesc_mxf8(int m, int n, uint32_t sf_id) {
    return (sf_id << 4)                                   // B scale id
           | (0u << 7) | (0u << 10)                       // A, B format: e4m3
           | (static_cast<uint32_t>(n >> 3) << 17)        // N / 8
           | (1u << 23)                                   // scale format: UE8M0
           | (static_cast<uint32_t>(m >> 4) << 24)        // M / 16
           | (sf_id << 29);                               // A scale id
}

// ---- k-grouped schedule of the pair kernel: G groups share the rows of A ([M, K_total], K-major copy) and of B
// ([N, K_total]); group g multiplies them over its K window and owns d[g].  Passed by value (up to 64 groups).
struct KgTable {
    int n;                 // groups
    int per_group;         // pair tiles per group: ceil(M/256) * column blocks
    int koff[64];          // first K element of each group
    int kb[64];            // K blocks (128) of each group
    int qoff[64];          // first scale word row (4 K blocks per word) of each group
};
struct KgNone {};
template <bool KG> struct KgArg { using type = KgNone; };
template <> struct KgArg<true> { using type = KgTable; };

template <bool MASKED, bool KG> struct MxSched;
template <bool MASKED>
struct MxSched<MASKED, false> : PairScheduler<MASKED> {
    __device__ __forceinline__ MxSched(const GGParams& p_, const int* prefix_, int lane_, int rank_, const KgNone&)
        : PairScheduler<MASKED>(p_, prefix_, lane_, rank_) {}
    static __device__ __forceinline__ int k_offset(const KgNone&, int) { return 0; }
    static __device__ __forceinline__ int k_blocks(const KgNone&, int, int KB) { return KB; }
    static __device__ __forceinline__ int quad_offset(const KgNone&, int) { return 0; }
};
template <>
struct MxSched<false, true> {
    const GGParams& p;
    const KgTable& kg;
    int t, stride, rank, total;
    __device__ __forceinline__ MxSched(const GGParams& p_, const int*, int, int rank_, const KgTable& kg_)
        : p(p_), kg(kg_), t(blockIdx.x >> 1), stride(gridDim.x >> 1), rank(rank_), total(kg_.n * kg_.per_group) {}
    __device__ __forceinline__ bool next(Tile& tile) {
        while (t < total) {
            const int g = t / kg.per_group, rem = t - g * kg.per_group;
            t += stride;
            if (kg.kb[g] == 0) continue;          // a group without K rows leaves its d untouched
            tile.g = g;
            tile.m0 = (rem / p.num_n_blocks) * 256 + rank * 128;
            tile.n_blk = rem % p.num_n_blocks;
            tile.rows = 128;
            return true;
        }
        return false;
    }
    static __device__ __forceinline__ int k_offset(const KgTable& k, int g) { return k.koff[g]; }
    static __device__ __forceinline__ int k_blocks(const KgTable& k, int g, int) { return k.kb[g]; }
    static __device__ __forceinline__ int quad_offset(const KgTable& k, int g) { return k.qoff[g]; }
};

template <bool MASKED, bool KG = false, bool MNMAJOR = false, int TILE_N = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(mx::THREADS, 1)
gg_fp8_mx_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                 const GGParams p, const int* __restrict__ flag, int quads, int* status,
                 const __grid_constant__ typename KgArg<KG>::type kg) {
    using namespace mx;
    static_assert(!(MASKED && KG), "the k-grouped schedule is a contiguous-layout mode");
    static_assert(!MNMAJOR || KG, "MN-major operands are the k-grouped layout's");
    // MNMAJOR: the operands stay as the caller has them, a [K_total, M] and b [K_total, N] (M / N contiguous); a stage
    // holds 128 K rows x 128 bytes of M (or N), the MMAs read it as an MN-major operand (instruction descriptor bits
    // 15 and 16) and step 32 K rows = 4096 bytes per instruction.
    // Column tile and accumulators: two 240-column accumulators, or (k-grouped modes) one of 256 columns.
    constexpr int TN = TILE_N ? TILE_N : BN;
    constexpr int ACCS = 2 * TN + 2 * TMEM_SF_STRIDE <= TMEM_COLS ? 2 : 1;
    constexpr int SF_BASE = ACCS * TN;                // scale columns behind the accumulators
    static_assert(SF_BASE + 2 * TMEM_SF_STRIDE <= TMEM_COLS, "accumulators and scale buffers must fit TMEM");
    using Sched = MxSched<MASKED, KG>;
    // some scale is not a power of two: the promotion kernel handles this call (packed UE8M0 scales: no flag to read)
    if (flag != nullptr && *flag == p.mode_gen) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
    uint8_t* smem_sfq = smem + OFF_SFQ;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
    // [0,S) full (leader's used), [S,2S) empty, [2S, 2S+2) tmem_full, [2S+2, 2S+4) tmem_empty (leader's used)
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    int* prefix = reinterpret_cast<int*>(smem + OFF_PREFIX);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);       // a value the compiler knows to be warp-uniform
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();

    const uint32_t full_bar = smem_u32(bars);
    const uint32_t empty_bar = smem_u32(bars + STAGES);
    const uint32_t tfull_bar = smem_u32(bars + 2 * STAGES);
    const uint32_t tempty_bar = smem_u32(bars + 2 * STAGES + 2);
    const uint32_t leader_full_bar = map_to_cta(full_bar, 0);
    const uint32_t leader_tempty_bar = map_to_cta(tempty_bar, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar + 8 * a, 1);
            mbar_init(tempty_bar + 8 * a, 16);        // the 16 epilogue warps of the pair
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_sfa);
        tma_prefetch_desc(&tmap_sfb);
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
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const int KB = p.num_k_blocks;
    // columns the pair multiplies for column tile n_blk: the full tile, or what is left of N rounded up to 16 (the
    // MMA's N granularity; columns past N are computed from whatever rows follow in B and never stored)
    auto tile_col0 = [&](int n_blk) { return mx_tile_col0(p.nt_base, p.nt_rem, n_blk); };
    auto tile_cols = [&](int n_blk) {
        if (KG) return TN;                  // MN-major operand stages are 128-byte swizzle rows of N: fixed halves of 128 columns
        const int w = mx_tile_width(p.nt_base, p.nt_rem, n_blk), left = ((p.N - tile_col0(n_blk)) + 15) & ~15;
        return left < w ? left : w;
    };

    if (warp < 4) {
        setmaxnreg_dec<72>();
        if (warp == 0) {
            // ------------------------------------------------ TMA producer (both CTAs)
            // The whole warp runs the loop and one elected lane issues: coordinates, barrier addresses and
            // descriptors then stay warp-uniform values, which is what the TMA and tcgen05 instructions take.
            Sched sched(p, prefix, lane, rank, kg);
            Tile tile;
            uint32_t stage = 0, phase = 0, qcount = 0;
            bool pdl_pending = p.pdl_scales != 0;
            long long tr_wait = 0;
            const long long tr_t0 = B200_TRACE(p.trace) ? clock64() : 0;
            bool ok = true;
            while (ok && sched.next(tile)) {
                // this CTA stages its half of the tile's columns; k-grouped: every group multiplies the same rows of
                // A and B over its own K window
                const int b_row = (KG ? 0 : tile.g * p.N) + tile_col0(tile.n_blk) + (int)rank * (tile_cols(tile.n_blk) >> 1);
                const int k0 = Sched::k_offset(kg, tile.g);
                const int KBt = Sched::k_blocks(kg, tile.g, KB);
                const int q0 = Sched::quad_offset(kg, tile.g);
                const int sfa_chunk = (tile.m0 >> 7) * quads + q0;                  // this CTA's 128 rows
                const int n_tiles = p.num_n_blocks;
                const int sfb_chunk = (((KG ? 0 : tile.g * n_tiles) + tile.n_blk) * quads + q0) * 2;  // two 128-entry halves per quad
                for (int kb = 0; kb < KBt; ++kb) {
                    const long long c0 = B200_TRACE(p.trace) ? clock64() : 0;
                    ok = mbar_wait_warp(empty_bar + 8 * stage, phase ^ 1, abort_flag, status,
                                        STATUS_TIMEOUT_SMEM_EMPTY);
                    if (B200_TRACE(p.trace)) tr_wait += clock64() - c0;
                    if (!ok) break;
                    const bool with_sf = (kb & 3) == 0;
                    if (elect_one_sync()) {
                        const uint32_t fb = leader_full_bar + 8 * stage;
                        constexpr int B_BYTES = (TN / 2) * BK;                          // bytes one TMA box of B delivers
                        if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * stage, 2 * (A_STAGE_BYTES + B_BYTES + (with_sf ? SFQ_SLOT_BYTES : 0)));
                        if (MNMAJOR) {
                            tma_load_2d_pair(smem_u32(smem_a + stage * A_STAGE_BYTES), &tmap_a, fb, tile.m0, k0 + kb * BK);
                            tma_load_2d_pair(smem_u32(smem_b + stage * B_STAGE_BYTES), &tmap_b, fb, b_row, k0 + kb * BK);
                        } else {
                            tma_load_2d_pair(smem_u32(smem_a + stage * A_STAGE_BYTES), &tmap_a, fb, k0 + kb * BK, tile.m0);
                            tma_load_2d_pair(smem_u32(smem_b + stage * B_STAGE_BYTES), &tmap_b, fb, k0 + kb * BK, b_row);
                        }
                        if (with_sf) {
                            if (pdl_pending) pdl_wait();          // the packed scale tiles are the predecessor's output
                            const int q = kb >> 2;
                            const uint32_t dst = smem_u32(smem_sfq + (qcount % SFQ_SLOTS) * SFQ_SLOT_BYTES);
                            tma_load_1d_pair(dst, &tmap_sfa, fb, (sfa_chunk + q) * 128);
                            tma_load_1d_pair(dst + 512, &tmap_sfb, fb, (sfb_chunk + 2 * q) * 128);
                            tma_load_1d_pair(dst + 1024, &tmap_sfb, fb, (sfb_chunk + 2 * q + 1) * 128);
                        }
                    }
                    if (with_sf) { ++qcount; pdl_pending = false; }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (B200_TRACE(p.trace) && lane == 0) {
                p.trace[blockIdx.x * 16 + 0] = tr_wait;
                p.trace[blockIdx.x * 16 + 1] = clock64() - tr_t0;
            }
        } else if (warp == 1 && rank == 0) {
            // ------------------------------------------------ MMA issuer (leader)
            // Warp-uniform loop, one elected lane issues.  The tensor pipe only queues a couple of MMAs, so what
            // this warp spends between two K blocks is a bubble: with the loop state in uniform registers a K block
            // costs the issuer well under the 512 cycles the pipe needs for it; a single diverged lane (every
            // operand moved from a vector register) needed more than that.
            Sched sched(p, prefix, lane, rank, kg);
            Tile tile;
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0, qcount = 0;
            bool ok = true;
            const uint64_t adesc0 = make_smem_desc_sw128(smem_u32(smem_a));
            const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(smem_b));
            constexpr uint64_t KSTEP = MNMAJOR ? (32 * 128) >> 4 : 2;      // descriptor units (16 bytes) per K = 32
            long long tr_te = 0, tr_full = 0, tr_issue = 0;
            const long long tr_m0 = B200_TRACE(p.trace) ? clock64() : 0;
            // The schedule of the NEXT tile is worked out right after the first K block of the current one has been
            // issued: the tensor pipe then has that block's MMAs to run, and the warp is not in the way at the tile border.
            Tile next_tile;
            bool have = sched.next(tile), have_next = false;
            while (ok && have) {
                // this tile's accumulator must have been drained by both CTAs' epilogues
                const long long c0 = B200_TRACE(p.trace) ? clock64() : 0;
                ok = mbar_wait_warp(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_TMEM_EMPTY);
                if (B200_TRACE(p.trace)) tr_te += clock64() - c0;
                if (!ok) break;
                tc_fence_after();
                const int KBt = Sched::k_blocks(kg, tile.g, KB);
                const uint32_t idesc0 = make_idesc_mxf8(2 * BM, tile_cols(tile.n_blk), 0) | (MNMAJOR ? (1u << 15) | (1u << 16) : 0u);
                const uint32_t tmem_d = tmem_base + acc * TN;
                for (int kb = 0; kb < KBt; ++kb) {
                    const long long c1 = B200_TRACE(p.trace) ? clock64() : 0;
                    ok = mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, status, STATUS_TIMEOUT_SMEM_FULL);
                    const long long c2 = B200_TRACE(p.trace) ? clock64() : 0;
                    tr_full += c2 - c1;
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sub = kb & 3;
                    if (elect_one_sync()) {
                        if (sub == 0) {
                            const uint32_t src = smem_u32(smem_sfq + (qcount % SFQ_SLOTS) * SFQ_SLOT_BYTES);
                            const uint32_t tsf = tmem_base + SF_BASE + (qcount & 1) * TMEM_SF_STRIDE;
                            tmem_cp_sf_pair(tsf, make_sf_desc(src));
                            tmem_cp_sf_pair(tsf + 4, make_sf_desc(src + 512));
                            tmem_cp_sf_pair(tsf + 8, make_sf_desc(src + 1024));
                        }
                        const uint32_t tsfa = tmem_base + SF_BASE + ((qcount - (sub == 0 ? 0u : 1u)) & 1) * TMEM_SF_STRIDE;
                        const uint32_t tsfb = tsfa + 4;
                        const uint32_t idesc = idesc0 | (sub << 4) | (sub << 29);
                        const uint64_t adesc = adesc0 + stage * (A_STAGE_BYTES >> 4);
                        const uint64_t bdesc = bdesc0 + stage * (B_STAGE_BYTES >> 4);
                        umma_mxf8_pair(tmem_d, adesc, bdesc, idesc, tsfa, tsfb, kb > 0 ? 1u : 0u);
                        umma_mxf8_pair(tmem_d, adesc + KSTEP, bdesc + KSTEP, idesc, tsfa, tsfb, 1u);
                        umma_mxf8_pair(tmem_d, adesc + 2 * KSTEP, bdesc + 2 * KSTEP, idesc, tsfa, tsfb, 1u);
                        umma_mxf8_pair(tmem_d, adesc + 3 * KSTEP, bdesc + 3 * KSTEP, idesc, tsfa, tsfb, 1u);
                        umma_commit_pair(empty_bar + 8 * stage, 3);
                        if (kb == KBt - 1) umma_commit_pair(tfull_bar + 8 * acc, 3);
                    }
                    if (sub == 0) ++qcount;
                    if (B200_TRACE(p.trace)) tr_issue += clock64() - c2;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    if (kb == 0) have_next = sched.next(next_tile);
                }
                tile = next_tile;
                have = have_next;
                if (++acc == ACCS) { acc = 0; acc_phase ^= 1; }
            }
            if (B200_TRACE(p.trace) && lane == 0) {
                p.trace[blockIdx.x * 16 + 2] = tr_te;
                p.trace[blockIdx.x * 16 + 3] = tr_full;
                p.trace[blockIdx.x * 16 + 4] = tr_issue;
                p.trace[blockIdx.x * 16 + 5] = clock64() - tr_m0;
            }
        }
    } else {
        // ---------------------------------------------------- epilogue (both CTAs): drains tile i while tile i+1 is multiplied
        setmaxnreg_inc<208>();
        const int ew = warp - 4;
        const int quarter = warp & 3;
        const int half = ew >> 2;
        const int row_in_tile = quarter * 32 + lane;
        Sched sched(p, prefix, lane, rank, kg);
        Tile tile;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        while (ok && sched.next(tile)) {
            // this warpgroup's columns: the first 128 of the tile, or what follows them (80 to 128 columns): both ranges
            // start on a multiple of 16 columns, i.e. on a 32-byte boundary of the bf16 output row
            const int tw = tile_cols(tile.n_blk);
            const int n0 = tile_col0(tile.n_blk) + half * 128;
            const int n_tile_end = tile_col0(tile.n_blk) + tw;
            const int n_end = n_tile_end < p.N ? n_tile_end : p.N;      // first column this thread must not store
            int row = tile.m0 + row_in_tile;
            bool row_valid;
            if (MASKED) row_valid = row_in_tile < tile.rows;
            else if (KG) row_valid = row < p.M;
            else row_valid = (row < p.M) && (__ldg(p.layout + row) == tile.g);
            if (KG) row += tile.g * p.M;          // d is [G, M, N]
            ok = mbar_wait_warp(tfull_bar + 8 * acc, acc_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
            if (!ok) break;
            tc_fence_after();
            // 128 columns from the accumulator's column 128 * half on (for the second warpgroup of a narrower tile the
            // last of them belong to whatever follows the accumulator in TMEM; they are loaded and never stored)
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * TN + half * 128;
            uint32_t v[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(taddr + c * 32, v[c]);
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_wait(v[c]);
            // the accumulator is in registers: the MMAs of the tile after next may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tempty_bar + 8 * acc);
            if (++acc == ACCS) { acc = 0; acc_phase ^= 1; }
            if (row_valid && p.d_f32) {
                float* drow = reinterpret_cast<float*>(p.d) + (long long)row * p.ldd + n0;
#pragma unroll
                for (int j = 0; j < 128; j += 4) {
                    if (n0 + j + 4 <= n_end) {
                        float4 o = make_float4(__uint_as_float(v[j / 32][j % 32]), __uint_as_float(v[j / 32][j % 32 + 1]),
                                               __uint_as_float(v[j / 32][j % 32 + 2]), __uint_as_float(v[j / 32][j % 32 + 3]));
                        if (p.d_accumulate) red_add_f32x4(drow + j, o);      // one contributor per element: same as load+add+store
                        else *reinterpret_cast<float4*>(drow + j) = o;
                    }
                }
            } else if (row_valid) {
                // bf16: every thread converts its row 16 columns at a time and stores them as ONE 32-byte sector
                // (st.global.v8): 32 lanes = 32 full sectors per instruction, nothing to stage and nothing to wait for.
                // Rows whose address is not 32-byte aligned (odd leading dimensions) take 16-byte stores.
                __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.d) + (long long)row * p.ldd + n0;
                const bool wide = (reinterpret_cast<uintptr_t>(drow) & 31u) == 0;
#pragma unroll
                for (int j = 0; j < 128; j += 16) {
                    if (n0 + j < n_end) {
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint32_t* sp = &v[(j + 2 * i) / 32][(j + 2 * i) % 32];
                            o[i] = cvt_bf16x2(pack_f32x2(__uint_as_float(sp[0]), __uint_as_float(sp[1])));
                        }
                        if (wide && n0 + j + 16 <= n_end) {
                            st_global_v8(drow + j, o);
                        } else {
                            if (n0 + j + 8 <= n_end) *reinterpret_cast<uint4*>(drow + j) = make_uint4(o[0], o[1], o[2], o[3]);
                            if (n0 + j + 16 <= n_end) *reinterpret_cast<uint4*>(drow + j + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------
// Single-CTA version of the same path: 128 x 256 tiles, cta_group::1, four 48 KB stages.  No cross-SM
// signalling at all and only 128 rows per tile (half the wasted MMA work on ragged or masked groups).
namespace mx1 {
constexpr int BM = 128, BN = 256, BK = 128;
constexpr int STAGES = 4;
constexpr int THREADS = 384;
constexpr int A_STAGE_BYTES = BM * BK;
constexpr int B_STAGE_BYTES = BN * BK;
constexpr int SMEM_TILE_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);
constexpr int SFQ_SLOTS = 4;
constexpr int SFQ_SLOT_BYTES = 512 + 2 * 512;
constexpr int OFF_SFQ = SMEM_TILE_BYTES;
constexpr int OFF_BARS = OFF_SFQ + SFQ_SLOTS * SFQ_SLOT_BYTES;
constexpr int OFF_PREFIX = OFF_BARS + 256;
constexpr int SMEM_BYTES = OFF_PREFIX + gg::MASKED_TABLE_INTS * 4 + 12 + 1024;
}  // namespace mx1
// (the single-CTA kernel keeps 256-column tiles and one accumulator: its use is the masked decode layout, which is
// bound by streaming the weights from HBM, not by the tensor pipe)

__device__ __forceinline__ void tma_load_1d(uint32_t smem_dst, const void* tmap, uint32_t bar, int32_t c0) {
    asm volatile(
        "cp.async.bulk.tensor.1d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3}], [%2];"
        ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(c0)
        : "memory");
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

template <bool MASKED>
__global__ void __launch_bounds__(mx1::THREADS, 1)
gg_fp8_mx1_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                  const GGParams p, const int* __restrict__ flag, int quads, int* status) {
    using namespace mx1;
    if (*flag == p.mode_gen) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
    uint8_t* smem_sfq = smem + OFF_SFQ;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    int* prefix = reinterpret_cast<int*>(smem + OFF_PREFIX);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);       // a value the compiler knows to be warp-uniform
    const int lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_u32(bars);
    const uint32_t empty_bar = smem_u32(bars + STAGES);
    const uint32_t tfull_bar = smem_u32(bars + 2 * STAGES);
    const uint32_t tempty_bar = smem_u32(bars + 2 * STAGES + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        mbar_init(tfull_bar, 1);
        mbar_init(tempty_bar, 8);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_sfa);
        tma_prefetch_desc(&tmap_sfb);
    }
    if (MASKED) build_masked_tables(p, prefix, 3);
    constexpr int TMEM_SF_BASE = BN;          // one 256-column accumulator, scale columns behind it
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), mx::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const int KB = p.num_k_blocks;

    if (warp < 4) {
        setmaxnreg_dec<72>();
        if (warp == 0) {
            // ------------------------------------------------ TMA producer
            Scheduler<MASKED> sched(p, prefix, lane);
            Tile tile;
            uint32_t stage = 0, phase = 0, qcount = 0;
            bool ok = true;
            while (ok && sched.next(tile)) {
                const int b_row = tile.g * p.N + tile.n_blk * BN;
                const int sfa_chunk = (tile.m0 >> 7) * quads;
                const int sfb_chunk = ((tile.g * p.num_n_blocks + tile.n_blk) * quads) * 2;      // two 128-entry halves per quad
                for (int kb = 0; kb < KB; ++kb) {
                    ok = mbar_wait_warp(empty_bar + 8 * stage, phase ^ 1, abort_flag, status, STATUS_TIMEOUT_SMEM_EMPTY);
                    if (!ok) break;
                    if (elect_one_sync()) {
                        const uint32_t fb = full_bar + 8 * stage;
                        const bool with_sf = (kb & 3) == 0;
                        mbar_arrive_expect_tx(fb, A_STAGE_BYTES + B_STAGE_BYTES + (with_sf ? SFQ_SLOT_BYTES : 0));
                        tma_load_2d(smem_u32(smem_a + stage * A_STAGE_BYTES), &tmap_a, fb, kb * BK, tile.m0);
                        tma_load_2d(smem_u32(smem_b + stage * B_STAGE_BYTES), &tmap_b, fb, kb * BK, b_row);
                        if (with_sf) {
                            const int q = kb >> 2;
                            const uint32_t dst = smem_u32(smem_sfq + (qcount % SFQ_SLOTS) * SFQ_SLOT_BYTES);
                            tma_load_1d(dst, &tmap_sfa, fb, (sfa_chunk + q) * 128);
                            tma_load_1d(dst + 512, &tmap_sfb, fb, (sfb_chunk + 2 * q) * 128);
                            tma_load_1d(dst + 1024, &tmap_sfb, fb, (sfb_chunk + 2 * q + 1) * 128);
                        }
                    }
                    __syncwarp();
                    if ((kb & 3) == 0) ++qcount;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------ MMA issuer (warp-uniform loop, one elected lane issues)
            Scheduler<MASKED> sched(p, prefix, lane);
            Tile tile;
            uint32_t stage = 0, phase = 0, tile_phase = 0, qcount = 0;
            bool ok = true;
            const uint64_t adesc0 = make_smem_desc_sw128(smem_u32(smem_a));
            const uint64_t bdesc0 = make_smem_desc_sw128(smem_u32(smem_b));
            const uint32_t idesc0 = make_idesc_mxf8(BM, BN, 0);
            while (ok && sched.next(tile)) {
                ok = mbar_wait_warp(tempty_bar, tile_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < KB; ++kb) {
                    ok = mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, status, STATUS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sub = kb & 3;
                    if (elect_one_sync()) {
                        if (sub == 0) {
                            const uint32_t src = smem_u32(smem_sfq + (qcount % SFQ_SLOTS) * SFQ_SLOT_BYTES);
                            const uint32_t tsf = tmem_base + TMEM_SF_BASE + (qcount & 1) * mx::TMEM_SF_STRIDE;
                            tmem_cp_sf(tsf, make_sf_desc(src));
                            tmem_cp_sf(tsf + 4, make_sf_desc(src + 512));
                            tmem_cp_sf(tsf + 8, make_sf_desc(src + 1024));
                        }
                        const uint32_t tsfa = tmem_base + TMEM_SF_BASE + ((qcount - (sub == 0 ? 0u : 1u)) & 1) * mx::TMEM_SF_STRIDE;
                        const uint32_t tsfb = tsfa + 4;
                        const uint32_t idesc = idesc0 | (sub << 4) | (sub << 29);
                        const uint64_t adesc = adesc0 + stage * (A_STAGE_BYTES >> 4);
                        const uint64_t bdesc = bdesc0 + stage * (B_STAGE_BYTES >> 4);
                        umma_mxf8(tmem_base, adesc, bdesc, idesc, tsfa, tsfb, kb > 0 ? 1u : 0u);
                        umma_mxf8(tmem_base, adesc + 2, bdesc + 2, idesc, tsfa, tsfb, 1u);
                        umma_mxf8(tmem_base, adesc + 4, bdesc + 4, idesc, tsfa, tsfb, 1u);
                        umma_mxf8(tmem_base, adesc + 6, bdesc + 6, idesc, tsfa, tsfb, 1u);
                        umma_commit(empty_bar + 8 * stage);
                        if (kb == KB - 1) umma_commit(tfull_bar);
                    }
                    if (sub == 0) ++qcount;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                tile_phase ^= 1;
            }
        }
    } else {
        // ---------------------------------------------------- epilogue: one drain per tile
        setmaxnreg_inc<208>();
        const int ew = warp - 4;
        const int quarter = warp & 3;
        const int half = ew >> 2;
        const int row_in_tile = quarter * 32 + lane;
        Scheduler<MASKED> sched(p, prefix, lane);
        Tile tile;
        uint32_t tile_phase = 0;
        bool ok = true;
        while (ok && sched.next(tile)) {
            const int n0 = tile.n_blk * BN + half * 128;
            const int row = tile.m0 + row_in_tile;
            bool row_valid;
            if (MASKED) row_valid = row_in_tile < tile.rows;
            else row_valid = (row < p.M) && (__ldg(p.layout + row) == tile.g);
            ok = mbar_wait_warp(tfull_bar, tile_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
            if (!ok) break;
            tile_phase ^= 1;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + half * 128;
            uint32_t v[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(taddr + c * 32, v[c]);
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_wait(v[c]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar);
            if (row_valid && p.d_f32) {
                float* drow = reinterpret_cast<float*>(p.d) + (long long)row * p.ldd + n0;
#pragma unroll
                for (int j = 0; j < 128; j += 4) {
                    if (n0 + j + 4 <= p.N) {
                        float4 o = make_float4(__uint_as_float(v[j / 32][j % 32]), __uint_as_float(v[j / 32][j % 32 + 1]),
                                               __uint_as_float(v[j / 32][j % 32 + 2]), __uint_as_float(v[j / 32][j % 32 + 3]));
                        if (p.d_accumulate) red_add_f32x4(drow + j, o);      // one contributor per element: same as load+add+store
                        else *reinterpret_cast<float4*>(drow + j) = o;
                    }
                }
            } else if (row_valid) {
                // one 32-byte sector per thread and store where the row is 32-byte aligned, else 16-byte stores
                __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.d) + (long long)row * p.ldd + n0;
                const bool wide = (reinterpret_cast<uintptr_t>(drow) & 31u) == 0;
#pragma unroll
                for (int j = 0; j < 128; j += 16) {
                    if (n0 + j < p.N) {
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint32_t* sp = &v[(j + 2 * i) / 32][(j + 2 * i) % 32];
                            o[i] = cvt_bf16x2(pack_f32x2(__uint_as_float(sp[0]), __uint_as_float(sp[1])));
                        }
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

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, mx::TMEM_COLS);
    }
}

}  // namespace b200
