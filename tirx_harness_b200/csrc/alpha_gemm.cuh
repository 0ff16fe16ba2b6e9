// Decode-regime expert GEMMs with the operands swapped: the expert's weight rows are the MMA's M dimension
// (128 output features per tile), the few tokens routed to the expert are its N dimension (32 columns).
// A 128 x 32 fp32 accumulator costs one tcgen05.ld per K block to drain instead of the 128 x 256 of the
// row-major tiling, eight accumulator buffers fit in TMEM, and the kernel streams weights at HBM speed.
//
//   PHASE 1  gate_up + SiLU(gate)*up + 1x128 requant: unit = (expert, chunk of <= 32 routed rows); per K block
//            the gate tile and the up tile of W13 (2 x 16 KB) and the rows' FP8 bytes (4 KB) are staged by TMA,
//            8 MMAs (M=128, N=32, K=32) accumulate into two TMEM buffers, the epilogue promotes them with
//            sfa[row,kb] * sfb[block,kb] into registers (thread = feature, register = row); after the last K
//            block the 128 features of each row are reduced to their amax across the four epilogue warps,
//            requantised and stored as the next GEMM's operand.  The fp32 gate_up row is stored as well
//            (inspection / tests; 1 KB per routed row).
//   PHASE 2  down projection: unit = (expert, chunk, 128-feature tile of the hidden size); one K block
//            (I = 128); the fp32 result goes to the route's row of d2 for the ordered bf16 reduction.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer (one thread), warp 2 scale loader (cp.async into a ring),
// warps 4-7 epilogue (TMEM lane quadrant = warp % 4).  All waits are bounded.
#pragma once

#include "gg_fp8.cuh"
#include "moe_ops.cuh"

namespace b200 {

namespace asw {
constexpr int NT = 32;                       // routed rows (MMA N) per unit
constexpr int BK = 128;
constexpr int W_TILE_BYTES = 128 * BK;       // 16 KB
constexpr int X_TILE_BYTES = NT * BK;        // 4 KB
constexpr int ACC_BUFS = 8;
constexpr int ACC_STRIDE = 64;               // TMEM columns per buffer: [0,32) first tile, [32,64) second tile
constexpr int TMEM_COLS = 512;
constexpr int SF_SLOTS = 16;
constexpr int SF_SLOT_FLOATS = 36;           // 32 row scales + 2 block scales (+ pad)
constexpr int UNIT_CAP = 2048;               // (expert, chunk) units: E + routes/32 <= 1024 + 1024
constexpr int MAX_E = 1024;
template <int PHASE> struct Cfg {
    // epilogue teams of four warps that take alternate units: with one K block per unit (PHASE 2) a unit is a
    // latency chain (barrier, TMEM load, stores) that only a second team can overlap
    static constexpr int TEAMS = PHASE == 1 ? 1 : 2;
    static constexpr int THREADS = 128 + TEAMS * 128;
    static constexpr int W_TILES = PHASE == 1 ? 2 : 1;
    static constexpr int STAGES = PHASE == 1 ? 5 : 8;
    static constexpr int STAGE_BYTES = W_TILES * W_TILE_BYTES + X_TILE_BYTES;
    static constexpr int OFF_BARS = STAGES * STAGE_BYTES;
    static constexpr int OFF_SF = OFF_BARS + 1024;
    static constexpr int OFF_AMAX = OFF_SF + SF_SLOTS * SF_SLOT_FLOATS * 4;
    static constexpr int OFF_TABLES = OFF_AMAX + 2 * 4 * NT * 4;
    static constexpr int SMEM_BYTES = OFF_TABLES + (MAX_E + 1 + UNIT_CAP) * 4 + 16 + 1024;
};
}  // namespace asw

struct AlphaGemmParams {
    const int* counts;          // routed rows per expert [E]
    int E, max_m;
    long long rows_total;       // E * max_m
    const float* s_rows;        // scale of (row, K block kb) at s_rows[kb * rows_total + row]
    const float* sfb;           // PHASE 1: w13_scale [E][2][KB];  PHASE 2: w2_scale [E][NF][1]
    int KB;                     // K blocks per unit (PHASE 2: 1)
    int NF;                     // PHASE 2: 128-feature tiles of the hidden size (PHASE 1: 1)
    uint8_t* a2;                // PHASE 1 out: e4m3 [rows_total, 128]
    float* s2;                  // PHASE 1 out: [rows_total]
    float* g1;                  // PHASE 1 out: fp32 [rows_total, 256] gate_up
    float* d2;                  // PHASE 2 out: fp32 [rows_total, H]
    int H;
    long long* trace;           // developer aid: per-CTA wait-cycle counters [grid][8], or nullptr
};

struct AlphaUnit {
    int e, row0, n_valid, f;    // expert, first row of the chunk, rows in use (<= NT), feature tile
};

// units in (expert, chunk, feature tile) order, round-robin over the CTAs
struct AlphaSched {
    const int* list;
    const int* counts_s;
    int t, total, nf, max_m;
    __device__ __forceinline__ AlphaSched(const int* tables, int nf_, int max_m_)
        : list(tables + asw::MAX_E + 1), counts_s(tables + 1), t(blockIdx.x), total(tables[0] * nf_), nf(nf_),
          max_m(max_m_) {}
    __device__ __forceinline__ bool next(AlphaUnit& u) {
        if (t >= total) return false;
        const int entry = list[t / nf];
        u.e = entry >> 16;
        const int chunk = entry & 0xFFFF;
        u.f = t % nf;
        u.row0 = u.e * max_m + chunk * asw::NT;
        const int left = counts_s[u.e] - chunk * asw::NT;
        u.n_valid = left < asw::NT ? left : asw::NT;
        t += gridDim.x;
        return true;
    }
};

// tables[0] = number of (expert, chunk) units, tables[1 + e] = clamped count, tables[1 + MAX_E + i] = unit i
__device__ __forceinline__ void alpha_build_units(const AlphaGemmParams& p, int* tables) {
    int* cnt = tables + 1;
    int* list = tables + 1 + asw::MAX_E;
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
        int c = __ldg(p.counts + e);
        cnt[e] = c < 0 ? 0 : (c > p.max_m ? p.max_m : c);
    }
    __syncthreads();
    if ((threadIdx.x >> 5) == 3) {
        const int lane = threadIdx.x & 31;
        int running = 0;
        for (int base = 0; base < p.E; base += 32) {
            const int e = base + lane;
            const int chunks = e < p.E ? (cnt[e] + asw::NT - 1) / asw::NT : 0;
            int incl = chunks;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int first = running + incl - chunks;
            for (int c = 0; c < chunks && first + c < asw::UNIT_CAP; ++c) list[first + c] = (e << 16) | c;
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) tables[0] = running < asw::UNIT_CAP ? running : asw::UNIT_CAP;
    }
}

template <int NC> struct TmemCols;
template <> struct TmemCols<16> {
    static __device__ __forceinline__ void load(uint32_t taddr, uint32_t (&v)[16]) { tmem_ld_32x32b_x16(taddr, v); }
};
template <> struct TmemCols<32> {
    static __device__ __forceinline__ void load(uint32_t taddr, uint32_t (&v)[32]) { tmem_ld_32x32b_x32(taddr, v); }
};

// State of one epilogue warp of alpha_swap_kernel; unit<NC>() processes one unit reading NC accumulator columns.
template <int PHASE>
struct AlphaEpilogue {
    const AlphaGemmParams& p;
    uint32_t tmem_base, tfull_bar, tempty_bar, sffull_bar, sfempty_bar, amax_bar;
    const float* sf_ring;
    float* amax_s;
    volatile int* abort_flag;
    int* status;
    int ew, lane;                              // ew == TMEM lane quadrant (warp % 4)
    uint32_t step = 0, unit_parity = 0;        // step = K blocks of this CTA handled so far (by any team)
    long long tr_tf = 0, tr_sf = 0;

    __device__ __forceinline__ void skip_unit() { step += p.KB; }

    template <int NC>
    __device__ __forceinline__ bool unit(const AlphaUnit& u) {
        using namespace asw;
        const int feat = ew * 32 + lane;
        float a0[NC], a1[NC];                  // PHASE 1: gate / up;  PHASE 2: a0 only
#pragma unroll
        for (int j = 0; j < NC; ++j) { a0[j] = 0.0f; a1[j] = 0.0f; }
        bool ok = true;
        for (int kb = 0; kb < p.KB; ++kb, ++step) {
            const uint32_t acc = step % ACC_BUFS, acc_phase = (step / ACC_BUFS) & 1u;
            const uint32_t slot = step % SF_SLOTS, sphase = (step / SF_SLOTS) & 1u;
            const long long c0 = B200_TRACE(p.trace) ? clock64() : 0;
            ok = mbar_wait_warp(tfull_bar + 8 * acc, acc_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
            if (B200_TRACE(p.trace)) tr_tf += clock64() - c0;
            if (!ok) return false;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t(ew * 32) << 16) + acc * ACC_STRIDE;
            uint32_t v0[NC], v1[NC];
            TmemCols<NC>::load(taddr, v0);
            if (PHASE == 1) TmemCols<NC>::load(taddr + NT, v1);
            const long long c1 = B200_TRACE(p.trace) ? clock64() : 0;
            ok = mbar_wait_warp(sffull_bar + 8 * slot, sphase, abort_flag, status, STATUS_TIMEOUT_SF_FULL);
            if (B200_TRACE(p.trace)) tr_sf += clock64() - c1;
            if (!ok) {                          // unwinding: the loads above must land before TMEM is freed
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                return false;
            }
            const float* sfp = sf_ring + slot * SF_SLOT_FLOATS;
            const float sb0 = sfp[NT], sb1 = sfp[NT + 1];
            tmem_ld_wait(v0);
            if (PHASE == 1) tmem_ld_wait(v1);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const float sr = sfp[j];
                a0[j] = fmaf(__uint_as_float(v0[j]), __fmul_rn(sr, sb0), a0[j]);
                if (PHASE == 1) a1[j] = fmaf(__uint_as_float(v1[j]), __fmul_rn(sr, sb1), a1[j]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sfempty_bar + 8 * slot);
        }
        if (PHASE == 1) {
            float* amax_w = amax_s + (unit_parity * 4 + ew) * NT;
            float* grow = p.g1 + (long long)u.row0 * 256 + feat;
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                if (j < u.n_valid) {            // warp-uniform
                    grow[j * 256] = a0[j];
                    grow[j * 256 + 128] = a1[j];
                    const float act = __fmul_rn(silu_f32(a0[j]), a1[j]);
                    a0[j] = act;
                    const float m = warp_max(fabsf(act));
                    if (lane == j) amax_w[j] = m;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(amax_bar);   // rendezvous of the four epilogue warps, bounded like every wait
            ok = mbar_wait_warp(amax_bar, unit_parity, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
            if (!ok) return false;
            const float* amax_r = amax_s + unit_parity * 4 * NT;
            uint8_t* qrow = p.a2 + (long long)u.row0 * 128 + feat;
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                if (j < u.n_valid) {
                    const float amax = fmaxf(fmaxf(amax_r[j], amax_r[NT + j]), fmaxf(amax_r[2 * NT + j], amax_r[3 * NT + j]));
                    const float sc = __fdiv_rn(fmaxf(amax, 1.0e-8f), 448.0f);
                    const float q = clamp448(__fdiv_rn(a0[j], sc));
                    qrow[j * 128] = (uint8_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3);
                    if (feat == 0) p.s2[u.row0 + j] = sc;
                }
            }
            unit_parity ^= 1;       // the other half of amax_s: the next unit's writes cannot race these reads
        } else {
            float* drow = p.d2 + (long long)u.row0 * p.H + u.f * 128 + feat;
#pragma unroll
            for (int j = 0; j < NC; ++j)
                if (j < u.n_valid) drow[(long long)j * p.H] = a0[j];
        }
        return true;
    }
};

template <int PHASE>
__global__ void __launch_bounds__(asw::Cfg<PHASE>::THREADS, 1)
alpha_swap_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                  const AlphaGemmParams p, int* status) {
    using namespace asw;
    using C = Cfg<PHASE>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BARS);
    // bars: full[STAGES], empty[STAGES], tfull[ACC_BUFS], tempty[ACC_BUFS], sffull[SF_SLOTS], sfempty[SF_SLOTS], amax
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC_BUFS + 2 * SF_SLOTS + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    float* sf_ring = reinterpret_cast<float*>(smem + C::OFF_SF);
    float* amax_s = reinterpret_cast<float*>(smem + C::OFF_AMAX);       // [2 parity][4 warps][NT]
    int* tables = reinterpret_cast<int*>(smem + C::OFF_TABLES);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);       // a value the compiler knows to be warp-uniform
    const int lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_u32(bars);
    const uint32_t empty_bar = smem_u32(bars + STAGES);
    const uint32_t tfull_bar = smem_u32(bars + 2 * STAGES);
    const uint32_t tempty_bar = smem_u32(bars + 2 * STAGES + ACC_BUFS);
    const uint32_t sffull_bar = smem_u32(bars + 2 * STAGES + 2 * ACC_BUFS);
    const uint32_t sfempty_bar = smem_u32(bars + 2 * STAGES + 2 * ACC_BUFS + SF_SLOTS);
    const uint32_t amax_bar = smem_u32(bars + 2 * STAGES + 2 * ACC_BUFS + 2 * SF_SLOTS);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int s = 0; s < ACC_BUFS; ++s) {
            mbar_init(tfull_bar + 8 * s, 1);
            mbar_init(tempty_bar + 8 * s, 4);      // one arrival per epilogue warp
        }
        for (int s = 0; s < SF_SLOTS; ++s) {
            mbar_init(sffull_bar + 8 * s, 32);     // one deferred arrival per lane of the loader warp
            mbar_init(sfempty_bar + 8 * s, 4);
        }
        mbar_init(amax_bar, 4);                    // the four epilogue warps, once per unit
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
    }
    pdl_launch_dependents();
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), TMEM_COLS);
        tmem_relinquish();
    }
    // everything above overlaps the previous kernel of the stream; its outputs (counts, operands) are read below
    pdl_wait();
    alpha_build_units(p, tables);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const int KB = p.KB;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        AlphaSched sched(tables, p.NF, p.max_m);
        AlphaUnit u;
        uint32_t stage = 0, phase = 0, issued = 0, issued_parity = 0;
        long long tr_wait = 0;
        const long long tr_t0 = B200_TRACE(p.trace) ? clock64() : 0;
        bool ok = true;
        while (ok && sched.next(u)) {
            const int w_row = PHASE == 1 ? u.e * 256 : u.e * p.H + u.f * 128;
            for (int kb = 0; kb < KB; ++kb) {
                const long long c0 = B200_TRACE(p.trace) ? clock64() : 0;
                ok = mbar_wait_warp(empty_bar + 8 * stage, phase ^ 1, abort_flag, status, STATUS_TIMEOUT_SMEM_EMPTY);
                if (B200_TRACE(p.trace)) tr_wait += clock64() - c0;
                if (!ok) break;
                if (elect_one_sync()) {
                    const uint32_t fb = full_bar + 8 * stage;
                    const uint32_t base = smem_u32(smem + stage * C::STAGE_BYTES);
                    mbar_arrive_expect_tx(fb, C::STAGE_BYTES);
                    tma_load_2d(base, &tmap_w, fb, kb * BK, w_row);
                    if (PHASE == 1) tma_load_2d(base + W_TILE_BYTES, &tmap_w, fb, kb * BK, w_row + 128);
                    tma_load_2d(base + C::W_TILES * W_TILE_BYTES, &tmap_x, fb, kb * BK, u.row0);
                }
                issued |= 1u << stage;
                issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (B200_TRACE(p.trace) && lane == 0) {
            p.trace[blockIdx.x * 8 + 0] = tr_wait;
            p.trace[blockIdx.x * 8 + 1] = clock64() - tr_t0;
        }
        // after a failed wait, give every copy this warp issued a bounded chance to land before the CTA exits
        if (!ok && lane == 0) {
            for (int s = 0; s < STAGES; ++s) {
                if (!((issued >> s) & 1u)) continue;
                const uint32_t par = (issued_parity >> s) & 1u;
                for (int it = 0; it < (1 << 20); ++it)
                    if (mbar_try_wait(full_bar + 8 * s, par)) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer: warp-uniform loop, one elected lane issues
        AlphaSched sched(tables, p.NF, p.max_m);
        AlphaUnit u;
        constexpr uint32_t idesc = make_idesc_e4m3_f32(128, NT);
        uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
        long long tr_te = 0, tr_full = 0, tr_issue = 0;
        bool ok = true;
        while (ok && sched.next(u)) {
            for (int kb = 0; kb < KB; ++kb) {
                const long long c0 = B200_TRACE(p.trace) ? clock64() : 0;
                ok = mbar_wait_warp(tempty_bar + 8 * acc, acc_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                const long long c1 = B200_TRACE(p.trace) ? clock64() : 0;
                ok = mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, status, STATUS_TIMEOUT_SMEM_FULL);
                if (!ok) break;
                const long long c2 = B200_TRACE(p.trace) ? clock64() : 0;
                tr_te += c1 - c0;
                tr_full += c2 - c1;
                tc_fence_after();
                if (elect_one_sync()) {
                    const uint32_t base = smem_u32(smem + stage * C::STAGE_BYTES);
                    const uint64_t wdesc = make_smem_desc_sw128(base);
                    const uint64_t xdesc = make_smem_desc_sw128(base + C::W_TILES * W_TILE_BYTES);
                    const uint32_t tmem_d = tmem_base + acc * ACC_STRIDE;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k) umma_f8f6f4(tmem_d, wdesc + 2 * k, xdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
                    if (PHASE == 1) {
                        const uint64_t wdesc2 = make_smem_desc_sw128(base + W_TILE_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k)
                            umma_f8f6f4(tmem_d + NT, wdesc2 + 2 * k, xdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar + 8 * stage);
                    umma_commit(tfull_bar + 8 * acc);
                }
                if (B200_TRACE(p.trace)) tr_issue += clock64() - c2;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
                if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1; }
            }
        }
        if (B200_TRACE(p.trace) && lane == 0) {
            p.trace[blockIdx.x * 8 + 2] = tr_te;
            p.trace[blockIdx.x * 8 + 3] = tr_full;
            p.trace[blockIdx.x * 8 + 4] = tr_issue;
        }
    } else if (warp == 2) {
        // ------------------------------------------------ scale loader: slot = 32 row scales + 2 block scales
        AlphaSched sched(tables, p.NF, p.max_m);
        AlphaUnit u;
        uint32_t slot = 0, sphase = 0;
        bool ok = true;
        while (ok && sched.next(u)) {
            long long r = (long long)u.row0 + lane;
            if (r >= p.rows_total) r = p.rows_total - 1;
            const float* rp = p.s_rows + r;
            const float* bp = PHASE == 1 ? p.sfb + ((long long)u.e * 2 + (lane & 1)) * KB
                                         : p.sfb + ((long long)u.e * p.NF + u.f);
            for (int kb = 0; kb < KB; ++kb) {
                ok = mbar_wait_warp(sfempty_bar + 8 * slot, sphase ^ 1, abort_flag, status, STATUS_TIMEOUT_SF_EMPTY);
                if (!ok) break;
                const uint32_t dst = smem_u32(sf_ring + slot * SF_SLOT_FLOATS);
                cp_async_4(dst + lane * 4, rp + (long long)kb * p.rows_total);
                if (lane < 2) cp_async_4(dst + (NT + lane) * 4, bp + kb);
                cp_async_mbar_arrive_noinc(sffull_bar + 8 * slot);
                if (++slot == SF_SLOTS) { slot = 0; sphase ^= 1; }
            }
        }
        cp_async_wait_all();
    } else if (warp >= 4) {
        // ------------------------------------------------ epilogue: thread = feature (TMEM lane), register = row
        AlphaEpilogue<PHASE> epi{p, tmem_base, tfull_bar, tempty_bar, sffull_bar, sfempty_bar, amax_bar, sf_ring, amax_s,
                                 abort_flag, status, warp & 3, lane};
        const int team = (warp - 4) >> 2;
        AlphaSched sched(tables, p.NF, p.max_m);
        AlphaUnit u;
        const long long tr_e0 = B200_TRACE(p.trace) ? clock64() : 0;
        bool ok = true;
        for (int i = 0; ok && sched.next(u); ++i) {
            if (C::TEAMS > 1 && (i % C::TEAMS) != team) {
                epi.skip_unit();
                continue;
            }
            // most decode units hold a handful of rows: drain and promote 16 accumulator columns instead of 32
            ok = u.n_valid <= 16 ? epi.template unit<16>(u) : epi.template unit<32>(u);
        }
        if (B200_TRACE(p.trace) && warp == 4 && lane == 0) {
            p.trace[blockIdx.x * 8 + 5] = epi.tr_tf;
            p.trace[blockIdx.x * 8 + 6] = epi.tr_sf;
            p.trace[blockIdx.x * 8 + 7] = clock64() - tr_e0;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace b200
