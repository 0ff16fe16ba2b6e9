// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM
// allocation, MMA, commit, load) and the bounded-wait helper every spin in this library uses.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ------------------------------------------------------------------ device status word
// One word per device (file-scope __device__ storage, no allocation).  Kernels OR an error code
// into it when a bounded wait runs out; the host reads and clears it.
enum : int {
    STATUS_TIMEOUT_SMEM_FULL = 1 << 0,    // MMA warp: TMA data never arrived
    STATUS_TIMEOUT_SMEM_EMPTY = 1 << 1,   // producer: stage never released
    STATUS_TIMEOUT_TMEM_FULL = 1 << 2,    // epilogue: accumulator never completed
    STATUS_TIMEOUT_TMEM_EMPTY = 1 << 3,   // MMA warp: accumulator never drained
    STATUS_TIMEOUT_PEER_FLAG = 1 << 4,    // exchange kernels: a peer flag never arrived
    STATUS_TIMEOUT_SF_FULL = 1 << 5,      // epilogue: block scales never arrived in shared memory
    STATUS_TIMEOUT_SF_EMPTY = 1 << 6,     // scale loader: ring slot never released
    STATUS_BAD_ARGUMENT = 1 << 8,
    STATUS_CAPACITY = 1 << 9,             // exchange: more rows were routed to a rank than its receive buffer holds
};

// Per-role wait-cycle counters (the `trace` pointers of the kernel parameter blocks) are compiled in only by a
// developer build with -DB200MOE_DEV_TRACE; the library as shipped never reads or writes through them.
#ifdef B200MOE_DEV_TRACE
#define B200_TRACE(ptr) ((ptr) != nullptr)
#else
#define B200_TRACE(ptr) false
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// One lane of the (converged) warp: the lane that issues TMA and tcgen05 instructions on the warp's behalf.  The code
// around it stays warp-uniform, so its operands live in uniform registers.
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// Bounded wait.  Every lane of the calling warp polls; the wait gives up after `limit_ns` of
// wall time (checked every 1024 failed polls) or as soon as another role of the CTA has raised
// the shared abort flag.  On expiry it raises the abort flag and ORs `code` into the device
// status word.  Returns true iff ALL lanes saw the phase complete (warp-uniform result).
constexpr uint64_t kWaitLimitNs = 2000ull * 1000ull * 1000ull;   // 2 s

__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int code) {
    bool ok = mbar_try_wait(bar, parity);
    if (!ok) {
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (true) {
            ok = mbar_try_wait(bar, parity);
            if (ok) break;
            if ((++spins & 1023u) == 0) {
                if (*abort_flag) break;
                uint64_t now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > kWaitLimitNs) {
                    *abort_flag = 1;
                    atomicOr(status, code);
                    break;
                }
            }
        }
    }
    return __all_sync(0xffffffffu, ok);
}

// one 32-byte sector per thread (256-bit store); the address must be 32-byte aligned
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&o)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
}

// d[0..3] += v, performed by the L2 (no read back into the SM); 16-byte aligned
__device__ __forceinline__ void red_add_f32x4(float* d, float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// ---- cp.async (LDGSTS): 4-byte global -> shared copies whose completion arrives on an mbarrier
__device__ __forceinline__ void cp_async_4(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
// one arrival on `bar` once all earlier cp.async of this thread have landed (the barrier's count must include it)
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may
// start while its predecessor in the stream is still running; it must call pdl_wait() before it touches anything the
// predecessor writes or reads.  pdl_launch_dependents() lets the successor's CTAs be scheduled from now on.
// Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Single-thread form of the bounded wait (no warp vote): used by the one thread that issues MMAs, where
// every instruction between "operands ready" and "MMA issued" is on the critical path.
__device__ __forceinline__ bool mbar_wait_thread(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                 int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 1023u) == 0) {
            if (*abort_flag) return false;
            uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(status, code);
                return false;
            }
        }
    }
}

// ------------------------------------------------------------------ TMA
// 2-D tiled load global -> shared, completion on an mbarrier (no multicast).
// c0 = innermost coordinate (elements), c1 = row.  c0 * element size must be a multiple of 16 B.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tmap, uint32_t bar,
                                            int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ------------------------------------------------------------------ tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_result_addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, e4m3 x e4m3 -> fp32, one elected thread issues.
__device__ __forceinline__ void umma_f8f6f4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier once all tcgen05 operations issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes, written by TMA with
// SWIZZLE_128B: 8-row groups are 1024 B apart (stride-dimension byte offset), version 1,
// layout type 2 (128-byte swizzle).  `saddr` must be 1024-byte aligned plus a multiple of 32 B
// inside the first row (the K step of one fp8 MMA).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);          // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                          // leading-dim offset (unused here)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                  // stride-dim offset: 8 rows * 128 B
    d |= static_cast<uint64_t>(1) << 46;                          // descriptor version (sm_100)
    d |= static_cast<uint64_t>(2) << 61;                          // SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f8f6f4, A = B = e4m3, D = fp32, both operands K-major, dense.
__host__ __device__ constexpr uint32_t make_idesc_e4m3_f32(int m, int n) {
    return (1u << 4)                                   // D format: fp32
           | (0u << 7) | (0u << 10)                    // A, B format: e4m3
           | (static_cast<uint32_t>(n >> 3) << 17)     // N / 8
           | (static_cast<uint32_t>(m >> 4) << 24);    // M / 16
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp reads TMEM lane (base lane + t),
// register i = column (base column + i).  No wait is issued here.
#define B200_R32(v)                                                                               \
    "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),          \
    "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),      \
    "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),   \
    "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),   \
    "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
#define B200_RW32(v)                                                                              \
    "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),          \
    "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]),      \
    "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]),   \
    "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]),   \
    "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : B200_R32(v)
        : "r"(taddr)
        : "memory");
}
// Waits for all of this thread's outstanding tcgen05.ld; the registers are listed as read-write
// operands so that no use of them can be scheduled above the wait.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : B200_RW32(v)::"memory");
}

// 16-column variants (half the registers in flight)
#define B200_R16(v)                                                                               \
    "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),          \
    "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),      \
    "=r"(v[14]), "=r"(v[15])
#define B200_RW16(v)                                                                              \
    "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]),          \
    "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]),      \
    "+r"(v[14]), "+r"(v[15])
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : B200_R16(v)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : B200_RW16(v)::"memory");
}

// ------------------------------------------------------------------ packed fp32 pairs
// sm_100 executes two fp32 FMAs per lane per instruction on 64-bit register pairs.
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// acc = {v0, v1} * s2 + acc, each half rounded to nearest even like fmaf
__device__ __forceinline__ void fma_f32x2(unsigned long long& acc, uint32_t v0, uint32_t v1,
                                          unsigned long long s2) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(v0), "r"(v1));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(v), "l"(s2));
}

// {lo, hi} fp32 pair -> packed bf16x2 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t cvt_bf16x2(unsigned long long v) {
    float lo, hi;
    unpack_f32x2(v, lo, hi);
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ------------------------------------------------------------------ register budget
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

}  // namespace b200
