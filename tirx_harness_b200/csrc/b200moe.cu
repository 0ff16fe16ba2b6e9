// Host side of the C ABI declared in include/b200moe.h: argument validation, TMA descriptor
// encoding, kernel launches and error reporting.  No torch types, no allocation on the GEMM path.
#include "b200moe.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>

#include "gg_fp8.cuh"
#include "pair_common.cuh"
#include "gg_fp8_mx.cuh"
#include "moe_ops.cuh"
#include "alpha_moe.cuh"
#include "alpha_gemm.cuh"
#include "alpha_gemv.cuh"

namespace {

using namespace b200;

// Device status word: kernels OR a code into it when a bounded wait runs out.
__device__ int g_status_word = 0;

// Process-wide modes (moe_set_option).  Plain atomics: a call reads each option once.
std::atomic<int> g_options[MOE_OPT_COUNT_] = {
    /* MOE_OPT_GG_BLOCK_SCALED */ {1},
    /* MOE_OPT_MX_TILE */ {MOE_MX_TILE_AUTO},
    /* MOE_OPT_ALPHA_PATH */ {MOE_ALPHA_PATH_AUTO},
    /* MOE_OPT_ALPHA_GEMV_MAX_ROUTES */ {160},
    /* MOE_OPT_KG_MODE */ {MOE_KG_MODE_MN_MAJOR},
    /* MOE_OPT_EP_WAIT_LIMIT_MS */ {2000},
};
inline int opt(int which) { return g_options[which].load(std::memory_order_relaxed); }

// Generation number of a call that takes the block-scaled path: the scale check marks "not all powers of two" by
// storing this number into the workspace flag, so nothing has to be cleared between calls.
std::atomic<unsigned> g_call_gen{1};
inline int next_gen() {
    unsigned g = g_call_gen.fetch_add(1, std::memory_order_relaxed);
    return (int)(g == 0 ? g_call_gen.fetch_add(1, std::memory_order_relaxed) : g);
}

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define CUDA_TRY(expr)                                                                       \
    do {                                                                                     \
        cudaError_t e_ = (expr);                                                             \
        if (e_ != cudaSuccess)                                                               \
            return fail(MOE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                                 \
    } while (0)

// cuTensorMapEncodeTiled is fetched through the runtime so that the library carries no link-time
// dependency on libcuda (it must load on machines without a driver, e.g. for symbol checks).
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    });
    return fn;
}

// 2-D K-major e4m3 matrix [rows, K]; box = box_rows x 128 bytes, SWIZZLE_128B, OOB reads give 0.
int encode_fp8_kmajor(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows,
                      uint64_t pitch = 0) {
    auto fn = get_encode_fn();
    if (!fn) return fail(MOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {pitch ? pitch : K};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return MOE_OK;
}

// 1-D array of 32-bit words, box = 128 words (one 512-byte scale tile)
int encode_words_1d(CUtensorMap* map, const void* base, uint64_t n_words) {
    auto fn = get_encode_fn();
    if (!fn) return fail(MOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[1] = {n_words};
    cuuint64_t strides[1] = {0};
    cuuint32_t box[1] = {128};
    cuuint32_t estr[1] = {1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 1, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MOE_ERR_CUDA, "cuTensorMapEncodeTiled (1-D) failed with CUresult %d", (int)r);
    return MOE_OK;
}

struct MxLayout {
    size_t flag_off, sfa_off, sfb_off, bytes;
    int row_blocks, quads;
};
// SFB tiles are packed per column tile of the kernel that will run (240 or 256 columns wide, two 512-byte halves
// each); the size covers the narrower tile, i.e. the larger count.
MxLayout mx_layout(int G, long long rows_total, int N, int K) {
    MxLayout l;
    l.row_blocks = (int)((rows_total + 127) / 128);
    l.quads = (K / 128 + 3) / 4;
    const int n_tiles = (N + 223) / 224;          // the narrowest tile any variant of the pair kernel uses
    l.flag_off = 0;
    l.sfa_off = 256;
    l.sfb_off = l.sfa_off + (size_t)l.row_blocks * l.quads * 512;
    l.bytes = l.sfb_off + (size_t)G * n_tiles * l.quads * 1024;
    return l;
}

struct DeviceInfo {
    int num_sms = 0;
    int max_pairs = 0;       // CTA pairs (clusters of 2) of the pair kernel that can be resident at once
    int* status = nullptr;   // device address of g_status_word on this device
    bool attr_set = false;
};

int device_info(DeviceInfo** out) {
    static DeviceInfo infos[64];
    static std::mutex mu;
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MOE_ERR_INVALID, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo& di = infos[dev];
    if (!di.attr_set) {
        cudaDeviceProp prop;
        CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10)
            return fail(MOE_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library needs sm_100a (B200)", dev,
                        prop.major, prop.minor);
        di.num_sms = prop.multiProcessorCount;
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      gg::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      gg::SMEM_BYTES_MASKED));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      gg::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      gg::SMEM_BYTES_SCATTER));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_kernel<false, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      gg::SMEM_BYTES_DISPATCH));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_kernel<false, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      gg::SMEM_BYTES_DISPATCH));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_mx_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_mx_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute((gg_fp8_mx_kernel<false, false, false, 240>), cudaFuncAttributeMaxDynamicSharedMemorySize, mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute((gg_fp8_mx_kernel<true, false, false, 240>), cudaFuncAttributeMaxDynamicSharedMemorySize, mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute((gg_fp8_mx_kernel<false, false, false, 224>), cudaFuncAttributeMaxDynamicSharedMemorySize, mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute((gg_fp8_mx_kernel<true, false, false, 224>), cudaFuncAttributeMaxDynamicSharedMemorySize, mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_mx_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_mx_kernel<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      mx::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_mx1_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      mx1::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(gg_fp8_mx1_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      mx1::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(ep_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, EP_DISPATCH_MAX_SMEM));
        CUDA_TRY(cudaFuncSetAttribute(alpha_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * asw::MAX_E * 4));
        CUDA_TRY(cudaFuncSetAttribute(alpha_swap_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, asw::Cfg<1>::SMEM_BYTES));
        CUDA_TRY(cudaFuncSetAttribute(alpha_swap_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, asw::Cfg<2>::SMEM_BYTES));
        {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * di.num_sms, 1, 1);
            cfg.blockDim = dim3(mx::THREADS, 1, 1);
            cfg.dynamicSmemBytes = mx::SMEM_BYTES;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gg_fp8_mx_kernel<false>, &cfg) != cudaSuccess || n <= 0) {
                (void)cudaGetLastError();
                n = di.num_sms / 2;
            }
            di.max_pairs = n < di.num_sms / 2 ? n : di.num_sms / 2;
        }
        int* sp = nullptr;
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&sp), g_status_word));
        if (sp == nullptr) return fail(MOE_ERR_CUDA, "cudaGetSymbolAddress returned NULL for the status word");
        di.status = sp;
        di.attr_set = true;
    }
    *out = &di;
    return MOE_OK;
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor in the stream
// still runs and orders itself with pdl_wait() (ptx.cuh).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <bool MASKED>
int launch_gg(const moe_gg_args* a, void* stream) {
    if (!a) return fail(MOE_ERR_INVALID, "args is NULL");
    if (a->M == 0 && a->G > 0 && a->N > 0 && a->K > 0) return MOE_OK;      // nothing to compute
    const bool packed_sf = a->sf_format == MOE_SF_UE8M0_PACKED;
    if (a->sf_format != MOE_SF_F32 && !packed_sf) return fail(MOE_ERR_INVALID, "sf_format must be MOE_SF_F32 or MOE_SF_UE8M0_PACKED");
    if (packed_sf) {
        if (!a->workspace) return fail(MOE_ERR_INVALID, "packed UE8M0 scales need workspace (moe_gg_workspace_bytes)");
        if (MASKED && a->M % 128 != 0) return fail(MOE_ERR_UNSUPPORTED, "packed UE8M0 scales with the masked layout need max_m %% 128 == 0");
        if (a->scatter_meta) return fail(MOE_ERR_UNSUPPORTED, "packed UE8M0 scales cannot be combined with scattered output");
    }
    if (!a->a || !a->b || !a->sfa || !a->sfb || !a->layout || (!a->d && !a->scatter_meta))
        return fail(MOE_ERR_INVALID, "a, b, sfa, sfb, layout and d must all be non-NULL");
    if (a->G <= 0 || a->N <= 0 || a->K <= 0 || a->M < 0)
        return fail(MOE_ERR_INVALID, "G, N, K must be positive and M non-negative (G=%d M=%d N=%d K=%d)", a->G,
                    a->M, a->N, a->K);
    if (a->K % 128 != 0) return fail(MOE_ERR_INVALID, "K=%d must be a multiple of 128", a->K);
    if (a->N % 8 != 0) return fail(MOE_ERR_INVALID, "N=%d must be a multiple of 8", a->N);
    if (a->d_dtype != MOE_DTYPE_BF16 && a->d_dtype != MOE_DTYPE_F32)
        return fail(MOE_ERR_INVALID, "d_dtype must be MOE_DTYPE_BF16 or MOE_DTYPE_F32");
    if (a->ldd < a->N || a->ldd % 8 != 0) return fail(MOE_ERR_INVALID, "ldd=%lld must be >= N and a multiple of 8", (long long)a->ldd);
    if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15) ||
        (reinterpret_cast<uintptr_t>(a->d) & 15))
        return fail(MOE_ERR_INVALID, "a, b and d must be 16-byte aligned");
    if (MASKED && a->G > gg::MAX_MASKED_GROUPS)
        return fail(MOE_ERR_INVALID, "masked layout supports at most %d groups", gg::MAX_MASKED_GROUPS);
    const long long rows_total = MASKED ? (long long)a->G * a->M : (long long)a->M;
    if (rows_total > 0x7FFFFFFFll || (long long)a->G * a->N > 0x7FFFFFFFll)
        return fail(MOE_ERR_INVALID, "row counts exceed 2^31-1");
    if (rows_total == 0) return MOE_OK;

    DeviceInfo* di = nullptr;
    int rc = device_info(&di);
    if (rc != MOE_OK) return rc;

    const bool allow_mx = opt(MOE_OPT_GG_BLOCK_SCALED) != 0;
    CUtensorMap tmap_a, tmap_b;
    if (a->lda != 0 && (a->lda < a->K || a->lda % 16)) return fail(MOE_ERR_INVALID, "lda must be 0 or >= K and a multiple of 16");
    if (a->ldb != 0 && (a->ldb < a->K || a->ldb % 16)) return fail(MOE_ERR_INVALID, "ldb must be 0 or >= K and a multiple of 16");
    if (a->accumulate && (a->d_dtype != MOE_DTYPE_F32 || a->scatter_meta || !packed_sf))
        return fail(MOE_ERR_UNSUPPORTED, "accumulate needs fp32 output, packed UE8M0 scales and no scattered output");
    rc = encode_fp8_kmajor(&tmap_a, a->a, (uint64_t)rows_total, (uint64_t)a->K, gg::BM, (uint64_t)a->lda);
    if (rc != MOE_OK) return rc;
    rc = encode_fp8_kmajor(&tmap_b, a->b, (uint64_t)a->G * a->N, (uint64_t)a->K, gg::BN, (uint64_t)a->ldb);
    if (rc != MOE_OK) return rc;

    GGParams p;
    p.sfa = a->sfa;
    p.sfa_sr = a->sfa_stride_row;
    p.sfa_sk = a->sfa_stride_kblk;
    p.sfb = a->sfb;
    p.layout = a->layout;
    p.rows_used = MASKED ? nullptr : a->rows_used;
    p.mode_flag = nullptr;
    p.mode_gen = 0;
    p.act_q = nullptr; p.act_s = nullptr; p.act_ss_r = 0; p.act_ss_b = 0; p.inter = 0; p.gate_first = 0;
    p.scatter_meta = MASKED ? nullptr : a->scatter_meta;
    p.scatter_meta_stride = a->scatter_meta_stride > 0 ? a->scatter_meta_stride : 1;
    for (int i = 0; i < 8; ++i) p.scatter_base[i] = static_cast<__nv_bfloat16*>(a->scatter_base[i]);
    if (p.scatter_meta != nullptr && a->d_dtype != MOE_DTYPE_BF16)
        return fail(MOE_ERR_INVALID, "scattered output is bf16 only");
    p.d = a->d;
    p.ldd = a->ldd;
    p.d_f32 = a->d_dtype == MOE_DTYPE_F32;
    p.d_accumulate = a->accumulate ? 1 : 0;
    p.trace = nullptr;
#ifdef B200MOE_DEV_TRACE
    // developer build only: device address of an int64 [grid][8] array of per-role wait-cycle counters
    if (const char* e = getenv("B200MOE_GG_TRACE")) p.trace = reinterpret_cast<long long*>(strtoull(e, nullptr, 10));
#endif
    p.G = a->G; p.M = a->M; p.N = a->N; p.K = a->K;
    p.rows_total = (int)rows_total;
    p.num_n_blocks = (a->N + gg::BN - 1) / gg::BN;
    p.num_k_blocks = a->K / 128;
    p.nb128 = (a->N + 127) / 128;
    p.num_m_blocks = (a->M + gg::BM - 1) / gg::BM;

    // ---- power-of-two-scale path: needs caller workspace; stands down on the device if a scale is not 2^e
    if ((allow_mx || packed_sf) && a->workspace != nullptr && (!MASKED || a->M % 128 == 0) && p.scatter_meta == nullptr) {
        const MxLayout ml = mx_layout(a->G, rows_total, a->N, a->K);
        if (a->workspace_bytes < ml.bytes)
            return fail(MOE_ERR_INVALID, "workspace too small: %llu < %zu bytes (moe_gg_workspace_bytes)",
                        (unsigned long long)a->workspace_bytes, ml.bytes);
        if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return fail(MOE_ERR_INVALID, "workspace must be 256-byte aligned");
        char* wsb = static_cast<char*>(a->workspace);
        MxWorkspace ws;
        ws.flag = reinterpret_cast<int*>(wsb + ml.flag_off);
        ws.sfa_packed = reinterpret_cast<uint32_t*>(wsb + ml.sfa_off);
        ws.sfb_packed = reinterpret_cast<uint32_t*>(wsb + ml.sfb_off);
        ws.row_blocks = ml.row_blocks;
        ws.quads = ml.quads;
        // measured: CTA pairs win on full 256-row blocks (contiguous layout), single CTAs on the masked
        // layout, where a pair multiplies up to 255 empty rows per group; among the pair tiles 240 columns with two
        // accumulators (the drain of tile i under the MMAs of tile i+1) beat 256 columns with one on every shape
        // measured against the same comparator, by 4 to 25 %, most on short K
        int mx_tile = a->mx_tile != 0 ? a->mx_tile : opt(MOE_OPT_MX_TILE);     // per call, else process-wide
        if (mx_tile < MOE_MX_TILE_AUTO || mx_tile > MOE_MX_TILE_PAIR_224) return fail(MOE_ERR_INVALID, "mx_tile out of range");
        if (mx_tile == MOE_MX_TILE_AUTO) mx_tile = MASKED ? MOE_MX_TILE_SINGLE : MOE_MX_TILE_PAIR_240;
        const bool mx_single = mx_tile == MOE_MX_TILE_SINGLE;
        // column tiles: 256 wide for the single-CTA kernel; for the pair kernel at most 240 wide and balanced in
        // units of 16 columns (all tiles 224 or 240 wide where N allows it: no narrow last tile)
        if (mx_single) {
            ws.n_tiles = (a->N + mx1::BN - 1) / mx1::BN;
            ws.nt_base = mx1::BN / 16; ws.nt_rem = 0;
        } else {
            const int tn = mx_tile == MOE_MX_TILE_PAIR_240 ? 240 : (mx_tile == MOE_MX_TILE_PAIR_224 ? 224 : mx::BN);
            const int units = (a->N + 15) / 16;
            ws.n_tiles = (a->N + tn - 1) / tn;
            ws.nt_base = units / ws.n_tiles; ws.nt_rem = units % ws.n_tiles;
        }
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        ws.gen = p.mode_gen = next_gen();
        dim3 pgrid(ml.row_blocks + a->G * ws.n_tiles * 2, ml.quads, 1);
        if (packed_sf)
            mx_prep_packed_kernel<<<pgrid, 128, 0, st>>>(
                reinterpret_cast<const uint32_t*>(a->sfa), a->sfa_stride_row, a->sfa_stride_kblk,
                reinterpret_cast<const uint32_t*>(a->sfb), a->sfb_stride[0], a->sfb_stride[1], a->sfb_stride[2],
                (int)rows_total, a->N, a->G, ws);
        else
            mx_prep_kernel<<<pgrid, 128, 0, st>>>(a->sfa, a->sfa_stride_row, a->sfa_stride_kblk, a->sfb, (int)rows_total,
                                                  p.num_k_blocks, a->G, p.nb128, ws, a->layout, MASKED ? a->M : 0,
                                                  p.rows_used);
        CUDA_TRY(cudaGetLastError());
        CUtensorMap tmap_b2, tmap_sfa, tmap_sfb;
        const int pair_tn = mx_tile == MOE_MX_TILE_PAIR_240 ? 240 : (mx_tile == MOE_MX_TILE_PAIR_224 ? 224 : mx::BN);
        rc = encode_fp8_kmajor(&tmap_b2, a->b, (uint64_t)a->G * a->N, (uint64_t)a->K, mx_single ? mx1::BN : pair_tn / 2,
                               (uint64_t)a->ldb);
        if (rc != MOE_OK) return rc;
        rc = encode_words_1d(&tmap_sfa, ws.sfa_packed, (uint64_t)ml.row_blocks * ml.quads * 128);
        if (rc != MOE_OK) return rc;
        rc = encode_words_1d(&tmap_sfb, ws.sfb_packed, (uint64_t)a->G * ws.n_tiles * ml.quads * 256);
        if (rc != MOE_OK) return rc;
        GGParams pm = p;                 // the block-scaled kernels count column tiles of their own width
        pm.num_n_blocks = ws.n_tiles;
        pm.nt_base = ws.nt_base; pm.nt_rem = ws.nt_rem;
        if (mx_single) {
            const long long tiles1 = (MASKED ? (long long)a->G * p.num_m_blocks : (long long)p.num_m_blocks) * pm.num_n_blocks;
            int grid1 = (int)(tiles1 < di->num_sms ? tiles1 : di->num_sms);
            if (grid1 < 1) grid1 = 1;
            gg_fp8_mx1_kernel<MASKED><<<grid1, mx1::THREADS, mx1::SMEM_BYTES, st>>>(tmap_a, tmap_b2, tmap_sfa, tmap_sfb, pm,
                                                                                   ws.flag, ml.quads, di->status);
        } else {
            const long long row_blocks256 = MASKED ? (long long)a->G * ((a->M + 255) / 256) : (a->M + 255) / 256;
            const long long tiles = row_blocks256 * pm.num_n_blocks;
            int pairs = (int)(tiles < di->max_pairs ? tiles : di->max_pairs);
            if (pairs < 1) pairs = 1;
            if (mx_tile == MOE_MX_TILE_PAIR_240 && packed_sf) {
                // packed scales: nothing but the re-tiled scale words comes from the kernel just launched, and no flag
                pm.pdl_scales = 1;
                CUDA_TRY(launch_pdl(gg_fp8_mx_kernel<MASKED, false, false, 240>, dim3(2 * pairs), dim3(mx::THREADS),
                                    (size_t)mx::SMEM_BYTES, st, tmap_a, tmap_b2, tmap_sfa, tmap_sfb, pm,
                                    (const int*)nullptr, ml.quads, di->status, KgNone{}));
            } else if (mx_tile == MOE_MX_TILE_PAIR_240)
                gg_fp8_mx_kernel<MASKED, false, false, 240><<<2 * pairs, mx::THREADS, mx::SMEM_BYTES, st>>>(
                    tmap_a, tmap_b2, tmap_sfa, tmap_sfb, pm, ws.flag, ml.quads, di->status, KgNone{});
            else if (mx_tile == MOE_MX_TILE_PAIR_224)
                gg_fp8_mx_kernel<MASKED, false, false, 224><<<2 * pairs, mx::THREADS, mx::SMEM_BYTES, st>>>(
                    tmap_a, tmap_b2, tmap_sfa, tmap_sfb, pm, ws.flag, ml.quads, di->status, KgNone{});
            else
                gg_fp8_mx_kernel<MASKED><<<2 * pairs, mx::THREADS, mx::SMEM_BYTES, st>>>(tmap_a, tmap_b2, tmap_sfa, tmap_sfb, pm,
                                                                                       ws.flag, ml.quads, di->status, KgNone{});
        }
        CUDA_TRY(cudaGetLastError());
        p.mode_flag = ws.flag;           // the promotion kernel below runs only if the flag was raised
        if (packed_sf) return MOE_OK;    // UE8M0 bytes are powers of two by construction: nothing else to run
    }
    long long max_tiles = MASKED ? (long long)a->G * p.num_m_blocks * p.num_n_blocks
                                 : (long long)p.num_m_blocks * p.num_n_blocks;
    int grid = (int)(max_tiles < di->num_sms ? max_tiles : di->num_sms);
    if (grid < 1) grid = 1;
    if constexpr (!MASKED) {
        if (p.scatter_meta != nullptr) {
            if (a->N % gg::BN != 0) return fail(MOE_ERR_INVALID, "scattered output needs N %% 256 == 0 (rows leave as 512-byte pieces)");
            gg_fp8_kernel<false, false, true><<<grid, gg::THREADS, gg::SMEM_BYTES_SCATTER, static_cast<cudaStream_t>(stream)>>>(
                tmap_a, tmap_b, tmap_a, p, di->status);
            CUDA_TRY(cudaGetLastError());
            return MOE_OK;
        }
    }
    CUtensorMap tmap_a_small = tmap_a;
    if (MASKED) {
        rc = encode_fp8_kmajor(&tmap_a_small, a->a, (uint64_t)rows_total, (uint64_t)a->K, gg::SMALL_A_ROWS, (uint64_t)a->lda);
        if (rc != MOE_OK) return rc;
    }
    gg_fp8_kernel<MASKED><<<grid, gg::THREADS, MASKED ? gg::SMEM_BYTES_MASKED : gg::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
        tmap_a, tmap_b, tmap_a_small, p, di->status);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}


inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// Carves the layer workspace.  Every region is 256-byte aligned.
struct LayerWorkspace {
    int32_t *ids, *counts, *offsets, *pos, *src_pair, *layout, *chunk_counts;
    float *weights, *s1, *s2;
    uint8_t *a1, *a2;
    __nv_bfloat16 *g1, *y;
    int64_t cap_rows;
    size_t bytes;
};

int64_t layer_cap_rows(int64_t n_pairs, int32_t E, int32_t align) {
    return (n_pairs + align - 1) / align * align + (int64_t)E * align;
}

LayerWorkspace carve_layer(void* base, int64_t T, int32_t H, int32_t I, int32_t E, int32_t top_k, int32_t align) {
    LayerWorkspace w;
    const int64_t n_pairs = T * top_k;
    const int64_t cap = layer_cap_rows(n_pairs, E, align);
    const int64_t n_chunks = (n_pairs + PLAN_CHUNK - 1) / PLAN_CHUNK;
    size_t off = 0;
    char* b = static_cast<char*>(base);
    auto take = [&](size_t bytes) { char* p = b ? b + off : nullptr; off += align256(bytes); return p; };
    w.ids = reinterpret_cast<int32_t*>(take(n_pairs * 4));
    w.weights = reinterpret_cast<float*>(take(n_pairs * 4));
    w.counts = reinterpret_cast<int32_t*>(take((size_t)E * 4));
    w.offsets = reinterpret_cast<int32_t*>(take((size_t)(E + 1) * 4));
    w.pos = reinterpret_cast<int32_t*>(take(n_pairs * 4));
    w.src_pair = reinterpret_cast<int32_t*>(take(cap * 4));
    w.layout = reinterpret_cast<int32_t*>(take(cap * 4));
    w.chunk_counts = reinterpret_cast<int32_t*>(take((size_t)n_chunks * E * 4));
    w.a1 = reinterpret_cast<uint8_t*>(take((size_t)cap * H));
    w.s1 = reinterpret_cast<float*>(take((size_t)cap * (H / 128) * 4));
    w.g1 = reinterpret_cast<__nv_bfloat16*>(take((size_t)cap * 2 * I * 2));
    w.a2 = reinterpret_cast<uint8_t*>(take((size_t)cap * I));
    w.s2 = reinterpret_cast<float*>(take((size_t)cap * (I / 128) * 4));
    w.y = reinterpret_cast<__nv_bfloat16*>(take((size_t)cap * H * 2));
    w.cap_rows = cap;
    w.bytes = off;
    return w;
}

int check_plan_args(int64_t n_pairs, int32_t E_local, int32_t align, int64_t cap_rows) {
    if (n_pairs < 0 || n_pairs > 0x7FFFFFFFll) return fail(MOE_ERR_INVALID, "n_pairs out of range");
    if (E_local <= 0 || E_local > 256) return fail(MOE_ERR_INVALID, "E_local=%d must be in [1, 256]", E_local);
    if (align <= 0) return fail(MOE_ERR_INVALID, "align must be positive");
    if (cap_rows < 0 || cap_rows > 0x7FFFFFFFll) return fail(MOE_ERR_INVALID, "cap_rows out of range");
    return MOE_OK;
}


// gate_up grouped GEMM with the SiLU*mul + 1x128 FP8 requantisation done in its epilogue.
int launch_gg_fused_act(const moe_gg_args* a, void* act_q, float* act_scales, int64_t ss_row, int64_t ss_blk,
                        int32_t gate_first, void* stream) {
    if (!a) return fail(MOE_ERR_INVALID, "args is NULL");
    if (a->M == 0 && a->G > 0 && a->N > 0 && a->K > 0) return MOE_OK;
    if (!a->a || !a->b || !a->sfa || !a->sfb || !a->layout || !act_q || !act_scales)
        return fail(MOE_ERR_INVALID, "a, b, sfa, sfb, layout, act_q and act_scales must all be non-NULL");
    if (a->G <= 0 || a->N <= 0 || a->K <= 0 || a->M < 0) return fail(MOE_ERR_INVALID, "G, N, K must be positive, M non-negative");
    if (a->K % 128 != 0) return fail(MOE_ERR_INVALID, "K=%d must be a multiple of 128", a->K);
    if (a->N % 256 != 0) return fail(MOE_ERR_INVALID, "N=%d (= 2 x intermediate) must be a multiple of 256", a->N);
    if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15) ||
        (reinterpret_cast<uintptr_t>(act_q) & 15))
        return fail(MOE_ERR_INVALID, "a, b and act_q must be 16-byte aligned");
    if ((long long)a->G * a->N > 0x7FFFFFFFll) return fail(MOE_ERR_INVALID, "row counts exceed 2^31-1");
    DeviceInfo* di = nullptr;
    int rc = device_info(&di);
    if (rc != MOE_OK) return rc;
    CUtensorMap tmap_a, tmap_b;
    if (a->lda != 0 && (a->lda < a->K || a->lda % 16)) return fail(MOE_ERR_INVALID, "lda must be 0 or >= K and a multiple of 16");
    if (a->ldb != 0 || a->accumulate) return fail(MOE_ERR_UNSUPPORTED, "ldb and accumulate are not supported by the fused-activation GEMM");
    rc = encode_fp8_kmajor(&tmap_a, a->a, (uint64_t)a->M, (uint64_t)a->K, gg::BM, (uint64_t)a->lda);
    if (rc != MOE_OK) return rc;
    rc = encode_fp8_kmajor(&tmap_b, a->b, (uint64_t)a->G * a->N, (uint64_t)a->K, gg::FUSE_B_BOX_ROWS);
    if (rc != MOE_OK) return rc;
    GGParams p = {};
    p.sfa = a->sfa; p.sfa_sr = a->sfa_stride_row; p.sfa_sk = a->sfa_stride_kblk;
    p.sfb = a->sfb; p.layout = a->layout; p.rows_used = a->rows_used; p.mode_flag = nullptr;
    p.d = nullptr; p.ldd = 0; p.d_f32 = 0; p.d_accumulate = 0; p.trace = nullptr;
    p.G = a->G; p.M = a->M; p.N = a->N; p.K = a->K;
    p.rows_total = a->M;
    p.inter = a->N / 2;
    p.num_n_blocks = p.inter / 128;          // one tile = 128 activation columns = 256 GEMM columns
    p.num_k_blocks = a->K / 128;
    p.nb128 = a->N / 128;
    p.num_m_blocks = (a->M + gg::BM - 1) / gg::BM;
    p.act_q = static_cast<uint8_t*>(act_q);
    p.act_s = act_scales;
    p.act_ss_r = ss_row; p.act_ss_b = ss_blk;
    p.gate_first = gate_first ? 1 : 0;
    long long max_tiles = (long long)p.num_m_blocks * p.num_n_blocks;
    int grid = (int)(max_tiles < di->num_sms ? max_tiles : di->num_sms);
    if (grid < 1) grid = 1;
    gg_fp8_kernel<false, true><<<grid, gg::THREADS, gg::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
        tmap_a, tmap_b, tmap_a, p, di->status);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

constexpr int ALPHA_FUSED_PLAN_MAX_ROUTES = 512;    // measured: the per-warp scan of the route list wins up to a few hundred routes
constexpr bool ALPHA_SWAP_GATE_UP_DEFAULT = true;
constexpr bool ALPHA_SWAP_DOWN_DEFAULT = true;

// out[c * R + r] = in[r * C + c] for a byte matrix in [R, C]; 128 x 128 tiles, full 128-byte lines in and out.
// Phase 1: the tile lands in shared memory as 32-bit words (row pitch 33 words); phase 2: thread (segment, column)
// gathers the 16 bytes of its column from 16 consecutive rows (a warp = 32 columns of one segment: 8 distinct
// banks, broadcast) into a second, transposed tile; phase 3: that tile leaves as 16-byte pieces of full lines.
// R % 128 == 0 and C % 16 == 0.
__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                                             long long R, int C) {
    __shared__ uint32_t t[128][33];
    __shared__ __align__(16) uint32_t tt[128][36];
    const long long r0 = (long long)blockIdx.y * 128;
    const int c0 = blockIdx.x * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + 256 * i, row = idx >> 3, seg = idx & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (c0 + seg * 16 < C) v = __ldg(reinterpret_cast<const uint4*>(in + (r0 + row) * C + c0 + seg * 16));
        t[row][seg * 4 + 0] = v.x; t[row][seg * 4 + 1] = v.y; t[row][seg * 4 + 2] = v.z; t[row][seg * 4 + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + 256 * i, seg = idx >> 7, c = idx & 127;
        const int sh = (c & 3) * 8;
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t x = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) x |= ((t[seg * 16 + q * 4 + k][c >> 2] >> sh) & 0xFFu) << (8 * k);
            w[q] = x;
        }
        *reinterpret_cast<uint4*>(&tt[c][seg * 4]) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + 256 * i, c = idx >> 3, seg = idx & 7;
        if (c0 + c < C)
            *reinterpret_cast<uint4*>(out + (long long)(c0 + c) * R + r0 + seg * 16) = *reinterpret_cast<const uint4*>(&tt[c][seg * 4]);
    }
}

struct KgWorkspace {
    uint8_t *at, *bt;
    int32_t* layout0;
    void* gg_ws;
    int* flag;
    uint32_t *sfa_tiles, *sfb_tiles;
    size_t gg_ws_bytes, bytes;
};

KgWorkspace carve_kg(void* base, int64_t M, int64_t N, int64_t K_total) {
    KgWorkspace w{};
    char* b = static_cast<char*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char* p = b ? b + off : nullptr; off += align256(bytes); return p; };
    w.at = reinterpret_cast<uint8_t*>(take((size_t)M * K_total));
    w.bt = reinterpret_cast<uint8_t*>(take((size_t)N * K_total));
    w.layout0 = reinterpret_cast<int32_t*>(take((size_t)M * 4));
    w.gg_ws_bytes = mx_layout(1, M, (int)N, (int)K_total).bytes;
    w.gg_ws = take(w.gg_ws_bytes);
    // single launch over all groups: scale tiles of every (128 rows or columns, scale word row); at most one word row
    // per 128 K rows
    const size_t max_quads = (size_t)(K_total / 128);
    w.flag = reinterpret_cast<int*>(take(256));
    w.sfa_tiles = reinterpret_cast<uint32_t*>(take((size_t)((M + 127) / 128) * max_quads * 512));
    w.sfb_tiles = reinterpret_cast<uint32_t*>(take((size_t)((N + mx::BN_WIDE - 1) / mx::BN_WIDE) * max_quads * 1024));
    w.bytes = off;
    return w;
}

struct AlphaWorkspace {
    int32_t *counts, *rowpos;
    float *s1, *s2, *g1, *d2;
    uint8_t *a1, *a2;
    int64_t max_m, rows_total;
    size_t bytes;
};

// Rows per expert: no expert can receive more than M routes (ids of a token are distinct); at least 128 rows in
// total so that a 128-row TMA box never exceeds the tensor.
AlphaWorkspace carve_alpha(void* base, int64_t M, int64_t H, int64_t I, int64_t E, int64_t top_k) {
    AlphaWorkspace w{};
    w.max_m = M > 0 ? M : 1;
    while (w.max_m * E < 128) ++w.max_m;
    w.rows_total = w.max_m * E;
    char* b = static_cast<char*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char* p = b ? b + off : nullptr; off += align256(bytes); return p; };
    w.counts = reinterpret_cast<int32_t*>(take((size_t)E * 4));
    w.rowpos = reinterpret_cast<int32_t*>(take((size_t)(M * top_k > 0 ? M * top_k : 1) * 4));
    w.a1 = reinterpret_cast<uint8_t*>(take((size_t)w.rows_total * H));
    w.s1 = reinterpret_cast<float*>(take((size_t)w.rows_total * (H / 128) * 4));
    w.g1 = reinterpret_cast<float*>(take((size_t)w.rows_total * 2 * I * 4));
    w.a2 = reinterpret_cast<uint8_t*>(take((size_t)w.rows_total * I));
    w.s2 = reinterpret_cast<float*>(take((size_t)w.rows_total * (I / 128) * 4));
    w.d2 = reinterpret_cast<float*>(take((size_t)w.rows_total * H * 4));
    w.bytes = off;
    return w;
}

int check_alpha_dims(int32_t M, int32_t H, int32_t I, int32_t E, int32_t top_k) {
    if (M < 0 || H <= 0 || H % 128) return fail(MOE_ERR_INVALID, "M must be non-negative and H a positive multiple of 128");
    if (I != 128) return fail(MOE_ERR_UNSUPPORTED, "the decode-regime layer supports I == 128 only (I=%d)", I);
    if (E <= 0 || E > gg::MAX_MASKED_GROUPS) return fail(MOE_ERR_INVALID, "E=%d must be in [1, %d]", E, gg::MAX_MASKED_GROUPS);
    if (top_k <= 0 || top_k > 32) return fail(MOE_ERR_INVALID, "top_k=%d must be in [1, 32]", top_k);
    if ((int64_t)M * top_k > 32768) return fail(MOE_ERR_UNSUPPORTED, "M*top_k=%lld exceeds 32768 routes", (long long)M * top_k);
    return MOE_OK;
}

}  // namespace

extern "C" {

int moe_gg_fp8_gate_up_act(const moe_gg_args* args, void* act_q, float* act_scales, int64_t ss_row, int64_t ss_blk,
                           int32_t gate_first, void* stream) {
    return launch_gg_fused_act(args, act_q, act_scales, ss_row, ss_blk, gate_first, stream);
}

size_t moe_gg_workspace_bytes(int32_t G, int64_t rows_total, int32_t N, int32_t K) {
    if (G <= 0 || rows_total < 0 || N <= 0 || K <= 0) return 0;
    return mx_layout(G, rows_total, N, K).bytes;
}

int moe_gg_fp8_contiguous(const moe_gg_args* args, void* stream) { return launch_gg<false>(args, stream); }
int moe_gg_fp8_masked(const moe_gg_args* args, void* stream) { return launch_gg<true>(args, stream); }

int moe_device_status(int32_t* status_out, void* stream) {
    CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    int v = 0;
    CUDA_TRY(cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)));
    if (v != 0) {
        int zero = 0;
        CUDA_TRY(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)));
    }
    if (status_out) *status_out = v;
    if (v != 0) return fail(MOE_ERR_DEVICE, "device status 0x%x: a bounded wait inside a kernel ran out", v);
    return MOE_OK;
}


int moe_quant_1x128(const void* x_bf16, void* q, float* scales, int64_t ss_row, int64_t ss_blk,
                    int32_t rows, int32_t cols, void* stream) {
    if (!x_bf16 || !q || !scales) return fail(MOE_ERR_INVALID, "x, q and scales must be non-NULL");
    if (rows < 0 || cols <= 0 || cols % 128) return fail(MOE_ERR_INVALID, "cols=%d must be a positive multiple of 128", cols);
    if (rows == 0) return MOE_OK;
    const long long warps = (long long)rows * (cols / 128);
    const int wpb = 8;
    quant_1x128_kernel<<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(q), scales, ss_row, ss_blk, rows, cols);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_silu_mul_requant(const void* gate_up_bf16, void* q, float* scales, int64_t ss_row, int64_t ss_blk,
                         const int32_t* layout, int32_t rows, int32_t inter, int32_t gate_first, void* stream) {
    if (!gate_up_bf16 || !q || !scales) return fail(MOE_ERR_INVALID, "gate_up, q and scales must be non-NULL");
    if (rows < 0 || inter <= 0 || inter % 128) return fail(MOE_ERR_INVALID, "inter=%d must be a positive multiple of 128", inter);
    if (rows == 0) return MOE_OK;
    const int wpb = 8;
    silu_mul_requant_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(gate_up_bf16), static_cast<uint8_t*>(q), scales, ss_row, ss_blk, layout,
        rows, inter, gate_first);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_route_topk(const float* logits, int32_t* ids, float* weights, int32_t T, int32_t E, int32_t top_k,
                   void* stream) {
    if (!logits || !ids || !weights) return fail(MOE_ERR_INVALID, "logits, ids and weights must be non-NULL");
    if (E <= 0 || E > 32 * ROUTE_MAX_PER_LANE) return fail(MOE_ERR_INVALID, "E=%d must be in [1, %d]", E, 32 * ROUTE_MAX_PER_LANE);
    if (top_k <= 0 || top_k > 32 || top_k > E) return fail(MOE_ERR_INVALID, "top_k=%d must be in [1, min(32, E)]", top_k);
    if (T < 0) return fail(MOE_ERR_INVALID, "T must be non-negative");
    if (T == 0) return MOE_OK;
    const int wpb = 8;
    route_softmax_topk_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, ids, weights, T, E, top_k);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_route_deepseek(const float* logits, const void* bias, int32_t bias_dtype, int32_t* ids, float* weights, int32_t T,
                       int32_t E, int32_t n_group, int32_t topk_group, int32_t top_k, float routed_scaling_factor,
                       void* stream) {
    if (!logits || !bias || !ids || !weights) return fail(MOE_ERR_INVALID, "logits, bias, ids and weights must be non-NULL");
    if (n_group <= 0 || n_group > DS_MAX_GROUPS || E != 32 * n_group)
        return fail(MOE_ERR_UNSUPPORTED, "E=%d must be 32 * n_group with n_group in [1, %d]", E, DS_MAX_GROUPS);
    if (topk_group <= 0 || topk_group > n_group) return fail(MOE_ERR_INVALID, "topk_group must be in [1, n_group]");
    if (top_k <= 0 || top_k > 32 || top_k > 32 * topk_group) return fail(MOE_ERR_INVALID, "top_k out of range");
    if (bias_dtype != MOE_DTYPE_BF16 && bias_dtype != MOE_DTYPE_F32) return fail(MOE_ERR_INVALID, "bias_dtype must be bf16 or f32");
    if (T <= 0) return T == 0 ? MOE_OK : fail(MOE_ERR_INVALID, "T must be non-negative");
    const int wpb = 8;
    route_deepseek_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        logits, bias, bias_dtype == MOE_DTYPE_BF16, ids, weights, T, n_group, topk_group, top_k, routed_scaling_factor);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

size_t moe_permute_workspace_bytes(int64_t n_pairs, int32_t E_local) {
    const int64_t n_chunks = (n_pairs + PLAN_CHUNK - 1) / PLAN_CHUNK;
    return align256((size_t)(n_chunks > 0 ? n_chunks : 1) * (size_t)E_local * 4);
}

int moe_permute_plan(const int32_t* ids, int64_t n_pairs, int32_t e_lo, int32_t E_local, int32_t align,
                     int32_t cap_rows, int32_t* counts, int32_t* offsets, int32_t* pos, int32_t* src_pair,
                     int32_t* grouped_layout, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_plan_args(n_pairs, E_local, align, cap_rows);
    if (rc != MOE_OK) return rc;
    if (!ids || !counts || !offsets || !pos || !src_pair || !grouped_layout || !workspace)
        return fail(MOE_ERR_INVALID, "all plan pointers must be non-NULL");
    if (workspace_bytes < moe_permute_workspace_bytes(n_pairs, E_local))
        return fail(MOE_ERR_INVALID, "plan workspace too small: %zu < %zu", workspace_bytes,
                    moe_permute_workspace_bytes(n_pairs, E_local));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* chunk_counts = static_cast<int*>(workspace);
    const int n_chunks = (int)((n_pairs + PLAN_CHUNK - 1) / PLAN_CHUNK);
    const size_t hist_bytes = (size_t)32 * E_local * 4;
    if (n_chunks > 0) {
        plan_count_kernel<<<n_chunks, PLAN_CHUNK, hist_bytes, st>>>(ids, n_pairs, e_lo, E_local, chunk_counts);
        CUDA_TRY(cudaGetLastError());
    }
    plan_scan_kernel<<<1, 256, (size_t)E_local * 4, st>>>(chunk_counts, n_chunks, E_local, align, counts, offsets);
    CUDA_TRY(cudaGetLastError());
    const int place_blocks = n_chunks > 0 ? n_chunks : 1;
    plan_place_kernel<<<place_blocks, PLAN_CHUNK, hist_bytes, st>>>(ids, n_pairs, e_lo, E_local, chunk_counts, counts,
                                                                   offsets, pos, src_pair, grouped_layout, cap_rows);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_permute(const void* x_q, const float* x_scale, int64_t xs_row, int64_t xs_blk, const int32_t* src_pair,
                int32_t top_k, void* a, float* a_scale, int64_t as_row, int64_t as_blk, int32_t rows, int32_t H,
                void* stream) {
    if (!x_q || !x_scale || !src_pair || !a || !a_scale) return fail(MOE_ERR_INVALID, "permute pointers must be non-NULL");
    if (H <= 0 || H % 128 || top_k <= 0) return fail(MOE_ERR_INVALID, "H must be a positive multiple of 128, top_k positive");
    if ((reinterpret_cast<uintptr_t>(x_q) & 15) || (reinterpret_cast<uintptr_t>(a) & 15))
        return fail(MOE_ERR_INVALID, "x_q and a must be 16-byte aligned");
    if (rows <= 0) return rows == 0 ? MOE_OK : fail(MOE_ERR_INVALID, "rows must be non-negative");
    const int wpb = 8;
    gather_rows_kernel<<<(rows + wpb - 1) / wpb, wpb * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x_q), x_scale, xs_row, xs_blk, src_pair, top_k, static_cast<uint8_t*>(a), a_scale,
        as_row, as_blk, rows, H);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_combine(const void* y_bf16, const int32_t* pos, const float* w, void* out_bf16, int32_t T, int32_t top_k,
                int32_t H, void* stream) {
    if (!y_bf16 || !pos || !w || !out_bf16) return fail(MOE_ERR_INVALID, "combine pointers must be non-NULL");
    if (H <= 0 || H % 8 || top_k <= 0 || top_k > 32) return fail(MOE_ERR_INVALID, "H must be a multiple of 8 and top_k in [1, 32]");
    if (T <= 0) return T == 0 ? MOE_OK : fail(MOE_ERR_INVALID, "T must be non-negative");
    combine_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(y_bf16), pos, w, static_cast<__nv_bfloat16*>(out_bf16), T, top_k, H);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

size_t moe_workspace_bytes(int32_t T, int32_t H, int32_t I, int32_t E, int32_t top_k, int32_t align) {
    if (T < 0 || H <= 0 || I <= 0 || E <= 0 || top_k <= 0 || align <= 0) return 0;
    return carve_layer(nullptr, T, H, I, E, top_k, align).bytes;
}

int moe_layer_forward(const moe_layer_args* L, void* stream) {
    if (!L) return fail(MOE_ERR_INVALID, "args is NULL");
    if (!L->x_q || !L->x_scale || !L->w13 || !L->w13_scale || !L->w2 || !L->w2_scale || !L->out || !L->workspace)
        return fail(MOE_ERR_INVALID, "x_q, x_scale, w13, w13_scale, w2, w2_scale, out and workspace must be non-NULL");
    if (!L->logits && !(L->topk_ids && L->topk_weights))
        return fail(MOE_ERR_INVALID, "pass router logits, or both topk_ids and topk_weights");
    if (L->H % 128 || L->I % 128) return fail(MOE_ERR_INVALID, "H and I must be multiples of 128");
    if (L->T < 0 || L->E <= 0 || L->E > 256 || L->top_k <= 0 || L->top_k > 32)
        return fail(MOE_ERR_INVALID, "T>=0, 1<=E<=256, 1<=top_k<=32 required");
    if (L->align <= 0 || L->align % 128) return fail(MOE_ERR_INVALID, "align must be a positive multiple of 128");
    const size_t need = moe_workspace_bytes(L->T, L->H, L->I, L->E, L->top_k, L->align);
    if (L->workspace_bytes < need)
        return fail(MOE_ERR_INVALID, "workspace too small: %zu < %zu bytes", (size_t)L->workspace_bytes, need);
    if (L->T == 0) return MOE_OK;
    LayerWorkspace w = carve_layer(L->workspace, L->T, L->H, L->I, L->E, L->top_k, L->align);
    const int64_t n_pairs = (int64_t)L->T * L->top_k;
    const int32_t cap = (int32_t)w.cap_rows;
    int rc;
    const int32_t* ids = L->topk_ids;
    const float* wts = L->topk_weights;
    if (L->logits) {
        const int32_t e_glob = L->E_global > 0 ? L->E_global : L->E;
        if (L->routing_bias != nullptr)      // DeepSeek-V3 no-aux routing of the registered `moe` workload
            rc = moe_route_deepseek(L->logits, L->routing_bias, MOE_DTYPE_BF16, w.ids, w.weights, L->T, e_glob,
                                    L->n_group > 0 ? L->n_group : 8, L->topk_group > 0 ? L->topk_group : 4, L->top_k,
                                    L->routed_scaling_factor, stream);
        else
            rc = moe_route_topk(L->logits, w.ids, w.weights, L->T, e_glob, L->top_k, stream);
        if (rc != MOE_OK) return rc;
        ids = w.ids;
        wts = w.weights;
    }
    rc = moe_permute_plan(ids, n_pairs, L->e_lo, L->E, L->align, cap, w.counts, w.offsets, w.pos, w.src_pair,
                          w.layout, w.chunk_counts, moe_permute_workspace_bytes(n_pairs, L->E), stream);
    if (rc != MOE_OK) return rc;
    // scales of the gathered rows are stored MN-major ([K/128, cap]) so that the GEMM's per-row
    // scale loads are coalesced
    rc = moe_permute(L->x_q, L->x_scale, L->xs_stride_row, L->xs_stride_blk, w.src_pair, L->top_k, w.a1, w.s1, 1, cap,
                     cap, L->H, stream);
    if (rc != MOE_OK) return rc;
    moe_gg_args g1 = {};
    g1.a = w.a1; g1.b = L->w13; g1.sfa = w.s1; g1.sfa_stride_row = 1; g1.sfa_stride_kblk = cap;
    g1.sfb = L->w13_scale; g1.layout = w.layout; g1.d = w.g1; g1.ldd = 2 * (int64_t)L->I;
    g1.rows_used = w.offsets + L->E;
    g1.G = L->E; g1.M = cap; g1.N = 2 * L->I; g1.K = L->H; g1.d_dtype = MOE_DTYPE_BF16;
    if (L->fuse_act) {
        rc = moe_gg_fp8_gate_up_act(&g1, w.a2, w.s2, 1, cap, L->gate_first, stream);
        if (rc != MOE_OK) return rc;
    } else {
        rc = moe_gg_fp8_contiguous(&g1, stream);
        if (rc != MOE_OK) return rc;
        rc = moe_silu_mul_requant(w.g1, w.a2, w.s2, 1, cap, w.layout, cap, L->I, L->gate_first, stream);
        if (rc != MOE_OK) return rc;
    }
    moe_gg_args g2 = {};
    g2.a = w.a2; g2.b = L->w2; g2.sfa = w.s2; g2.sfa_stride_row = 1; g2.sfa_stride_kblk = cap;
    g2.sfb = L->w2_scale; g2.layout = w.layout; g2.d = w.y; g2.ldd = L->H;
    g2.rows_used = w.offsets + L->E;
    g2.G = L->E; g2.M = cap; g2.N = L->H; g2.K = L->I; g2.d_dtype = MOE_DTYPE_BF16;
    rc = moe_gg_fp8_contiguous(&g2, stream);
    if (rc != MOE_OK) return rc;
    return moe_combine(w.y, w.pos, wts, L->out, L->T, L->top_k, L->H, stream);
}

int moe_layer_workspace_view(void* workspace, int32_t T, int32_t H, int32_t I, int32_t E, int32_t top_k,
                             int32_t align, moe_layer_view* view) {
    if (!view) return fail(MOE_ERR_INVALID, "view is NULL");
    LayerWorkspace w = carve_layer(workspace, T, H, I, E, top_k, align);
    view->ids = w.ids; view->weights = w.weights; view->counts = w.counts; view->offsets = w.offsets;
    view->pos = w.pos; view->src_pair = w.src_pair; view->grouped_layout = w.layout;
    view->a1 = w.a1; view->s1 = w.s1; view->g1 = w.g1; view->a2 = w.a2; view->s2 = w.s2; view->y = w.y;
    view->cap_rows = w.cap_rows;
    return MOE_OK;
}

/* ---------------------------------------------------------------- k-grouped layout */
size_t moe_kg_workspace_bytes(int32_t M, int32_t N, int64_t K_total) {
    if (M <= 0 || N <= 0 || K_total <= 0 || K_total % 128 || K_total > 0x7FFFFFFFll) return 0;
    return carve_kg(nullptr, M, N, K_total).bytes;
}

int moe_kg_fp8_contiguous(const moe_kg_args* A, void* stream) {
    if (!A) return fail(MOE_ERR_INVALID, "args is NULL");
    if (!A->a || !A->b || !A->sfa || !A->sfb || !A->d || !A->ks || !A->workspace)
        return fail(MOE_ERR_INVALID, "a, b, sfa, sfb, d, ks and workspace must be non-NULL");
    if (A->G <= 0 || A->M <= 0 || A->N <= 0 || A->M % 128 || A->N % 16)
        return fail(MOE_ERR_INVALID, "G, M, N must be positive, M a multiple of 128 and N of 16 (G=%d M=%d N=%d)", A->G, A->M, A->N);
    int64_t k_sum = 0;
    for (int g = 0; g < A->G; ++g) {
        if (A->ks[g] < 0 || A->ks[g] % 128) return fail(MOE_ERR_INVALID, "ks[%d]=%d must be a non-negative multiple of 128", g, A->ks[g]);
        k_sum += A->ks[g];
    }
    if (k_sum != A->K_total || k_sum <= 0 || k_sum > 0x7FFFFFFFll)
        return fail(MOE_ERR_INVALID, "sum(ks)=%lld must equal K_total=%lld (positive, < 2^31)", (long long)k_sum, (long long)A->K_total);
    if ((reinterpret_cast<uintptr_t>(A->a) & 15) || (reinterpret_cast<uintptr_t>(A->b) & 15) || (reinterpret_cast<uintptr_t>(A->d) & 15) ||
        (reinterpret_cast<uintptr_t>(A->workspace) & 255))
        return fail(MOE_ERR_INVALID, "a, b, d must be 16-byte aligned and workspace 256-byte aligned");
    const size_t need = moe_kg_workspace_bytes(A->M, A->N, A->K_total);
    if (A->workspace_bytes < need) return fail(MOE_ERR_INVALID, "workspace too small: %zu < %zu bytes", (size_t)A->workspace_bytes, need);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    KgWorkspace w = carve_kg(A->workspace, A->M, A->N, A->K_total);
    // default: the MN-major operands go to the tensor core as they are (MOE_OPT_KG_MODE selects the other two forms)
    const int kg_mode = opt(MOE_OPT_KG_MODE);
    const bool single_launch = A->G <= 64 && kg_mode != MOE_KG_MODE_PER_GROUP;
    const bool mn_major = single_launch && kg_mode == MOE_KG_MODE_MN_MAJOR && A->M % 16 == 0;
    CUDA_TRY(cudaMemsetAsync(w.layout0, 0, (size_t)A->M * 4, st));        // every row belongs to group 0 of its launch
    if (!mn_major) {
    transpose_u8_kernel<<<dim3((A->M + 127) / 128, (unsigned)(A->K_total / 128)), 256, 0, st>>>(
        static_cast<const uint8_t*>(A->a), w.at, A->K_total, A->M);
    CUDA_TRY(cudaGetLastError());
    transpose_u8_kernel<<<dim3((A->N + 127) / 128, (unsigned)(A->K_total / 128)), 256, 0, st>>>(
        static_cast<const uint8_t*>(A->b), w.bt, A->K_total, A->N);
    CUDA_TRY(cudaGetLastError());
    }
    if (single_launch) {
        // one launch over all groups (per-group launches round 6.05 waves of tiles up to 7, eight times)
        DeviceInfo* di = nullptr;
        int rc = device_info(&di);
        if (rc != MOE_OK) return rc;
        KgTable kg = {};
        kg.n = A->G;
        int64_t ko = 0, qo = 0;
        for (int g = 0; g < A->G; ++g) {
            kg.koff[g] = (int)ko; kg.kb[g] = A->ks[g] / 128; kg.qoff[g] = (int)qo;
            ko += A->ks[g];
            qo += (A->ks[g] + 511) / 512;
        }
        const int quads = (int)qo;
        GGParams p = {};
        p.d = A->d; p.ldd = A->N; p.d_f32 = 1; p.d_accumulate = 1;
        p.G = A->G; p.M = A->M; p.N = A->N; p.K = (int)A->K_total;
        p.rows_total = A->M;
        p.num_n_blocks = (A->N + mx::BN_WIDE - 1) / mx::BN_WIDE;
        p.num_k_blocks = 0;
        p.nb128 = (A->N + 127) / 128;
        p.num_m_blocks = (A->M + 127) / 128;
        kg.per_group = ((A->M + 255) / 256) * p.num_n_blocks;
        MxWorkspace ws;
        ws.flag = w.flag; ws.sfa_packed = w.sfa_tiles; ws.sfb_packed = w.sfb_tiles;
        ws.row_blocks = (A->M + 127) / 128; ws.quads = quads;
        ws.n_tiles = p.num_n_blocks; ws.nt_base = mx::BN_WIDE / 16; ws.nt_rem = 0;
        p.nt_base = ws.nt_base; p.nt_rem = 0;
        ws.gen = p.mode_gen = next_gen();
        dim3 pgrid(ws.row_blocks + ws.n_tiles * 2, quads, 1);
        mx_prep_packed_kernel<<<pgrid, 128, 0, st>>>(reinterpret_cast<const uint32_t*>(A->sfa), 1, A->M,
                                                     reinterpret_cast<const uint32_t*>(A->sfb), 0, 1, A->N, A->M, A->N, 1, ws);
        CUDA_TRY(cudaGetLastError());
        CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
        if (mn_major) {      // the caller's matrices as they are: [K_total rows, M or N bytes], box = 128 K rows x 128 bytes
            rc = encode_fp8_kmajor(&tm_a, A->a, (uint64_t)A->K_total, (uint64_t)A->M, 128);
            if (rc != MOE_OK) return rc;
            rc = encode_fp8_kmajor(&tm_b, A->b, (uint64_t)A->K_total, (uint64_t)A->N, 128);
            if (rc != MOE_OK) return rc;
        } else {
            rc = encode_fp8_kmajor(&tm_a, w.at, (uint64_t)A->M, (uint64_t)A->K_total, 128);
            if (rc != MOE_OK) return rc;
            rc = encode_fp8_kmajor(&tm_b, w.bt, (uint64_t)A->N, (uint64_t)A->K_total, mx::BN_WIDE / 2);
            if (rc != MOE_OK) return rc;
        }
        rc = encode_words_1d(&tm_sfa, ws.sfa_packed, (uint64_t)ws.row_blocks * quads * 128);
        if (rc != MOE_OK) return rc;
        rc = encode_words_1d(&tm_sfb, ws.sfb_packed, (uint64_t)ws.n_tiles * quads * 256);
        if (rc != MOE_OK) return rc;
        const long long tiles = (long long)kg.n * kg.per_group;
        int pairs = (int)(tiles < di->max_pairs ? tiles : di->max_pairs);
        if (pairs < 1) pairs = 1;
        if (mn_major)
            gg_fp8_mx_kernel<false, true, true><<<2 * pairs, mx::THREADS, mx::SMEM_BYTES, st>>>(tm_a, tm_b, tm_sfa, tm_sfb, p, ws.flag,
                                                                                              quads, di->status, kg);
        else
            gg_fp8_mx_kernel<false, true><<<2 * pairs, mx::THREADS, mx::SMEM_BYTES, st>>>(tm_a, tm_b, tm_sfa, tm_sfb, p, ws.flag, quads,
                                                                                        di->status, kg);
        CUDA_TRY(cudaGetLastError());
        return MOE_OK;
    }
    int64_t koff = 0, srow = 0;
    for (int g = 0; g < A->G; ++g) {
        const int32_t k = A->ks[g];
        if (k == 0) continue;
        moe_gg_args gg = {};
        gg.a = w.at + koff; gg.lda = A->K_total;
        gg.b = w.bt + koff; gg.ldb = A->K_total;
        gg.sfa = reinterpret_cast<const float*>(A->sfa + srow * A->M); gg.sfa_stride_row = 1; gg.sfa_stride_kblk = A->M;
        gg.sfb = reinterpret_cast<const float*>(A->sfb + srow * A->N);
        gg.sfb_stride[0] = 0; gg.sfb_stride[1] = 1; gg.sfb_stride[2] = A->N;
        gg.layout = w.layout0;
        gg.d = A->d + (int64_t)g * A->M * A->N; gg.ldd = A->N;
        gg.G = 1; gg.M = A->M; gg.N = A->N; gg.K = k;
        gg.d_dtype = MOE_DTYPE_F32; gg.accumulate = 1; gg.sf_format = MOE_SF_UE8M0_PACKED;
        gg.workspace = w.gg_ws; gg.workspace_bytes = w.gg_ws_bytes;
        int rc = launch_gg<false>(&gg, stream);
        if (rc != MOE_OK) return rc;
        koff += k;
        srow += (k + 511) / 512;
    }
    return MOE_OK;
}

/* ---------------------------------------------------------------- decode-regime layer (alphamoe task) */
size_t moe_alpha_workspace_bytes(int32_t M, int32_t H, int32_t I, int32_t E, int32_t top_k) {
    if (M < 0 || H <= 0 || I <= 0 || E <= 0 || top_k <= 0) return 0;
    return carve_alpha(nullptr, M, H, I, E, top_k).bytes;
}

int moe_alpha_workspace_view(void* workspace, int32_t M, int32_t H, int32_t I, int32_t E, int32_t top_k,
                             moe_alpha_view* view) {
    if (!view) return fail(MOE_ERR_INVALID, "view is NULL");
    int rc = check_alpha_dims(M, H, I, E, top_k);
    if (rc != MOE_OK) return rc;
    AlphaWorkspace w = carve_alpha(workspace, M, H, I, E, top_k);
    view->counts = w.counts; view->rowpos = w.rowpos; view->s1 = w.s1; view->s2 = w.s2; view->g1 = w.g1;
    view->d2 = w.d2; view->a1 = w.a1; view->a2 = w.a2; view->max_m = w.max_m;
    return MOE_OK;
}

int moe_alpha_forward(const moe_alpha_args* A, void* stream) {
    if (!A) return fail(MOE_ERR_INVALID, "args is NULL");
    int rc = check_alpha_dims(A->M, A->H, A->I, A->E, A->top_k);
    if (rc != MOE_OK) return rc;
    if (!A->hidden || !A->topk_ids || !A->topk_weights || !A->w13 || !A->w13_scale || !A->w2 || !A->w2_scale || !A->out ||
        !A->workspace)
        return fail(MOE_ERR_INVALID, "hidden, topk_ids, topk_weights, weights, scales, out and workspace must be non-NULL");
    if ((reinterpret_cast<uintptr_t>(A->hidden) & 15) || (reinterpret_cast<uintptr_t>(A->out) & 15) ||
        (reinterpret_cast<uintptr_t>(A->workspace) & 255))
        return fail(MOE_ERR_INVALID, "hidden and out must be 16-byte aligned, workspace 256-byte aligned");
    const size_t need = moe_alpha_workspace_bytes(A->M, A->H, A->I, A->E, A->top_k);
    if (A->workspace_bytes < need)
        return fail(MOE_ERR_INVALID, "workspace too small: %zu < %zu bytes", (size_t)A->workspace_bytes, need);
    if (A->M == 0) return MOE_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AlphaWorkspace w = carve_alpha(A->workspace, A->M, A->H, A->I, A->E, A->top_k);
    const int n_pairs = A->M * A->top_k;
    const size_t hist_bytes = (size_t)32 * A->E * 4;
    DeviceInfo* di = nullptr;      // also raises the kernels' dynamic shared-memory limits, once per device
    rc = device_info(&di);
    if (rc != MOE_OK) return rc;
    // A handful of tokens (default: up to 160 routes = 16 tokens x top-10): two CUDA-core kernels that stream each
    // routed expert's weights once (alpha_gemv.cuh).  MOE_OPT_ALPHA_GEMV_MAX_ROUTES moves the threshold (0 = never);
    // any MOE_OPT_ALPHA_PATH other than AUTO selects the tensor-core pipeline below.
    const int alpha_path = opt(MOE_OPT_ALPHA_PATH);
    {
        const int gemv_max = opt(MOE_OPT_ALPHA_GEMV_MAX_ROUTES);
        if (n_pairs <= gemv_max && A->H <= AGV_MAX_H && alpha_path == MOE_ALPHA_PATH_AUTO) {
            float* act = w.d2;                  // [n_pairs, 128] fp32, indexed by route
            CUDA_TRY(launch_pdl(alpha_gemv_gate_up_kernel, dim3(n_pairs * AGV_SLICES), dim3(256), 0, st,
                                static_cast<const __nv_bfloat16*>(A->hidden), A->topk_ids, static_cast<const uint8_t*>(A->w13),
                                A->w13_scale, A->top_k, A->E, A->H, act, w.g1));
            CUDA_TRY(launch_pdl(alpha_gemv_down_kernel, dim3(A->M * (A->H / 32)), dim3(128), 0, st, (const float*)act, A->topk_ids,
                                A->topk_weights, static_cast<const uint8_t*>(A->w2), A->w2_scale, A->routed_scaling_factor,
                                A->top_k, A->E, A->H, static_cast<__nv_bfloat16*>(A->out)));
            return MOE_OK;
        }
    }
    const int wpb = 8;
    const int route_blocks = (n_pairs + wpb - 1) / wpb;
    const int quant_blocks = (n_pairs * (A->H / 128) + wpb - 1) / wpb;
    if (n_pairs <= ALPHA_FUSED_PLAN_MAX_ROUTES) {
        // decode regime: every quantisation warp finds its route's slot itself, no separate plan launch
        CUDA_TRY(cudaMemsetAsync(w.counts, 0, (size_t)A->E * 4, st));
        alpha_plan_quant_kernel<<<quant_blocks, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(A->hidden), A->topk_ids, n_pairs,
                                                                 A->top_k, A->E, (int)w.max_m, A->H, w.rows_total, w.counts, w.rowpos,
                                                                 w.a1, w.s1, di->status);
        CUDA_TRY(cudaGetLastError());
    } else {
        CUDA_TRY(launch_pdl(alpha_plan_kernel, dim3(1), dim3(ALPHA_PLAN_THREADS), hist_bytes, st, A->topk_ids, n_pairs, A->E,
                            (int)w.max_m, w.counts, w.rowpos, di->status));
        CUDA_TRY(launch_pdl(alpha_quant_scatter_kernel, dim3(quant_blocks), dim3(wpb * 32), 0, st,
                            static_cast<const __nv_bfloat16*>(A->hidden), w.rowpos, n_pairs, A->top_k, A->H, w.rows_total, w.a1, w.s1));
    }
    (void)route_blocks;
    // The two projections run either as swapped-operand decode kernels (weights = MMA rows, 32 routed rows = MMA
    // columns) or as row-major masked-layout grouped GEMMs (128 x 256 tiles); the intermediates have the same layout
    // either way.  MOE_OPT_ALPHA_PATH = SWAP | MASKED | MIXED (masked gate_up, swapped down).
    bool swap1 = ALPHA_SWAP_GATE_UP_DEFAULT, swap2 = ALPHA_SWAP_DOWN_DEFAULT;
    if (alpha_path != MOE_ALPHA_PATH_AUTO) {
        swap1 = alpha_path == MOE_ALPHA_PATH_SWAP;
        swap2 = alpha_path == MOE_ALPHA_PATH_SWAP || alpha_path == MOE_ALPHA_PATH_MIXED;
    }
    // (expert, chunk) units: at most one per expert that has rows plus one per further 32 rows
    const long long unit_bound = (n_pairs < A->E ? n_pairs : A->E) + n_pairs / asw::NT;
    long long* trace = nullptr;
    AlphaGemmParams gp{};
    gp.counts = w.counts; gp.E = A->E; gp.max_m = (int)w.max_m; gp.rows_total = w.rows_total;
    gp.a2 = w.a2; gp.s2 = w.s2; gp.g1 = w.g1; gp.d2 = w.d2; gp.H = A->H;
    if (swap1) {
        CUtensorMap tm_w13, tm_x1;
        rc = encode_fp8_kmajor(&tm_w13, A->w13, (uint64_t)A->E * 2 * A->I, (uint64_t)A->H, 128);
        if (rc != MOE_OK) return rc;
        rc = encode_fp8_kmajor(&tm_x1, w.a1, (uint64_t)w.rows_total, (uint64_t)A->H, asw::NT);
        if (rc != MOE_OK) return rc;
        gp.trace = trace;
        gp.s_rows = w.s1; gp.sfb = A->w13_scale; gp.KB = A->H / 128; gp.NF = 1;
        int grid1 = (int)(unit_bound < di->num_sms ? unit_bound : di->num_sms);
        CUDA_TRY(launch_pdl(alpha_swap_kernel<1>, dim3(grid1), dim3(asw::Cfg<1>::THREADS), asw::Cfg<1>::SMEM_BYTES, st, tm_w13, tm_x1,
                            gp, di->status));
    } else {
        moe_gg_args g1 = {};
        g1.a = w.a1; g1.b = A->w13; g1.sfa = w.s1; g1.sfa_stride_row = 1; g1.sfa_stride_kblk = w.rows_total;
        g1.sfb = A->w13_scale; g1.layout = w.counts; g1.d = w.g1; g1.ldd = 2 * (int64_t)A->I;
        g1.G = A->E; g1.M = (int32_t)w.max_m; g1.N = 2 * A->I; g1.K = A->H; g1.d_dtype = MOE_DTYPE_F32;
        rc = moe_gg_fp8_masked(&g1, stream);
        if (rc != MOE_OK) return rc;
        CUDA_TRY(launch_pdl(alpha_silu_requant_kernel, dim3(route_blocks), dim3(wpb * 32), 0, st, (const float*)w.g1,
                            (const int*)w.rowpos, n_pairs, A->I, 1, w.rows_total, w.a2, w.s2));
    }
    if (swap2) {
        CUtensorMap tm_w2, tm_x2;
        rc = encode_fp8_kmajor(&tm_w2, A->w2, (uint64_t)A->E * A->H, (uint64_t)A->I, 128);
        if (rc != MOE_OK) return rc;
        rc = encode_fp8_kmajor(&tm_x2, w.a2, (uint64_t)w.rows_total, (uint64_t)A->I, asw::NT);
        if (rc != MOE_OK) return rc;
        gp.s_rows = w.s2; gp.sfb = A->w2_scale; gp.KB = 1; gp.NF = A->H / 128;
        gp.trace = trace ? trace + 148 * 8 : nullptr;
        const long long units2 = unit_bound * gp.NF;
        int grid2 = (int)(units2 < di->num_sms ? units2 : di->num_sms);
        CUDA_TRY(launch_pdl(alpha_swap_kernel<2>, dim3(grid2), dim3(asw::Cfg<2>::THREADS), asw::Cfg<2>::SMEM_BYTES, st, tm_w2, tm_x2,
                            gp, di->status));
    } else {
        moe_gg_args g2 = {};
        g2.a = w.a2; g2.b = A->w2; g2.sfa = w.s2; g2.sfa_stride_row = 1; g2.sfa_stride_kblk = w.rows_total;
        g2.sfb = A->w2_scale; g2.layout = w.counts; g2.d = w.d2; g2.ldd = A->H;
        g2.G = A->E; g2.M = (int32_t)w.max_m; g2.N = A->H; g2.K = A->I; g2.d_dtype = MOE_DTYPE_F32;
        rc = moe_gg_fp8_masked(&g2, stream);
        if (rc != MOE_OK) return rc;
    }
    CUDA_TRY(launch_pdl(alpha_combine_kernel, dim3(A->M), dim3(A->H >= 2048 ? 512 : 256), 0, st, (const float*)w.d2, A->topk_ids,
                        A->topk_weights, (const int*)w.rowpos, A->routed_scaling_factor, A->top_k, A->H,
                        static_cast<__nv_bfloat16*>(A->out)));
    return MOE_OK;
}

/* ---------------------------------------------------------------- expert parallelism */

int moe_ipc_alloc(size_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return fail(MOE_ERR_INVALID, "ptr must be non-NULL and bytes positive");
    CUDA_TRY(cudaMalloc(ptr, bytes));
    CUDA_TRY(cudaMemset(*ptr, 0, bytes));
    return MOE_OK;
}
int moe_ipc_free(void* ptr) {
    if (ptr) CUDA_TRY(cudaFree(ptr));
    return MOE_OK;
}
int moe_ipc_get_handle(void* ptr, void* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    if (!ptr || !handle64) return fail(MOE_ERR_INVALID, "ptr and handle must be non-NULL");
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle64, &h, 64);
    return MOE_OK;
}
int moe_ipc_open(const void* handle64, void** ptr) {
    if (!ptr || !handle64) return fail(MOE_ERR_INVALID, "ptr and handle must be non-NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return MOE_OK;
}
int moe_ipc_close(void* ptr) {
    if (ptr) CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return MOE_OK;
}

static int ep_check(const moe_ep_peers* P, int rank, int world) {
    if (!P) return fail(MOE_ERR_INVALID, "peers is NULL");
    if (world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world)
        return fail(MOE_ERR_INVALID, "world=%d must be in [1, %d] and rank=%d inside it", world, EP_MAX_WORLD, rank);
    for (int i = 0; i < world; ++i)
        if (!P->a[i] || !P->sa[i] || !P->y[i] || !P->counts[i] || !P->flags[i] || !P->meta[i])
            return fail(MOE_ERR_INVALID, "peer table entry %d has a NULL pointer", i);
    return MOE_OK;
}
static EpPeers ep_convert(const moe_ep_peers* P) {
    EpPeers d;
    for (int i = 0; i < EP_MAX_WORLD; ++i) {
        d.a[i] = static_cast<uint8_t*>(P->a[i]);
        d.sa[i] = P->sa[i];
        d.y[i] = static_cast<const __nv_bfloat16*>(P->y[i]);
        d.counts[i] = P->counts[i];
        d.flags[i] = P->flags[i];
        d.meta[i] = P->meta[i];
    }
    return d;
}

int moe_ep_barrier(const moe_ep_peers* P, int32_t rank, int32_t world, int32_t epoch, void* stream) {
    int rc = ep_check(P, rank, world);
    if (rc != MOE_OK) return rc;
    DeviceInfo* di = nullptr;
    rc = device_info(&di);
    if (rc != MOE_OK) return rc;
    const unsigned long long limit_ns = (unsigned long long)opt(MOE_OPT_EP_WAIT_LIMIT_MS) * 1000000ull;
    ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ep_convert(P), rank, world, epoch, limit_ns, di->status);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

size_t moe_ep_workspace_bytes(int64_t n_pairs, int32_t E_total) {
    return moe_permute_workspace_bytes(n_pairs, E_total) + align256((size_t)(E_total + 1) * 4);
}

int moe_ep_count_publish(const moe_ep_peers* P, const int32_t* ids, int64_t n_pairs, int32_t rank, int32_t world,
                         int32_t E_total, int32_t* my_counts, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = ep_check(P, rank, world);
    if (rc != MOE_OK) return rc;
    rc = check_plan_args(n_pairs, E_total, 1, 0);
    if (rc != MOE_OK) return rc;
    if (!ids || !my_counts || !workspace) return fail(MOE_ERR_INVALID, "ids, my_counts and workspace must be non-NULL");
    if (workspace_bytes < moe_ep_workspace_bytes(n_pairs, E_total)) return fail(MOE_ERR_INVALID, "EP workspace too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* chunk_counts = static_cast<int*>(workspace);
    int* scratch_offsets = reinterpret_cast<int*>(static_cast<char*>(workspace) + moe_permute_workspace_bytes(n_pairs, E_total));
    const int n_chunks = (int)((n_pairs + PLAN_CHUNK - 1) / PLAN_CHUNK);
    if (n_chunks > 0) {
        plan_count_kernel<<<n_chunks, PLAN_CHUNK, (size_t)32 * E_total * 4, st>>>(ids, n_pairs, 0, E_total, chunk_counts);
        CUDA_TRY(cudaGetLastError());
    }
    plan_scan_kernel<<<1, 256, (size_t)E_total * 4, st>>>(chunk_counts, n_chunks, E_total, 1, my_counts, scratch_offsets);
    CUDA_TRY(cudaGetLastError());
    ep_publish_counts_kernel<<<1, 256, 0, st>>>(ep_convert(P), my_counts, rank, world, E_total);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_ep_plan(const moe_ep_peers* P, const int32_t* ids, int64_t n_pairs, int32_t rank, int32_t world,
                int32_t E_total, int32_t E_local, int32_t align, int32_t cap_rows, int32_t* counts_local,
                int32_t* offsets, int32_t* grouped_layout, int32_t* dst_base, int32_t* pos, int32_t* send_order,
                void* workspace, size_t workspace_bytes, void* stream) {
    int rc = ep_check(P, rank, world);
    if (rc != MOE_OK) return rc;
    rc = check_plan_args(n_pairs, E_total, align, cap_rows);
    if (rc != MOE_OK) return rc;
    if (E_local * world != E_total) return fail(MOE_ERR_INVALID, "E_total must equal world * E_local");
    if (!ids || !counts_local || !offsets || !grouped_layout || !dst_base || !pos || !workspace)
        return fail(MOE_ERR_INVALID, "plan pointers must be non-NULL");
    if (workspace_bytes < moe_ep_workspace_bytes(n_pairs, E_total)) return fail(MOE_ERR_INVALID, "EP workspace too small");
    DeviceInfo* di = nullptr;
    rc = device_info(&di);
    if (rc != MOE_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int* chunk_offsets = static_cast<const int*>(workspace);      // left by moe_ep_count_publish
    // first slot of every global expert in this rank's sending order: the scratch behind the chunk counters
    int* send_base = send_order ? reinterpret_cast<int*>(static_cast<char*>(workspace) + moe_permute_workspace_bytes(n_pairs, E_total))
                                : nullptr;
    ep_plan_kernel<<<1, 256, (size_t)2 * E_total * 4, st>>>(P->counts[rank], rank, world, E_total, E_local, align,
                                                          cap_rows, counts_local, offsets, dst_base, send_base, di->status);
    CUDA_TRY(cudaGetLastError());
    ep_layout_kernel<<<(cap_rows + 1023) / 1024, 1024, 0, st>>>(offsets, counts_local, E_local, grouped_layout, cap_rows);
    CUDA_TRY(cudaGetLastError());
    const int n_chunks = (int)((n_pairs + PLAN_CHUNK - 1) / PLAN_CHUNK);
    if (n_chunks > 0) {
        // cap = INT_MAX: destination rows live in the owners' buffers; the owner bounds them by its own capacity
        plan_place_kernel<<<n_chunks, PLAN_CHUNK, (size_t)32 * E_total * 4, st>>>(
            ids, n_pairs, 0, E_total, chunk_offsets, nullptr, dst_base, pos, nullptr, nullptr, 0x7FFFFFFF, send_base, send_order);
        CUDA_TRY(cudaGetLastError());
    }
    return MOE_OK;
}

int moe_ep_dispatch(const moe_ep_peers* P, const void* x_q, const float* x_scale, int64_t xs_row, int64_t xs_blk,
                    const int32_t* ids, const int32_t* pos, int64_t n_pairs, int32_t top_k, int32_t E_local, int32_t H,
                    int32_t cap_rows, int64_t pitch, int32_t rank, int32_t world, void* stream) {
    int rc = ep_check(P, rank, world);
    if (rc != MOE_OK) return rc;
    if (!x_q || !x_scale || !ids || !pos) return fail(MOE_ERR_INVALID, "dispatch pointers must be non-NULL");
    if (H <= 0 || H % 128 || top_k <= 0 || E_local <= 0)
        return fail(MOE_ERR_INVALID, "H must be a positive multiple of 128; top_k, E_local positive");
    if (n_pairs <= 0) return n_pairs == 0 ? MOE_OK : fail(MOE_ERR_INVALID, "n_pairs must be non-negative");
    if (n_pairs % top_k) return fail(MOE_ERR_INVALID, "n_pairs must be a multiple of top_k");
    if (top_k > 32) return fail(MOE_ERR_INVALID, "top_k must be at most 32");
    if (n_pairs > (1ll << 24)) return fail(MOE_ERR_INVALID, "n_pairs must be at most 2^24 (a row's return address packs the pair index into 24 bits)");
    const long long rec = ((long long)H + H / 32 + 15) & ~15ll;
    if (pitch < rec || pitch % 16) return fail(MOE_ERR_INVALID, "pitch must be >= H + H/32 (rounded up to 16) and a multiple of 16");
    if ((reinterpret_cast<uintptr_t>(x_q) & 15)) return fail(MOE_ERR_INVALID, "x_q must be 16-byte aligned");
    const long long tokens = n_pairs / top_k;
    DeviceInfo* di = nullptr;      // also raises the dispatch kernel's dynamic shared-memory limit, once per device
    rc = device_info(&di);
    if (rc != MOE_OK) return rc;
    const size_t smem = (size_t)DISPATCH_WARPS * rec;
    if (smem > (size_t)EP_DISPATCH_MAX_SMEM) return fail(MOE_ERR_INVALID, "H too large for the dispatch staging buffer");
    ep_dispatch_kernel<<<(unsigned)((tokens + DISPATCH_WARPS - 1) / DISPATCH_WARPS), DISPATCH_WARPS * 32, smem,
                         static_cast<cudaStream_t>(stream)>>>(
        ep_convert(P), static_cast<const uint8_t*>(x_q), x_scale, xs_row, xs_blk, ids, pos, n_pairs, top_k, E_local, H,
        cap_rows, rank, pitch, di->status);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_ep_gate_up_dispatch(const moe_gg_args* a, const moe_ep_send_args* S, void* act_q, float* act_scales, int64_t ss_row,
                            int64_t ss_blk, int32_t gate_first, void* stream) {
    if (!a || !S) return fail(MOE_ERR_INVALID, "args is NULL");
    int rc = ep_check(S->peers, S->rank, S->world);
    if (rc != MOE_OK) return rc;
    const bool fused = act_q != nullptr;
    if (!a->a || !a->b || !a->sfa || !a->sfb || !a->layout || !a->rows_used || (fused ? !act_scales : !a->d))
        return fail(MOE_ERR_INVALID, "a, b, sfa, sfb, layout, rows_used and the output must be non-NULL");
    if (!S->x_q || !S->x_scale || !S->ids || !S->pos || !S->send_order || !S->counts_local)
        return fail(MOE_ERR_INVALID, "send pointers must be non-NULL");
    if (a->G <= 0 || a->G != S->E_local || a->N <= 0 || a->K <= 0 || a->M <= 0 || a->K != S->H)
        return fail(MOE_ERR_INVALID, "G must equal E_local, K must equal H, M (capacity) positive");
    if (a->K % 128 || a->N % (fused ? 256 : 8)) return fail(MOE_ERR_INVALID, "K must be a multiple of 128, N of %d", fused ? 256 : 8);
    if (a->sf_format != MOE_SF_F32 || a->scatter_meta || a->accumulate || a->ldb)
        return fail(MOE_ERR_UNSUPPORTED, "the dispatching GEMM takes fp32 scales and writes plain output");
    if (!fused && (a->d_dtype != MOE_DTYPE_BF16 || a->ldd < a->N || a->ldd % 8)) return fail(MOE_ERR_INVALID, "d must be bf16 with ldd >= N, ldd %% 8 == 0");
    if (S->n_pairs < 0 || S->n_pairs > (1ll << 24) || S->top_k <= 0 || S->n_pairs % S->top_k)
        return fail(MOE_ERR_INVALID, "n_pairs must be a multiple of top_k and at most 2^24");
    const long long rec = ((long long)S->H + S->H / 32 + 4 + 15) & ~15ll;       // row, scales, return address
    if (rec > EP_SEND_RECORD_MAX) return fail(MOE_ERR_UNSUPPORTED, "H=%d: a token record must fit %d bytes", S->H, EP_SEND_RECORD_MAX);
    if (S->pitch < rec || S->pitch % 16 || a->lda != S->pitch) return fail(MOE_ERR_INVALID, "pitch must be >= H + H/32 + 4, a multiple of 16, and equal to lda");
    if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15) || (reinterpret_cast<uintptr_t>(S->x_q) & 15) ||
        (reinterpret_cast<uintptr_t>(fused ? act_q : a->d) & 15))
        return fail(MOE_ERR_INVALID, "a, b, x_q and the output must be 16-byte aligned");
    if ((long long)a->G * a->N > 0x7FFFFFFFll) return fail(MOE_ERR_INVALID, "row counts exceed 2^31-1");
    DeviceInfo* di = nullptr;
    rc = device_info(&di);
    if (rc != MOE_OK) return rc;
    CUtensorMap tmap_a, tmap_b;
    rc = encode_fp8_kmajor(&tmap_a, a->a, (uint64_t)a->M, (uint64_t)a->K, gg::BM, (uint64_t)a->lda);
    if (rc != MOE_OK) return rc;
    rc = encode_fp8_kmajor(&tmap_b, a->b, (uint64_t)a->G * a->N, (uint64_t)a->K, fused ? gg::FUSE_B_BOX_ROWS : gg::BN);
    if (rc != MOE_OK) return rc;
    GGParams p = {};
    p.sfa = a->sfa; p.sfa_sr = a->sfa_stride_row; p.sfa_sk = a->sfa_stride_kblk;
    p.sfb = a->sfb; p.layout = a->layout; p.rows_used = a->rows_used;
    p.d = a->d; p.ldd = a->ldd;
    p.G = a->G; p.M = a->M; p.N = a->N; p.K = a->K;
    p.rows_total = a->M;
    p.num_k_blocks = a->K / 128;
    p.nb128 = (a->N + 127) / 128;
    p.num_m_blocks = (a->M + gg::BM - 1) / gg::BM;
#ifdef B200MOE_DEV_TRACE
    if (const char* ev = getenv("B200MOE_GG_TRACE")) p.trace = reinterpret_cast<long long*>(strtoull(ev, nullptr, 10));
#endif
    if (fused) {
        p.inter = a->N / 2;
        p.num_n_blocks = p.inter / 128;
        p.act_q = static_cast<uint8_t*>(act_q);
        p.act_s = act_scales;
        p.act_ss_r = ss_row; p.act_ss_b = ss_blk;
        p.gate_first = gate_first ? 1 : 0;
    } else {
        p.num_n_blocks = (a->N + gg::BN - 1) / gg::BN;
    }
    EpSend& e = p.ep;
    for (int i = 0; i < EP_MAX_WORLD; ++i) {
        e.a[i] = static_cast<uint8_t*>(S->peers->a[i]);
        e.arrive[i] = S->peers->flags[i] ? S->peers->flags[i] + EP_ARRIVE_OFFSET : nullptr;
    }
    e.x = static_cast<const uint8_t*>(S->x_q); e.xs = S->x_scale; e.xs_r = S->xs_row; e.xs_b = S->xs_blk; e.pitch = S->pitch;
    e.ids = S->ids; e.pos = S->pos; e.order = S->send_order; e.expected = S->counts_local;
    e.n_pairs = (int)S->n_pairs; e.top_k = S->top_k; e.E_local = S->E_local; e.H = S->H; e.cap_rows = S->cap_rows; e.rank = S->rank;
    // every CTA must be resident (its sending warp's rows are awaited by other GPUs): a persistent grid of one CTA
    // per SM; CTAs beyond the tile count only send
    const int grid = di->num_sms;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (fused)
        gg_fp8_kernel<false, true, false, true><<<grid, gg::THREADS, gg::SMEM_BYTES_DISPATCH, st>>>(tmap_a, tmap_b, tmap_a, p, di->status);
    else
        gg_fp8_kernel<false, false, false, true><<<grid, gg::THREADS, gg::SMEM_BYTES_DISPATCH, st>>>(tmap_a, tmap_b, tmap_a, p, di->status);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_ep_combine(const moe_ep_peers* P, const int32_t* ids, const int32_t* pos, const float* w, void* out_bf16,
                   int32_t T, int32_t top_k, int32_t E_local, int32_t H, int32_t world, void* stream) {
    int rc = ep_check(P, 0, world);
    if (rc != MOE_OK) return rc;
    if (!ids || !pos || !w || !out_bf16) return fail(MOE_ERR_INVALID, "combine pointers must be non-NULL");
    if (H <= 0 || H % 8 || top_k <= 0 || top_k > 32) return fail(MOE_ERR_INVALID, "H must be a multiple of 8 and top_k in [1, 32]");
    if (T <= 0) return T == 0 ? MOE_OK : fail(MOE_ERR_INVALID, "T must be non-negative");
    ep_combine_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(ep_convert(P), ids, pos, w,
                                                                        static_cast<__nv_bfloat16*>(out_bf16), T, top_k,
                                                                        E_local, H);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

/* ---------------------------------------------------------------- allocation-free permutation plan */

// Scratch of moe_permute_plan_static: the per-chunk expert counters, kept in the library's own device
// image instead of caller memory.  128 KiB per GPU that loads the library, held until the process exits.
constexpr int kPlanStaticMaxInts = 32768;
static __device__ __align__(256) int g_plan_static_scratch[kPlanStaticMaxInts];

// The array's name is only a host-side handle; kernels need its device address, which is looked up
// once per device (with that device current) and cached.
static int plan_static_scratch(int** out) {
    static int* ptrs[64] = {};
    static std::mutex mu;
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MOE_ERR_INVALID, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        int* p = nullptr;
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_plan_static_scratch));
        if (p == nullptr) return fail(MOE_ERR_CUDA, "cudaGetSymbolAddress returned a NULL scratch address");
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return MOE_OK;
}

int moe_permute_plan_static(const int32_t* ids, int64_t n_pairs, int32_t e_lo, int32_t E_local, int32_t align,
                            int32_t cap_rows, int32_t* counts, int32_t* offsets, int32_t* pos, int32_t* src_pair,
                            int32_t* grouped_layout, void* stream) {
    int rc = check_plan_args(n_pairs, E_local, align, cap_rows);
    if (rc != MOE_OK) return rc;
    if (!ids || !counts || !offsets || !pos || !src_pair || !grouped_layout)
        return fail(MOE_ERR_INVALID, "all plan pointers must be non-NULL");
    const int64_t n_chunks64 = (n_pairs + PLAN_CHUNK - 1) / PLAN_CHUNK;
    if (n_chunks64 * (int64_t)E_local > kPlanStaticMaxInts)
        return fail(MOE_ERR_INVALID,
                    "moe_permute_plan_static: ceil(n_pairs/1024) * E_local = %lld exceeds the built-in scratch of %d "
                    "counters (e.g. 131072 pairs x 256 experts); use moe_permute_plan with caller workspace",
                    (long long)(n_chunks64 * E_local), kPlanStaticMaxInts);
    int* chunk_counts = nullptr;
    rc = plan_static_scratch(&chunk_counts);
    if (rc != MOE_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int n_chunks = (int)n_chunks64;
    const size_t hist_bytes = (size_t)32 * E_local * 4;
    // Nothing in the scratch has to start at zero: the count kernel writes every counter the later
    // kernels read, so contents left by an earlier call are simply overwritten.
    if (n_chunks > 0) {
        plan_count_kernel<<<n_chunks, PLAN_CHUNK, hist_bytes, st>>>(ids, n_pairs, e_lo, E_local, chunk_counts);
        CUDA_TRY(cudaGetLastError());
    }
    plan_scan_kernel<<<1, 256, (size_t)E_local * 4, st>>>(chunk_counts, n_chunks, E_local, align, counts, offsets);
    CUDA_TRY(cudaGetLastError());
    plan_place_kernel<<<n_chunks > 0 ? n_chunks : 1, PLAN_CHUNK, hist_bytes, st>>>(
        ids, n_pairs, e_lo, E_local, chunk_counts, counts, offsets, pos, src_pair, grouped_layout, cap_rows);
    CUDA_TRY(cudaGetLastError());
    return MOE_OK;
}

int moe_set_option(int32_t option, int32_t value) {
    if (option < 0 || option >= MOE_OPT_COUNT_) return fail(MOE_ERR_INVALID, "unknown option %d", option);
    bool ok = true;
    switch (option) {
        case MOE_OPT_GG_BLOCK_SCALED: ok = value == 0 || value == 1; break;
        case MOE_OPT_MX_TILE: ok = value >= MOE_MX_TILE_AUTO && value <= MOE_MX_TILE_PAIR_224; break;
        case MOE_OPT_ALPHA_PATH: ok = value >= MOE_ALPHA_PATH_AUTO && value <= MOE_ALPHA_PATH_MIXED; break;
        case MOE_OPT_ALPHA_GEMV_MAX_ROUTES: ok = value >= 0 && value <= 32768; break;
        case MOE_OPT_KG_MODE: ok = value >= MOE_KG_MODE_MN_MAJOR && value <= MOE_KG_MODE_PER_GROUP; break;
        case MOE_OPT_EP_WAIT_LIMIT_MS: ok = value >= 1 && value <= 60000; break;
    }
    if (!ok) return fail(MOE_ERR_INVALID, "value %d is out of range for option %d", value, option);
    g_options[option].store(value, std::memory_order_relaxed);
    return MOE_OK;
}

int moe_get_option(int32_t option, int32_t* value) {
    if (option < 0 || option >= MOE_OPT_COUNT_ || !value) return fail(MOE_ERR_INVALID, "unknown option %d or NULL value", option);
    *value = opt(option);
    return MOE_OK;
}

const char* moe_last_error(void) { return g_err; }
const char* moe_version(void) { return "b200moe 0.1 sm_100a"; }

}  // extern "C"
