/*
 * b200moe -- C ABI of the B200 (sm_100a) MoE grouped-FP8-GEMM hot path.
 *
 * Plain C: device pointers, sizes and strides only.  Every entry point returns
 * 0 on success and a negative code on failure; moe_last_error() then holds a
 * message for the calling thread.  All launches go to the stream passed in
 * (a cudaStream_t cast to void*, NULL = the legacy default stream) on the
 * CURRENT device of the calling thread, which must own the pointers.
 *
 * Citations name the interface of mlc-ai/TIRx-harness each entry point stands
 * in for (paths inside that project).
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)   /* the library is built with hidden visibility */
#endif

#define MOE_OK 0
#define MOE_ERR_INVALID (-1)   /* bad argument (shape, alignment, null pointer) */
#define MOE_ERR_CUDA (-2)      /* a CUDA runtime / driver call failed */
#define MOE_ERR_DEVICE (-3)    /* a kernel reported a device-side error (bounded wait ran out) */
#define MOE_ERR_UNSUPPORTED (-4)

#define MOE_DTYPE_BF16 0
#define MOE_DTYPE_F32 1

#define MOE_SF_F32 0            /* block scales as fp32 values */
#define MOE_SF_UE8M0_PACKED 1   /* block scales as UE8M0 bytes, four consecutive 128-K blocks per int32 */

/* Arguments of the m-grouped FP8 block-scaled GEMM  D_g = deq(A_g) * deq(B_g)^T.
 *   a       e4m3, K-major.  contiguous: [M, K];  masked: [G, M, K] with M = max rows per group
 *   b       e4m3 [G, N, K], K-major
 *   sfa     fp32, one scale per (row, 128-wide K block); element (row r, block kb) is
 *           sfa[r * sfa_stride_row + kb * sfa_stride_kblk]   (masked: r = g * M + row)
 *           -> row-major [rows, K/128] is (K/128, 1); MN-major [K/128, rows] is (1, rows)
 *   sfb     fp32 [G, ceil(N/128), K/128] row major: one scale per 128x128 block of B_g
 *   layout  contiguous: grouped_layout int32[M], group id per row, negative = padding row
 *           masked:     masked_m int32[G], number of valid rows of each group
 *   d       contiguous [M, N] / masked [G, M, N]; row stride ldd elements; bf16 (d_dtype =
 *           MOE_DTYPE_BF16, the workload's output type) or the unrounded fp32 accumulator
 *           (MOE_DTYPE_F32).  Only valid rows are written; padding / masked-out rows are left
 *           untouched.
 *   rows_used  contiguous layout only, may be NULL: device pointer to the number of leading rows of
 *           a/d that are in use (<= M).  Lets a fixed-capacity buffer be passed with M = capacity
 *           while the kernel only visits the rows a routing step actually filled.
 *   workspace  may be NULL.  If given (256-byte aligned, >= moe_gg_workspace_bytes), each call first
 *           checks on the device whether every scale is an exact power of two; if so the scales are
 *           applied inside the tensor core (block-scaled MMA, CTA pairs) instead of by per-K-block
 *           promotion -- same exact products, fp32 accumulation, about 1.5x faster.  Otherwise, and
 *           always without workspace, the promotion kernel runs.  The decision is taken per call on
 *           the device from the current scale values; nothing is cached between calls.
 *   lda     row pitch of a in bytes; 0 = K (dense).  A larger pitch (multiple of 16) lets rows carry a
 *           trailer, e.g. their own scales, as the expert-parallel receive buffer does.
 *   sf_format  MOE_SF_F32 (default, 0) or MOE_SF_UE8M0_PACKED: the scale format of the registered
 *           grouped_gemm/fp8 workload (evolution/tasks/grouped_gemm_fp8.yaml:16-19; packing as in
 *           tools/tests/numsim/corpus/kernels/gemm.py:252-263: byte j of a word = K block 4*word+j).
 *           Then sfa / sfb point to int32 words: word (row r, q) of A at sfa[r*sfa_stride_row + q*sfa_stride_kblk],
 *           word (group g, column n, q) of B at sfb[g*sfb_stride[0] + n*sfb_stride[1] + q*sfb_stride[2]]
 *           (B scales per column, as that format stores them).  Needs workspace; always takes the
 *           block-scaled-MMA path.
 *   ldb     row pitch of b in bytes; 0 = K (dense).  With lda it lets a K window of wider matrices be multiplied.
 *   accumulate  non-zero: d (fp32 only) is added to instead of overwritten (d += a*b^T), block-scaled path only.
 *   scatter_meta  contiguous layout, bf16 output only, may be NULL.  If given (int32 [M]), valid row r is not
 *           stored at d + r*ldd but at scatter_base[meta >> 24] + (meta & 0xFFFFFF)*ldd, meta = scatter_meta[r]:
 *           the expert-parallel down GEMM uses it to store every output row directly into the slot of the
 *           rank that owns the token (bases may be peer-mapped memory of other GPUs; plain stores).
 *   scatter_meta_stride  distance in int32 elements between the entries of consecutive rows (0 = 1: a dense array).
 *           The dispatching GEMM (moe_ep_gate_up_dispatch) leaves every row's return address inside its record, at
 *           byte H + H/32: pass that word of the first record with a stride of pitch / 4.
 *   mx_tile  tiling of the block-scaled kernels for THIS call (a MOE_MX_TILE_* value); 0 = the process-wide option
 *           MOE_OPT_MX_TILE.  (Measured on a Zipf-distributed batch of 64 groups, where CTA pairs multiply 15 % more
 *           rows than 128-row tiles would: the pairs are still 3 to 9 % faster, so the default does not look at the
 *           group sizes.)
 * Requirements: K % 128 == 0, N % 8 == 0, a/b 16-byte aligned, d 16-byte aligned, ldd % 8 == 0.
 */
typedef struct moe_gg_args {
    const void* a;
    const void* b;
    const float* sfa;
    int64_t sfa_stride_row;
    int64_t sfa_stride_kblk;
    const float* sfb;
    const int32_t* layout;
    void* d;
    int64_t ldd;
    int32_t G, M, N, K;
    int32_t d_dtype;
    const int32_t* rows_used;
    void* workspace;
    uint64_t workspace_bytes;
    const int32_t* scatter_meta;
    void* scatter_base[8];
    int32_t sf_format;
    int64_t sfb_stride[3];
    int64_t lda;
    int64_t ldb;
    int32_t accumulate;
    int64_t scatter_meta_stride;
    int32_t mx_tile;
} moe_gg_args;

/* Scratch for the power-of-two-scale path (rows_total = M contiguous, G*M masked).  With
 * args.workspace = NULL the GEMM always takes the promotion path. */
size_t moe_gg_workspace_bytes(int32_t G, int64_t rows_total, int32_t N, int32_t K);

/* Contiguous layout.  Stands in for the timed call of the registered workload
 * `grouped_gemm/fp8`: DeepGEMM m_grouped_fp8_gemm_nt_contiguous as launched by
 * evolution/benchmark/flashinfer_bench_evolve/tasks/grouped_gemm_fp8/baseline.py:30-42, with the
 * tensor contract of evolution/tasks/grouped_gemm_fp8.yaml:15-25. */
int moe_gg_fp8_contiguous(const moe_gg_args* args, void* stream);

/* Masked layout.  Stands in for the masked grouped kernel exercised by
 * tools/tests/numsim/corpus/kernels/gemm.py:705-795 (deepgemm_sm100_m_grouped_fp8_gemm_masked). */
int moe_gg_fp8_masked(const moe_gg_args* args, void* stream);


/* ---- k-grouped layout (weight-gradient shape) ------------------------------------------------ */
/* D_g [M, N] (fp32) += A_g^T * B_g for g < G, where group g owns the K rows [sum(ks[:g]), +ks[g]) of the
 * MN-major operands a e4m3 [K_total, M] and b e4m3 [K_total, N]; scales are the packed UE8M0 words of that
 * layout, one word per (row m or n, four 128-K blocks of one group): sfa int32 [sum(ceil(ks[g]/512)), M],
 * sfb likewise [.., N]; d fp32 [G, M, N] is accumulated into.  Stands in for the k-grouped entry of the
 * reference's DeepGEMM kernel family (deepgemm_sm100_k_grouped_fp8_gemm_contiguous as exercised by
 * tools/tests/numsim/corpus/kernels/gemm.py:610-702: per-group K cursors, MN-major operands, fp32 accumulation
 * onto the existing D).  `ks` is a HOST array (the shapes of a weight gradient are known on the host);
 * every ks[g] must be a multiple of 128, M % 128 == 0, N % 16 == 0.  Up to 64 groups run as ONE launch of the
 * block-scaled kernel that reads a and b as MN-major operands where they are; more groups run one launch per
 * group on K-major copies made in the workspace.  workspace: moe_kg_workspace_bytes, 256-byte aligned. */
typedef struct moe_kg_args {
    const void* a;                /* e4m3 [K_total, M] */
    const void* b;                /* e4m3 [K_total, N] */
    const int32_t* sfa;           /* packed UE8M0 [scale_rows, M] */
    const int32_t* sfb;           /* packed UE8M0 [scale_rows, N] */
    float* d;                     /* fp32 [G, M, N], accumulated into */
    const int32_t* ks;            /* host pointer, int32 [G] */
    int32_t G, M, N;
    int64_t K_total;
    void* workspace;
    uint64_t workspace_bytes;
} moe_kg_args;
size_t moe_kg_workspace_bytes(int32_t M, int32_t N, int64_t K_total);
int moe_kg_fp8_contiguous(const moe_kg_args* args, void* stream);


/* ---- memory-bound stages around the GEMMs ------------------------------------------------- */

/* Per-token 1x128 activation quantisation: s = max(amax,1e-8)/448, q = e4m3(clamp(x/s, +-448)),
 * true division.  x bf16 [rows, cols] -> q e4m3 [rows, cols], scale (r, block b) stored at
 * scales[r*ss_row + b*ss_blk].  Stands in for alphamoe/baseline.py:14-26 (`_quantize`) and the
 * rule `_quantize_per_token_group` of tasks/alphamoe/definition.json. */
int moe_quant_1x128(const void* x_bf16, void* q, float* scales, int64_t ss_row, int64_t ss_blk,
                    int32_t rows, int32_t cols, void* stream);

/* Fused SiLU(gate)*up + 1x128 FP8 requantisation between the gate_up and down GEMMs.
 * gate_up bf16 [rows, 2*inter]; gate_first != 0: gate = columns [0, inter) (alphamoe/definition.json
 * `_reference_quantized`), else gate = [inter, 2*inter) (moe/definition.json: silu(G1[:, I:]) * G1[:, :I]).
 * layout (nullable): rows with a negative entry are skipped.  q e4m3 [rows, inter]. */
int moe_silu_mul_requant(const void* gate_up_bf16, void* q, float* scales, int64_t ss_row, int64_t ss_blk,
                         const int32_t* layout, int32_t rows, int32_t inter, int32_t gate_first, void* stream);

/* Softmax-of-logits top-k routing (ties -> lowest expert index; weights = selected probabilities
 * renormalised to sum 1; ids in descending score order).  logits f32 [T, E], E <= 512, top_k <= 32.
 * The routing rule of the MoE-layer workload; takes the place of the routing block inside
 * trtllm_fp8_block_scale_moe as called at tasks/moe/baseline.py:31-51. */
int moe_route_topk(const float* logits, int32_t* ids, float* weights, int32_t T, int32_t E, int32_t top_k,
                   void* stream);

/* DeepSeek-V3 "no-aux" routing, the routing block of the registered `moe` workload
 * (tasks/moe/definition.json, "2) No-aux routing"; called inside trtllm_fp8_block_scale_moe with
 * routing_method_type=2, n_group=8, topk_group=4 at tasks/moe/baseline.py:31-51): s = sigmoid(logit),
 * selection on s + bias by groups of 32 experts (sum of the two best per group, topk_group groups kept, top_k
 * experts among them), weight = s / (sum of selected s + 1e-20) * routed_scaling_factor.  bias: E values,
 * bf16 (MOE_DTYPE_BF16, the task's dtype) or f32.  E = 32 * n_group, n_group <= 16. */
int moe_route_deepseek(const float* logits, const void* bias, int32_t bias_dtype, int32_t* ids, float* weights, int32_t T,
                       int32_t E, int32_t n_group, int32_t topk_group, int32_t top_k, float routed_scaling_factor,
                       void* stream);

/* Stable permutation plan into the contiguous grouped layout for local experts
 * [e_lo, e_lo + E_local): counts[E_local], offsets[E_local+1] (each expert padded to `align` rows,
 * offsets[E_local] = rows in use), pos[n_pairs] (destination row of pair p = t*top_k + j, -1 if
 * not local), src_pair[cap_rows] (pair stored in a row, -1 on padding) and
 * grouped_layout[cap_rows] (local expert id, -1 on padding).  Pairs keep their order inside an
 * expert.  cap_rows >= n_pairs rounded up to align + E_local*align always suffices.
 * Replaces the permute stage inside trtllm_fp8_block_scale_moe (tasks/moe/baseline.py:31-51);
 * the counts equal bincount(routes) as the reference checks for its receive counters
 * (tools/tests/numsim/corpus/kernels/deepgemm.py:1444-1491). */
size_t moe_permute_workspace_bytes(int64_t n_pairs, int32_t E_local);
int moe_permute_plan(const int32_t* ids, int64_t n_pairs, int32_t e_lo, int32_t E_local, int32_t align,
                     int32_t cap_rows, int32_t* counts, int32_t* offsets, int32_t* pos, int32_t* src_pair,
                     int32_t* grouped_layout, void* workspace, size_t workspace_bytes, void* stream);

/* Allocation-free form of moe_permute_plan.  It has no counterpart in the reference.
 * Some hosts cannot give this library device memory at call time: a serving engine that reserved the
 * whole GPU for its own pool at start-up, or a plugin host that forbids driver allocations once it is
 * running (cudaMalloc may fail there, and it stalls the device while it runs).  For them the plan's
 * only scratch, the per-chunk expert counters, lives in a 128 KiB array inside the library's device
 * image; the call itself never allocates (no cudaMalloc/cudaFree, no torch or other allocating
 * routine).  Inputs and outputs are still the caller's, with the same meaning as in moe_permute_plan.
 * Limit: ceil(n_pairs / 1024) * E_local <= 32768 (for example 131072 pairs x 256 experts); larger
 * requests return MOE_ERR_INVALID and leave the outputs untouched.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call during start-up, before any stream capture begins.
 * All calls on a device share the one array.  Nothing in it has to be cleared between calls (every
 * counter that is read is written first by the same call), but two calls whose kernels overlap on
 * the GPU -- different streams, or different host threads -- race on it: serialise them.
 * Every GPU that loads the library keeps the 128 KiB until the process exits. */
int moe_permute_plan_static(const int32_t* ids, int64_t n_pairs, int32_t e_lo, int32_t E_local, int32_t align,
                            int32_t cap_rows, int32_t* counts, int32_t* offsets, int32_t* pos, int32_t* src_pair,
                            int32_t* grouped_layout, void* stream);

/* Row gather: for each row with src_pair >= 0 copies token (src_pair / top_k)'s e4m3 row (H bytes)
 * and its H/128 scales.  Source scale (t, b) at x_scale[t*xs_row + b*xs_blk]; destination
 * (row, b) at a_scale[row*as_row + b*as_blk]. */
int moe_permute(const void* x_q, const float* x_scale, int64_t xs_row, int64_t xs_blk, const int32_t* src_pair,
                int32_t top_k, void* a, float* a_scale, int64_t as_row, int64_t as_blk, int32_t rows, int32_t H,
                void* stream);

/* Weighted combine: out[t,:] = bf16( sum_j w[t,j] * y[pos[t,j],:] ), fp32 multiply-then-add in
 * slot order, pos < 0 skipped: the fp32 weighted accumulation of tasks/moe/definition.json
 * (output.index_add_(0, token_idx, O * w_tok) ... .to(bfloat16)). */
int moe_combine(const void* y_bf16, const int32_t* pos, const float* w, void* out_bf16, int32_t T, int32_t top_k,
                int32_t H, void* stream);

/* ---- one MoE layer on one GPU --------------------------------------------------------------- */

/* route -> plan -> gather -> gate_up grouped GEMM -> SiLU*mul requant -> down grouped GEMM ->
 * combine, all on `stream`, using caller-provided workspace (moe_workspace_bytes).  Mirrors the
 * candidate contract of the registered `moe` workload (tasks/moe/benchmark.py:143-182:
 * setup(data, T) -> callable writing the preallocated bf16 output).
 *   x_q e4m3 [T,H], x_scale f32 at [t*xs_stride_row + b*xs_stride_blk]
 *   logits f32 [T, E_global]: softmax top-k routing, or DeepSeek-V3 no-aux routing when routing_bias is
 *   given (the registered `moe` task; only experts [e_lo, e_lo+E) contribute, as with its
 *   local_expert_offset); if logits is NULL, topk_ids/topk_weights [T, top_k] are used as they are
 *   w13 e4m3 [E, 2I, H], w13_scale f32 [E, 2I/128, H/128]; w2 e4m3 [E, H, I], w2_scale f32 [E, H/128, I/128]
 *   E local experts = global ids [e_lo, e_lo+E); out bf16 [T, H] */
typedef struct moe_layer_args {
    const void* x_q;
    const float* x_scale;
    int64_t xs_stride_row, xs_stride_blk;
    const float* logits;
    const int32_t* topk_ids;
    const float* topk_weights;
    const void* w13;
    const float* w13_scale;
    const void* w2;
    const float* w2_scale;
    void* out;
    void* workspace;
    uint64_t workspace_bytes;
    int32_t T, H, I, E, E_global, e_lo, top_k, align, gate_first;
    int32_t fuse_act;        /* != 0: SiLU*mul requant inside the gate_up GEMM (no gate_up matrix in memory) */
    const void* routing_bias; /* bf16 [E_global] or NULL.  Non-NULL selects DeepSeek-V3 no-aux routing on `logits` */
    int32_t n_group, topk_group;   /* 0 = the task's 8 and 4 */
    float routed_scaling_factor;
} moe_layer_args;

size_t moe_workspace_bytes(int32_t T, int32_t H, int32_t I, int32_t E, int32_t top_k, int32_t align);
int moe_layer_forward(const moe_layer_args* args, void* stream);

/* Where moe_layer_forward keeps its intermediates inside the workspace (for inspection / tests). */
typedef struct moe_layer_view {
    int32_t *ids, *counts, *offsets, *pos, *src_pair, *grouped_layout;
    float *weights, *s1, *s2;
    void *a1, *g1, *a2, *y;
    int64_t cap_rows;
} moe_layer_view;
int moe_layer_workspace_view(void* workspace, int32_t T, int32_t H, int32_t I, int32_t E, int32_t top_k,
                             int32_t align, moe_layer_view* view);

/* ---- decode-regime layer from bf16 activations and preselected routes ------------------------ */
/* Replaces the timed callable of the reference's `alphamoe` task: `setup(data, M)` of
 * candidates/alphamoe/<name>/solution.py (evolution/tasks/alphamoe.yaml:17-47; data keys and shapes
 * flashinfer_bench_evolve/tasks/alphamoe/benchmark.py, oracle `run` in its definition.json).  Everything the
 * task times is inside the call: 1x128 quantisation of hidden_states (s = max(amax,1e-8)/448, true
 * division), expert alignment, gate_up GEMM on rows stacked [gate; up] (fp32 kept), SiLU(gate)*up, 1x128
 * requantisation, down GEMM, and the reduction: each route's down contribution times
 * fp32(topk_weight * routed_scaling_factor) is rounded to bf16 and added to a zero bf16 accumulator with a
 * rounding per update, experts in ascending id (definition.json `_reference_quantized`).
 * Limits: I == 128 (one down contribution per route, as in the task's rows), H % 128 == 0, E <= 1024,
 * top_k <= 32, M * top_k <= 32768, ids of one token distinct (an expert that receives more than M routes
 * raises status bit 4096 and the excess routes are dropped).  The call launches on `stream`, allocates
 * nothing and never synchronises (graph-capturable).                                             */
typedef struct moe_alpha_args {
    const void* hidden;           /* bf16 [M, H] */
    const int32_t* topk_ids;      /* [M, top_k]; ids outside [0, E) are skipped */
    const float* topk_weights;    /* [M, top_k] */
    const void* w13;              /* e4m3 [E, 2I, H], rows [gate; up] */
    const float* w13_scale;       /* [E, 2I/128, H/128] */
    const void* w2;               /* e4m3 [E, H, I] */
    const float* w2_scale;        /* [E, H/128, I/128] */
    void* out;                    /* bf16 [M, H], overwritten */
    int32_t M, H, I, E, top_k;
    float routed_scaling_factor;
    void* workspace;              /* moe_alpha_workspace_bytes(M, H, I, E, top_k), 256-byte aligned */
    uint64_t workspace_bytes;
} moe_alpha_args;
size_t moe_alpha_workspace_bytes(int32_t M, int32_t H, int32_t I, int32_t E, int32_t top_k);
int moe_alpha_forward(const moe_alpha_args* args, void* stream);

/* Where moe_alpha_forward keeps its intermediates (for inspection / tests).  Expert e owns rows
 * [e*max_m, e*max_m + counts[e]) of a1/g1/a2/d2; rowpos[p] is the row of route p (-1 = skipped);
 * s1/s2 are MN-major: scale of (row, block b) at s[b*E*max_m + row].                             */
typedef struct moe_alpha_view {
    int32_t *counts, *rowpos;
    float *s1, *s2, *g1, *d2;     /* g1 fp32 [E*max_m, 2I], d2 fp32 [E*max_m, H] */
    void *a1, *a2;                /* e4m3 [E*max_m, H], [E*max_m, I] */
    int64_t max_m;
} moe_alpha_view;
int moe_alpha_workspace_view(void* workspace, int32_t M, int32_t H, int32_t I, int32_t E, int32_t top_k,
                             moe_alpha_view* view);

/* ---- expert parallelism over NVLink peer memory --------------------------------------------- */
/* The reference has no multi-GPU path: it emulates expert parallelism on one GPU through
 * `local_expert_offset` (tasks/moe/definition.json, inputs `local_expert_offset`; offsets 0..224 in
 * tasks/moe/workload.jsonl).  These entry points are the real exchange for that sharding: rank r owns
 * experts [r*E_local, (r+1)*E_local) and a slice of the tokens, one process per GPU.            */

/* Device memory that can be mapped by the other ranks of the node (CUDA IPC).  alloc zero-fills. */
int moe_ipc_alloc(size_t bytes, void** ptr);
int moe_ipc_free(void* ptr);
int moe_ipc_get_handle(void* ptr, void* handle64);         /* 64-byte handle to send to the peers */
int moe_ipc_open(const void* handle64, void** ptr);        /* map a peer's allocation */
int moe_ipc_close(void* ptr);

/* Peer table: entry i = rank i's buffers as mapped in THIS process (own buffers at i == rank).
 *   a      cap_rows records of `pitch` bytes in the contiguous grouped layout: H e4m3 bytes, then the row's
 *          H/128 fp32 scales (pitch >= H + H/32, multiple of 16)
 *   sa     = a + H: scales of (row r, block b) at sa[r*pitch/4 + b]
 *   y      bf16 [cap_rows, H]       down-GEMM output rows
 *   counts int32 [world, E_total]   row s = number of pairs rank s routes to each expert
 *   flags  int32 [64 + E_local]     [0, world): barrier epochs; [64, 64 + E_local): arrival counters of the local experts
 *   meta   int32 [cap_rows]         (source rank << 24) | source pair index of each received row           */
typedef struct moe_ep_peers {
    void* a[8];
    float* sa[8];
    const void* y[8];
    int32_t* counts[8];
    int32_t* flags[8];
    int32_t* meta[8];
} moe_ep_peers;

/* Cross-GPU barrier on `stream`: publishes `epoch` (strictly increasing per call) to every peer and
 * waits, at most MOE_OPT_EP_WAIT_LIMIT_MS (2 s by default), for theirs; a wait that runs out sets bit 16 of the
 * device status word (moe_device_status) instead of hanging, and the kernel returns. */
int moe_ep_barrier(const moe_ep_peers* peers, int32_t rank, int32_t world, int32_t epoch, void* stream);

size_t moe_ep_workspace_bytes(int64_t n_pairs, int32_t E_total);

/* Step 1 (before the first barrier): count this rank's pairs per global expert (my_counts[E_total]) and
 * store them into row `rank` of every peer's counts table. */
int moe_ep_count_publish(const moe_ep_peers* peers, const int32_t* ids, int64_t n_pairs, int32_t rank, int32_t world,
                         int32_t E_total, int32_t* my_counts, void* workspace, size_t workspace_bytes, void* stream);

/* Step 2 (after that barrier): from the gathered counts derive the receive side (counts_local[E_local],
 * offsets[E_local+1], grouped_layout[cap_rows]) and the send side (dst_base[E_total], pos[n_pairs] =
 * destination row of every pair inside its owner's buffer; rows are ordered by source rank, then by pair
 * order, so the result is independent of timing).  send_order (int32 [n_pairs], may be NULL): this rank's pairs in
 * the order moe_ep_gate_up_dispatch sends them -- by local expert index first, destination rank second, pair order
 * inside -- so that every rank's first expert is complete first.  `workspace` must be the one step 1 used. */
int moe_ep_plan(const moe_ep_peers* peers, const int32_t* ids, int64_t n_pairs, int32_t rank, int32_t world,
                int32_t E_total, int32_t E_local, int32_t align, int32_t cap_rows, int32_t* counts_local,
                int32_t* offsets, int32_t* grouped_layout, int32_t* dst_base, int32_t* pos, int32_t* send_order,
                void* workspace, size_t workspace_bytes, void* stream);

/* Dispatch all-to-all fused with the permutation: every pair's e4m3 row and scales are stored directly
 * into the owner rank's grouped-layout buffers, together with the row's return address (meta). */
int moe_ep_dispatch(const moe_ep_peers* peers, const void* x_q, const float* x_scale, int64_t xs_row, int64_t xs_blk,
                    const int32_t* ids, const int32_t* pos, int64_t n_pairs, int32_t top_k, int32_t E_local, int32_t H,
                    int32_t cap_rows, int64_t pitch, int32_t rank, int32_t world, void* stream);

/* gate_up grouped GEMM that carries the dispatch all-to-all itself (ONE kernel: the transfer overlaps the GEMM tile
 * by tile and needs neither moe_ep_dispatch nor the barrier behind it).  One warp of every CTA stores this rank's
 * token records into the owners' receive buffers in `send_order`, and counts each row into the owner's arrival
 * counter of its expert once the store has completed (a record = H e4m3 bytes, H/128 fp32 scales, then the row's
 * return address (rank << 24) | pair as one int32: pitch >= H + H/32 + 4); the GEMM's loader warps wait, per expert and with the usual
 * 2 s bound, until counts_local[expert] rows have arrived, then multiply them.  The counters live at
 * peers->flags[r] + 64 (int32 [E_local]); moe_ep_count_publish clears them at the start of every forward.
 *   gemm   the gate_up GEMM over this rank's receive buffer exactly as moe_gg_fp8_contiguous would get it
 *          (a = peers->a[rank], lda = pitch, sfa = peers->sa[rank], rows_used = offsets + E_local, G = E_local,
 *          M = cap_rows, fp32 scales, bf16 d); no workspace: the promotion kernel runs
 *   act_q  NULL: plain bf16 output to gemm->d.  Non-NULL: SiLU*mul + 1x128 requant in the epilogue, as
 *          moe_gg_fp8_gate_up_act (then act_scales / ss_row / ss_blk / gate_first as there)
 * Every rank of the group must call it in the same forward (the waits are for the other ranks' sends).  No peer
 * memory is ever read: peer traffic is bulk stores, plain stores and reductions.  The reference has no multi-GPU
 * path; this is the exchange behind its single-GPU `local_expert_offset` emulation. */
typedef struct moe_ep_send_args {
    const moe_ep_peers* peers;
    const void* x_q;                /* e4m3 [T_local, H] */
    const float* x_scale;           /* scale of (t, block b) at x_scale[t*xs_row + b*xs_blk] */
    int64_t xs_row, xs_blk;
    const int32_t* ids;             /* [n_pairs] */
    const int32_t* pos;             /* [n_pairs], from moe_ep_plan */
    const int32_t* send_order;      /* [n_pairs], from moe_ep_plan */
    const int32_t* counts_local;    /* [E_local], from moe_ep_plan */
    int64_t n_pairs;
    int64_t pitch;
    int32_t top_k, E_local, H, cap_rows, rank, world;
} moe_ep_send_args;
int moe_ep_gate_up_dispatch(const moe_gg_args* gemm, const moe_ep_send_args* send, void* act_q, float* act_scales,
                            int64_t ss_row, int64_t ss_blk, int32_t gate_first, void* stream);

/* Combine all-to-all fused with the weighted sum: each token loads its top_k expert rows from the owners'
 * y buffers and accumulates w * row in fp32 (slot order), writing bf16. */
int moe_ep_combine(const moe_ep_peers* peers, const int32_t* ids, const int32_t* pos, const float* w, void* out_bf16,
                   int32_t T, int32_t top_k, int32_t E_local, int32_t H, int32_t world, void* stream);

/* gate_up grouped GEMM (contiguous layout, N = 2*inter) whose epilogue applies SiLU(gate)*up to the fp32
 * accumulators and requantises to e4m3 with 1x128 scales, writing act_q [M, inter] and
 * act_scales[(row)*ss_row + (block)*ss_blk]; the gate_up matrix is never stored (args->d is ignored).
 * This is the "fused SiLU-mul-FP8 requant between the two GEMMs": same rule as moe_silu_mul_requant
 * (alphamoe/definition.json `_reference_quantized`: gate_up and SwiGLU stay fp32 up to the requant),
 * gate_first as there.  Requires N % 256 == 0. */
int moe_gg_fp8_gate_up_act(const moe_gg_args* args, void* act_q, float* act_scales, int64_t ss_row, int64_t ss_blk,
                           int32_t gate_first, void* stream);

/* ---- process-wide modes ----------------------------------------------------------------------- */
/* None is needed for normal use: the defaults are the measured-fastest choices.  Each mode exists because a
 * test or a measurement selects it; they replace nothing in the reference (its candidates are single kernels).
 * Values are read once per call, so a change applies from the next call of any thread. */
#define MOE_OPT_GG_BLOCK_SCALED 0        /* 1 (default): power-of-two scales take the block-scaled-MMA kernels when
                                          * workspace is given; 0: always the promotion kernel */
#define MOE_OPT_MX_TILE 1                /* block-scaled kernel: AUTO = CTA pairs with 240-column tiles and two
                                          * accumulators for the contiguous layout, one CTA per tile for the masked layout */
#define MOE_MX_TILE_AUTO 0
#define MOE_MX_TILE_PAIR 1               /* CTA pairs, 256-column tiles, one accumulator (measurement variant) */
#define MOE_MX_TILE_SINGLE 2
#define MOE_MX_TILE_PAIR_240 3           /* CTA pairs, column tiles of at most 240 (balanced in units of 16), two accumulators */
#define MOE_MX_TILE_PAIR_224 4           /* CTA pairs, column tiles of at most 224, two accumulators (measurement variant) */
#define MOE_OPT_ALPHA_PATH 2             /* decode-regime layer: AUTO = two CUDA-core kernels up to the route
                                          * threshold, else swapped-operand tensor-core kernels; the others force
                                          * the tensor-core pipeline and choose the tiling of its two projections */
#define MOE_ALPHA_PATH_AUTO 0
#define MOE_ALPHA_PATH_SWAP 1
#define MOE_ALPHA_PATH_MASKED 2          /* both projections as masked-layout grouped GEMMs */
#define MOE_ALPHA_PATH_MIXED 3           /* masked gate_up, swapped down */
#define MOE_OPT_ALPHA_GEMV_MAX_ROUTES 3  /* largest M*top_k that takes the CUDA-core kernels (default 160, 0 = never) */
#define MOE_OPT_KG_MODE 4                /* k-grouped GEMM */
#define MOE_KG_MODE_MN_MAJOR 0           /* default: one launch, operands read MN-major as the caller has them */
#define MOE_KG_MODE_TRANSPOSE 1          /* one launch on K-major copies made by a transposing pre-pass */
#define MOE_KG_MODE_PER_GROUP 2          /* one launch per group (what more than 64 groups always get) */
#define MOE_OPT_EP_WAIT_LIMIT_MS 5       /* bound of the cross-GPU flag waits of moe_ep_barrier, 1..60000 ms (default 2000) */
#define MOE_OPT_COUNT_ 6
int moe_set_option(int32_t option, int32_t value);
int moe_get_option(int32_t option, int32_t* value);

/* Reads (and clears) the device-side status word of the current device; synchronises the
 * stream first.  0 = no kernel reported a problem.  Non-zero: a bounded wait inside a kernel ran
 * out (value encodes which) -- the failure surface that replaces a hang; the reference reports
 * failures as Python exceptions (benchmark_common.py:1013-1020), the host wrapper raises. */
int moe_device_status(int32_t* status_out, void* stream);

/* Message describing the last failure on the calling thread ("" if none). */
const char* moe_last_error(void);

/* Library / build description, e.g. "b200moe 0.1 sm_100a". */
const char* moe_version(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
