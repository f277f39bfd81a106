/*
 * dgb200 -- C ABI of the B200 (sm_100a) block-scaled FP8/FP4 GEMM library.
 *
 * This is the boundary a host in another language binds to.  Each entry point
 * names the interface of the reference crate (idrees2516/deepgemm-rust, paths
 * relative to that crate) it stands in for.  All pointers named "device" are
 * raw CUDA device addresses; nothing here takes or returns a framework type.
 * Work is enqueued on the context's stream and the call returns without
 * synchronising, like the reference.  Every function returns a dg_status;
 * dg_last_error() gives the message of the calling thread's last failure.
 *
 * There is no CPU fallback: without a CUDA device dg_ctx_create fails.
 */
#ifndef DGB200_H_
#define DGB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* deepgemm/src/types.rs:9-21 (DgError) plus a code for a device-side wait that ran out. */
typedef enum {
    DG_OK = 0,
    DG_ERR_DRIVER = 1,
    DG_ERR_SHAPE = 2,
    DG_ERR_UNSUPPORTED = 3,
    DG_ERR_TIMEOUT = 4
} dg_status;

typedef struct dg_ctx dg_ctx;

/* deepgemm/src/device.rs:40-56 (DgContext::new): one device, one stream. */
int dg_ctx_create(int ordinal, dg_ctx** out);
/* Same, adopting a stream the caller owns (e.g. the current stream of a tensor library). */
int dg_ctx_create_on_stream(int ordinal, void* cuda_stream, dg_ctx** out);
int dg_ctx_destroy(dg_ctx* ctx);
/* device.rs:129 (sync).  Also reports DG_ERR_TIMEOUT if a kernel gave up on a wait. */
int dg_ctx_sync(dg_ctx* ctx);
/* device.rs:124 (num_sms) */
int dg_ctx_num_sms(const dg_ctx* ctx, int* out);
void* dg_ctx_stream(const dg_ctx* ctx);
int dg_ctx_set_stream(dg_ctx* ctx, void* cuda_stream);
/* Reads the device status word without synchronising the stream first (the caller has). */
int dg_ctx_check_status(dg_ctx* ctx);
const char* dg_last_error(void);

/* deepgemm/src/ops_sm100.rs:33-45 (LpOperand).  data: (rows, ld) K-major e4m3 bytes, or packed
 * e2m1 with ld counted in logical elements; sf: packed UE8M0 words, see dg_sf_words. */
typedef struct {
    const void* data;     /* device */
    const uint32_t* sf;   /* device */
    uint32_t rows, k, ld;
    uint32_t bits;        /* 8 = e4m3, 4 = packed e2m1 */
    uint32_t gran_k;      /* 32 or 128 */
    uint32_t major_mn;    /* 0: K-major, (rows, ld) with ld >= k.  1 (e4m3 only): MN-major, (k, ld) bytes per group with ld >= rows and
                           * ld a multiple of 16: element (row r, k) at data[(group * k_total + k) * ld + r] (ops_sm100.rs:336-362) */
    size_t data_len;      /* bytes available at data */
    size_t sf_len;        /* words available at sf */
} dg_lp_operand;

/* ops_sm100.rs:95-110 (Sm100Out) */
/* DG_OUT_SWIGLU_FP8 (no counterpart as one call in the reference: moe.rs:254-296 runs the gate/up GEMM, then
 * deepgemm_silu_mul_bf16, and would then have to quantise): b holds, per group, n gate rows followed by n up rows
 * (b.rows = groups * 2n); the output is e4m3(silu(gate) * up), (rows, n) bytes at buf, with one UE8M0 scale per 32
 * columns in sfd, laid out as for DG_OUT_FP8 -- i.e. the next GEMM's A operand with gran_k = 32.  The gate and up products
 * are rounded to bf16 before the activation, as the unfused sequence does.  e4m3 operands, per-128 weight scales,
 * n a multiple of 128.  Exercised through the dense and the contiguous grouped entry points. */
enum { DG_OUT_BF16 = 0, DG_OUT_F32 = 1, DG_OUT_FP8 = 2, DG_OUT_SWIGLU_FP8 = 3 };
typedef struct {
    int kind;
    void* buf;            /* device; (rows, ld) elements of the kind */
    uint32_t ld;
    uint32_t* sfd;        /* device; DG_OUT_FP8 only: (ceil(n/128) [* groups], align4(m)) words */
    size_t buf_len;       /* elements available at buf */
    size_t sfd_len;       /* words available at sfd */
} dg_out;

/* ops_sm100.rs:114-131 (Sm100Epilogue) */
typedef struct {
    float alpha;
    int has_alpha;
    int accumulate;       /* D += A.B^T (dense, masked and batched calls; bf16 or f32 outputs; not with alpha) */
    uint32_t tc_util;     /* tensor-core duty cycle in percent (cuda/bf16_gemm_sm100.rs:358-371): below 100 the UMMA warp pauses after
                             every k-block for (100 - tc_util) / tc_util of that k-block's tensor time; 0 or 100 = no pause */
} dg_epilogue;

/* ops_sm100.rs:719 (fp8_fp4_gemm_dev): D[m,n] = alpha * A[m,k] . B[n,k]^T */
int dg_fp8_fp4_gemm(dg_ctx* ctx, const dg_lp_operand* a, const dg_lp_operand* b, const dg_out* out, const dg_epilogue* epi);

/* ops_sm100.rs:893 (bf16_gemm_dev; ops.rs:769 bf16_gemm_nt_dev routes here on Blackwell): D[m,n] = A[m,k] . B[n,k]^T
 * with bf16 K-major operands (leading dimensions in elements, multiples of 8), f32 accumulation, bf16 or f32
 * output; alpha and accumulate as for the FP8 GEMM.  Same kernel skeleton with kind::f16 UMMAs and no scale path. */
int dg_bf16_gemm(dg_ctx* ctx, const uint16_t* a, uint32_t a_ld, uint32_t m, const uint16_t* b, uint32_t b_ld, uint32_t n, uint32_t k,
                 const dg_out* out, const dg_epilogue* epi);

/* ops_sm100.rs:759 (m_grouped_fp8_fp4_gemm_contiguous_dev).  a: (m_total, k) arena, every group
 * starts at a multiple of the mk alignment; m_indices (device, m_total int32): group of each
 * row, -1 for padding; b.rows = num_groups * n.  The group-end table is built in a scratch
 * buffer the context owns. */
int dg_m_grouped_fp8_fp4_gemm_contiguous(dg_ctx* ctx, const dg_lp_operand* a, const int32_t* m_indices, const dg_lp_operand* b,
                                         const dg_out* out, uint32_t num_groups, const dg_epilogue* epi);
/* Same with a caller-built group-end table (device, num_groups uint32, non-decreasing):
 * group_ends[g] = one past the last row of group g (what dg_group_ends_from_m_indices writes). */
int dg_m_grouped_fp8_fp4_gemm_contiguous_ends(dg_ctx* ctx, const dg_lp_operand* a, const uint32_t* group_ends, const dg_lp_operand* b,
                                              const dg_out* out, uint32_t num_groups, const dg_epilogue* epi);

/* No counterpart in the reference.  The contiguous grouped GEMM for hosts that must not touch the
 * device allocator once they are running -- for instance a serving process that handed every byte of
 * device memory to its own pool at start-up (so a cudaMalloc can only fail), or a latency-critical
 * loop where the implicit device-wide synchronisation of cudaMalloc / cudaFree would stall every
 * stream.  It needs no dg_ctx and allocates nothing, neither on the device nor through any
 * allocating library routine: the group-end table it builds from m_indices, and the record its
 * kernels write if a bounded wait runs out, live in an array that is part of the library image
 * (about 16.3 KB on every GPU that loads the library, held until the process exits).
 *   - num_groups may be at most DG_STATIC_MAX_GROUPS; larger values return DG_ERR_SHAPE.
 *   - The first call on a device looks up the array's device address and opts every kernel this
 *     path can launch into the large shared-memory carve-out (once, with that device current).
 *     Make that first call before any stream capture.
 *   - Every call on a device uses the same array, which still holds the previous call's table; the
 *     call clears the entries it needs on `cuda_stream` first.  Two calls whose GPU work can overlap
 *     (different streams, or different threads) race on it: keep them on one stream.
 *   - Arguments and results are those of dg_m_grouped_fp8_fp4_gemm_contiguous; `cuda_stream` is the
 *     cudaStream_t to enqueue on. */
#define DG_STATIC_MAX_GROUPS 4096
int dg_m_grouped_fp8_fp4_gemm_contiguous_static(int device, void* cuda_stream, const dg_lp_operand* a, const int32_t* m_indices,
                                                const dg_lp_operand* b, const dg_out* out, uint32_t num_groups, const dg_epilogue* epi);
/* No counterpart in the reference.  What dg_ctx_sync is to the context-based calls: waits for `cuda_stream`, then reads
 * the 16-byte record in the built-in array that a kernel of the call above writes when one of its bounded waits runs
 * out (the kernel then stops early and leaves the output incomplete).  Returns DG_ERR_TIMEOUT with the block and wait
 * site and clears the record, or DG_OK.  Allocates nothing.  A host that uses the allocation-free call should poll this
 * whenever it synchronises: without it such an event goes unnoticed and the record stays set until the process exits. */
int dg_static_check_status(int device, void* cuda_stream);

/* ops_sm100.rs:815 (m_grouped_fp8_fp4_gemm_masked_dev).  a.rows = m_max (per group), data
 * (num_groups, m_max, k); b.rows = num_groups * n; masked_m (device, int32 per group) is read on
 * the device.  Unlike the reference, DG_OUT_FP8 is accepted here: D is (num_groups, m_max, n)
 * e4m3 and sfd takes the grouped packed layout with gran 32 along n. */
int dg_m_grouped_fp8_fp4_gemm_masked(dg_ctx* ctx, const dg_lp_operand* a, const int32_t* masked_m, const dg_lp_operand* b,
                                     const dg_out* out, uint32_t num_groups, uint32_t expected_m, const dg_epilogue* epi);

/* ops_sm100.rs:864 (fp8_fp4_bmm_dev): a (num_groups, m, k), b (num_groups, n, k); a.rows = m, b.rows = n. */
int dg_fp8_fp4_bmm(dg_ctx* ctx, const dg_lp_operand* a, const dg_lp_operand* b, const dg_out* out, uint32_t num_groups,
                   const dg_epilogue* epi);

/* The older f32-scale API (deepgemm/src/ops.rs:328 fp8_gemm_nt_dev, :422 / :535 the grouped variants, :635
 * fp8_bmm_nt_dev), which on Blackwell the reference routes through ops_sm100.rs:1414-1605.  a: e4m3 (rows, a_ld);
 * a_sf_t: the output of dg_transform_sf for a's (rows, k/128) f32 scales; b: e4m3 (num_groups * n, b_ld); sfb:
 * (num_groups * n / 128, k/128) f32 tile scales; out: bf16.  Exactly like the reference's bridge, only the exponent of
 * each f32 scale is used (scales must be powers of two to be exact).  Packed scale words are built in
 * context-owned scratch. */
int dg_fp8_gemm_nt(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld, const float* sfb, uint32_t m,
                   uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld);
int dg_m_grouped_fp8_gemm_nt_contiguous(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld,
                                        const float* sfb, uint32_t m_total, uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld,
                                        const int32_t* m_indices, uint32_t num_groups);
int dg_m_grouped_fp8_gemm_nt_masked(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld,
                                    const float* sfb, uint32_t m_max, uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld,
                                    const int32_t* masked_m, uint32_t num_groups, uint32_t expected_m);
int dg_fp8_bmm_nt(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld, const float* sfb, uint32_t m,
                  uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld, uint32_t num_groups);

/* ops_sm100.rs:1091-1098 (sf_packed_cols, sf_aligned_rows) and the size of alloc_sf (:1107). */
uint32_t dg_sf_packed_cols(uint32_t k, uint32_t gran_k);
uint32_t dg_sf_aligned_rows(uint32_t rows);
size_t dg_sf_words(uint32_t rows, uint32_t k, uint32_t gran_k, uint32_t num_groups);

/* Scale selection rule of the FP4 quantiser.  0: the rule of the reference's CPU quantiser
 * (deepgemm/src/reference.rs:273, exponent max(rounded, 128)); 1: smallest power of two that
 * maps the block maximum into [-6, 6]. */
enum { DG_SF_RULE_REFERENCE_CPU = 0, DG_SF_RULE_RANGE_FIT = 1 };

/* ops_sm100.rs:1186 (cast_bf16_to_fp8_sf_dev).  Outputs are caller-allocated: dst rows*k bytes,
 * sf dg_sf_words(rows, k, gran_k, num_groups) words (every word is written, no pre-zeroing needed
 * except for the alignment padding rows, which are left untouched). */
int dg_cast_bf16_to_fp8_sf(dg_ctx* ctx, const uint16_t* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t gran_k,
                           uint32_t num_groups, uint8_t* dst, uint32_t* sf);
/* moe.rs:273-296 with layout.rs:218-233 (deepgemm_silu_mul_bf16), fused with the activation quantiser the
 * second grouped GEMM needs: gate_up is (rows, 2n) bf16 with gate = [:, :n] and up = [:, n:]; the value
 * quantised is bf16(silu(gate) * up), silu(g) = g / (1 + exp(-g)); output as dg_cast_bf16_to_fp8_sf gives
 * for that bf16 matrix ((rows, n) e4m3 and packed UE8M0 words), without writing it.  live_rows (may be
 * NULL): a device word; rows from its value (rounded up to 8) on are left untouched, for an arena whose
 * row count only the device knows. */
int dg_silu_mul_cast_fp8_sf(dg_ctx* ctx, const uint16_t* gate_up, uint32_t src_ld, uint32_t rows, uint32_t n, uint32_t gran_k,
                            uint32_t num_groups, uint8_t* dst, uint32_t* sf, const uint32_t* live_rows);

/* ops_sm100.rs:1135 (cast_bf16_to_fp4_packed_sf_dev): dst rows*k/2 bytes. */
int dg_cast_bf16_to_fp4_packed_sf(dg_ctx* ctx, const uint16_t* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t num_groups,
                                  int sf_rule, uint8_t* dst, uint32_t* sf);

/* deepgemm/src/ops.rs:52 (transform_sf_dev): (batches, mn, sf_k) f32 -> (batches*sf_k, align4(mn)) f32. */
int dg_transform_sf(dg_ctx* ctx, const float* sf, uint32_t mn, uint32_t sf_k, uint32_t num_batches, float* dst);
/* ops_sm100.rs:1250 / :1294 / :1372 (transform_sf{1d,2d,_t}_packed_ue8m0_dev) */
int dg_transform_sf1d_packed_ue8m0(dg_ctx* ctx, const float* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t gran_k,
                                   uint32_t num_groups, uint32_t* dst);
int dg_transform_sf2d_packed_ue8m0(dg_ctx* ctx, const float* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t num_groups,
                                   uint32_t* dst);
int dg_transform_sf_t_packed_ue8m0(dg_ctx* ctx, const float* src, uint32_t rows, uint32_t k, uint32_t gran_k, uint32_t num_groups,
                                   uint32_t* dst);
/* ops_sm100.rs:1073 (run_psum_kernel): group_ends[g] = 1 + last row with m_indices == g; a group
 * without rows takes the previous group's end. */
int dg_group_ends_from_m_indices(dg_ctx* ctx, const int32_t* m_indices, uint32_t m, uint32_t num_groups, uint32_t* group_ends);
/* ops_sm100.rs:1338 (unpack_fp4_raw_dev) */
int dg_unpack_fp4_raw(dg_ctx* ctx, const uint8_t* src, size_t packed_len, uint8_t* dst);

/* Row movers either side of the expert-sharded grouped GEMM (the reference's single-GPU versions are
 * deepgemm/src/cuda/layout.rs:174 gather_rows_fp8 and :192 scatter_rows_f32_acc; here they feed and
 * drain an all-to-all).  All index arrays are device int32.
 * dg_gather_rows: dst row i = src row idx[i] (row_bytes, multiple of 16); idx[i] < 0 writes zeros. */
int dg_gather_rows(dg_ctx* ctx, const void* src, size_t src_pitch, const int32_t* idx, uint32_t n_dst, uint32_t row_bytes, void* dst,
                   size_t dst_pitch);
/* Send row i = [k e4m3 bytes of token idx[i] | its sf_cols packed scale words | zeros up to out_pitch]. */
int dg_moe_pack_rows(dg_ctx* ctx, const uint8_t* data, uint32_t k, const uint32_t* sf, uint32_t sf_stride, uint32_t sf_cols, const int32_t* idx,
                     uint32_t n, uint8_t* out, size_t out_pitch);
/* Arena row i = received row idx[i]: data to dst_data (n_dst, k), scale words to the packed layout
 * dst_sf[c * dst_sf_stride + i]; idx[i] < 0 (alignment padding) writes zero data and scales. */
int dg_moe_unpack_rows(dg_ctx* ctx, const uint8_t* in, size_t in_pitch, uint32_t k, uint32_t sf_cols, const int32_t* idx, uint32_t n_dst,
                       uint8_t* dst_data, uint32_t* dst_sf, uint32_t dst_sf_stride);
/* out[t, :] = bf16(sum_j weights[t, j] * rows[pos[t, j], :]): f32, terms in order, one fused
 * multiply-add each; pos < 0 skips a term.  rows / out are bf16 with pitches in elements. */
int dg_moe_combine(dg_ctx* ctx, const uint16_t* rows, size_t pitch, const int32_t* pos, const float* weights, uint32_t tokens, uint32_t topk,
                   uint32_t n, uint16_t* out, size_t out_pitch);

/* ---- Expert-parallel exchange over peer memory (multi-GPU form of moe.rs:120-252 and :314-360; the
 * reference is single-GPU).  Rank r owns experts [r * E / W, (r + 1) * E / W).  Each rank exposes its
 * arena, the arena's packed scale words and its result rows to the other ranks' GPUs; rows are
 * written to (dispatch) and read from (combine) the owner's memory directly.  Nothing here waits on
 * another rank: the caller orders the ranks with a collective on the same stream between dispatch and
 * the grouped GEMM, and between the last GEMM and combine. ---- */
#define DG_PEER_HANDLE_BYTES 64
/* Device buffer other processes can map: *ptr is this process's address, handle64 what to send them
 * (NULL: no handle is made, the buffer stays private to this process). */
int dg_peer_alloc(dg_ctx* ctx, size_t bytes, void** ptr, unsigned char* handle64);
/* Map another process's buffer from its handle (same node); *ptr is valid on ctx's device. */
int dg_peer_open(dg_ctx* ctx, const unsigned char* handle64, void** ptr);
int dg_peer_close(dg_ctx* ctx, void* ptr);   /* unmap what dg_peer_open returned */
int dg_peer_free(dg_ctx* ctx, void* ptr);    /* free what dg_peer_alloc returned */

/* Words of the block_hist scratch of dg_ep_count: ceil(pairs / 256) * num_experts. */
size_t dg_ep_block_hist_words(uint32_t pairs, uint32_t num_experts);
/* moe.rs:120-173 (expert counts, offsets, destination positions), this rank's part.
 * expert_of_pair (pairs = tokens * topk, int32, token-major): local_rank[p] = position of pair p among the pairs
 * of its 256-pair chunk with the same expert (-1 for an expert id outside [0, num_experts): the pair is dropped);
 * block_hist becomes, per chunk and expert, the number of such pairs in earlier chunks; counts[e] = this rank's
 * pairs for expert e.  Pairs of one expert keep their order (stable). */
int dg_ep_count(dg_ctx* ctx, const int32_t* expert_of_pair, uint32_t pairs, uint32_t num_experts, int32_t* local_rank, uint32_t* block_hist,
                uint32_t* counts);
/* all_counts (world, num_experts): every rank's counts (all-gathered by the caller).  Groups sit on their owner in
 * expert order, each starting at a multiple of `alignment`, rows ordered by (source rank, pair index).
 * pair_base[e] = arena row of this rank's first pair for expert e; group_ends[l] (num_experts / world words) = one
 * past the last valid row of local expert l, the table dg_m_grouped_fp8_fp4_gemm_contiguous_ends takes;
 * totals[0..3] = arena rows in use here, valid rows here, 1 if some rank's arena needs more than `capacity` rows
 * (dispatch then drops the rows that do not fit, and combine skips them), the largest arena in use.
 * slot_rows != 0 selects the masked layout of ops_sm100.rs:815 instead (decode-style steps): local expert l owns rows
 * [l * slot_rows, (l + 1) * slot_rows) of the arena, group_ends[l] becomes its valid row count (the masked_m array of
 * dg_m_grouped_fp8_fp4_gemm_masked with m_max = slot_rows), and the flag is also raised when an expert receives more than
 * slot_rows rows. */
int dg_ep_layout(dg_ctx* ctx, const uint32_t* all_counts, uint32_t world, uint32_t rank, uint32_t num_experts, uint32_t alignment,
                 uint32_t capacity, uint32_t slot_rows, uint32_t* pair_base, uint32_t* group_ends, uint32_t* totals);
/* moe.rs:176-206 (gather of token rows and scale rows into the grouped layout), across ranks: pair p's e4m3 row
 * (k bytes) and its sf_cols scale words go to row pos_of_pair[p] of the arena of the rank that owns its expert.
 * peer_data / peer_sf: device arrays of `world` pointers (every rank's arena (capacity, k) and its scale words
 * sf[c * peer_sf_stride + row]), entry `rank` being the local buffers.  Padding rows are not written.
 * slot_rows: as given to dg_ep_layout; in the masked layout the scale words go to the per-slot layout the masked GEMM
 * reads, sf[(slot * sf_cols + c) * peer_sf_stride + row in slot] with peer_sf_stride = dg_sf_aligned_rows(slot_rows).
 * max_blocks: 0 launches one warp per pair; a positive value bounds the grid (256-thread blocks striding over the
 * pairs), e.g. 2 x the SM count to leave room on every SM for a GEMM running beside the exchange. */
int dg_ep_dispatch(dg_ctx* ctx, const int32_t* expert_of_pair, const int32_t* local_rank, const uint32_t* block_base, const uint32_t* pair_base,
                   uint32_t pairs, uint32_t topk, uint32_t num_experts, uint32_t world, const uint8_t* data, uint32_t k, const uint32_t* sf,
                   uint32_t sf_stride, uint32_t sf_cols, void* const* peer_data, void* const* peer_sf, uint32_t peer_sf_stride,
                   uint32_t capacity, uint32_t slot_rows, int32_t* pos_of_pair, uint32_t max_blocks);
/* moe.rs:314-360 (weighted scatter-accumulate and f32 -> bf16), across ranks and as a gather: out[t, :] =
 * bf16(sum_j weights[t, j] * rows_j[pos_of_pair[t, j], :]) with rows_j the result buffer (bf16, `pitch` elements per
 * row) of the rank owning expert_of_pair[t, j]; same arithmetic as dg_moe_combine.  max_blocks as for dg_ep_dispatch. */
int dg_ep_combine(dg_ctx* ctx, const int32_t* expert_of_pair, const int32_t* pos_of_pair, const float* weights, uint32_t tokens, uint32_t topk,
                  uint32_t num_experts, uint32_t world, const void* const* peer_rows, size_t pitch, uint32_t n, uint16_t* out, size_t out_pitch,
                  uint32_t max_blocks);

/* No counterpart in the reference (its device waits spin without bound, deepgemm/src/cuda/common.rs:74-85).
 * Self-test of the bounded wait all kernels here use: launches one warp that waits, for at most limit_us, on a
 * barrier nothing signals.  The kernel finishes normally; the next dg_ctx_sync returns DG_ERR_TIMEOUT (site 0x700)
 * and clears the record, after which the context works as before. */
int dg_debug_expire_wait(dg_ctx* ctx, uint32_t limit_us);

/* deepgemm/src/types.rs:195-219 (mk alignment knob; process-global, power of two in [16,256]). */
int dg_set_mk_alignment_for_contiguous_layout(uint32_t value);
uint32_t dg_get_mk_alignment_for_contiguous_layout(void);
uint32_t dg_get_theoretical_mk_alignment_for_contiguous_layout(uint32_t arch_major);

/* deepgemm/src/heuristics_sm100.rs:61-87 (Sm100Desc) and :17-57 (Sm100Layout/Storage/Config). */
enum { DG_GEMM_NORMAL = 0, DG_GEMM_M_GROUPED_CONTIGUOUS = 1, DG_GEMM_M_GROUPED_MASKED = 2, DG_GEMM_BATCHED = 3 };
typedef struct {
    uint32_t gemm_type;
    uint32_t m, n, k, num_groups, expected_m;
    uint32_t a_bits, b_bits;
    uint32_t gran_a, gran_b;
    uint32_t cd_dtype;   /* DG_OUT_* */
    uint32_t num_sms;
    uint32_t major_a_mn, major_b_mn;   /* heuristics_sm100.rs:72-73 */
} dg_desc;
typedef struct {
    uint32_t swap_ab;            /* always 0: A rows ride the UMMA M dimension */
    uint32_t block_m, block_n, block_k;
    uint32_t cluster_m, cluster_n;
    uint32_t num_stages;
    uint32_t num_accum_stages;   /* TMEM accumulator buffers (2 = epilogue overlaps the next tile) */
    uint32_t smem_size;
    uint32_t num_tiles;          /* expected tiles (from expected_m for grouped layouts) */
    uint32_t num_splits;         /* dense GEMMs with few tiles: K ranges computed by different CTAs and summed in f32 */
} dg_config;
/* heuristics_sm100.rs:455 (best_config) */
int dg_best_config(const dg_desc* desc, dg_config* out);

#ifdef __cplusplus
}
#endif
#endif /* DGB200_H_ */
