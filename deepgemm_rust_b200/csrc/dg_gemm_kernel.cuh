// Persistent, warp-specialised block-scaled GEMM for sm_100a.
//
//   D[g][m, n] = epilogue( sum_k (A[g][m, k] * 2^(sfa-127)) * (B[g][n, k] * 2^(sfb-127)) )
//
// A and B are K-major e4m3 bytes (kind::mxf8f6f4) or packed e2m1 nibbles (kind::mxf4); the
// UE8M0 scale factors arrive as packed u32 words (rows contiguous, one word per 4 scale
// blocks along K) and are applied by the tensor core itself (tcgen05.mma ... block_scale).
//
// Roles inside one 256-thread CTA (one CTA per SM, looping over output tiles):
//   warp 0      issues every TMA load: A/B tiles into a ring of 128B-swizzled stages,
//               scale-factor words into the same stage's raw scale area
//   warp 1      allocates TMEM; copies scales smem->TMEM (tcgen05.cp) and issues the
//               UMMAs; tcgen05.commit releases the stage and, after the last k-block,
//               publishes the accumulator
//   warp 2      re-orders each 128-word scale chunk from row order to the 32x4 order the
//               tensor core reads (row r -> lane r%32, column r/32)
//   warp 3      idle
//   warps 4-7   epilogue: TMEM -> registers -> {bf16 | f32 | e4m3 + UE8M0 row scales}
//               -> swizzled staging -> TMA store; each warp owns 32 rows and stores on its own
// With kCtas = 2 two CTAs of a cluster share one 256 x BLOCK_N tile (tcgen05 cta_group::2): each
// loads its own 128 rows of A and half of the B rows, rank 0 issues the UMMAs for both, each
// CTA's TMEM receives its own 128 accumulator rows and runs its own epilogue.
// Accumulators are double-buffered in TMEM whenever 2*BLOCK_N plus the scale columns fit
// in 512 columns, so the epilogue of tile i overlaps the main loop of tile i+1.
//
// kSwap = true is the second tile family, for few activation rows per weight matrix (skinny dense
// GEMMs, small expert groups): the WEIGHT rows ride the UMMA M dimension (128 per CTA, 256 per
// pair) and the activation rows the UMMA N dimension, whose width follows the rows a tile really
// has (a multiple of 16, up to BLOCK_N).  The host hands the operands over with their roles
// exchanged, so loads, scale path and UMMA issue are the code above; what differs is the tile
// walk and the epilogue, which holds D transposed (lane = output column, TMEM column = output
// row) and writes it with plain stores, 32 consecutive columns of one output row per warp.
// Dense GEMMs with few tiles also cut K into ranges, one per CTA (or pair) of a cluster; the
// partial tiles are exchanged through distributed shared memory (every CTA sums a slice of the
// tile's rows over all ranges, in range order) and each CTA stores its slice: one launch, no
// workspace, a deterministic sum.
#pragma once
#include "dg_ptx.cuh"
#include "dg_activation.cuh"

namespace dg {

enum GemmType : uint32_t { kGemmNormal = 0, kGemmContiguous = 1, kGemmMasked = 2, kGemmBatched = 3 };
// kOutSwiGluFp8: B holds, per group, n gate rows followed by n up rows; a tile's accumulator is [gate columns | up columns] of
// the same n-range and the epilogue writes e4m3(silu(gate) * up) with one UE8M0 scale per 32 columns (CTA pairs only:
// rank 0 loads the gate rows of B, rank 1 the up rows).
enum OutKind : uint32_t { kOutBf16 = 0, kOutF32 = 1, kOutFp8 = 2, kOutSwiGluFp8 = 3 };
enum OperandFmt : uint32_t { kFmtMxf8f6f4 = 0, kFmtMxf4 = 1, kFmtBf16 = 2 };

constexpr uint32_t kBlockM = 128;          // UMMA M, rows of A per tile
constexpr uint32_t kBlockKBytes = 128;     // one 128-byte swizzle row of K per TMA box / UMMA group ("half" of a double stage)
constexpr uint32_t kUmmaKBytes = 32;       // K bytes consumed by one UMMA
constexpr uint32_t kMaxStages = 12;
constexpr uint32_t kNumThreads = 256;
// staging buffer of one epilogue warp: 32 rows x 64 bytes (bf16, 32 columns) or x 128 bytes (f32 / e4m3)
// (the fused activation stages 32 rows x 32 bytes)
constexpr uint32_t epilogue_buf_bytes(uint32_t out_kind) { return out_kind == 0 ? 2048u : (out_kind == 3 ? 1024u : 4096u); }
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
    uint32_t m, n, k;          // m: rows per group (contiguous: rows of the whole arena); n: output columns
    uint32_t num_groups;
    uint32_t gemm_type;
    uint32_t block_n;          // UMMA N = accumulator columns of a tile
    uint32_t tile_n;           // output columns of a tile: block_n, or block_n / 2 for the fused gate/up activation
    uint32_t block_k_elems;    // 128 (e4m3) or 256 (packed e2m1)
    uint32_t num_stages;
    uint32_t num_accum_stages;
    uint32_t gran_a, gran_b;   // K elements per scale factor (32 or 128)
    uint32_t tx_shift_a, tx_shift_b;   // 1 if the TMA load of that operand signals half the bytes its tile occupies (expanded e2m1)
    uint32_t fmt_a, fmt_b;     // kind::mxf8f6f4 operand formats: 0 = e4m3, 5 = e2m1 held one code per byte in shared memory
    uint32_t sf_a_cols, sf_b_cols;  // packed words per row (per group) along K
    uint32_t num_splits;       // dense only: K is cut into this many ranges, each writing its own f32 partial (D's 3rd coordinate)
    uint32_t kb_per_split;     // k-blocks per range (a multiple of every scale-word period)
    uint32_t mk_alignment;     // contiguous layout: every group starts at a multiple of this
    uint32_t has_alpha;
    uint32_t mask_rows;        // contiguous layout whose groups start at multiples of 16 rows: a 32-row store box can reach
                               // into the next group, so boxes that cross the group end are written row by row instead
    void* out_ptr;             // output base and leading dimension (elements), used by those row-by-row stores only
    uint32_t out_ld;
    uint32_t accumulate;       // D += A.B^T: tiles are added to the output with TMA reduce-add instead of stored
    uint32_t stream_a, stream_b;   // that operand is read from DRAM once by the whole launch (weights of a skinny or small-group
                                   // problem): its loads carry the L2 evict-first hint
    uint32_t wide_k;           // both operand maps are 4-D (128 bytes, rows, K slabs, groups): one load brings the two K slabs of a stage
    uint32_t mn_a, mn_b;       // that operand is MN-major in memory ((k, ld) bytes, rows contiguous; e4m3 only): its tiles arrive as
                               // boxes of 128 rows x 128 k and the UMMA descriptors walk them with the MN-major strides
    uint32_t tc_util;          // tensor-core duty cycle in percent (100: no pause); below 100 the UMMA warp idles after every k-block
                               // for (100 - tc_util) / tc_util times the k-block's tensor time (bf16_gemm_sm100.rs:358-371)
    float alpha;
    uint32_t sfd_stride;       // output scale words: stride between word columns (fp8 output)
    uint32_t cluster_splits;   // kSwap, dense: K ranges handled by the CTAs (pairs) of one cluster and summed through shared memory
    uint32_t out_group_rows;   // kSwap: output rows between two groups' outputs (masked / batched layouts)
    const uint32_t* grouped_layout;  // contiguous: end row of each group; masked: valid rows per group
    uint32_t* sfd;
    Status* status;
    long long* prof;           // debug builds only
    uint32_t debug_flags;      // debug builds only: 1 = epilogue only releases the accumulator, 2 = no scale-factor traffic
};

// Optional cycle accounting of the UMMA warp (debug builds with -DDG_PROFILE): p.prof[block*8 + i]
// i = 0 loop total, 1 wait for tiles, 2 wait for scales, 3 issue, 4 wait for a free accumulator.
#ifdef DG_PROFILE
#define DG_PROF_T(var) const long long var = clock64()
#define DG_PROF_ADD(slot, t0) prof_acc[slot] += clock64() - (t0)
#else
#define DG_PROF_T(var)
#define DG_PROF_ADD(slot, t0)
#endif

struct Tile {
    uint32_t m0, n0;     // first row / column of the tile (row is group-local except in the contiguous arena)
    uint32_t m_end;      // rows at or beyond this one belong to someone else (next group / out of range): never stored
    uint32_t n_end;      // kSwap: rows of the N-side operand at or beyond this one are not part of the tile (group end / matrix end)
    uint32_t ga, gb;     // group coordinate of A/SFA and of B/SFB
    uint32_t gd;         // third coordinate of D: the group, or the K range when K is split
    uint32_t kb0, kb1;   // k-block range of this tile
};

// Walks the tile list of one CTA.  Every role runs its own copy and sees the same sequence.
// In the swapped family "m" is the weight dimension (rows of the UMMA M side, per group) and "n" the
// activation rows (UMMA N side): p.m / num_m_blocks count weight rows, groups are ranges of N-side rows.
struct Scheduler {
    const GemmParams& p;
    bool swap;
    uint32_t tile_m, worker, num_workers, split;   // rows per tile; cluster index and count; K range of this CTA (pair)
    uint32_t num_m_blocks, num_n_blocks, iter;
    uint32_t cur_group, cum_begin, cur_m_blocks, cur_row_start, cur_row_end;

    DG_DEVICE Scheduler(const GemmParams& params, uint32_t ctas, bool swapped = false, uint32_t cluster_rank = 0) : p(params) {
        swap = swapped;
        tile_m = kBlockM * ctas;
        const uint32_t per_cluster = ctas * (swap ? p.cluster_splits : 1u);
        worker = blockIdx.x / per_cluster;
        num_workers = gridDim.x / per_cluster;
        split = swap ? cluster_rank / ctas : 0u;
        num_m_blocks = (p.m + tile_m - 1) / tile_m;
        num_n_blocks = (p.n + p.tile_n - 1) / p.tile_n;
        iter = 0;
        cur_group = 0;
        cum_begin = 0;
        cur_m_blocks = 0;
        cur_row_start = 0;
        cur_row_end = swap ? p.n : p.m;
        if (p.gemm_type == kGemmContiguous || p.gemm_type == kGemmMasked) load_group();
    }

    // rows of the current group, and how many row blocks they make (of tile_m rows, or of block_n rows when swapped)
    DG_DEVICE void load_group() {
        if (cur_group >= p.num_groups) return;
        const uint32_t limit = swap ? p.n : p.m, block = swap ? p.block_n : tile_m;
        if (p.gemm_type == kGemmContiguous) {
            const uint32_t prev_end = cur_group == 0 ? 0u : __ldg(p.grouped_layout + cur_group - 1);
            const uint32_t end = __ldg(p.grouped_layout + cur_group);
            cur_row_start = (prev_end + p.mk_alignment - 1) / p.mk_alignment * p.mk_alignment;
            const uint32_t rows = end > cur_row_start ? end - cur_row_start : 0u;
            cur_row_end = end < limit ? end : limit;
            cur_m_blocks = (rows + block - 1) / block;
        } else {
            const int32_t valid = static_cast<int32_t>(__ldg(p.grouped_layout + cur_group));
            const uint32_t rows = valid <= 0 ? 0u : (static_cast<uint32_t>(valid) < limit ? static_cast<uint32_t>(valid) : limit);
            cur_row_start = 0;
            cur_row_end = rows;      // nothing is stored (and a pair's second CTA loads nothing) past the group's valid rows
            cur_m_blocks = (rows + block - 1) / block;
        }
    }

    DG_DEVICE bool next(Tile& t) {
        uint32_t idx = worker + (iter++) * num_workers;
        const uint32_t total_kb = (p.k + p.block_k_elems - 1) / p.block_k_elems;
        t.kb0 = 0;
        t.kb1 = total_kb;
        t.n_end = p.n;
        if (swap) {
            if (p.cluster_splits > 1) {
                // k-blocks dealt out evenly: no range is empty as long as there are at least as many k-blocks as ranges
                t.kb0 = split * total_kb / p.cluster_splits;
                t.kb1 = (split + 1) * total_kb / p.cluster_splits;
            }
            t.m_end = p.m;
            if (p.gemm_type == kGemmNormal || p.gemm_type == kGemmBatched) {
                const uint32_t per_group = num_m_blocks * num_n_blocks;
                if (idx >= per_group * p.num_groups) return false;
                const uint32_t g = idx / per_group, r = idx - g * per_group;
                const uint32_t nb = r / num_m_blocks, mb = r - nb * num_m_blocks;     // weight blocks fastest: CTAs in flight share the rows
                t.m0 = mb * tile_m;
                t.n0 = nb * p.block_n;
                t.ga = t.gb = t.gd = g;
                return true;
            }
            while (true) {
                if (cur_group >= p.num_groups) return false;
                const uint32_t end = cum_begin + cur_m_blocks * num_m_blocks;
                if (idx < end) break;
                cum_begin = end;
                ++cur_group;
                load_group();
            }
            const uint32_t in_group = idx - cum_begin;
            const uint32_t nb = in_group / num_m_blocks, mb = in_group - nb * num_m_blocks;
            t.m0 = mb * tile_m;
            t.n0 = cur_row_start + nb * p.block_n;
            t.n_end = cur_row_end;
            t.ga = cur_group;
            t.gb = p.gemm_type == kGemmContiguous ? 0u : cur_group;
            t.gd = t.gb;
            return true;
        }
        if (p.gemm_type == kGemmNormal || p.gemm_type == kGemmBatched) {
            const uint32_t per_group = num_m_blocks * num_n_blocks;
            uint32_t split_k = 0;
            if (p.num_splits > 1) {
                // K ranges of one output tile sit next to each other in the tile order
                if (idx >= per_group * p.num_splits) return false;
                split_k = idx % p.num_splits;
                idx /= p.num_splits;
                t.kb0 = split_k * p.kb_per_split;
                t.kb1 = t.kb0 + p.kb_per_split < total_kb ? t.kb0 + p.kb_per_split : total_kb;
            } else if (idx >= per_group * p.num_groups) {
                return false;
            }
            const uint32_t g = idx / per_group, r = idx - g * per_group;
            // bands of 2048 rows, rows fastest inside a band: the tiles in flight at any moment form a
            // patch about as tall as it is wide (148 tiles of 128 x 224..256), which is what minimises the
            // A rows plus B rows a wave pulls from DRAM, and a band's A rows stay in L2 for its next wave
            const uint32_t kBand = 2048 / tile_m;
            const uint32_t per_band = kBand * num_n_blocks;
            const uint32_t band = r / per_band, in_band = r - band * per_band;
            const uint32_t first_m = band * kBand;
            const uint32_t rows_here = num_m_blocks - first_m < kBand ? num_m_blocks - first_m : kBand;
            const uint32_t nb = in_band / rows_here, mb = first_m + (in_band - nb * rows_here);
            t.m0 = mb * tile_m;
            t.m_end = p.m;
            t.n0 = nb * p.tile_n;
            t.ga = t.gb = g;
            t.gd = p.num_splits > 1 ? split_k : g;
            return true;
        }
        while (true) {
            if (cur_group >= p.num_groups) return false;
            const uint32_t end = cum_begin + cur_m_blocks * num_n_blocks;
            if (idx < end) break;
            cum_begin = end;
            ++cur_group;
            load_group();
        }
        const uint32_t in_group = idx - cum_begin;
        const uint32_t nb = in_group / cur_m_blocks, ml = in_group - nb * cur_m_blocks;
        t.m0 = cur_row_start + ml * tile_m;
        t.m_end = cur_row_end;
        t.n0 = nb * p.tile_n;
        t.gb = cur_group;
        t.ga = p.gemm_type == kGemmContiguous ? 0u : cur_group;
        t.gd = t.ga;
        return true;
    }

    // UMMA N of a tile: the whole BLOCK_N, or in the swapped family the rows the tile really has, rounded up to what
    // the instruction (and, for a pair, the split of the rows between the two CTAs) allows
    DG_DEVICE uint32_t umma_n(const Tile& t, uint32_t ctas) const {
        if (!swap) return p.block_n;
        const uint32_t rows = t.n_end > t.n0 ? t.n_end - t.n0 : 0u;
        const uint32_t step = 16 * ctas;
        const uint32_t n = (rows + step - 1) / step * step;
        return n < p.block_n ? (n == 0 ? step : n) : p.block_n;
    }
};

// How often a scale word must be (re)loaded and how many words one k-block needs.
//   block_k_elems = 128 (e4m3) or 256 (e2m1 pairs).  A word covers 4*gran elements.
struct SfPlan {
    uint32_t period;  // load on k-blocks where kb % period == 0; a power of two (1, 2 or 4)
    uint32_t shift;   // log2(period): the loops use masks and shifts instead of dividing by a run-time value every k-block
    uint32_t words;   // words per row per load
};
DG_DEVICE SfPlan sf_plan(uint32_t gran, uint32_t block_k_elems) {
    const uint32_t per_word = 4 * gran;
    SfPlan s;
    if (per_word >= block_k_elems) { s.period = per_word / block_k_elems; s.words = 1; }
    else { s.period = 1; s.words = block_k_elems / per_word; }
    s.shift = 31 - __clz(s.period);
    return s;
}

// One output element of the swapped family: alpha, optional accumulation into what the output holds, rounding.
template <uint32_t kOut>
DG_DEVICE void store_output(uint8_t* dst, float x, const GemmParams& p) {
    if (p.has_alpha) x *= p.alpha;
    if constexpr (kOut == kOutBf16) {
        uint16_t* d = reinterpret_cast<uint16_t*>(dst);
        // like the reduce-add store of the other family: the product is rounded to bf16, added to the bf16 addend, rounded again
        if (p.accumulate) x = __uint_as_float((pack_bf16x2(x, 0.0f) & 0xFFFFu) << 16) + __uint_as_float(static_cast<uint32_t>(*d) << 16);
        *d = static_cast<uint16_t>(pack_bf16x2(x, 0.0f) & 0xFFFFu);
    } else {
        float* d = reinterpret_cast<float*>(dst);
        *d = p.accumulate ? *d + x : x;
    }
}

// kFmt: kFmtMxf8f6f4 (e4m3 / expanded e2m1 operands, block-scaled), kFmtMxf4 (packed e2m1, block-scaled) or
// kFmtBf16 (bf16 operands seen as K-major rows of 2k bytes, kind::f16, no scale factors: bf16_gemm_sm100.rs).
template <uint32_t kFmt, uint32_t kOut, uint32_t kCtas, bool kSwap = false>
__global__ void __launch_bounds__(kNumThreads, 1)
dg_gemm_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
               const __grid_constant__ CUtensorMap tmap_d) {
    // a stage holds one or two 128-byte K slabs per operand (block_k_elems = halves x 128 e4m3 / 256 e2m1):
    // two slabs halve the per-stage bookkeeping (waits, commits) the UMMA warp does per UMMA
    constexpr bool kMXF4 = kFmt == kFmtMxf4, kScaled = kFmt != kFmtBf16;
    constexpr uint32_t kHalfElems = kMXF4 ? 256 : 128;
    const uint32_t kBlockKElems = p.block_k_elems;
    const uint32_t halves = kBlockKElems / kHalfElems;
    constexpr uint32_t kEpiBufBytes = kSwap ? 0u : epilogue_buf_bytes(kOut);   // the swapped family stores from registers
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    // CTA pair: rank 0 issues the UMMAs for both, each CTA owns 128 rows of the 256-row tile
    // and loads half of the B tile
    // (a cluster may hold several pairs: the K ranges of one tile in the swapped family; a pair is ranks 2i and 2i + 1)
    const uint32_t cluster_rank = (kCtas == 2 || kSwap) ? cluster_cta_rank() : 0u;
    const uint32_t cta_rank = kCtas == 2 ? (cluster_rank & 1u) : 0u;
    const uint32_t leader_rank = cluster_rank & ~1u;       // kCtas == 2: the CTA of this pair that issues the UMMAs
    const uint32_t block_n = p.block_n;
    const uint32_t load_n = block_n / kCtas;
    const uint32_t sf_block_n = (block_n + 127) / 128 * 128;
    const SfPlan plan_a = sf_plan(p.gran_a, kBlockKElems), plan_b = sf_plan(p.gran_b, kBlockKElems);
    const uint32_t sfa_bytes = 512 * plan_a.words, sfb_bytes = sf_block_n * 4 * plan_b.words;
    const uint32_t a_half = kBlockM * kBlockKBytes, b_half = load_n * kBlockKBytes;
    const uint32_t a_bytes = a_half * halves, b_bytes = b_half * halves;
    const uint32_t num_stages = p.num_stages;

    // shared memory carve-up (every tile base stays 1024-byte aligned)
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem_a + num_stages * a_bytes;
    uint8_t* smem_epi = smem_b + num_stages * b_bytes;
    uint8_t* smem_sfa = smem_epi + 8 * kEpiBufBytes;
    uint8_t* smem_sfb = smem_sfa + num_stages * sfa_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_sfb + num_stages * sfb_bytes);
    uint64_t* bar_full = bars;                       // A/B tiles of a stage landed (pair: both CTAs' tiles, on rank 0)
    uint64_t* bar_empty = bars + kMaxStages;         // the UMMAs reading a stage finished
    uint64_t* bar_sf_raw = bars + 2 * kMaxStages;    // scale words of a stage landed (per CTA)
    uint64_t* bar_tmem_full = bars + 4 * kMaxStages;
    uint64_t* bar_tmem_empty = bars + 4 * kMaxStages + 2;
    uint64_t* bar_tc = bars + 4 * kMaxStages + 4;     // the UMMAs of a k-block finished (only with a tensor-core duty cycle below 100 %)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kMaxStages + 5);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < num_stages; ++s) {
            // a stage is ready for the UMMA warp when both producer warps have arrived (operand A, operand B; their bytes are
            // counted on the same barrier) and, for the block-scaled kinds, the scale words of every CTA of the pair are in place:
            // on the k-blocks that bring new scale words the re-ordering warp arrives when it is done, on the others the A-side
            // producer arrives in its place, so the UMMA warp has one barrier to wait for per stage
            mbar_init(bar_full + s, 2 + (kScaled ? kCtas : 0u));
            mbar_init(bar_empty + s, 1);
            mbar_init(bar_sf_raw + s, 2);
        }
        for (uint32_t e = 0; e < 2; ++e) {
            mbar_init(bar_tmem_full + e, 1);
            mbar_init(bar_tmem_empty + e, 4 * kCtas);
        }
        mbar_init(bar_tc, 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_sfa);
        tma_prefetch_desc(&tmap_sfb);
        tma_prefetch_desc(&tmap_d);
    }
    if (warp == 1) {
        tmem_alloc<kCtas>(tmem_slot, kTmemCols);
        tmem_relinquish<kCtas>();
    }
    tc_fence_before();
    if constexpr (kCtas == 2 || kSwap) cluster_sync(); else __syncthreads();
    tc_fence_after();
    // up to here nothing read or wrote global memory: the set-up above may overlap the previous kernel of the stream
    griddep_wait();
    griddep_launch_dependents();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sfa = tmem_base + p.num_accum_stages * block_n;
    const uint32_t tmem_sfb = tmem_sfa + 4 * plan_a.words;

    // The producer and UMMA warps run their loops with all 32 lanes and guard only the issuing
    // instructions with lane 0: addresses and descriptors stay warp-uniform, so they live in
    // uniform registers instead of being moved there one by one for every tcgen05 / TMA
    // instruction (which alone costs ~190 cycles per UMMA).
    if (warp == 0 || warp == 3) {
        // ------------------------------------------------------------ TMA producers
        // Two warps, one per operand: warp 0 brings A and its scale words, warp 3 B and its scale words.  Issuing a stage's four
        // to six loads from one lane took ~450 cycles per 128 bytes of K, more than the tensor pipe needs for them at N = 224;
        // halved, the loads of a stage are on their way sooner after its buffer is released.  Both warps arrive on the stage's
        // barriers (count 2), each with the bytes of its own operand.
        const bool b_side = warp == 3;
        Scheduler sched(p, kCtas, kSwap, cluster_rank);
        Tile t;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        const uint32_t full_bar_leader = kCtas == 2 ? mapa_u32(smem_u32(bar_full), leader_rank) : 0u;
        const uint64_t stream_policy = (p.stream_a | p.stream_b) ? l2_policy_evict_first() : 0ull;
        const bool leader_lane = elect_one();      // the lane that issues; the same one for the whole kernel
        const uint32_t a_tx = a_bytes >> p.tx_shift_a, b_tx = b_bytes >> p.tx_shift_b;
        while (ok && sched.next(t)) {
            const int32_t row_a = static_cast<int32_t>(t.m0 + cta_rank * kBlockM);
            // fused gate/up activation: rank 0 takes the gate rows [n0, n0 + load_n) of the group's B block, rank 1 the up rows
            // of the same range, which start p.n rows further down.  Swapped family: the UMMA takes the first half of its N
            // rows from rank 0 and the second half from rank 1, so rank 1's box starts where that half starts.
            const int32_t row_b = static_cast<int32_t>(kOut == kOutSwiGluFp8 ? t.n0 + cta_rank * p.n
                                                       : (kSwap ? t.n0 + cta_rank * (sched.umma_n(t, kCtas) / 2) : t.n0 + cta_rank * load_n));
            // a pair's second CTA whose 128 rows all lie past the end of the group (or of the matrix) loads no A rows: its
            // accumulator rows are never stored, and the operand stream from L2 is what bounds these tiles
            const bool load_a = kCtas == 1 || static_cast<uint32_t>(row_a) < t.m_end;
            for (uint32_t kb = t.kb0; kb < t.kb1; ++kb) {
                if (!mbar_wait_warp(bar_empty + stage, phase ^ 1, abort_flag, p.status, (b_side ? 0x180 : 0x100) + stage)) { ok = false; break; }
                // a scale word is loaded where it starts and, for a K range that begins inside a word, at the range's first k-block
                bool need_a = kScaled && ((kb & (plan_a.period - 1)) == 0 || kb == t.kb0), need_b = kScaled && ((kb & (plan_b.period - 1)) == 0 || kb == t.kb0);
#ifdef DG_PROFILE
                if (p.debug_flags & 2) need_a = need_b = false;
#endif
                const uint32_t bar_addr = full_bar_leader + stage * 8;
                if (!b_side) {
                    if (leader_lane) {
                        if (need_a || need_b) {
                            mbar_arrive_expect_tx(bar_sf_raw + stage, need_a ? sfa_bytes : 0u);
                            if (need_a)
                                tma_load_2d(smem_sfa + stage * sfa_bytes, &tmap_sfa, bar_sf_raw + stage, row_a,
                                            static_cast<int32_t>(t.ga * p.sf_a_cols + (kb >> plan_a.shift) * plan_a.words));
                        }
                        if constexpr (kCtas == 1) mbar_arrive_expect_tx(bar_full + stage, a_tx);
                        // both CTAs' tiles complete on rank 0's barrier; rank 0 expects the bytes of the pair
                        else if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + stage, (t.m0 + kBlockM < t.m_end ? 2u : 1u) * a_tx);
                        if (p.wide_k) {
                            uint8_t* dst_a = smem_a + stage * a_bytes;
                            if constexpr (kCtas == 1) tma_load_4d(dst_a, &tmap_a, bar_full + stage, 0, row_a, static_cast<int32_t>(kb * 2), static_cast<int32_t>(t.ga));
                            else if (load_a) tma_load_4d_2cta(dst_a, &tmap_a, bar_addr, 0, row_a, static_cast<int32_t>(kb * 2), static_cast<int32_t>(t.ga));
                        } else
                        for (uint32_t h = 0; h < halves; ++h) {
                            const int32_t kx = static_cast<int32_t>(kb * kBlockKElems + h * kHalfElems);
                            uint8_t* dst_a = smem_a + stage * a_bytes + h * a_half;
                            // an MN-major operand comes as boxes of 128 rows (innermost) x one slab of K, 16 KB each, one box per 128 rows
                            if constexpr (kCtas == 1) {
                                if (p.mn_a) tma_load_3d(dst_a, &tmap_a, bar_full + stage, row_a, kx, static_cast<int32_t>(t.ga));
                                else if (p.stream_a) tma_load_3d_hint(dst_a, &tmap_a, bar_full + stage, kx, row_a, static_cast<int32_t>(t.ga), stream_policy);
                                else tma_load_3d(dst_a, &tmap_a, bar_full + stage, kx, row_a, static_cast<int32_t>(t.ga));
                            } else if (load_a) {
                                if (p.mn_a) tma_load_3d_2cta(dst_a, &tmap_a, bar_addr, row_a, kx, static_cast<int32_t>(t.ga));
                                else if (p.stream_a) tma_load_3d_2cta_hint(dst_a, &tmap_a, bar_addr, kx, row_a, static_cast<int32_t>(t.ga), stream_policy);
                                else tma_load_3d_2cta(dst_a, &tmap_a, bar_addr, kx, row_a, static_cast<int32_t>(t.ga));
                            }
                        }
                        if (kScaled && !(need_a || need_b)) {
                            // no new scale words on this k-block: stand in for this CTA's re-ordering warp
                            if constexpr (kCtas == 1) mbar_arrive(bar_full + stage);
                            else mbar_arrive_remote(bar_full + stage, leader_rank);
                        }
                    }
                } else {
                    if (leader_lane) {
                        if (need_a || need_b) {
                            // fused gate/up activation: the scale words of the gate rows and of the up rows come as two boxes of
                            // block_n / 2 words (one word per row and stage: per-128 scales only)
                            const uint32_t sfb_tx = kOut == kOutSwiGluFp8 ? block_n * 4 : sfb_bytes;
                            mbar_arrive_expect_tx(bar_sf_raw + stage, need_b ? sfb_tx : 0u);
                            if (need_b) {
                                const int32_t sf_y = static_cast<int32_t>(t.gb * p.sf_b_cols + (kb >> plan_b.shift) * plan_b.words);
                                tma_load_2d(smem_sfb + stage * sfb_bytes, &tmap_sfb, bar_sf_raw + stage, static_cast<int32_t>(t.n0), sf_y);
                                if constexpr (kOut == kOutSwiGluFp8)
                                    tma_load_2d(smem_sfb + stage * sfb_bytes + block_n * 2, &tmap_sfb, bar_sf_raw + stage,
                                                static_cast<int32_t>(t.n0 + p.n), sf_y);
                            }
                        }
                        if constexpr (kCtas == 1) mbar_arrive_expect_tx(bar_full + stage, b_tx);
                        else if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + stage, 2 * b_tx);
                        if (p.wide_k) {
                            uint8_t* dst_b = smem_b + stage * b_bytes;
                            if constexpr (kCtas == 1) tma_load_4d(dst_b, &tmap_b, bar_full + stage, 0, row_b, static_cast<int32_t>(kb * 2), static_cast<int32_t>(t.gb));
                            else tma_load_4d_2cta(dst_b, &tmap_b, bar_addr, 0, row_b, static_cast<int32_t>(kb * 2), static_cast<int32_t>(t.gb));
                        } else
                        for (uint32_t h = 0; h < halves; ++h) {
                            const int32_t kx = static_cast<int32_t>(kb * kBlockKElems + h * kHalfElems);
                            uint8_t* dst_b = smem_b + stage * b_bytes + h * b_half;
                            if constexpr (kCtas == 1) {
                                if (p.mn_b) {
                                    for (uint32_t j = 0; j < load_n / 128; ++j)
                                        tma_load_3d(dst_b + j * 16384, &tmap_b, bar_full + stage, row_b + static_cast<int32_t>(j * 128), kx, static_cast<int32_t>(t.gb));
                                } else if (p.stream_b) tma_load_3d_hint(dst_b, &tmap_b, bar_full + stage, kx, row_b, static_cast<int32_t>(t.gb), stream_policy);
                                else tma_load_3d(dst_b, &tmap_b, bar_full + stage, kx, row_b, static_cast<int32_t>(t.gb));
                            } else {
                                if (p.mn_b) {
                                    for (uint32_t j = 0; j < load_n / 128; ++j)
                                        tma_load_3d_2cta(dst_b + j * 16384, &tmap_b, bar_addr, row_b + static_cast<int32_t>(j * 128), kx, static_cast<int32_t>(t.gb));
                                } else if (p.stream_b) tma_load_3d_2cta_hint(dst_b, &tmap_b, bar_addr, kx, row_b, static_cast<int32_t>(t.gb), stream_policy);
                                else tma_load_3d_2cta(dst_b, &tmap_b, bar_addr, kx, row_b, static_cast<int32_t>(t.gb));
                            }
                        }
                    }
                }
                __syncwarp();
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- UMMA issuer
        if (cta_rank == 0) {
            Scheduler sched(p, kCtas, kSwap, cluster_rank);
            Tile t;
            uint32_t stage = 0, phase = 0, it = 0, tc_phase = 0;
            const uint32_t chunks_b = plan_b.words * (sf_block_n / 128);
            bool ok = true;
            const bool leader_lane = elect_one();      // the lane that issues; the same one for the whole kernel
#ifdef DG_PROFILE
            long long prof_acc[5] = {0, 0, 0, 0, 0};
#endif
            DG_PROF_T(t_loop);
            while (ok && sched.next(t)) {
                const uint32_t e = it % p.num_accum_stages, acc_phase = (it / p.num_accum_stages) & 1;
                ++it;
                DG_PROF_T(t_acc);
                if (!mbar_wait_warp(bar_tmem_empty + e, acc_phase ^ 1, abort_flag, p.status, 0x200 + e)) break;
                DG_PROF_ADD(4, t_acc);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + e * block_n;
                const uint32_t n_tile = sched.umma_n(t, kCtas);
                const uint32_t idesc = (kScaled ? make_idesc_block_scaled(kBlockM * kCtas, n_tile, kMXF4 ? 1u : p.fmt_a, kMXF4 ? 1u : p.fmt_b)
                                                : make_idesc_bf16(kBlockM * kCtas, n_tile)) | (p.mn_a << 15) | (p.mn_b << 16);
                // MN-major tiles: 8 k-rows of 128 row-bytes form a 1024-byte swizzle atom (stride byte offset), the next 128 rows
                // lie one box (16 KB) further (leading byte offset), and one UMMA (32 k) advances by 32 x 128 bytes
                const uint32_t a_lbo = p.mn_a ? 16384u : 0u, b_lbo = p.mn_b ? 16384u : 0u;
                const uint32_t a_kstep = (p.mn_a ? 4096u : kUmmaKBytes) >> 4, b_kstep = (p.mn_b ? 4096u : kUmmaKBytes) >> 4;
                for (uint32_t kb = t.kb0; kb < t.kb1; ++kb) {
                    bool need_a = kScaled && ((kb & (plan_a.period - 1)) == 0 || kb == t.kb0), need_b = kScaled && ((kb & (plan_b.period - 1)) == 0 || kb == t.kb0);
#ifdef DG_PROFILE
                    if (p.debug_flags & 2) need_a = need_b = false;
#endif
                    DG_PROF_T(t_full);
                    if (!mbar_wait_warp(bar_full + stage, phase, abort_flag, p.status, 0x300 + stage)) { ok = false; break; }
                    DG_PROF_ADD(1, t_full);
                    DG_PROF_T(t_sf);
                    DG_PROF_ADD(2, t_sf);
                    DG_PROF_T(t_issue);
                    tc_fence_after();
                    // One single-lane region per stage holds the scale copies, every UMMA of the stage and the commits; all operands
                    // are computed before it by the whole warp (warp-uniform values).  Measured on 4096 x 7168 x 16384: with one region
                    // per K slab plus one each for the copies and the commits this warp spent 435 cycles per 128 bytes of K issuing
                    // (the tensor pipe needs 512 / 448 at N = 256 / 224 and was starved by the rest of the loop); with one region 283.
                    const uint32_t sfa_addr = smem_u32(smem_sfa + stage * sfa_bytes), sfb_addr = smem_u32(smem_sfb + stage * sfb_bytes);
                    const uint64_t sfa_desc = make_smem_desc(sfa_addr, 0, 128, 0), sfb_desc = make_smem_desc(sfb_addr, 0, 128, 0);
                    const bool last = kb + 1 == t.kb1;
                    uint32_t idescs[2][4], a_cols[2][4], b_cols[2][4];
                    uint64_t a_descs[2], b_descs[2];
                    #pragma unroll
                    for (uint32_t h = 0; h < 2; ++h) {
                        #pragma unroll
                        for (uint32_t k = 0; k < 4; ++k) {
                            uint32_t a_id, b_id;
                            if constexpr (kMXF4) {
                                a_id = (k & 1) * 2; b_id = (k & 1) * 2;
                                a_cols[h][k] = tmem_sfa + 4 * (h * 2 + k / 2); b_cols[h][k] = tmem_sfb + 4 * (h * 2 + k / 2) * (sf_block_n / 128);
                            } else {
                                a_id = p.gran_a == 128 ? (kb * halves + h) % 4 : k;
                                b_id = p.gran_b == 128 ? (kb * halves + h) % 4 : k;
                                a_cols[h][k] = tmem_sfa + (p.gran_a == 128 ? 0u : 4 * h);
                                b_cols[h][k] = tmem_sfb + (p.gran_b == 128 ? 0u : 4 * h * (sf_block_n / 128));
                            }
                            idescs[h][k] = idesc_with_sf_ids(idesc, a_id, b_id);
                        }
                        a_descs[h] = make_smem_desc(smem_u32(smem_a + stage * a_bytes + h * a_half), a_lbo, 1024, 2);
                        b_descs[h] = make_smem_desc(smem_u32(smem_b + stage * b_bytes + h * b_half), b_lbo, 1024, 2);
                    }
                    if (leader_lane) {
                        if (need_a)
                            for (uint32_t c = 0; c < plan_a.words; ++c) utccp_32x128b_warpx4<kCtas>(tmem_sfa + 4 * c, sfa_desc + c * (512 >> 4));
                        if (need_b)
                            for (uint32_t c = 0; c < chunks_b; ++c) utccp_32x128b_warpx4<kCtas>(tmem_sfb + 4 * c, sfb_desc + c * (512 >> 4));
                        #pragma unroll
                        for (uint32_t h = 0; h < 2; ++h) {
                            if (h < halves) {
                                #pragma unroll
                                for (uint32_t k = 0; k < kBlockKBytes / kUmmaKBytes; ++k) {
                                    const uint32_t accumulate = (kb != t.kb0 || h != 0 || k != 0) ? 1u : 0u;
                                    if constexpr (kScaled)
                                        umma_block_scaled<kCtas, kMXF4>(d_tmem, a_descs[h] + k * a_kstep, b_descs[h] + k * b_kstep, idescs[h][k],
                                                                        a_cols[h][k], b_cols[h][k], accumulate);
                                    else
                                        umma_f16<kCtas>(d_tmem, a_descs[h] + k * (kUmmaKBytes >> 4), b_descs[h] + k * (kUmmaKBytes >> 4), idesc, accumulate);
                                }
                            }
                        }
                        if constexpr (kCtas == 1) {
                            umma_commit(bar_empty + stage);
                            if (last) umma_commit(bar_tmem_full + e);
                        } else {
                            umma_commit_2cta(bar_empty + stage, static_cast<uint16_t>(3u << leader_rank));
                            if (last) umma_commit_2cta(bar_tmem_full + e, static_cast<uint16_t>(3u << leader_rank));
                        }
                    }
                    __syncwarp();
                    if (p.tc_util < 100) {
                        // let the tensor cores rest: wait until this k-block's UMMAs are done, then idle for the requested share
                        if (leader_lane) {
                            if constexpr (kCtas == 1) umma_commit(bar_tc);
                            else umma_commit_2cta(bar_tc, static_cast<uint16_t>(1u << leader_rank));
                        }
                        __syncwarp();
                        if (!mbar_wait_warp(bar_tc, tc_phase, abort_flag, p.status, 0x480)) { ok = false; break; }
                        tc_phase ^= 1;
                        const long long busy = 4ll * n_tile * halves;      // 2 * 128 * N * (128 * halves) / 8192 cycles per k-block and SM
                        const long long idle = (100ll - p.tc_util) * busy / p.tc_util;
                        const long long t0 = clock64();
                        while (clock64() - t0 < idle) {}
                        __syncwarp();
                    }
                    DG_PROF_ADD(3, t_issue);
                    if (++stage == num_stages) { stage = 0; phase ^= 1; }
                }
            }
#ifdef DG_PROFILE
            DG_PROF_ADD(0, t_loop);
            if (lane == 0 && p.prof != nullptr)
                for (int i = 0; i < 5; ++i) p.prof[blockIdx.x * 8 + i] = prof_acc[i];
#endif
        }
        __syncwarp();
    } else if (warp == 2) {
        // -------------------------------------------------- scale-factor re-ordering
        Scheduler sched(p, kCtas, kSwap, cluster_rank);
        Tile t;
        uint32_t stage = 0, sf_phase_bits = 0;
        bool ok = true;
        while (ok && sched.next(t)) {
            for (uint32_t kb = t.kb0; kb < t.kb1; ++kb) {
                bool need_a = kScaled && ((kb & (plan_a.period - 1)) == 0 || kb == t.kb0), need_b = kScaled && ((kb & (plan_b.period - 1)) == 0 || kb == t.kb0);
#ifdef DG_PROFILE
                if (p.debug_flags & 2) need_a = need_b = false;
#endif
                if (need_a || need_b) {
                    if (!mbar_wait(bar_sf_raw + stage, (sf_phase_bits >> stage) & 1, abort_flag, p.status, 0x500 + stage)) { ok = false; break; }
                    sf_phase_bits ^= 1u << stage;
                    // word r of a 128-word chunk moves to position (r % 32) * 4 + r / 32
                    const uint32_t chunks_a = need_a ? plan_a.words : 0u;
                    const uint32_t chunks_b = need_b ? plan_b.words * (sf_block_n / 128) : 0u;
                    for (uint32_t c = 0; c < chunks_a + chunks_b; ++c) {
                        uint32_t* chunk = reinterpret_cast<uint32_t*>(c < chunks_a ? smem_sfa + stage * sfa_bytes + c * 512
                                                                                   : smem_sfb + stage * sfb_bytes + (c - chunks_a) * 512);
                        const uint32_t w0 = chunk[lane], w1 = chunk[32 + lane], w2 = chunk[64 + lane], w3 = chunk[96 + lane];
                        __syncwarp();
                        st_shared_v4(smem_u32(chunk + lane * 4), w0, w1, w2, w3);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (kCtas == 1) mbar_arrive(bar_full + stage);
                        else mbar_arrive_remote(bar_full + stage, leader_rank);
                    }
                }
                if (++stage == num_stages) stage = 0;
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
      if constexpr (kSwap) {
        // ------------------------------------------------- epilogue of the swapped family
        // The accumulator holds D transposed: TMEM lane = output column (a weight row), TMEM column = output row.  For one
        // output row the 32 lanes of a warp hold 32 consecutive columns, so every store instruction of a warp writes one
        // 64-byte (bf16) or 128-byte (f32) run of a row; rows past the tile's last valid row are skipped.
        static_assert(kOut == kOutBf16 || kOut == kOutF32, "the swapped tile family writes bf16 or f32");
        const uint32_t ew = warp - 4;
        Scheduler sched(p, kCtas, true, cluster_rank);
        Tile t;
        uint32_t it = 0;
        if (p.cluster_splits > 1) {
            // K ranges: the partial sums stay in TMEM until every CTA of the cluster has finished its range (after the roles)
            if (sched.next(t)) mbar_wait(bar_tmem_full, 0, abort_flag, p.status, 0x600);
        } else {
            while (sched.next(t)) {
                const uint32_t e = it % p.num_accum_stages, acc_phase = (it / p.num_accum_stages) & 1;
                ++it;
                if (!mbar_wait(bar_tmem_full + e, acc_phase, abort_flag, p.status, 0x600 + e)) break;
                tc_fence_after();
                const uint32_t n_tile = sched.umma_n(t, kCtas);
                const uint32_t rows_left = t.n_end > t.n0 ? t.n_end - t.n0 : 0u;
                const uint32_t valid = rows_left < n_tile ? rows_left : n_tile;
                const uint32_t taddr = tmem_base + ((ew * 32) << 16) + e * block_n;
                const uint32_t col_out = t.m0 + cta_rank * kBlockM + ew * 32 + lane;
                const bool col_ok = col_out < t.m_end;
                constexpr uint32_t kElem = kOut == kOutBf16 ? 2 : 4;
                uint8_t* base = static_cast<uint8_t*>(p.out_ptr) +
                                ((static_cast<size_t>(t.gd) * p.out_group_rows + t.n0) * p.out_ld + col_out) * kElem;
                const size_t row_pitch = static_cast<size_t>(p.out_ld) * kElem;
                auto release_accumulator = [&]() {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (kCtas == 1) mbar_arrive(bar_tmem_empty + e);
                        else mbar_arrive_remote(bar_tmem_empty + e, leader_rank);
                    }
                };
                auto store_rows = [&](uint32_t (&v)[32], uint32_t s) {
                    #pragma unroll
                    for (uint32_t c = 0; c < 32; ++c) {
                        const uint32_t row = s * 32 + c;
                        if (row < valid && col_ok) store_output<kOut>(base + row * row_pitch, __uint_as_float(v[c]), p);
                    }
                };
                const uint32_t chunks = (n_tile + 31) / 32;
                uint32_t va[32], vb[32];
                tmem_ld_32x32b_x32(taddr, va);
                for (uint32_t s = 0; s < chunks; s += 2) {
                    tmem_ld_wait_x32(va);
                    const bool has_b = s + 1 < chunks;
                    if (has_b) tmem_ld_32x32b_x32(taddr + (s + 1) * 32, vb);
                    else release_accumulator();
                    store_rows(va, s);
                    if (has_b) {
                        tmem_ld_wait_x32(vb);
                        if (s + 2 < chunks) tmem_ld_32x32b_x32(taddr + (s + 2) * 32, va);
                        else release_accumulator();
                        store_rows(vb, s + 1);
                    }
                }
            }
        }
      } else {
        // ------------------------------------------------------------------ epilogue
        // 32 accumulator columns at a time: one tcgen05.ld per step; bf16 / f32 / e4m3 rows are staged
        // in rows of kRowBytes (64 / 128 / 128 bytes, swizzled like the store's tensor map) and
        // every kSubsPerBuf steps one TMA store writes 32 rows
        const uint32_t ew = warp - 4;  // TMEM lane quadrant and 32-row slice of this CTA's 128 rows
        uint8_t* buf0 = smem_epi + ew * 2 * kEpiBufBytes;
        constexpr uint32_t kSubsPerBuf = kOut == kOutFp8 ? 4 : 1;
        constexpr uint32_t kColsPerBuf = 32 * kSubsPerBuf;
        constexpr uint32_t kRowBytes = kOut == kOutBf16 ? 64 : 128;
        Scheduler sched(p, kCtas);
        Tile t;
        uint32_t it = 0, buf_idx = 0;
        while (sched.next(t)) {
            const uint32_t e = it % p.num_accum_stages, acc_phase = (it / p.num_accum_stages) & 1;
            ++it;
            if (!mbar_wait(bar_tmem_full + e, acc_phase, abort_flag, p.status, 0x600 + e)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((ew * 32) << 16) + e * block_n;
            const uint32_t row0 = t.m0 + cta_rank * kBlockM + ew * 32;
            const uint32_t row = row0 + lane;  // row this thread owns
            const uint32_t num_subs = block_n / 32;
            uint32_t sf_word = 0;
#ifdef DG_PROFILE
            if (p.debug_flags & 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (kCtas == 1) mbar_arrive(bar_tmem_empty + e);
                    else mbar_arrive_remote(bar_tmem_empty + e, leader_rank);
                }
                continue;
            }
#endif
            // hand the TMEM stage back to the UMMA warp once its last columns are in registers
            auto release_accumulator = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (kCtas == 1) mbar_arrive(bar_tmem_empty + e);
                    else mbar_arrive_remote(bar_tmem_empty + e, leader_rank);
                }
            };
            if constexpr (kOut == kOutSwiGluFp8) {
                // accumulator columns [0, block_n / 2) are gate, [block_n / 2, block_n) up, for the same output columns.
                // Per 32 output columns: both halves to registers, round to bf16 (what an unfused GEMM would have stored),
                // act = bf16(silu(gate) * up), one power-of-two scale for the 32 values, e4m3, 32-byte rows staged for a
                // TMA store, the scale byte straight to the packed scale words of the next GEMM's operand.
                const uint32_t half_n = block_n / 2, num_out_subs = half_n / 32;
                for (uint32_t s = 0; s < num_out_subs; ++s) {
                    uint32_t g[32], u[32];
                    tmem_ld_32x32b_x32(taddr + s * 32, g);
                    tmem_ld_32x32b_x32(taddr + half_n + s * 32, u);
                    tmem_ld_wait_x32(g);
                    tmem_ld_wait_x32(u);
                    if (s + 1 == num_out_subs) release_accumulator();
                    uint8_t* buf = buf0 + buf_idx * kEpiBufBytes;
                    if (lane == 0) tma_store_wait_read<1>();   // the store issued two buffers ago has finished reading this buffer
                    __syncwarp();
                    uint32_t amax = 0;
                    #pragma unroll
                    for (uint32_t i = 0; i < 32; i += 2) {
                        const uint32_t gb = pack_bf16x2(__uint_as_float(g[i]), __uint_as_float(g[i + 1]));
                        const uint32_t ub = pack_bf16x2(__uint_as_float(u[i]), __uint_as_float(u[i + 1]));
                        const float2 act = silu_mul_bf16x2(make_float2(__uint_as_float(gb << 16), __uint_as_float(gb & 0xFFFF0000u)),
                                                           make_float2(__uint_as_float(ub << 16), __uint_as_float(ub & 0xFFFF0000u)));
                        g[i] = __float_as_uint(act.x);         // bf16 values, widened
                        g[i + 1] = __float_as_uint(act.y);
                        amax = max(amax, max((g[i] >> 16) & 0x7FFFu, (g[i + 1] >> 16) & 0x7FFFu));
                    }
                    const uint32_t rounded = (amax + 0x7Fu - 0x60u) >> 7;
                    uint32_t sf_exp = (rounded < 8u ? 8u : rounded) - 8u;
                    sf_exp = sf_exp < 105u ? 105u : sf_exp;
                    const float inv = __uint_as_float((254u - sf_exp) << 23);
                    const uint32_t row_addr = smem_u32(buf) + lane * 32;
                    #pragma unroll
                    for (uint32_t j = 0; j < 2; ++j) {
                        uint32_t w[4];
                        #pragma unroll
                        for (uint32_t q = 0; q < 4; ++q)
                            w[q] = cvt_e4m3x4(scale_pos_zero(__uint_as_float(g[16 * j + 4 * q + 0]), inv), scale_pos_zero(__uint_as_float(g[16 * j + 4 * q + 1]), inv),
                                              scale_pos_zero(__uint_as_float(g[16 * j + 4 * q + 2]), inv), scale_pos_zero(__uint_as_float(g[16 * j + 4 * q + 3]), inv));
                        st_shared_v4(row_addr + j * 16, w[0], w[1], w[2], w[3]);
                    }
                    const uint32_t col0 = t.n0 + s * 32;
                    if (row < t.m_end && col0 < p.n)
                        reinterpret_cast<uint8_t*>(p.sfd)[(static_cast<size_t>(t.ga * (p.n / 128) + col0 / 128) * p.sfd_stride + row) * 4 + (col0 % 128) / 32] =
                            static_cast<uint8_t>(sf_exp);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (col0 < p.n && row0 < t.m_end)
                            tma_store_3d(&tmap_d, buf, static_cast<int32_t>(col0), static_cast<int32_t>(row0), static_cast<int32_t>(t.gd));
                        tma_store_commit();
                    }
                    buf_idx ^= 1;
                }
                continue;
            }
            auto process = [&](uint32_t (&v)[32], uint32_t s) {
                const uint32_t sub_in_buf = s % kSubsPerBuf;
                uint8_t* buf = buf0 + buf_idx * kEpiBufBytes;
                if (sub_in_buf == 0) {
                    // the store issued two buffers ago must have finished reading this buffer
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                }
                if (p.has_alpha) {
                    #pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * p.alpha);
                }
                const uint32_t row_addr = smem_u32(buf) + lane * kRowBytes;
                if constexpr (kOut == kOutBf16) {
                    // 64-byte rows, 64B swizzle: 16-byte chunk index ^ ((row / 2) % 4)
                    #pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        const uint32_t chunk = j ^ ((lane >> 1) & 3);
                        st_shared_v4(row_addr + chunk * 16,
                                     pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1])),
                                     pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                                     pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                                     pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
                    }
                } else if constexpr (kOut == kOutF32) {
                    #pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        const uint32_t chunk = j ^ (lane & 7);
                        st_shared_v4(row_addr + chunk * 16, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                } else {
                    // round to bf16 first, take the block maximum on the bf16 bit patterns, pick the
                    // power-of-two scale that brings it under 448, quantise the rounded values
                    uint32_t amax = 0;
                    #pragma unroll
                    for (uint32_t i = 0; i < 32; i += 2) {
                        const uint32_t pk = pack_bf16x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                        v[i] = pk << 16;            // bf16 widened back to f32 bits
                        v[i + 1] = pk & 0xFFFF0000u;
                        amax = max(amax, max((pk & 0x7FFFu), ((pk >> 16) & 0x7FFFu)));
                    }
                    const uint32_t rounded = (amax + 0x7Fu - 0x60u) >> 7;
                    uint32_t sf_exp = (rounded < 8u ? 8u : rounded) - 8u;
                    sf_exp = sf_exp < 105u ? 105u : sf_exp;
                    const float inv = __uint_as_float((254u - sf_exp) << 23);
                    sf_word |= sf_exp << (8 * sub_in_buf);
                    #pragma unroll
                    for (uint32_t j = 0; j < 2; ++j) {
                        const uint32_t chunk = (sub_in_buf * 2 + j) ^ (lane & 7);
                        uint32_t w[4];
                        #pragma unroll
                        for (uint32_t q = 0; q < 4; ++q)
                            w[q] = cvt_e4m3x4(scale_pos_zero(__uint_as_float(v[16 * j + 4 * q + 0]), inv), scale_pos_zero(__uint_as_float(v[16 * j + 4 * q + 1]), inv),
                                              scale_pos_zero(__uint_as_float(v[16 * j + 4 * q + 2]), inv), scale_pos_zero(__uint_as_float(v[16 * j + 4 * q + 3]), inv));
                        st_shared_v4(row_addr + chunk * 16, w[0], w[1], w[2], w[3]);
                    }
                }
                if constexpr (kOut != kOutFp8) {
                    if (p.mask_rows && row0 < t.m_end && row0 + 32 > t.m_end) {
                        // this box crosses the end of the group: each lane writes its own row's 32 columns, if the row is valid
                        const uint32_t col0 = t.n0 + s * 32;
                        if (row < t.m_end) {
                            constexpr uint32_t kElem = kOut == kOutBf16 ? 2 : 4;
                            uint8_t* dst = static_cast<uint8_t*>(p.out_ptr) + (static_cast<size_t>(row) * p.out_ld + col0) * kElem;
                            #pragma unroll
                            for (uint32_t i = 0; i < 32; ++i) {
                                if (col0 + i < p.n) {
                                    if constexpr (kOut == kOutBf16)
                                        reinterpret_cast<uint16_t*>(dst)[i] = static_cast<uint16_t>(pack_bf16x2(__uint_as_float(v[i]), 0.0f) & 0xFFFFu);
                                    else
                                        reinterpret_cast<uint32_t*>(dst)[i] = v[i];
                                }
                            }
                        }
                        return;
                    }
                }
                if (sub_in_buf + 1 == kSubsPerBuf) {
                    const uint32_t col0 = t.n0 + (s / kSubsPerBuf) * kColsPerBuf;
                    if constexpr (kOut == kOutFp8) {
                        if (row < t.m_end && col0 < p.n)
                            p.sfd[static_cast<size_t>(t.ga * (p.n / 128) + col0 / 128) * p.sfd_stride + row] = sf_word;
                        sf_word = 0;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (col0 < p.n && row0 < t.m_end) {
                            if (p.accumulate) tma_reduce_add_3d(&tmap_d, buf, static_cast<int32_t>(col0), static_cast<int32_t>(row0), static_cast<int32_t>(t.gd));
                            else tma_store_3d(&tmap_d, buf, static_cast<int32_t>(col0), static_cast<int32_t>(row0), static_cast<int32_t>(t.gd));
                        }
                        tma_store_commit();
                    }
                    buf_idx ^= 1;
                }
            };
            // two register sets: the TMEM load of the next 32 columns is in flight while the current ones are
            // converted and staged
            uint32_t va[32], vb[32];
            tmem_ld_32x32b_x32(taddr, va);
            for (uint32_t s = 0; s < num_subs; s += 2) {
                tmem_ld_wait_x32(va);
                const bool has_b = s + 1 < num_subs;
                if (has_b) tmem_ld_32x32b_x32(taddr + (s + 1) * 32, vb);
                else release_accumulator();
                process(va, s);
                if (has_b) {
                    tmem_ld_wait_x32(vb);
                    if (s + 2 < num_subs) tmem_ld_32x32b_x32(taddr + (s + 2) * 32, va);
                    else release_accumulator();
                    process(vb, s + 1);
                }
            }
        }
        if (lane == 0) tma_store_wait<0>();
        __syncwarp();
      }
    }

    if constexpr (kSwap) {
        if (p.cluster_splits > 1) {
            // Every CTA (pair) of the cluster now holds, in TMEM, the partial sums of one K range of the same tile.  Output rows
            // (accumulator columns) are dealt out in slices, one per K range: every CTA sends each slice to the CTA that owns it
            // (same rank within the pair), the owner adds the slices in range order and stores its rows.  The exchange buffer
            // lies over the stage buffers, which nobody touches once all main loops of the cluster are over.
            Scheduler sched(p, kCtas, true, cluster_rank);
            Tile t;
            const bool has_tile = sched.next(t);
            const uint32_t num_ranges = p.cluster_splits;
            const uint32_t n_tile = has_tile ? sched.umma_n(t, kCtas) : 0u;
            const uint32_t rows_per = (n_tile + num_ranges - 1) / num_ranges;
            float* red = reinterpret_cast<float*>(smem);       // [source range][row of the slice][128 lanes]
            tc_fence_before();
            cluster_sync();
            tc_fence_after();
            if (warp >= 4 && has_tile && *abort_flag == 0) {
                const uint32_t ew = warp - 4;
                const uint32_t taddr = tmem_base + ((ew * 32) << 16);
                const uint32_t my_slot = smem_u32(red) + (sched.split * rows_per * kBlockM + ew * 32 + lane) * 4;
                for (uint32_t s = 0; s * 32 < n_tile; ++s) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + s * 32, v);
                    tmem_ld_wait_x32(v);
                    #pragma unroll
                    for (uint32_t c = 0; c < 32; ++c) {
                        const uint32_t row = s * 32 + c;
                        if (row < n_tile) {
                            const uint32_t owner = row / rows_per, local = row - owner * rows_per;
                            st_shared_cluster_u32(mapa_u32(my_slot + local * kBlockM * 4, owner * kCtas + cta_rank), v[c]);
                        }
                    }
                }
            }
            cluster_sync();      // release / acquire across the cluster: every slice has arrived
            if (has_tile && *abort_flag == 0) {
                const uint32_t rows_left = t.n_end > t.n0 ? t.n_end - t.n0 : 0u;
                const uint32_t valid = rows_left < n_tile ? rows_left : n_tile;
                const uint32_t row_lo = sched.split * rows_per;
                const uint32_t rows_here = row_lo < valid ? (valid - row_lo < rows_per ? valid - row_lo : rows_per) : 0u;
                constexpr uint32_t kElem = kOut == kOutBf16 ? 2 : 4;
                for (uint32_t i = threadIdx.x; i < rows_here * kBlockM; i += kNumThreads) {
                    const uint32_t local = i / kBlockM, col = i % kBlockM;
                    float acc = red[local * kBlockM + col];
                    for (uint32_t src = 1; src < num_ranges; ++src) acc += red[(src * rows_per + local) * kBlockM + col];
                    const uint32_t col_out = t.m0 + cta_rank * kBlockM + col;
                    if (col_out < t.m_end) {
                        uint8_t* dst = static_cast<uint8_t*>(p.out_ptr) +
                                       ((static_cast<size_t>(t.gd) * p.out_group_rows + t.n0 + row_lo + local) * p.out_ld + col_out) * kElem;
                        if constexpr (kOut == kOutBf16 || kOut == kOutF32) store_output<kOut>(dst, acc, p);
                    }
                }
            }
        }
    }

    tc_fence_before();
    if constexpr (kCtas == 2) cluster_sync(); else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<kCtas>(tmem_base, kTmemCols);
    }
}

// Bytes of dynamic shared memory the kernel needs for a configuration (host side).
inline uint32_t gemm_smem_bytes(uint32_t block_n, uint32_t ctas, uint32_t out_kind, uint32_t stages, uint32_t sfa_words, uint32_t sfb_words,
                                uint32_t halves, bool swap = false) {
    const uint32_t sf_block_n = (block_n + 127) / 128 * 128;
    const uint32_t per_stage = halves * (kBlockM * kBlockKBytes + block_n / ctas * kBlockKBytes) + 512 * sfa_words + sf_block_n * 4 * sfb_words;
    return 1024 + stages * per_stage + (swap ? 0u : 8 * epilogue_buf_bytes(out_kind)) + (4 * kMaxStages + 5) * 8 + 16;
}
// Bytes of the operand stage buffers alone: the K-range exchange of the swapped family lays its buffer over them.
inline uint32_t gemm_stage_bytes(uint32_t block_n, uint32_t ctas, uint32_t stages, uint32_t halves) {
    return stages * halves * (kBlockM * kBlockKBytes + block_n / ctas * kBlockKBytes);
}

}  // namespace dg
