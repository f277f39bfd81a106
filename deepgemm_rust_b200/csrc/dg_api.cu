// Host side of the C ABI declared in include/dgb200.h: context, argument validation, tile
// configuration, tensor-map encoding and kernel launches.  No CPU compute path exists here:
// every entry point either launches sm_100a kernels or returns an error.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/dgb200.h"
#include "dg_cast_kernels.cuh"
#include "dg_gemm_kernel.cuh"
#include "dg_gemm_f32scale.cuh"
#include "dg_moe_kernels.cuh"

namespace {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define DG_CUDA(expr)                                                                            \
    do {                                                                                         \
        cudaError_t e_ = (expr);                                                                 \
        if (e_ != cudaSuccess) return fail(DG_ERR_DRIVER, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

std::atomic<uint32_t> g_mk_alignment{128};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

constexpr uint32_t kSmemCapacity = 232448;  // 227 KB opt-in maximum per CTA on sm_100

uint32_t align4(uint32_t x) { return (x + 3) / 4 * 4; }
uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

}  // namespace

struct dg_ctx {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int num_sms = 0;
    dg::Status* status = nullptr;       // device word block the kernels report into
    uint32_t* group_ends = nullptr;     // scratch for the contiguous layout's group-end table
    uint32_t group_ends_cap = 0;
    float* splitk_ws = nullptr;         // scratch for the f32 partial products of K-split GEMMs
    size_t splitk_ws_cap = 0;           // in floats
    uint32_t* bridge_sf[2] = {nullptr, nullptr};   // packed scale words built from f32 scales by the f32-scale entry points
    size_t bridge_sf_cap[2] = {0, 0};              // in words
};

extern "C" {

const char* dg_last_error(void) { return g_last_error.c_str(); }

static int ctx_create(int ordinal, void* stream, bool adopt, dg_ctx** out) {
    if (out == nullptr) return fail(DG_ERR_SHAPE, "null output pointer");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(DG_ERR_DRIVER, "no CUDA device available (%s); this library has no CPU path", cudaGetErrorString(e));
    if (ordinal < 0 || ordinal >= count) return fail(DG_ERR_SHAPE, "device ordinal %d out of range (0..%d)", ordinal, count - 1);
    DG_CUDA(cudaSetDevice(ordinal));
    cudaDeviceProp prop;
    DG_CUDA(cudaGetDeviceProperties(&prop, ordinal));
    if (prop.major != 10)
        return fail(DG_ERR_UNSUPPORTED, "device %d is sm_%d%d; these kernels are built for sm_100a only", ordinal, prop.major, prop.minor);
    if (encode_tiled_fn() == nullptr) return fail(DG_ERR_DRIVER, "cuTensorMapEncodeTiled not found in the driver");
    dg_ctx* c = new dg_ctx();
    c->ordinal = ordinal;
    c->num_sms = prop.multiProcessorCount;
    if (adopt) {
        c->stream = static_cast<cudaStream_t>(stream);
    } else {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return fail(DG_ERR_DRIVER, "cudaStreamCreate failed"); }
        c->owns_stream = true;
    }
    if (cudaMalloc(&c->status, sizeof(dg::Status)) != cudaSuccess || cudaMemset(c->status, 0, sizeof(dg::Status)) != cudaSuccess) {
        delete c;
        return fail(DG_ERR_DRIVER, "allocating the device status word failed");
    }
    *out = c;
    return DG_OK;
}

int dg_ctx_create(int ordinal, dg_ctx** out) { return ctx_create(ordinal, nullptr, false, out); }
int dg_ctx_create_on_stream(int ordinal, void* cuda_stream, dg_ctx** out) { return ctx_create(ordinal, cuda_stream, true, out); }

int dg_ctx_destroy(dg_ctx* ctx) {
    if (ctx == nullptr) return DG_OK;
    cudaSetDevice(ctx->ordinal);
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->group_ends) cudaFree(ctx->group_ends);
    if (ctx->splitk_ws) cudaFree(ctx->splitk_ws);
    for (int i = 0; i < 2; ++i)
        if (ctx->bridge_sf[i]) cudaFree(ctx->bridge_sf[i]);
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return DG_OK;
}

int dg_ctx_check_status(dg_ctx* ctx) {
    if (ctx == nullptr) return fail(DG_ERR_SHAPE, "null context");
    dg::Status st;
    DG_CUDA(cudaMemcpy(&st, ctx->status, sizeof(st), cudaMemcpyDeviceToHost));
    if (st.code != 0) {
        cudaMemset(ctx->status, 0, sizeof(st));
        return fail(DG_ERR_TIMEOUT, "a device-side wait ran out: block %u, site 0x%x, parity %u", st.block, st.site, st.extra);
    }
    return DG_OK;
}

int dg_ctx_sync(dg_ctx* ctx) {
    if (ctx == nullptr) return fail(DG_ERR_SHAPE, "null context");
    DG_CUDA(cudaStreamSynchronize(ctx->stream));
    return dg_ctx_check_status(ctx);
}

int dg_ctx_num_sms(const dg_ctx* ctx, int* out) {
    if (ctx == nullptr || out == nullptr) return fail(DG_ERR_SHAPE, "null argument");
    *out = ctx->num_sms;
    return DG_OK;
}
void* dg_ctx_stream(const dg_ctx* ctx) { return ctx ? ctx->stream : nullptr; }
int dg_ctx_set_stream(dg_ctx* ctx, void* cuda_stream) {
    if (ctx == nullptr) return fail(DG_ERR_SHAPE, "null context");
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    ctx->owns_stream = false;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    return DG_OK;
}

// ------------------------------------------------------------------ size helpers / knobs
uint32_t dg_sf_packed_cols(uint32_t k, uint32_t gran_k) { return gran_k ? ceil_div(k, gran_k * 4) : 0; }
uint32_t dg_sf_aligned_rows(uint32_t rows) { return align4(rows); }
size_t dg_sf_words(uint32_t rows, uint32_t k, uint32_t gran_k, uint32_t num_groups) {
    const uint32_t g = num_groups ? num_groups : 1;
    return static_cast<size_t>(dg_sf_packed_cols(k, gran_k)) * g * align4(rows / g);
}

int dg_set_mk_alignment_for_contiguous_layout(uint32_t value) {
    if (value < 16 || value > 256 || (value & (value - 1)) != 0)
        return fail(DG_ERR_SHAPE, "mk alignment must be a power of two in [16, 256], got %u", value);
    g_mk_alignment.store(value);
    return DG_OK;
}
uint32_t dg_get_mk_alignment_for_contiguous_layout(void) { return g_mk_alignment.load(); }
uint32_t dg_get_theoretical_mk_alignment_for_contiguous_layout(uint32_t arch_major) { return arch_major == 10 ? 256u : 128u; }

// ------------------------------------------------------------------------- heuristics
// Tile choice for 148 SMs / 227 KB shared memory / 512 TMEM columns.  A rows always ride the
// UMMA M dimension (128 per tile); BLOCK_N is picked from the widths the epilogue of the output
// type can store, minimising waves x per-tile cost; stages fill the shared memory left over.
// What the launcher needs to know about a choice (the public dg_config describes the same choice in the reference's terms).
struct KernelPlan {
    bool swap;                 // weights on the UMMA M dimension, activation rows on UMMA N
    uint32_t ctas, umma_n, halves, stages, accum, smem;
    uint32_t splits;           // K ranges summed by a second kernel (first tile family)
    uint32_t cluster_splits;   // K ranges summed inside a cluster (swapped family)
    uint32_t tiles;
};
static int choose_config(const dg_desc* d, uint32_t no_k_ranges, dg_config* out, KernelPlan* plan);
int dg_best_config(const dg_desc* d, dg_config* out) {
    KernelPlan plan;
    return choose_config(d, 0, out, &plan);
}

// no_k_ranges: the caller adds into the output (K ranges would need the sum to be written, not added)
static int choose_config(const dg_desc* d, uint32_t no_k_ranges, dg_config* out, KernelPlan* plan) {
    if (d == nullptr || out == nullptr) return fail(DG_ERR_SHAPE, "null argument");
    if ((d->a_bits != 8 && d->a_bits != 4) || (d->b_bits != 8 && d->b_bits != 4)) return fail(DG_ERR_SHAPE, "operand bits must be 8 or 4");
    if ((d->major_a_mn && d->a_bits == 4) || (d->major_b_mn && d->b_bits == 4)) return fail(DG_ERR_SHAPE, "FP4 operands must be K-major");
    // two packed e2m1 operands run on kind::mxf4 (256 elements per 128-byte slab); an e4m3 x e2m1 pair runs on
    // kind::mxf8f6f4 with the e2m1 side expanded to one code per byte by the TMA load (128 elements per slab)
    const bool mxf4 = d->a_bits == 4 && d->b_bits == 4;
    const uint32_t half_k = mxf4 ? 256 : 128;     // K elements of one 128-byte slab
    const uint32_t sms = d->num_sms ? d->num_sms : 148;
    const uint32_t groups = d->num_groups ? d->num_groups : 1;
    // the fused gate/up activation writes block_n / 2 columns per tile in 32-column scale blocks: widths of 64
    const bool swiglu = d->cd_dtype == DG_OUT_SWIGLU_FP8;
    const uint32_t step = d->cd_dtype == DG_OUT_FP8 ? 128 : (swiglu ? 64 : 32);
    const uint32_t align = g_mk_alignment.load();
    const char* force_n = getenv("DG_BLOCK_N");
    const char* force_ctas = getenv("DG_CTAS");
    const char* force_stages = getenv("DG_STAGES");

    const char* force_splits = getenv("DG_SPLITS");
    const char* force_halves = getenv("DG_K_SLABS");
    uint32_t best_n = 0, best_accum = 0, best_tiles = 0, best_ctas = 0, best_stages = 0, best_splits = 1, best_halves = 1;
    double best_cost = 0;
    // a stage holds one or two 128-byte K slabs per operand; two slabs halve the per-stage bookkeeping per UMMA
    for (uint32_t halves = 1; halves <= 2; ++halves) {
    if (force_halves && static_cast<uint32_t>(atoi(force_halves)) != halves) continue;
    const uint32_t block_k = half_k * halves;
    const uint32_t sfa_words = 4 * d->gran_a >= block_k ? 1 : block_k / (4 * d->gran_a);
    const uint32_t sfb_words = 4 * d->gran_b >= block_k ? 1 : block_k / (4 * d->gran_b);
    for (uint32_t ctas = 1; ctas <= 2; ++ctas) {
        if (force_ctas && static_cast<uint32_t>(atoi(force_ctas)) != ctas) continue;
        const uint32_t tile_m = 128 * ctas;
        // contiguous layout: a tile may run past its group's end into the next groups' rows; those rows are computed but
        // never stored (stores are 32 rows tall and stop at the group end; an alignment of 16 switches the last box of a
        // group to row-exact stores), so every alignment from 16 to 256 works with 128- and 256-row tiles
        if (ctas == 2 && sms < 2) continue;
        if (swiglu && ctas != 2) continue;        // gate rows on one CTA of the pair, up rows on the other
        // expected row-tiles.  Grouped layouts: a group of r valid rows needs ceil(r / tile_m) tiles, on average
        // r / tile_m + 1/2 when group sizes are spread out; the contiguous arena's m includes about half an alignment of
        // padding per group.
        double m_blocks;
        if (d->gemm_type == DG_GEMM_M_GROUPED_CONTIGUOUS) {
            const double per_group = groups ? static_cast<double>(d->m) / groups : d->m;
            const double valid = per_group > align / 2.0 ? per_group - align / 2.0 : per_group;
            m_blocks = groups > 1 ? groups * (valid / tile_m + 0.5) : ceil_div(d->m, tile_m);
        } else if (d->gemm_type == DG_GEMM_M_GROUPED_MASKED) {
            const double e = d->expected_m ? d->expected_m : d->m;
            m_blocks = groups * (e / tile_m + 0.5);
        } else {
            m_blocks = groups * ceil_div(d->m, tile_m);
        }
        const uint32_t workers = sms / ctas;
        for (uint32_t bn = step; bn <= 256; bn += step) {
            if (bn % (16 * ctas) != 0) continue;
            if (d->major_b_mn && (bn / ctas) % 128 != 0) continue;    // an MN-major B tile is made of whole 128-row boxes per CTA
            if (force_n && static_cast<uint32_t>(atoi(force_n)) != bn) continue;
            const uint32_t sf_cols = 4 * sfa_words + ceil_div(bn, 128) * 4 * sfb_words;
            if (bn + sf_cols > 512) continue;
            const uint32_t accum = 2 * bn + sf_cols <= 512 ? 2 : 1;
            if (swiglu && accum == 1 && !force_n) continue;   // its epilogue is long: only worth it behind a second accumulator
            const uint32_t tiles = static_cast<uint32_t>(m_blocks * ceil_div(d->n, bn) + 0.999);
            // cycles per tile, fitted to measurements on B200 (dense 4096x7168x4096, every width, 1 and 2 CTAs):
            // per k-block max(UMMA time, load time) + ~150 of issue-side overhead, where one UMMA (K = 32 bytes) takes
            // max(~118, bn / 2) cycles and a CTA receives its A tile (16 KB) plus bn/ctas rows of B at ~77 bytes per cycle;
            // a single-buffered accumulator exposes the whole epilogue (~10.5 cycles per column).
            const uint32_t total_kb = ceil_div(d->k, block_k);
            const double mma = 4.0 * (bn * 0.5 > 118.0 ? bn * 0.5 : 118.0);
            const double feed = (16384.0 + bn / ctas * 128.0) / 77.0;
            const double epilogue = swiglu ? (accum == 1 ? 40.0 * bn : 1.0 * bn) : (accum == 1 ? 10.5 * bn : 1.0 * bn);
            const double per_kb = halves * (mma > feed ? mma : feed) + 150.0;
            // K ranges (dense GEMMs with f32-summable outputs only): each range is a multiple of 4 k-blocks so scale words
            // never straddle ranges; the partial sums cost a second small kernel (launch + S reads of the M x N f32 tile set)
            const bool may_split = d->gemm_type == DG_GEMM_NORMAL && d->cd_dtype != DG_OUT_FP8 && !swiglu && d->n % 4 == 0 && !no_k_ranges;
            for (uint32_t splits = 1; splits <= 16; ++splits) {
                if (splits > 1 && (!may_split || halves > 1)) break;
                if (force_splits && static_cast<uint32_t>(atoi(force_splits)) != splits) continue;
                uint32_t kb_per = ceil_div(ceil_div(total_kb, splits), 4) * 4;
                if (splits > 1 && (kb_per < 8 || kb_per * (splits - 1) >= total_kb)) continue;   // every range non-empty, at least 8 k-blocks
                if (splits == 1) kb_per = total_kb;
                // K ranges store f32 partials whatever the caller's output type: size the staging buffers for that
                const uint32_t kernel_out = splits > 1 ? static_cast<uint32_t>(DG_OUT_F32) : d->cd_dtype;
                uint32_t stages = force_stages ? static_cast<uint32_t>(atoi(force_stages)) : dg::kMaxStages;
                if (stages > dg::kMaxStages) stages = dg::kMaxStages;
                while (stages > 1 && dg::gemm_smem_bytes(bn, ctas, kernel_out, stages, sfa_words, sfb_words, halves) > kSmemCapacity) --stages;
                if (stages < 1 || dg::gemm_smem_bytes(bn, ctas, kernel_out, stages, sfa_words, sfb_words, halves) > kSmemCapacity) continue;
                if (stages < 3 && !force_stages) continue;
                const uint32_t waves = ceil_div(tiles * splits, workers);
                const double tile_cost = kb_per * per_kb + (splits > 1 ? 2.0 * bn : epilogue) + 600.0;
                const double reduce = splits > 1 ? 9000.0 + static_cast<double>(splits) * d->m * d->n * 4.0 / 3000.0 : 0.0;
                // every CTA pulls its A slab (16 KB) and its share of B from L2 for each 128 bytes of K; with many small groups
                // (weights read once, little reuse) that aggregate stream, ~9000 bytes per cycle on this part, is the limit
                const double l2_bytes = static_cast<double>(tiles) * ctas * ceil_div(d->k, half_k) * (16384.0 + bn / ctas * 128.0);
                const double l2_floor = l2_bytes / 9000.0;
                const double compute = waves * tile_cost;
                const double cost = (compute > l2_floor ? compute : l2_floor) + reduce;
                if (best_n == 0 || cost < best_cost * (1.0 - 1e-9)) {
                    best_n = bn; best_cost = cost; best_accum = accum; best_tiles = tiles; best_ctas = ctas; best_stages = stages;
                    best_splits = splits; best_halves = halves;
                }
            }
        }
    }
    }
    // ---- the swapped family: weight rows on UMMA M, activation rows on UMMA N (bf16 / f32 outputs).  DG_SWAP=1 selects it
    // wherever it applies.  It is not the default anywhere yet: measured on B200 it streams the weights of skinny and
    // small-group problems more slowly than the first family, which keeps more weight bytes in flight per SM.
    {
        const char* force_swap = getenv("DG_SWAP");
        const bool forced = force_swap && atoi(force_swap) != 0, forbidden = force_swap && atoi(force_swap) == 0;
        const bool plain_out = d->cd_dtype == DG_OUT_BF16 || d->cd_dtype == DG_OUT_F32;
        const bool dense = d->gemm_type == DG_GEMM_NORMAL || d->gemm_type == DG_GEMM_BATCHED;
        const bool want = forced && !d->major_a_mn && !d->major_b_mn;   // MN-major operands: first family only
        if (plain_out && want && !forbidden) {
            uint32_t s_n = 0, s_ctas = 0, s_halves = 0, s_stages = 0, s_accum = 0, s_split = 1, s_tiles = 0;
            double s_cost = 0;
            for (uint32_t halves = 1; halves <= 2; ++halves) {
                if (force_halves && static_cast<uint32_t>(atoi(force_halves)) != halves) continue;
                const uint32_t block_k = half_k * halves;
                // kernel operand A is the caller's b (weights), kernel operand B the caller's a (activation rows)
                const uint32_t sfa_words = 4 * d->gran_b >= block_k ? 1 : block_k / (4 * d->gran_b);
                const uint32_t sfb_words = 4 * d->gran_a >= block_k ? 1 : block_k / (4 * d->gran_a);
                const uint32_t total_kb = ceil_div(d->k, block_k);
                for (uint32_t ctas = 1; ctas <= 2; ++ctas) {
                    if (force_ctas && static_cast<uint32_t>(atoi(force_ctas)) != ctas) continue;
                    if (ctas == 2 && sms < 2) continue;
                    const uint32_t step_n = 16 * ctas;
                    // rows a tile may have: everything a dense problem has (up to 256), else 256 and the tile's UMMA N follows the group
                    uint32_t bn = dense && d->m <= 256 ? ceil_div(d->m, step_n) * step_n : 256;
                    if (force_n) bn = static_cast<uint32_t>(atoi(force_n));
                    if (bn == 0 || bn > 256 || bn % step_n != 0) continue;
                    const uint32_t sf_cols = 4 * sfa_words + ceil_div(bn, 128) * 4 * sfb_words;
                    if (bn + sf_cols > 512) continue;
                    const uint32_t accum = 2 * bn + sf_cols <= 512 ? 2 : 1;
                    const uint32_t a_blocks = ceil_div(d->n, 128 * ctas);
                    double row_blocks;
                    if (dense) row_blocks = static_cast<double>(groups) * ceil_div(d->m, bn);
                    else if (d->gemm_type == DG_GEMM_M_GROUPED_CONTIGUOUS) {
                        const double per_group = static_cast<double>(d->m) / groups;
                        row_blocks = groups * ((per_group > align / 2.0 ? per_group - align / 2.0 : per_group) / bn + 0.5);
                    } else row_blocks = groups * (static_cast<double>(d->expected_m ? d->expected_m : d->m) / bn + 0.5);
                    const uint32_t tiles = static_cast<uint32_t>(row_blocks * a_blocks + 0.999);
                    const uint32_t max_split = d->gemm_type == DG_GEMM_NORMAL ? 8 / ctas : 1;
                    for (uint32_t split = 1; split <= max_split; ++split) {
                        if (force_splits && static_cast<uint32_t>(atoi(force_splits)) != split) continue;
                        const uint32_t kb_per = ceil_div(total_kb, split);
                        if (split > 1 && total_kb < 2 * split) continue;       // at least two k-blocks per range
                        uint32_t stages = force_stages ? static_cast<uint32_t>(atoi(force_stages)) : dg::kMaxStages;
                        if (stages > dg::kMaxStages) stages = dg::kMaxStages;
                        while (stages > 1 && dg::gemm_smem_bytes(bn, ctas, d->cd_dtype, stages, sfa_words, sfb_words, halves, true) > kSmemCapacity) --stages;
                        if (dg::gemm_smem_bytes(bn, ctas, d->cd_dtype, stages, sfa_words, sfb_words, halves, true) > kSmemCapacity) continue;
                        if (stages < 3 && !force_stages) continue;
                        // the exchange buffer of the K ranges lies over the stage buffers
                        if (split > 1 && dg::gemm_stage_bytes(bn, ctas, stages, halves) < split * ceil_div(bn, split) * 512) continue;
                        const double bytes_kb = halves * (16384.0 + bn / ctas * 128.0);                  // per CTA and k-block
                        const double stream = kb_per * bytes_kb / 64.0;
                        const double mma = kb_per * halves * 4.0 * (bn * 0.5 > 118.0 ? bn * 0.5 : 118.0);
                        const double per_tile = (stream > mma ? stream : mma) + (split > 1 ? 3500.0 : (accum == 1 ? 12.0 * bn : 2.0 * bn)) + 2500.0;
                        const double ctas_total = static_cast<double>(tiles) * split * ctas;
                        const double waves = ctas_total <= sms ? 1.0 : ctas_total / sms;               // the hardware refills SMs as clusters finish
                        const double hbm = (static_cast<double>(d->n) * groups * d->k * (d->b_bits / 8.0) + static_cast<double>(d->m) * d->k + 2.0 * d->m * d->n) / 3300.0;
                        const double l2 = ctas_total * kb_per * bytes_kb / 9000.0;
                        double cost = waves * per_tile;
                        if (hbm > cost) cost = hbm;
                        if (l2 > cost) cost = l2;
                        cost += 0.1 * per_tile + l2 * 0.01;      // among equals: more CTAs in flight, fewer bytes through L2
                        if (s_n == 0 || cost < s_cost * (1.0 - 1e-9)) {
                            s_n = bn; s_ctas = ctas; s_halves = halves; s_stages = stages; s_accum = accum; s_split = split; s_tiles = tiles;
                            s_cost = cost;
                        }
                    }
                }
            }
            if (s_n != 0) {
                const uint32_t block_k = half_k * s_halves;
                const uint32_t sfa_words = 4 * d->gran_b >= block_k ? 1 : block_k / (4 * d->gran_b);
                const uint32_t sfb_words = 4 * d->gran_a >= block_k ? 1 : block_k / (4 * d->gran_a);
                plan->swap = true;
                plan->ctas = s_ctas; plan->umma_n = s_n; plan->halves = s_halves; plan->stages = s_stages; plan->accum = s_accum;
                plan->splits = 1; plan->cluster_splits = s_split; plan->tiles = s_tiles;
                plan->smem = dg::gemm_smem_bytes(s_n, s_ctas, d->cd_dtype, s_stages, sfa_words, sfb_words, s_halves, true);
                out->swap_ab = 1;
                out->block_m = s_n;            // activation rows per tile (an upper bound: a tile's UMMA N follows its rows)
                out->block_n = 128 * s_ctas;   // weight rows per tile
                out->block_k = block_k;
                out->cluster_m = 1;
                out->cluster_n = s_ctas;
                out->num_stages = s_stages;
                out->num_accum_stages = s_accum;
                out->smem_size = plan->smem;
                out->num_tiles = s_tiles;
                out->num_splits = s_split;
                return DG_OK;
            }
            if (forced) return fail(DG_ERR_SHAPE, "no tile configuration of the swapped family fits (DG_BLOCK_N=%s DG_CTAS=%s)", force_n ? force_n : "",
                                    force_ctas ? force_ctas : "");
        }
    }
    if (best_n == 0) return fail(DG_ERR_SHAPE, "no tile configuration fits (DG_BLOCK_N=%s DG_CTAS=%s)", force_n ? force_n : "", force_ctas ? force_ctas : "");
    const uint32_t stages = best_stages;
    plan->swap = false;
    plan->ctas = best_ctas; plan->umma_n = best_n; plan->halves = best_halves; plan->stages = best_stages; plan->accum = best_accum;
    plan->splits = best_splits; plan->cluster_splits = 1; plan->tiles = best_tiles;
    out->swap_ab = 0;
    out->block_m = 128 * best_ctas;
    out->block_n = best_n;
    const uint32_t block_k = half_k * best_halves;
    const uint32_t sfa_words = 4 * d->gran_a >= block_k ? 1 : block_k / (4 * d->gran_a);
    const uint32_t sfb_words = 4 * d->gran_b >= block_k ? 1 : block_k / (4 * d->gran_b);
    out->block_k = block_k;
    out->cluster_m = best_ctas;
    out->cluster_n = 1;
    out->num_stages = stages;
    out->num_accum_stages = best_accum;
    out->smem_size = dg::gemm_smem_bytes(best_n, best_ctas, best_splits > 1 ? static_cast<uint32_t>(DG_OUT_F32) : d->cd_dtype, stages, sfa_words,
                                         sfb_words, best_halves);
    out->num_tiles = best_tiles;
    out->num_splits = best_splits;
    plan->smem = out->smem_size;
    return DG_OK;
}

}  // extern "C"

namespace {

// ----------------------------------------------------------------------- tensor maps
int encode_map(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, const void* base, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle, const char* what) {
    cuuint64_t gdim[4], gstride[3];
    cuuint32_t gbox[4], estride[4] = {1, 1, 1, 1};
    for (uint32_t i = 0; i < rank; ++i) { gdim[i] = dims[i]; gbox[i] = box[i]; }
    for (uint32_t i = 0; i + 1 < rank; ++i) gstride[i] = strides_bytes[i];
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return fail(DG_ERR_SHAPE, "%s: base address must be 16-byte aligned", what);
    for (uint32_t i = 0; i + 1 < rank; ++i)
        if (gstride[i] % 16 != 0) return fail(DG_ERR_SHAPE, "%s: stride %llu bytes is not a multiple of 16", what, (unsigned long long)gstride[i]);
    CUresult r = encode_tiled_fn()(map, dtype, rank, const_cast<void*>(base), gdim, gstride, gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DG_ERR_DRIVER, "cuTensorMapEncodeTiled(%s) failed with %d", what, static_cast<int>(r));
    return DG_OK;
}

int check_operand(const dg_lp_operand* op, const char* name, uint32_t total_rows, uint32_t groups) {
    if (op == nullptr || op->data == nullptr || op->sf == nullptr) return fail(DG_ERR_SHAPE, "%s: null operand", name);
    if (op->bits != 8 && op->bits != 4) return fail(DG_ERR_SHAPE, "invalid bits %u", op->bits);
    if (op->gran_k != 32 && op->gran_k != 128) return fail(DG_ERR_SHAPE, "invalid gran_k %u", op->gran_k);
    if (op->major_mn && op->bits == 4) return fail(DG_ERR_SHAPE, "%s: FP4 operands must be K-major", name);
    if (op->bits == 4 && (op->k % 128 != 0 || op->ld % 128 != 0)) return fail(DG_ERR_SHAPE, "FP4 k and ld must be multiples of 128");
    if (op->bits == 4 && op->gran_k != 32) return fail(DG_ERR_UNSUPPORTED, "FP4 operands need gran_k = 32");
    if (op->k == 0 || op->k % op->gran_k != 0) return fail(DG_ERR_SHAPE, "k (%u) must be a multiple of the SF granularity (%u)", op->k, op->gran_k);
    if (op->major_mn) {
        // (groups, k, ld) bytes: the rows of a group are contiguous, ld is the pitch between two k
        const uint32_t g = groups ? groups : 1;
        if (op->ld < total_rows / g) return fail(DG_ERR_SHAPE, "%s: MN-major ld (%u) smaller than the rows of a group (%u)", name, op->ld, total_rows / g);
        if (op->ld % 16 != 0) return fail(DG_ERR_SHAPE, "%s: MN-major pitch %u bytes must be a multiple of 16", name, op->ld);
        const size_t need = static_cast<size_t>(g) * op->k * op->ld;
        if (op->data_len < need) return fail(DG_ERR_SHAPE, "data buffer too small: %zu < %zu", op->data_len, need);
        const size_t sf_words = dg_sf_words(total_rows, op->k, op->gran_k, groups);
        if (op->sf_len < sf_words) return fail(DG_ERR_SHAPE, "sf buffer too small: %zu < %zu", op->sf_len, sf_words);
        return DG_OK;
    }
    if (op->ld < op->k) return fail(DG_ERR_SHAPE, "%s: ld (%u) smaller than k (%u)", name, op->ld, op->k);
    const uint32_t row_bytes = op->bits == 4 ? op->ld / 2 : op->ld;
    if (row_bytes % 16 != 0) return fail(DG_ERR_SHAPE, "%s: row pitch %u bytes must be a multiple of 16", name, row_bytes);
    const size_t storage = static_cast<size_t>(total_rows) * row_bytes;
    if (op->data_len < storage) return fail(DG_ERR_SHAPE, "data buffer too small: %zu < %zu", op->data_len, storage);
    const size_t sf_need = dg_sf_words(total_rows, op->k, op->gran_k, groups);
    if (op->sf_len < sf_need) return fail(DG_ERR_SHAPE, "sf buffer too small: %zu < %zu", op->sf_len, sf_need);
    return DG_OK;
}

struct Problem {
    uint32_t type;
    uint32_t m;            // rows per group (contiguous: whole arena)
    uint32_t n, k, groups;
    uint32_t expected_m;
    const uint32_t* layout;
    bool bf16 = false;     // operands are bf16 rows described as 2k bytes each; no scale factors (dg_bf16_gemm)
};

// DG_PDL=0 launches every kernel fully serialised (for comparisons and debugging).
bool pdl_enabled() {
    static const bool on = [] { const char* v = getenv("DG_PDL"); return !(v && strcmp(v, "0") == 0); }();
    return on;
}

template <bool kBf16>
cudaError_t launch_reduce(uint32_t blocks, cudaStream_t stream, const float* partial, uint32_t splits, uint32_t m, uint32_t n, uint32_t pitch,
                          float alpha, void* out, uint32_t out_ld) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dg::dg_splitk_reduce_kernel<kBf16>, partial, splits, m, n, pitch, alpha, out, out_ld);
}

// The opt-in to the full shared-memory carve-out is per kernel instantiation and per device; the first
// call also makes the runtime load that kernel's image.
template <uint32_t kFmt, uint32_t kOut, uint32_t kCtas, bool kSwap = false>
cudaError_t configure_kernel() {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && (configured.load() & (1ull << dev))) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(dg::dg_gemm_kernel<kFmt, kOut, kCtas, kSwap>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kSmemCapacity));
    if (e == cudaSuccess && dev < 64) configured.fetch_or(1ull << dev);
    return e;
}

template <uint32_t kFmt, uint32_t kOut, uint32_t kCtas, bool kSwap = false>
cudaError_t launch_kernel(const dg::GemmParams& p, uint32_t grid, uint32_t smem, cudaStream_t stream, const CUtensorMap* maps) {
    auto kernel = dg::dg_gemm_kernel<kFmt, kOut, kCtas, kSwap>;
    cudaError_t e = configure_kernel<kFmt, kOut, kCtas, kSwap>();
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(dg::kNumThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCtas * (kSwap ? p.cluster_splits : 1u);   // swapped family: the K ranges of a tile share a cluster
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // the kernel waits for its predecessor itself (griddep_wait) after its set-up: let the two overlap
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, p, maps[0], maps[1], maps[2], maps[3], maps[4]);
}

template <uint32_t kFmt, uint32_t kCtas>
cudaError_t launch_swapped(int kind, const dg::GemmParams& p, uint32_t grid, uint32_t smem, cudaStream_t stream, const CUtensorMap* maps) {
    if (kind == DG_OUT_BF16) return launch_kernel<kFmt, dg::kOutBf16, kCtas, true>(p, grid, smem, stream, maps);
    if (kind == DG_OUT_F32) return launch_kernel<kFmt, dg::kOutF32, kCtas, true>(p, grid, smem, stream, maps);
    return cudaErrorInvalidValue;
}

template <uint32_t kFmt, uint32_t kCtas>
cudaError_t launch_by_out(int kind, const dg::GemmParams& p, uint32_t grid, uint32_t smem, cudaStream_t stream, const CUtensorMap* maps) {
    if (kind == DG_OUT_BF16) return launch_kernel<kFmt, dg::kOutBf16, kCtas>(p, grid, smem, stream, maps);
    if (kind == DG_OUT_F32) return launch_kernel<kFmt, dg::kOutF32, kCtas>(p, grid, smem, stream, maps);
    if constexpr (kFmt == dg::kFmtMxf8f6f4 && kCtas == 2)
        if (kind == DG_OUT_SWIGLU_FP8) return launch_kernel<kFmt, dg::kOutSwiGluFp8, kCtas>(p, grid, smem, stream, maps);
    if constexpr (kFmt != dg::kFmtBf16)
        if (kind == DG_OUT_FP8) return launch_kernel<kFmt, dg::kOutFp8, kCtas>(p, grid, smem, stream, maps);
    return cudaErrorInvalidValue;
}

template <uint32_t kFmt>
cudaError_t configure_contiguous_kernels_of() {
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutBf16, 1>();
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutBf16, 2>();
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutF32, 1>();
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutF32, 2>();
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutBf16, 1, true>();
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutBf16, 2, true>();
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutF32, 1, true>();
    if (e == cudaSuccess) e = configure_kernel<kFmt, dg::kOutF32, 2, true>();
    return e;
}
// Everything dg_m_grouped_fp8_fp4_gemm_contiguous[_ends] can launch, configured (and loaded) for the current device.
cudaError_t configure_contiguous_kernels() {
    cudaError_t e = configure_contiguous_kernels_of<dg::kFmtMxf8f6f4>();
    if (e == cudaSuccess) e = configure_contiguous_kernels_of<dg::kFmtMxf4>();
    if (e == cudaSuccess) e = configure_kernel<dg::kFmtMxf8f6f4, dg::kOutSwiGluFp8, 2>();
    cudaFuncAttributes fa;
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, dg::dg_group_ends_kernel);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, dg::dg_group_ends_scan_kernel);
    return e;
}

int launch_gemm(dg_ctx* ctx, const dg_lp_operand* a, const dg_lp_operand* b, const dg_out* out, const dg_epilogue* epi, const Problem& pr) {
    if (out == nullptr || out->buf == nullptr) return fail(DG_ERR_SHAPE, "null output");
    if (out->kind < DG_OUT_BF16 || out->kind > DG_OUT_SWIGLU_FP8) return fail(DG_ERR_SHAPE, "invalid output kind %d", out->kind);
    dg_epilogue e = {1.0f, 0, 0, 100};
    if (epi) e = *epi;
    const bool swiglu = out->kind == DG_OUT_SWIGLU_FP8;
    const bool fp8_out = out->kind == DG_OUT_FP8 || swiglu;
    if (fp8_out && (e.has_alpha || e.accumulate))
        return fail(DG_ERR_SHAPE, "the FP8-quantized output cannot combine alpha/accumulation");
    if (swiglu) {
        if (pr.bf16 || a->bits != 8 || b->bits != 8 || b->gran_k != 128)
            return fail(DG_ERR_UNSUPPORTED, "the fused gate/up activation takes e4m3 operands with per-128 weight scales");
        if (pr.n % 256 != 0) return fail(DG_ERR_SHAPE, "gate|up weights: rows per group (%u) must be 2 x a multiple of 128", pr.n);
    }
    if (e.accumulate && e.has_alpha) return fail(DG_ERR_SHAPE, "alpha and accumulation are mutually exclusive");
    const bool any_mn = !pr.bf16 && (a->major_mn || b->major_mn);
    if (any_mn && swiglu) return fail(DG_ERR_UNSUPPORTED, "the fused gate/up activation takes K-major operands");
    if (a->k != b->k) return fail(DG_ERR_SHAPE, "a.k (%u) != b.k (%u)", a->k, b->k);
    if (pr.m == 0 || pr.n == 0) return DG_OK;
    const bool contiguous = pr.type == DG_GEMM_M_GROUPED_CONTIGUOUS;
    const uint32_t a_groups = contiguous || pr.type == DG_GEMM_NORMAL ? 1 : pr.groups;
    const uint32_t b_groups = pr.type == DG_GEMM_NORMAL ? 1 : pr.groups;
    int rc = pr.bf16 ? DG_OK : check_operand(a, "a", pr.m * a_groups, a_groups);
    if (rc) return rc;
    rc = pr.bf16 ? DG_OK : check_operand(b, "b", pr.n * b_groups, b_groups);
    if (rc) return rc;
    const uint32_t d_rows = pr.m * a_groups;
    const uint32_t d_elem = out->kind == DG_OUT_F32 ? 4 : (fp8_out ? 1 : 2);
    const uint32_t n_out = swiglu ? pr.n / 2 : pr.n;     // output columns (the fused activation halves them)
    if (out->ld < n_out) return fail(DG_ERR_SHAPE, "output ld (%u) smaller than n (%u)", out->ld, n_out);
    if ((static_cast<size_t>(out->ld) * d_elem) % 16 != 0) return fail(DG_ERR_SHAPE, "output row pitch must be a multiple of 16 bytes");
    if (out->buf_len < static_cast<size_t>(d_rows - 1) * out->ld + n_out) return fail(DG_ERR_SHAPE, "output buffer too small");
    if (fp8_out) {
        if (out->sfd == nullptr) return fail(DG_ERR_SHAPE, "FP8 output needs sfd");
        if (n_out % 128 != 0) return fail(DG_ERR_SHAPE, "FP8 output needs n to be a multiple of 128");
        if (out->sfd_len < static_cast<size_t>(n_out / 128) * a_groups * align4(pr.m)) return fail(DG_ERR_SHAPE, "sfd buffer too small");
    }
    const uint32_t align = g_mk_alignment.load();
    if (swiglu && contiguous && align % 32 != 0)
        return fail(DG_ERR_UNSUPPORTED, "the fused gate/up activation needs an mk alignment of at least 32");

    dg_desc desc = {pr.type, pr.m, pr.n, pr.k, pr.groups, pr.expected_m, a->bits, b->bits, a->gran_k, b->gran_k,
                    static_cast<uint32_t>(out->kind), static_cast<uint32_t>(ctx->num_sms), (!pr.bf16 && a->major_mn) ? 1u : 0u,
                    (!pr.bf16 && b->major_mn) ? 1u : 0u};
    dg_config cfg;
    KernelPlan plan;
    rc = choose_config(&desc, e.accumulate ? 1u : 0u, &cfg, &plan);
    if (rc) return rc;
    const bool swap = plan.swap;
    // the swapped family runs the same kernel with the operands' roles exchanged: its operand A (UMMA M side) is the weights
    const dg_lp_operand* ka = swap ? b : a;
    const dg_lp_operand* kb = swap ? a : b;
    const uint32_t ka_rows = swap ? pr.n : pr.m, kb_rows = swap ? pr.m : pr.n;              // per group
    const uint32_t ka_groups = swap ? b_groups : a_groups, kb_groups = swap ? a_groups : b_groups;
    static const bool print_cfg = [] { const char* v = getenv("DG_PRINT_CONFIGS"); return v && strcmp(v, "0") != 0; }();
    if (print_cfg)
        fprintf(stderr, "[dgb200] type=%u m=%u n=%u k=%u groups=%u -> swap_ab=%u block=%ux%ux%u ctas=%u stages=%u accum=%u smem=%u tiles~%u splits=%u\n",
                pr.type, pr.m, pr.n, pr.k, pr.groups, cfg.swap_ab, cfg.block_m, cfg.block_n, cfg.block_k, plan.ctas, cfg.num_stages,
                cfg.num_accum_stages, cfg.smem_size, cfg.num_tiles, cfg.num_splits);

    const bool mxf4 = a->bits == 4 && b->bits == 4;
    const uint32_t block_k = cfg.block_k;
    const uint32_t splits = plan.splits;
    const uint32_t ws_pitch = align4(pr.n);
    if (splits > 1) {
        const size_t need = static_cast<size_t>(splits) * pr.m * ws_pitch;
        if (ctx->splitk_ws_cap < need) {
            DG_CUDA(cudaSetDevice(ctx->ordinal));
            if (ctx->splitk_ws) { cudaFree(ctx->splitk_ws); ctx->splitk_ws = nullptr; ctx->splitk_ws_cap = 0; }
            DG_CUDA(cudaMalloc(&ctx->splitk_ws, need * sizeof(float)));
            ctx->splitk_ws_cap = need;
        }
    }
    const uint32_t sfa_words = 4 * ka->gran_k >= block_k ? 1 : block_k / (4 * ka->gran_k);
    const uint32_t sfb_words = 4 * kb->gran_k >= block_k ? 1 : block_k / (4 * kb->gran_k);
    const uint32_t sf_block_n = ceil_div(plan.umma_n, 128) * 128;

    CUtensorMap maps[5];
    bool wide_k = false;
    {
        // packed e2m1 stays packed in shared memory for kind::mxf4 (16U4_ALIGN8B) and is expanded to one code per byte
        // for the mixed kind (16U4_ALIGN16B); dims and boxes of both are in logical 4-bit elements, pitches in bytes
        auto map_dtype = [&](uint32_t bits) {
            return bits == 8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : (mxf4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B);
        };
        const uint64_t a_pitch = ka->bits == 4 ? ka->ld / 2 : ka->ld, b_pitch = kb->bits == 4 ? kb->ld / 2 : kb->ld;
        uint64_t dims[3] = {pr.k, ka_rows, ka_groups};
        uint64_t strides[2] = {a_pitch, a_pitch * ka_rows};
        const uint32_t slab = mxf4 ? 256u : 128u;    // one 128-byte slab of K per TMA box
        uint32_t box[3] = {slab, dg::kBlockM, 1};
        if (!pr.bf16 && ka->major_mn) {
            // (groups, k, ld): rows innermost; a box is 128 rows x one slab of K
            dims[0] = ka_rows; dims[1] = pr.k; strides[0] = ka->ld; strides[1] = static_cast<uint64_t>(ka->ld) * pr.k;
            box[0] = 128; box[1] = slab;
        }
        // Two-slab stages of plain K-major byte operands: the operand is described as (128 bytes, rows, K slabs, groups) so that one
        // load brings both slabs of a stage (half as many TMA instructions per stage).  K must be whole slabs for that (a partial
        // last slab would read into the next row), otherwise the 3-D maps and one load per slab stay.
        const char* wide_env = getenv("DG_WIDE_K");
        // (not where the loads carry the evict-first hint: dense problems of a single row block, see below)
        const bool hinted = pr.type == DG_GEMM_NORMAL && pr.m <= (swap ? plan.umma_n : 128 * plan.ctas);
        wide_k = plan.halves == 2 && !mxf4 && ka->bits == 8 && kb->bits == 8 && pr.k % 128 == 0 && !(!pr.bf16 && (ka->major_mn || kb->major_mn)) &&
                 !hinted && !(wide_env && strcmp(wide_env, "0") == 0);
        if (wide_k) {
            uint64_t d4[4] = {128, ka_rows, pr.k / 128, ka_groups};
            uint64_t s4[3] = {a_pitch, 128, a_pitch * ka_rows};
            uint32_t b4[4] = {128, dg::kBlockM, 2, 1};
            rc = encode_map(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, ka->data, d4, s4, b4, CU_TENSOR_MAP_SWIZZLE_128B, "A");
            if (rc) return rc;
            uint64_t e4[4] = {128, kb_rows, pr.k / 128, kb_groups};
            uint64_t t4[3] = {b_pitch, 128, b_pitch * kb_rows};
            uint32_t c4[4] = {128, plan.umma_n / plan.ctas, 2, 1};
            rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, kb->data, e4, t4, c4, CU_TENSOR_MAP_SWIZZLE_128B, "B");
            if (rc) return rc;
        } else {
        rc = encode_map(&maps[0], map_dtype(ka->bits), 3, ka->data, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "A");
        if (rc) return rc;
        uint64_t bdims[3] = {pr.k, kb_rows, kb_groups};
        uint64_t bstrides[2] = {b_pitch, b_pitch * kb_rows};
        uint32_t bbox[3] = {slab, plan.umma_n / plan.ctas, 1};
        if (!pr.bf16 && kb->major_mn) {
            bdims[0] = kb_rows; bdims[1] = pr.k; bstrides[0] = kb->ld; bstrides[1] = static_cast<uint64_t>(kb->ld) * pr.k;
            bbox[0] = 128; bbox[1] = slab;
        }
        rc = encode_map(&maps[1], map_dtype(kb->bits), 3, kb->data, bdims, bstrides, bbox, CU_TENSOR_MAP_SWIZZLE_128B, "B");
        if (rc) return rc;
        }
    }
    const uint32_t sfa_cols = dg_sf_packed_cols(pr.k, ka->gran_k), sfb_cols = dg_sf_packed_cols(pr.k, kb->gran_k);
    {
        // bf16 operands carry no scales: the kernel never issues these loads, the maps only have to be well-formed
        uint64_t dims[2] = {align4(ka_rows), static_cast<uint64_t>(sfa_cols) * ka_groups};
        uint64_t strides[1] = {static_cast<uint64_t>(align4(ka_rows)) * 4};
        uint32_t box[2] = {128, sfa_words};
        rc = encode_map(&maps[2], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, pr.bf16 ? ka->data : ka->sf, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, "SFA");
        if (rc) return rc;
        uint64_t bdims[2] = {align4(kb_rows), static_cast<uint64_t>(sfb_cols) * kb_groups};
        uint64_t bstrides[1] = {static_cast<uint64_t>(align4(kb_rows)) * 4};
        uint32_t bbox[2] = {swiglu ? plan.umma_n / 2 : sf_block_n, sfb_words};   // fused activation: gate rows and up rows as two boxes
        rc = encode_map(&maps[3], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, pr.bf16 ? kb->data : kb->sf, bdims, bstrides, bbox, CU_TENSOR_MAP_SWIZZLE_NONE, "SFB");
        if (rc) return rc;
    }
    {
        // 32 rows per store; 32 columns of bf16 (64-byte rows) or f32, 128 columns of e4m3 (128-byte rows)
        if (splits > 1) {
            // K ranges write f32 partial tiles into the workspace, one plane per range
            uint64_t dims[3] = {pr.n, pr.m, splits};
            uint64_t strides[2] = {static_cast<uint64_t>(ws_pitch) * 4, static_cast<uint64_t>(ws_pitch) * 4 * pr.m};
            uint32_t box[3] = {32, 32, 1};
            rc = encode_map(&maps[4], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ctx->splitk_ws, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "D partials");
        } else {
            const CUtensorMapDataType dt = out->kind == DG_OUT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                           : (fp8_out ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
            const uint64_t pitch = static_cast<uint64_t>(out->ld) * d_elem;
            uint64_t dims[3] = {n_out, pr.m, a_groups};
            uint64_t strides[2] = {pitch, pitch * pr.m};
            uint32_t box[3] = {out->kind == DG_OUT_FP8 ? 128u : 32u, 32, 1};   // the fused activation stores 32 x 32 bytes, unswizzled
            rc = encode_map(&maps[4], dt, 3, out->buf, dims, strides, box,
                            swiglu ? CU_TENSOR_MAP_SWIZZLE_NONE : (out->kind == DG_OUT_BF16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B), "D");
        }
        if (rc) return rc;
    }

    dg::GemmParams p;
    memset(&p, 0, sizeof(p));
    p.m = swap ? pr.n : pr.m;     // rows of the kernel's operand A per group (swapped family: weight rows)
    p.n = swap ? pr.m : n_out;
    p.k = pr.k;
    p.tile_n = swiglu ? plan.umma_n / 2 : plan.umma_n;
    p.num_groups = pr.groups;
    p.gemm_type = pr.type;
    p.block_n = plan.umma_n;
    p.block_k_elems = block_k;
    p.num_splits = splits;
    p.cluster_splits = plan.cluster_splits;
    p.kb_per_split = splits > 1 ? ceil_div(ceil_div(ceil_div(pr.k, block_k), splits), 4) * 4 : ceil_div(ceil_div(pr.k, block_k), plan.cluster_splits);
    p.out_group_rows = (pr.type == DG_GEMM_M_GROUPED_MASKED || pr.type == DG_GEMM_BATCHED) ? pr.m : 0;
    p.num_stages = plan.stages;
    p.num_accum_stages = plan.accum;
    p.gran_a = ka->gran_k;
    p.gran_b = kb->gran_k;
    // measured on B200: a 16U4_ALIGN16B load (e2m1 expanded to one code per byte) fills 128 bytes of shared memory per
    // 128 elements but signals only the 64 packed bytes it read on its barrier
    p.tx_shift_a = (!mxf4 && ka->bits == 4) ? 1 : 0;
    p.tx_shift_b = (!mxf4 && kb->bits == 4) ? 1 : 0;
    p.fmt_a = ka->bits == 8 ? 0u : 5u;
    p.fmt_b = kb->bits == 8 ? 0u : 5u;
    p.sf_a_cols = sfa_cols;
    p.sf_b_cols = sfb_cols;
    p.mk_alignment = align;
    // groups start at multiples of `align` rows; tiles stay 128 (or 256) rows tall and simply run into the next group's rows,
    // which are computed and not stored.  Stores go out in 32-row boxes, so only an alignment of 16 needs row-exact stores.
    p.mask_rows = (contiguous && align % 32 != 0) ? 1 : 0;
    p.out_ptr = out->buf;
    p.out_ld = out->ld;
    {
        // dense problems of a single row block read every weight byte exactly once: those loads carry the L2 evict-first hint
        // (+9 % on 128 x 7168 x 16384).  Grouped problems with small groups were measured 4 % slower with it (a group's second row
        // block, running on a neighbouring CTA pair, finds its weight tile gone) and keep plain loads.  DG_STREAM_HINT=0 turns it off.
        const uint32_t row_block = swap ? plan.umma_n : 128 * plan.ctas;
        const char* v = getenv("DG_STREAM_HINT");
        const bool once = pr.type == DG_GEMM_NORMAL && pr.m <= row_block && !(v && strcmp(v, "0") == 0);
        p.stream_a = (once && swap) ? 1 : 0;
        p.stream_b = (once && !swap) ? 1 : 0;
    }
    p.wide_k = wide_k ? 1 : 0;
    p.mn_a = (!pr.bf16 && ka->major_mn) ? 1 : 0;
    p.mn_b = (!pr.bf16 && kb->major_mn) ? 1 : 0;
    p.accumulate = e.accumulate ? 1 : 0;
    p.tc_util = (e.tc_util == 0 || e.tc_util > 100) ? 100 : e.tc_util;      // 0 means "unset", as in ops_sm100.rs:518-522
    p.has_alpha = (e.has_alpha && splits == 1) ? 1 : 0;   // with K ranges summed by the second kernel alpha is applied there
    p.alpha = e.alpha;
    p.sfd = out->sfd;
    p.sfd_stride = align4(pr.m);
    p.grouped_layout = pr.layout;
    p.status = ctx->status;
#ifdef DG_PROFILE
    {   // debug builds: DG_PROF_PTR carries a device buffer address (8 x int64 per CTA)
        const char* pp = getenv("DG_PROF_PTR");
        p.prof = pp ? reinterpret_cast<long long*>(strtoull(pp, nullptr, 0)) : nullptr;
        const char* df = getenv("DG_DEBUG_FLAGS");
        p.debug_flags = df ? static_cast<uint32_t>(atoi(df)) : 0;
    }
#endif

    const uint32_t ctas = plan.ctas;
    uint32_t grid = static_cast<uint32_t>(ctx->num_sms) / ctas * ctas;
    if (pr.type == DG_GEMM_NORMAL || pr.type == DG_GEMM_BATCHED)
        grid = plan.tiles * splits * ctas < grid ? plan.tiles * splits * ctas : grid;
    // K ranges summed inside a cluster: one cluster per output tile, as many clusters as tiles
    if (swap && plan.cluster_splits > 1) grid = plan.tiles * plan.cluster_splits * ctas;
    const int kernel_out = splits > 1 ? DG_OUT_F32 : out->kind;
    const uint32_t smem = plan.smem;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    cudaError_t ce;
    if (swap) {
        if (pr.bf16) ce = ctas == 2 ? launch_swapped<dg::kFmtBf16, 2>(kernel_out, p, grid, smem, ctx->stream, maps)
                                    : launch_swapped<dg::kFmtBf16, 1>(kernel_out, p, grid, smem, ctx->stream, maps);
        else if (mxf4) ce = ctas == 2 ? launch_swapped<dg::kFmtMxf4, 2>(kernel_out, p, grid, smem, ctx->stream, maps)
                                      : launch_swapped<dg::kFmtMxf4, 1>(kernel_out, p, grid, smem, ctx->stream, maps);
        else ce = ctas == 2 ? launch_swapped<dg::kFmtMxf8f6f4, 2>(kernel_out, p, grid, smem, ctx->stream, maps)
                            : launch_swapped<dg::kFmtMxf8f6f4, 1>(kernel_out, p, grid, smem, ctx->stream, maps);
    } else if (pr.bf16) ce = ctas == 2 ? launch_by_out<dg::kFmtBf16, 2>(kernel_out, p, grid, smem, ctx->stream, maps)
                                : launch_by_out<dg::kFmtBf16, 1>(kernel_out, p, grid, smem, ctx->stream, maps);
    else if (mxf4) ce = ctas == 2 ? launch_by_out<dg::kFmtMxf4, 2>(kernel_out, p, grid, smem, ctx->stream, maps)
                                  : launch_by_out<dg::kFmtMxf4, 1>(kernel_out, p, grid, smem, ctx->stream, maps);
    else ce = ctas == 2 ? launch_by_out<dg::kFmtMxf8f6f4, 2>(kernel_out, p, grid, smem, ctx->stream, maps)
                        : launch_by_out<dg::kFmtMxf8f6f4, 1>(kernel_out, p, grid, smem, ctx->stream, maps);
    if (ce == cudaSuccess && splits > 1) {
        const uint64_t threads = static_cast<uint64_t>(pr.m) * ceil_div(pr.n, 4);
        const uint32_t blocks = static_cast<uint32_t>((threads + 255) / 256);
        const float alpha = e.has_alpha ? e.alpha : 1.0f;
        ce = out->kind == DG_OUT_BF16 ? launch_reduce<true>(blocks, ctx->stream, ctx->splitk_ws, splits, pr.m, pr.n, ws_pitch, alpha, out->buf, out->ld)
                                      : launch_reduce<false>(blocks, ctx->stream, ctx->splitk_ws, splits, pr.m, pr.n, ws_pitch, alpha, out->buf, out->ld);
    }
    if (ce != cudaSuccess) return fail(DG_ERR_DRIVER, "kernel launch failed: %s", cudaGetErrorString(ce));
    return DG_OK;
}

int ensure_group_ends(dg_ctx* ctx, uint32_t groups) {
    if (ctx->group_ends_cap >= groups) return DG_OK;
    if (ctx->group_ends) { cudaFree(ctx->group_ends); ctx->group_ends = nullptr; ctx->group_ends_cap = 0; }
    const uint32_t cap = groups < 1024 ? 1024 : groups;
    DG_CUDA(cudaMalloc(&ctx->group_ends, static_cast<size_t>(cap) * 4));
    ctx->group_ends_cap = cap;
    return DG_OK;
}

int run_group_ends(dg_ctx* ctx, const int32_t* m_indices, uint32_t m, uint32_t groups, uint32_t* ends) {
    DG_CUDA(cudaMemsetAsync(ends, 0, static_cast<size_t>(groups) * 4, ctx->stream));
    if (m > 0) dg::dg_group_ends_kernel<<<ceil_div(m, 256), 256, 0, ctx->stream>>>(m_indices, ends, groups, m);
    dg::dg_group_ends_scan_kernel<<<1, 1024, 0, ctx->stream>>>(ends, groups);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

}  // namespace

extern "C" {

int dg_fp8_fp4_gemm(dg_ctx* ctx, const dg_lp_operand* a, const dg_lp_operand* b, const dg_out* out, const dg_epilogue* epi) {
    if (!ctx || !a || !b || !out) return fail(DG_ERR_SHAPE, "null argument");
    if (out->kind == DG_OUT_FP8) return fail(DG_ERR_SHAPE, "the dynamic FP8 output is only supported by the batched and masked APIs");
    Problem pr = {DG_GEMM_NORMAL, a->rows, b->rows, a->k, 1, a->rows, nullptr};
    return launch_gemm(ctx, a, b, out, epi, pr);
}

int dg_bf16_gemm(dg_ctx* ctx, const uint16_t* a, uint32_t a_ld, uint32_t m, const uint16_t* b, uint32_t b_ld, uint32_t n, uint32_t k,
                 const dg_out* out, const dg_epilogue* epi) {
    if (!ctx || !a || !b || !out) return fail(DG_ERR_SHAPE, "null argument");
    if (out->kind == DG_OUT_FP8) return fail(DG_ERR_UNSUPPORTED, "the bf16 GEMM writes bf16 or f32 outputs");
    if (k == 0 || k % 8 != 0) return fail(DG_ERR_SHAPE, "bf16 k (%u) must be a positive multiple of 8", k);
    if (a_ld < k || b_ld < k || a_ld % 8 != 0 || b_ld % 8 != 0) return fail(DG_ERR_SHAPE, "leading dimensions must be >= k and multiples of 8 elements");
    // the kernel sees K-major rows of 2k bytes: same tiles, same TMA boxes, same 32-byte UMMA steps as the 8-bit formats
    dg_lp_operand a8 = {a, nullptr, m, 2 * k, 2 * a_ld, 8, 128, 0, static_cast<size_t>(m) * 2 * a_ld, 0};
    dg_lp_operand b8 = {b, nullptr, n, 2 * k, 2 * b_ld, 8, 128, 0, static_cast<size_t>(n) * 2 * b_ld, 0};
    Problem pr = {DG_GEMM_NORMAL, m, n, 2 * k, 1, m, nullptr, true};
    return launch_gemm(ctx, &a8, &b8, out, epi, pr);
}

int dg_m_grouped_fp8_fp4_gemm_contiguous_ends(dg_ctx* ctx, const dg_lp_operand* a, const uint32_t* group_ends, const dg_lp_operand* b,
                                              const dg_out* out, uint32_t num_groups, const dg_epilogue* epi) {
    if (!ctx || !a || !b || !out || !group_ends) return fail(DG_ERR_SHAPE, "null argument");
    if (num_groups == 0 || b->rows % num_groups != 0) return fail(DG_ERR_SHAPE, "b.rows (%u) must be num_groups (%u) x n", b->rows, num_groups);
    if (out->kind == DG_OUT_FP8) return fail(DG_ERR_SHAPE, "the dynamic FP8 output is only supported by the batched and masked APIs");
    if (epi && epi->accumulate) return fail(DG_ERR_SHAPE, "accumulation is not supported by the grouped contiguous layout");
    Problem pr = {DG_GEMM_M_GROUPED_CONTIGUOUS, a->rows, b->rows / num_groups, a->k, num_groups, a->rows, group_ends};
    return launch_gemm(ctx, a, b, out, epi, pr);
}

int dg_m_grouped_fp8_fp4_gemm_contiguous(dg_ctx* ctx, const dg_lp_operand* a, const int32_t* m_indices, const dg_lp_operand* b,
                                         const dg_out* out, uint32_t num_groups, const dg_epilogue* epi) {
    if (!ctx || !a || !b || !out || !m_indices) return fail(DG_ERR_SHAPE, "null argument");
    if (num_groups == 0) return fail(DG_ERR_SHAPE, "num_groups must be positive");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    int rc = ensure_group_ends(ctx, num_groups);
    if (rc) return rc;
    rc = run_group_ends(ctx, m_indices, a->rows, num_groups, ctx->group_ends);
    if (rc) return rc;
    return dg_m_grouped_fp8_fp4_gemm_contiguous_ends(ctx, a, ctx->group_ends, b, out, num_groups, epi);
}

int dg_m_grouped_fp8_fp4_gemm_masked(dg_ctx* ctx, const dg_lp_operand* a, const int32_t* masked_m, const dg_lp_operand* b,
                                     const dg_out* out, uint32_t num_groups, uint32_t expected_m, const dg_epilogue* epi) {
    if (!ctx || !a || !b || !out || !masked_m) return fail(DG_ERR_SHAPE, "null argument");
    if (num_groups == 0 || b->rows % num_groups != 0) return fail(DG_ERR_SHAPE, "b.rows (%u) must be num_groups (%u) x n", b->rows, num_groups);
    Problem pr = {DG_GEMM_M_GROUPED_MASKED, a->rows, b->rows / num_groups, a->k, num_groups, expected_m ? expected_m : 1,
                  reinterpret_cast<const uint32_t*>(masked_m)};
    return launch_gemm(ctx, a, b, out, epi, pr);
}

int dg_fp8_fp4_bmm(dg_ctx* ctx, const dg_lp_operand* a, const dg_lp_operand* b, const dg_out* out, uint32_t num_groups,
                   const dg_epilogue* epi) {
    if (!ctx || !a || !b || !out) return fail(DG_ERR_SHAPE, "null argument");
    if (num_groups == 0) return fail(DG_ERR_SHAPE, "num_groups must be positive");
    Problem pr = {DG_GEMM_BATCHED, a->rows, b->rows, a->k, num_groups, a->rows, nullptr};
    return launch_gemm(ctx, a, b, out, epi, pr);
}

// ------------------------------------------------------------ f32-scale entry points
// The reference's older API hands scales over as f32 (activations transposed by transform_sf, weights one per
// 128x128 tile).  By default they are applied exactly, K block by K block, as the reference's CPU definition does
// (reference.rs:85-208): dg_gemm_f32scale_kernel.  With DG_F32_SCALES=exponent the calls do what the reference itself does on
// Blackwell (ops_sm100.rs:1414-1605): pack the exponents into UE8M0 words (mantissas are dropped, so the scales must be powers
// of two to be exact) and run the block-scaled kernel, which is about three times faster.
static int launch_f32scale(dg_ctx* ctx, uint32_t type, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld,
                           const float* sfb, uint32_t m, uint32_t n, uint32_t k, uint32_t groups, const uint32_t* layout, uint16_t* out,
                           uint32_t out_ld) {
    if (m == 0 || n == 0) return DG_OK;
    const bool contiguous = type == DG_GEMM_M_GROUPED_CONTIGUOUS;
    const uint32_t a_groups = (type == DG_GEMM_NORMAL || contiguous) ? 1 : groups;
    const uint32_t b_groups = type == DG_GEMM_NORMAL ? 1 : groups;
    const uint32_t align = g_mk_alignment.load();
    if (contiguous && align % 32 != 0) return fail(DG_ERR_UNSUPPORTED, "the exact f32-scale path needs an mk alignment of at least 32");
    if (a_ld < k || b_ld < k || a_ld % 16 != 0 || b_ld % 16 != 0) return fail(DG_ERR_SHAPE, "leading dimensions must be >= k and multiples of 16 bytes");
    if (out_ld < n || (static_cast<size_t>(out_ld) * 2) % 16 != 0) return fail(DG_ERR_SHAPE, "output ld (%u) must be >= n and a multiple of 8 elements", out_ld);
    CUtensorMap maps[3];
    int rc;
    {
        uint64_t dims[3] = {k, m, a_groups};
        uint64_t strides[2] = {a_ld, static_cast<uint64_t>(a_ld) * m};
        uint32_t box[3] = {128, dg::kBlockM, 1};
        rc = encode_map(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "A");
        if (rc) return rc;
        uint64_t bdims[3] = {k, n, b_groups};
        uint64_t bstrides[2] = {b_ld, static_cast<uint64_t>(b_ld) * n};
        uint32_t bbox[3] = {128, dg::kF32BlockN, 1};
        rc = encode_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, b, bdims, bstrides, bbox, CU_TENSOR_MAP_SWIZZLE_128B, "B");
        if (rc) return rc;
        const uint64_t pitch = static_cast<uint64_t>(out_ld) * 2;
        uint64_t ddims[3] = {n, m, a_groups};
        uint64_t dstrides[2] = {pitch, pitch * m};
        uint32_t dbox[3] = {32, 32, 1};
        rc = encode_map(&maps[2], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, out, ddims, dstrides, dbox, CU_TENSOR_MAP_SWIZZLE_64B, "D");
        if (rc) return rc;
    }
    dg::F32ScaleParams q;
    memset(&q, 0, sizeof(q));
    dg::GemmParams& p = q.g;
    p.m = m; p.n = n; p.k = k;
    p.num_groups = groups;
    p.gemm_type = type;
    p.block_n = p.tile_n = dg::kF32BlockN;
    p.block_k_elems = 128;
    p.num_splits = 1;
    p.cluster_splits = 1;
    p.num_accum_stages = 2;
    p.mk_alignment = align;
    p.grouped_layout = layout;
    p.status = ctx->status;
    uint32_t stages = dg::kMaxStages;
    while (stages > 1 && dg::f32scale_smem_bytes(stages) > kSmemCapacity) --stages;
    p.num_stages = stages;
    q.sfa_t = a_sf_t;
    q.sfb = sfb;
    q.sfa_stride = align4(m);
    q.k_blocks = k / 128;
    q.n_blocks128 = ceil_div(n, 128);
    const uint32_t smem = dg::f32scale_smem_bytes(stages);
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    {
        static std::atomic<uint64_t> configured{0};
        if (ctx->ordinal >= 64 || !(configured.load() & (1ull << ctx->ordinal))) {
            DG_CUDA(cudaFuncSetAttribute(dg::dg_gemm_f32scale_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemCapacity)));
            if (ctx->ordinal < 64) configured.fetch_or(1ull << ctx->ordinal);
        }
    }
    uint32_t grid = static_cast<uint32_t>(ctx->num_sms);
    if (type == DG_GEMM_NORMAL || type == DG_GEMM_BATCHED) {
        const uint64_t tiles = static_cast<uint64_t>(ceil_div(m, dg::kBlockM)) * ceil_div(n, dg::kF32BlockN) * (type == DG_GEMM_BATCHED ? groups : 1);
        if (tiles < grid) grid = static_cast<uint32_t>(tiles);
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(dg::kF32Threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, dg::dg_gemm_f32scale_kernel, q, maps[0], maps[1], maps[2]);
    if (ce != cudaSuccess) return fail(DG_ERR_DRIVER, "kernel launch failed: %s", cudaGetErrorString(ce));
    return DG_OK;
}

static int bridge_common(dg_ctx* ctx, uint32_t type, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld,
                         const float* sfb, uint32_t m, uint32_t n, uint32_t k, uint32_t groups, const uint32_t* layout, uint32_t expected_m,
                         uint16_t* out, uint32_t out_ld) {
    if (!ctx || !a || !a_sf_t || !b || !sfb || !out) return fail(DG_ERR_SHAPE, "null argument");
    if (k == 0 || k % 128 != 0) return fail(DG_ERR_SHAPE, "k (%u) must be a multiple of 128 (per-128-channel scaling)", k);
    if (n % 8 != 0) return fail(DG_ERR_SHAPE, "n (%u) must be a multiple of 8", n);
    if (groups == 0) return fail(DG_ERR_SHAPE, "num_groups must be positive");
    const bool contiguous = type == DG_GEMM_M_GROUPED_CONTIGUOUS;
    const uint32_t a_groups = (type == DG_GEMM_NORMAL || contiguous) ? 1 : groups;
    const uint32_t b_groups = type == DG_GEMM_NORMAL ? 1 : groups;
    {
        const char* mode = getenv("DG_F32_SCALES");
        if (!(mode && strcmp(mode, "exponent") == 0)) {
            const uint32_t* table = layout;
            if (contiguous) {
                // the group-end table the scheduler walks, built from m_indices in the context's scratch
                int rc = ensure_group_ends(ctx, groups);
                if (rc) return rc;
                DG_CUDA(cudaSetDevice(ctx->ordinal));
                rc = run_group_ends(ctx, reinterpret_cast<const int32_t*>(layout), m, groups, ctx->group_ends);
                if (rc) return rc;
                table = ctx->group_ends;
            }
            return launch_f32scale(ctx, type, a, a_ld, a_sf_t, b, b_ld, sfb, m, n, k, groups, table, out, out_ld);
        }
    }
    const size_t need[2] = {dg_sf_words(m * a_groups, k, 128, a_groups), dg_sf_words(n * b_groups, k, 128, b_groups)};
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    for (int i = 0; i < 2; ++i) {
        if (ctx->bridge_sf_cap[i] >= need[i]) continue;
        if (ctx->bridge_sf[i]) { cudaFree(ctx->bridge_sf[i]); ctx->bridge_sf[i] = nullptr; ctx->bridge_sf_cap[i] = 0; }
        DG_CUDA(cudaMalloc(&ctx->bridge_sf[i], need[i] * 4));
        ctx->bridge_sf_cap[i] = need[i];
    }
    // padding rows of the packed layouts must read as a valid exponent
    DG_CUDA(cudaMemsetAsync(ctx->bridge_sf[0], 0, need[0] * 4, ctx->stream));
    DG_CUDA(cudaMemsetAsync(ctx->bridge_sf[1], 0, need[1] * 4, ctx->stream));
    int rc = dg_transform_sf_t_packed_ue8m0(ctx, a_sf_t, m * a_groups, k, 128, a_groups, ctx->bridge_sf[0]);
    if (rc) return rc;
    rc = dg_transform_sf2d_packed_ue8m0(ctx, sfb, k / 128, n * b_groups, k, b_groups, ctx->bridge_sf[1]);
    if (rc) return rc;
    dg_lp_operand a_op = {a, ctx->bridge_sf[0], m, k, a_ld, 8, 128, 0, static_cast<size_t>(m) * a_groups * a_ld, need[0]};
    dg_lp_operand b_op = {b, ctx->bridge_sf[1], type == DG_GEMM_BATCHED || type == DG_GEMM_NORMAL ? n : n * groups, k, b_ld, 8, 128, 0,
                          static_cast<size_t>(n) * b_groups * b_ld, need[1]};
    dg_out o = {DG_OUT_BF16, out, out_ld, nullptr, static_cast<size_t>(m) * a_groups * out_ld, 0};
    switch (type) {
        case DG_GEMM_NORMAL: return dg_fp8_fp4_gemm(ctx, &a_op, &b_op, &o, nullptr);
        case DG_GEMM_M_GROUPED_CONTIGUOUS:
            return dg_m_grouped_fp8_fp4_gemm_contiguous(ctx, &a_op, reinterpret_cast<const int32_t*>(layout), &b_op, &o, groups, nullptr);
        case DG_GEMM_M_GROUPED_MASKED:
            return dg_m_grouped_fp8_fp4_gemm_masked(ctx, &a_op, reinterpret_cast<const int32_t*>(layout), &b_op, &o, groups, expected_m, nullptr);
        default: return dg_fp8_fp4_bmm(ctx, &a_op, &b_op, &o, groups, nullptr);
    }
}

int dg_fp8_gemm_nt(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld, const float* sfb, uint32_t m,
                   uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld) {
    return bridge_common(ctx, DG_GEMM_NORMAL, a, a_ld, a_sf_t, b, b_ld, sfb, m, n, k, 1, nullptr, m, out, out_ld);
}
int dg_m_grouped_fp8_gemm_nt_contiguous(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld,
                                        const float* sfb, uint32_t m_total, uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld,
                                        const int32_t* m_indices, uint32_t num_groups) {
    if (!m_indices) return fail(DG_ERR_SHAPE, "null argument");
    return bridge_common(ctx, DG_GEMM_M_GROUPED_CONTIGUOUS, a, a_ld, a_sf_t, b, b_ld, sfb, m_total, n, k, num_groups,
                         reinterpret_cast<const uint32_t*>(m_indices), m_total, out, out_ld);
}
int dg_m_grouped_fp8_gemm_nt_masked(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld,
                                    const float* sfb, uint32_t m_max, uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld,
                                    const int32_t* masked_m, uint32_t num_groups, uint32_t expected_m) {
    if (!masked_m) return fail(DG_ERR_SHAPE, "null argument");
    return bridge_common(ctx, DG_GEMM_M_GROUPED_MASKED, a, a_ld, a_sf_t, b, b_ld, sfb, m_max, n, k, num_groups,
                         reinterpret_cast<const uint32_t*>(masked_m), expected_m, out, out_ld);
}
int dg_fp8_bmm_nt(dg_ctx* ctx, const uint8_t* a, uint32_t a_ld, const float* a_sf_t, const uint8_t* b, uint32_t b_ld, const float* sfb, uint32_t m,
                  uint32_t n, uint32_t k, uint16_t* out, uint32_t out_ld, uint32_t num_groups) {
    return bridge_common(ctx, DG_GEMM_BATCHED, a, a_ld, a_sf_t, b, b_ld, sfb, m, n, k, num_groups, nullptr, m, out, out_ld);
}

// ------------------------------------------------------- entry point that allocates nothing
// Scratch for dg_m_grouped_fp8_fp4_gemm_contiguous_static: words [0, 4) are the record a kernel
// writes when one of its bounded waits runs out, words [64, 64 + kStaticMaxGroups) hold the
// group-end table.  One copy per GPU that loads the library, kept until the process exits.
constexpr uint32_t kStaticMaxGroups = DG_STATIC_MAX_GROUPS;
constexpr uint32_t kStaticEndsOffset = 64;
static __device__ __align__(256) uint32_t g_static_scratch[kStaticEndsOffset + kStaticMaxGroups];

namespace {
struct StaticDevice {
    bool ready = false;
    uint32_t* scratch = nullptr;   // device address of g_static_scratch on this device
    int num_sms = 0;
};
StaticDevice g_static_devices[64];
std::mutex g_static_mutex;

// Once per device, with that device current: ask the runtime for the device address of the array.
// In host code the array's name is only a handle for this lookup, never a pointer a kernel can use.
int static_device_setup(int device, StaticDevice** out) {
    if (device < 0 || device >= 64) return fail(DG_ERR_SHAPE, "device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticDevice& d = g_static_devices[device];
    if (!d.ready) {
        DG_CUDA(cudaSetDevice(device));
        int major = 0;
        DG_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        if (major != 10) return fail(DG_ERR_UNSUPPORTED, "device %d is not sm_100; these kernels are built for sm_100a only", device);
        if (encode_tiled_fn() == nullptr) return fail(DG_ERR_DRIVER, "cuTensorMapEncodeTiled not found in the driver");
        DG_CUDA(cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, device));
        uint32_t* ptr = nullptr;
        DG_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch));
        d.scratch = ptr;
        // every kernel the contiguous path can reach gets its shared-memory opt-in (and its image loaded) now, so that later
        // calls with another output kind, operand format or tile choice do no set-up work
        DG_CUDA(configure_contiguous_kernels());
        d.ready = true;
    }
    *out = &d;
    return DG_OK;
}
}  // namespace

int dg_m_grouped_fp8_fp4_gemm_contiguous_static(int device, void* cuda_stream, const dg_lp_operand* a, const int32_t* m_indices,
                                                const dg_lp_operand* b, const dg_out* out, uint32_t num_groups, const dg_epilogue* epi) {
    if (!a || !b || !out || !m_indices) return fail(DG_ERR_SHAPE, "null argument");
    if (num_groups == 0) return fail(DG_ERR_SHAPE, "num_groups must be positive");
    if (num_groups > kStaticMaxGroups)
        return fail(DG_ERR_SHAPE, "num_groups (%u) exceeds the %u groups the built-in scratch holds; use dg_m_grouped_fp8_fp4_gemm_contiguous",
                    num_groups, kStaticMaxGroups);
    StaticDevice* dev = nullptr;
    int rc = static_device_setup(device, &dev);
    if (rc) return rc;
    DG_CUDA(cudaSetDevice(device));
    // a context view on the stack: nothing is created, nothing has to be destroyed
    dg_ctx view;
    view.ordinal = device;
    view.stream = static_cast<cudaStream_t>(cuda_stream);
    view.num_sms = dev->num_sms;
    view.status = reinterpret_cast<dg::Status*>(dev->scratch);
    uint32_t* ends = dev->scratch + kStaticEndsOffset;
    // the table keeps the previous call's contents: run_group_ends clears the entries it is about to fill
    rc = run_group_ends(&view, m_indices, a->rows, num_groups, ends);
    if (rc) return rc;
    return dg_m_grouped_fp8_fp4_gemm_contiguous_ends(&view, a, ends, b, out, num_groups, epi);
}

int dg_static_check_status(int device, void* cuda_stream) {
    StaticDevice* dev = nullptr;
    int rc = static_device_setup(device, &dev);
    if (rc) return rc;
    DG_CUDA(cudaSetDevice(device));
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    dg::Status st;
    // a stack destination and 16 bytes: the copy allocates nothing; it is ordered after the GEMMs enqueued on `stream`
    DG_CUDA(cudaMemcpyAsync(&st, dev->scratch, sizeof(st), cudaMemcpyDeviceToHost, stream));
    DG_CUDA(cudaStreamSynchronize(stream));
    if (st.code != 0) {
        DG_CUDA(cudaMemsetAsync(dev->scratch, 0, sizeof(st), stream));
        DG_CUDA(cudaStreamSynchronize(stream));
        return fail(DG_ERR_TIMEOUT, "a device-side wait ran out: block %u, site 0x%x, parity %u", st.block, st.site, st.extra);
    }
    return DG_OK;
}

// ------------------------------------------------------------------ quantise / re-layout
static int cast_common(dg_ctx* ctx, const uint16_t* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t gran, uint32_t groups, int rule,
                       bool fp4, uint8_t* dst, uint32_t* sf, bool silu_mul = false, const uint32_t* live_rows = nullptr) {
    if (!ctx || !src || !dst || !sf) return fail(DG_ERR_SHAPE, "null argument");
    if (groups == 0) groups = 1;
    if (rows % groups != 0) return fail(DG_ERR_SHAPE, "rows (%u) must be a multiple of num_groups (%u)", rows, groups);
    if (src_ld < (silu_mul ? 2 * k : k) || src_ld % 8 != 0)
        return fail(DG_ERR_SHAPE, "src_ld (%u) must cover the %u source columns and be a multiple of 8 elements", src_ld, silu_mul ? 2 * k : k);
    if (reinterpret_cast<uintptr_t>(src) % 16 != 0 || reinterpret_cast<uintptr_t>(dst) % 16 != 0)
        return fail(DG_ERR_SHAPE, "src and dst must be 16-byte aligned");
    if (rows == 0) return DG_OK;
    dg::CastParams p;
    p.src = src; p.dst = dst; p.sf = sf;
    p.src_ld = src_ld; p.rows = rows; p.k = k; p.group_rows = rows / groups;
    p.sf_cols = dg_sf_packed_cols(k, gran);
    p.sf_stride = align4(rows / groups);
    p.rule = rule;
    p.live_rows = live_rows;
    // one block per 8 consecutive rows x one 1024-element segment (one warp per row)
    const uint64_t units = static_cast<uint64_t>(ceil_div(rows, 8)) * ceil_div(k, 1024);
    if (units > 0x7FFFFFFFull) return fail(DG_ERR_SHAPE, "matrix too large for one launch");
    const uint32_t blocks = static_cast<uint32_t>(units);
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    if (silu_mul && gran == 32) dg::dg_cast_kernel<32, false, true><<<blocks, 256, 0, ctx->stream>>>(p);
    else if (silu_mul) dg::dg_cast_kernel<128, false, true><<<blocks, 256, 0, ctx->stream>>>(p);
    else if (fp4) dg::dg_cast_kernel<32, true><<<blocks, 256, 0, ctx->stream>>>(p);
    else if (gran == 32) dg::dg_cast_kernel<32, false><<<blocks, 256, 0, ctx->stream>>>(p);
    else dg::dg_cast_kernel<128, false><<<blocks, 256, 0, ctx->stream>>>(p);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_cast_bf16_to_fp8_sf(dg_ctx* ctx, const uint16_t* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t gran_k,
                           uint32_t num_groups, uint8_t* dst, uint32_t* sf) {
    if (gran_k != 32 && gran_k != 128) return fail(DG_ERR_SHAPE, "gran_k must be 32 or 128");
    if (k == 0 || k % (gran_k * 4) != 0) return fail(DG_ERR_SHAPE, "k must be a multiple of %u for gran %u", gran_k * 4, gran_k);
    return cast_common(ctx, src, src_ld, rows, k, gran_k, num_groups, 0, false, dst, sf);
}

int dg_silu_mul_cast_fp8_sf(dg_ctx* ctx, const uint16_t* gate_up, uint32_t src_ld, uint32_t rows, uint32_t n, uint32_t gran_k,
                            uint32_t num_groups, uint8_t* dst, uint32_t* sf, const uint32_t* live_rows) {
    if (gran_k != 32 && gran_k != 128) return fail(DG_ERR_SHAPE, "gran_k must be 32 or 128");
    if (n == 0 || n % (gran_k * 4) != 0) return fail(DG_ERR_SHAPE, "n must be a multiple of %u for gran %u", gran_k * 4, gran_k);
    return cast_common(ctx, gate_up, src_ld, rows, n, gran_k, num_groups, 0, false, dst, sf, true, live_rows);
}

int dg_cast_bf16_to_fp4_packed_sf(dg_ctx* ctx, const uint16_t* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t num_groups,
                                  int sf_rule, uint8_t* dst, uint32_t* sf) {
    if (k == 0 || k % 128 != 0) return fail(DG_ERR_SHAPE, "fp4 k must be a multiple of 128");
    if (sf_rule != DG_SF_RULE_REFERENCE_CPU && sf_rule != DG_SF_RULE_RANGE_FIT) return fail(DG_ERR_SHAPE, "unknown sf_rule %d", sf_rule);
    return cast_common(ctx, src, src_ld, rows, k, 32, num_groups, sf_rule, true, dst, sf);
}

int dg_transform_sf(dg_ctx* ctx, const float* sf, uint32_t mn, uint32_t sf_k, uint32_t num_batches, float* dst) {
    if (!ctx || !sf || !dst) return fail(DG_ERR_SHAPE, "null argument");
    if (mn == 0 || sf_k == 0 || num_batches == 0) return DG_OK;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    dim3 grid(ceil_div(align4(mn), 32), ceil_div(sf_k, 32), num_batches);
    dg::dg_transpose_sf_kernel<<<grid, 256, 0, ctx->stream>>>(sf, dst, mn, sf_k, align4(mn));
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

static int sf_pack_common(dg_ctx* ctx, const float* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t gran, uint32_t groups,
                          uint32_t mode, uint32_t* dst) {
    if (!ctx || !src || !dst) return fail(DG_ERR_SHAPE, "null argument");
    if (gran != 32 && gran != 128) return fail(DG_ERR_SHAPE, "gran_k must be 32 or 128");
    if (groups == 0) groups = 1;
    if (rows % groups != 0) return fail(DG_ERR_SHAPE, "rows (%u) must be a multiple of num_groups (%u)", rows, groups);
    if (rows == 0 || k == 0) return DG_OK;
    dg::SfPackParams p;
    p.src = src; p.dst = dst; p.src_ld = src_ld; p.rows = rows; p.group_rows = rows / groups;
    p.k_blocks = ceil_div(k, gran);
    p.cols = ceil_div(p.k_blocks, 4);
    p.dst_stride = align4(rows / groups);
    p.mode = mode;
    const uint64_t total = static_cast<uint64_t>(rows) * p.cols;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    dg::dg_sf_pack_kernel<<<static_cast<uint32_t>((total + 255) / 256), 256, 0, ctx->stream>>>(p);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_transform_sf1d_packed_ue8m0(dg_ctx* ctx, const float* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t gran_k,
                                   uint32_t num_groups, uint32_t* dst) {
    return sf_pack_common(ctx, src, src_ld, rows, k, gran_k, num_groups, 0, dst);
}
int dg_transform_sf2d_packed_ue8m0(dg_ctx* ctx, const float* src, uint32_t src_ld, uint32_t rows, uint32_t k, uint32_t num_groups,
                                   uint32_t* dst) {
    const uint32_t g = num_groups ? num_groups : 1;
    if (g > 1 && (rows / g) % 128 != 0) return fail(DG_ERR_SHAPE, "2-D SF groups must own whole 128-row tiles (group rows %u)", rows / g);
    return sf_pack_common(ctx, src, src_ld, rows, k, 128, num_groups, 1, dst);
}
int dg_transform_sf_t_packed_ue8m0(dg_ctx* ctx, const float* src, uint32_t rows, uint32_t k, uint32_t gran_k, uint32_t num_groups,
                                   uint32_t* dst) {
    const uint32_t g = num_groups ? num_groups : 1;
    return sf_pack_common(ctx, src, align4(rows / g), rows, k, gran_k, num_groups, 2, dst);
}

int dg_group_ends_from_m_indices(dg_ctx* ctx, const int32_t* m_indices, uint32_t m, uint32_t num_groups, uint32_t* group_ends) {
    if (!ctx || !m_indices || !group_ends) return fail(DG_ERR_SHAPE, "null argument");
    if (num_groups == 0) return DG_OK;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    return run_group_ends(ctx, m_indices, m, num_groups, group_ends);
}

int dg_unpack_fp4_raw(dg_ctx* ctx, const uint8_t* src, size_t packed_len, uint8_t* dst) {
    if (!ctx || !src || !dst) return fail(DG_ERR_SHAPE, "null argument");
    if (packed_len == 0) return DG_OK;
    if (reinterpret_cast<uintptr_t>(src) % 16 != 0 || reinterpret_cast<uintptr_t>(dst) % 16 != 0)
        return fail(DG_ERR_SHAPE, "src and dst must be 16-byte aligned");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    const uint64_t threads = (packed_len + 15) / 16;
    dg::dg_unpack_fp4_kernel<<<static_cast<uint32_t>((threads + 255) / 256), 256, 0, ctx->stream>>>(src, dst, packed_len);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_debug_expire_wait(dg_ctx* ctx, uint32_t limit_us) {
    if (!ctx) return fail(DG_ERR_SHAPE, "null context");
    if (limit_us == 0 || limit_us > 1000000) return fail(DG_ERR_SHAPE, "limit must be between 1 us and 1 s");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    dg::dg_expire_wait_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status, static_cast<uint64_t>(limit_us) * 1000ull);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

// ------------------------------------------------------------------ MoE row movers
static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int dg_gather_rows(dg_ctx* ctx, const void* src, size_t src_pitch, const int32_t* idx, uint32_t n_dst, uint32_t row_bytes, void* dst,
                   size_t dst_pitch) {
    if (!ctx || !src || !idx || !dst) return fail(DG_ERR_SHAPE, "null argument");
    if (row_bytes % 16 || src_pitch % 16 || dst_pitch % 16 || !aligned16(src) || !aligned16(dst))
        return fail(DG_ERR_SHAPE, "rows, pitches and base addresses must be multiples of 16 bytes");
    if (n_dst == 0) return DG_OK;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    dg::dg_gather_rows_kernel<<<ceil_div(n_dst, 8), 256, 0, ctx->stream>>>(static_cast<const uint8_t*>(src), src_pitch, idx, n_dst, row_bytes,
                                                                           static_cast<uint8_t*>(dst), dst_pitch);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_moe_pack_rows(dg_ctx* ctx, const uint8_t* data, uint32_t k, const uint32_t* sf, uint32_t sf_stride, uint32_t sf_cols, const int32_t* idx,
                     uint32_t n, uint8_t* out, size_t out_pitch) {
    if (!ctx || !data || !sf || !idx || !out) return fail(DG_ERR_SHAPE, "null argument");
    if (k % 16 || out_pitch % 16 || out_pitch < static_cast<size_t>(k) + 4 * sf_cols || !aligned16(data) || !aligned16(out))
        return fail(DG_ERR_SHAPE, "k and out_pitch must be multiples of 16 and out_pitch >= k + 4 * sf_cols");
    if (n == 0) return DG_OK;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    dg::dg_moe_pack_rows_kernel<<<ceil_div(n, 8), 256, 0, ctx->stream>>>(data, k, sf, sf_stride, sf_cols, idx, n, out, out_pitch);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_moe_unpack_rows(dg_ctx* ctx, const uint8_t* in, size_t in_pitch, uint32_t k, uint32_t sf_cols, const int32_t* idx, uint32_t n_dst,
                       uint8_t* dst_data, uint32_t* dst_sf, uint32_t dst_sf_stride) {
    if (!ctx || !in || !idx || !dst_data || !dst_sf) return fail(DG_ERR_SHAPE, "null argument");
    if (k % 16 || in_pitch % 16 || in_pitch < static_cast<size_t>(k) + 4 * sf_cols || !aligned16(in) || !aligned16(dst_data))
        return fail(DG_ERR_SHAPE, "k and in_pitch must be multiples of 16 and in_pitch >= k + 4 * sf_cols");
    if (dst_sf_stride < n_dst) return fail(DG_ERR_SHAPE, "scale stride smaller than the row count");
    if (n_dst == 0) return DG_OK;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    dg::dg_moe_unpack_rows_kernel<<<ceil_div(n_dst, 8), 256, 0, ctx->stream>>>(in, in_pitch, k, sf_cols, idx, n_dst, dst_data, dst_sf, dst_sf_stride);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_moe_combine(dg_ctx* ctx, const uint16_t* rows, size_t pitch, const int32_t* pos, const float* weights, uint32_t tokens, uint32_t topk,
                   uint32_t n, uint16_t* out, size_t out_pitch) {
    if (!ctx || !rows || !pos || !weights || !out) return fail(DG_ERR_SHAPE, "null argument");
    if (n % 8 || pitch % 8 || out_pitch % 8 || !aligned16(rows) || !aligned16(out)) return fail(DG_ERR_SHAPE, "n and pitches must be multiples of 8 elements");
    if (tokens == 0 || n == 0) return DG_OK;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    const uint64_t threads = static_cast<uint64_t>(tokens) * (n / 8);
    dg::dg_moe_combine_kernel<<<static_cast<uint32_t>((threads + 255) / 256), 256, 0, ctx->stream>>>(rows, pitch, pos, weights, tokens, topk, n, out,
                                                                                                    out_pitch);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

// ------------------------------------------------------------------------------------------------
// Buffers other processes' GPUs can map, and the expert-parallel exchange over them
// ------------------------------------------------------------------------------------------------
int dg_peer_alloc(dg_ctx* ctx, size_t bytes, void** ptr, unsigned char* handle64) {
    if (!ctx || !ptr || bytes == 0) return fail(DG_ERR_SHAPE, "null argument or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == DG_PEER_HANDLE_BYTES, "handle size");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    void* p = nullptr;
    DG_CUDA(cudaMalloc(&p, bytes));
    if (handle64 != nullptr) {
        cudaIpcMemHandle_t h;
        const cudaError_t e = cudaIpcGetMemHandle(&h, p);
        if (e != cudaSuccess) {
            cudaFree(p);
            return fail(DG_ERR_DRIVER, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
        }
        memcpy(handle64, &h, sizeof(h));
    }
    *ptr = p;
    return DG_OK;
}

int dg_peer_open(dg_ctx* ctx, const unsigned char* handle64, void** ptr) {
    if (!ctx || !ptr || !handle64) return fail(DG_ERR_SHAPE, "null argument");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    DG_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return DG_OK;
}

int dg_peer_close(dg_ctx* ctx, void* ptr) {
    if (!ctx || !ptr) return fail(DG_ERR_SHAPE, "null argument");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    DG_CUDA(cudaIpcCloseMemHandle(ptr));
    return DG_OK;
}

int dg_peer_free(dg_ctx* ctx, void* ptr) {
    if (!ctx || !ptr) return fail(DG_ERR_SHAPE, "null argument");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    DG_CUDA(cudaFree(ptr));
    return DG_OK;
}

size_t dg_ep_block_hist_words(uint32_t pairs, uint32_t num_experts) {
    return static_cast<size_t>(ceil_div(pairs, dg::kEpChunk)) * num_experts;
}

int dg_ep_count(dg_ctx* ctx, const int32_t* expert_of_pair, uint32_t pairs, uint32_t num_experts, int32_t* local_rank, uint32_t* block_hist,
                uint32_t* counts) {
    if (!ctx || !expert_of_pair || !local_rank || !block_hist || !counts) return fail(DG_ERR_SHAPE, "null argument");
    if (num_experts == 0 || num_experts > 8192) return fail(DG_ERR_SHAPE, "num_experts must be in [1, 8192]");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    const uint32_t chunks = ceil_div(pairs, dg::kEpChunk);
    if (chunks > 0)
        dg::dg_ep_rank_pairs_kernel<<<chunks, dg::kEpChunk, num_experts * sizeof(uint32_t), ctx->stream>>>(expert_of_pair, pairs, num_experts,
                                                                                                         local_rank, block_hist);
    dg::dg_ep_block_scan_kernel<<<ceil_div(num_experts, 8), 256, 0, ctx->stream>>>(block_hist, chunks, num_experts, counts);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_ep_layout(dg_ctx* ctx, const uint32_t* all_counts, uint32_t world, uint32_t rank, uint32_t num_experts, uint32_t alignment,
                 uint32_t capacity, uint32_t slot_rows, uint32_t* pair_base, uint32_t* group_ends, uint32_t* totals) {
    if (!ctx || !all_counts || !pair_base || !group_ends || !totals) return fail(DG_ERR_SHAPE, "null argument");
    if (world == 0 || world > 1024 || rank >= world || num_experts == 0 || num_experts > 4096 || num_experts % world != 0)
        return fail(DG_ERR_SHAPE, "need 1 <= world <= 1024, rank < world, num_experts <= 4096 and a multiple of world");
    if (alignment == 0) return fail(DG_ERR_SHAPE, "alignment must be positive");
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    dg::dg_ep_layout_kernel<<<1, 1024, 3 * num_experts * sizeof(uint32_t), ctx->stream>>>(all_counts, world, rank, num_experts, alignment, capacity,
                                                                                         slot_rows, pair_base, group_ends, totals);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_ep_dispatch(dg_ctx* ctx, const int32_t* expert_of_pair, const int32_t* local_rank, const uint32_t* block_base, const uint32_t* pair_base,
                   uint32_t pairs, uint32_t topk, uint32_t num_experts, uint32_t world, const uint8_t* data, uint32_t k, const uint32_t* sf,
                   uint32_t sf_stride, uint32_t sf_cols, void* const* peer_data, void* const* peer_sf, uint32_t peer_sf_stride,
                   uint32_t capacity, uint32_t slot_rows, int32_t* pos_of_pair, uint32_t max_blocks) {
    if (!ctx || !expert_of_pair || !local_rank || !block_base || !pair_base || !data || !sf || !peer_data || !peer_sf || !pos_of_pair)
        return fail(DG_ERR_SHAPE, "null argument");
    if (k % 16 || !aligned16(data)) return fail(DG_ERR_SHAPE, "k and the token rows must be multiples of 16 bytes");
    if (topk == 0 || pairs % topk != 0) return fail(DG_ERR_SHAPE, "pairs (%u) must be tokens x topk (%u)", pairs, topk);
    if (world == 0 || num_experts % world != 0) return fail(DG_ERR_SHAPE, "num_experts (%u) must be a multiple of world (%u)", num_experts, world);
    if (peer_sf_stride < (slot_rows ? slot_rows : capacity)) return fail(DG_ERR_SHAPE, "arena scale stride smaller than the rows it indexes");
    if (pairs == 0) return DG_OK;
    dg::EpDispatchParams p;
    p.expert_of_pair = expert_of_pair; p.local_rank = local_rank; p.block_base = block_base; p.pair_base = pair_base;
    p.data = data; p.sf = sf;
    p.peer_data = reinterpret_cast<uint8_t* const*>(peer_data); p.peer_sf = reinterpret_cast<uint32_t* const*>(peer_sf);
    p.pos_of_pair = pos_of_pair;
    p.pairs = pairs; p.topk = topk; p.k = k; p.sf_cols = sf_cols; p.sf_stride = sf_stride; p.peer_sf_stride = peer_sf_stride;
    p.num_experts = num_experts; p.experts_per_rank = num_experts / world; p.capacity = capacity; p.slot_rows = slot_rows;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    uint32_t blocks = ceil_div(pairs, 8);
    if (max_blocks != 0 && blocks > max_blocks) blocks = max_blocks;
    dg::dg_ep_dispatch_kernel<<<blocks, 256, 0, ctx->stream>>>(p);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_ep_combine(dg_ctx* ctx, const int32_t* expert_of_pair, const int32_t* pos_of_pair, const float* weights, uint32_t tokens, uint32_t topk,
                  uint32_t num_experts, uint32_t world, const void* const* peer_rows, size_t pitch, uint32_t n, uint16_t* out, size_t out_pitch,
                  uint32_t max_blocks) {
    if (!ctx || !expert_of_pair || !pos_of_pair || !weights || !peer_rows || !out) return fail(DG_ERR_SHAPE, "null argument");
    if (n % 8 || pitch % 8 || out_pitch % 8 || !aligned16(out)) return fail(DG_ERR_SHAPE, "n and pitches must be multiples of 8 elements");
    if (world == 0 || num_experts % world != 0) return fail(DG_ERR_SHAPE, "num_experts (%u) must be a multiple of world (%u)", num_experts, world);
    if (tokens == 0 || n == 0) return DG_OK;
    dg::EpCombineParams p;
    p.expert_of_pair = expert_of_pair; p.pos_of_pair = pos_of_pair; p.weights = weights;
    p.peer_rows = reinterpret_cast<const uint16_t* const*>(peer_rows);
    p.out = out; p.pitch = pitch; p.out_pitch = out_pitch;
    p.tokens = tokens; p.topk = topk; p.n = n; p.experts_per_rank = num_experts / world;
    DG_CUDA(cudaSetDevice(ctx->ordinal));
    const uint64_t threads = static_cast<uint64_t>(tokens) * (n / 8);
    if (threads > 0xFFFFFF00ull) return fail(DG_ERR_SHAPE, "tokens x n / 8 must fit 32 bits");
    uint32_t blocks = static_cast<uint32_t>((threads + 255) / 256);
    if (max_blocks != 0 && blocks > max_blocks) blocks = max_blocks;
    dg::dg_ep_combine_kernel<<<blocks, 256, 0, ctx->stream>>>(p);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

}  // extern "C"
