// Memory-bound kernels either side of the GEMM: bf16 -> e4m3 / e2m1 quantisation with packed
// UE8M0 scale factors, f32 scale-factor re-layouts, and the group-end table of the contiguous
// MoE layout.  All of them are HBM-bound byte/integer work: 16-byte loads and stores, one warp
// per 1024-element row segment, scale words written straight into the packed layout
//   word(group g, local row r, column c) = sf[(g * cols + c) * align4(group_rows) + r],
//   byte j of a word = exponent of K block 4c + j.
#pragma once
#include "dg_ptx.cuh"
#include "dg_activation.cuh"

namespace dg {

DG_DEVICE float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
DG_DEVICE float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Biased exponent of amax, plus one if its mantissa exceeds the largest mantissa of the
// target format (qmant = 0x600000 for 448, 0x400000 for 6).
DG_DEVICE uint32_t rounded_exp(float amax, uint32_t qmant) { return (__float_as_uint(amax) + 0x7FFFFFu - qmant) >> 23; }

DG_DEVICE uint32_t sf_exp_e4m3(float amax) {
    const uint32_t r = rounded_exp(amax, 0x600000u);
    const uint32_t e = (r < 8u ? 8u : r) - 8u;
    return e < 105u ? 105u : e;
}
// rule 0: the reference crate's CPU MXFP4 rule max(rounded, 128); rule 1: smallest power of two
// that brings the block maximum to 6 or below.
DG_DEVICE uint32_t sf_exp_e2m1(float amax, int rule) {
    const uint32_t r = rounded_exp(amax, 0x400000u);
    if (rule == 0) { const uint32_t e = r < 128u ? 128u : r; return e > 255u ? 255u : e; }
    const uint32_t e = (r < 2u ? 2u : r) - 2u;
    return e < 1u ? 1u : e;
}

struct CastParams {
    const uint16_t* src;   // (rows, src_ld) bf16; with kSiluMul: gate at [0, k), up at [k, 2k) of each row
    uint8_t* dst;          // (rows, k) e4m3 or (rows, k/2) packed e2m1
    uint32_t* sf;          // packed scale words
    uint32_t src_ld, rows, k, group_rows, sf_cols, sf_stride;
    int rule;
    const uint32_t* live_rows;   // optional device word: rows at or beyond it are skipped (a row count only the device knows)
};

// One warp quantises 1024 consecutive K elements of one row: four 16-byte loads per lane, all issued
// before the first use (elements [256*h + 8*lane, +8) for h = 0..3).  kGran = 128: 16 lanes share a scale,
// the warp produces two scale words.  kGran = 32: 4 lanes share a scale, the warp produces 8 words.
// kSiluMul: the value quantised is bf16(silu(gate) * up) (moe.rs:273-296, layout.rs:218-233 followed by the
// activation quantiser), read from a (rows, 2k) gate|up matrix; the bf16 activation never reaches memory.
template <uint32_t kGran, bool kFp4, bool kSiluMul = false>
__global__ void __launch_bounds__(256) dg_cast_kernel(const CastParams p) {
    constexpr uint32_t kLoads = 4, kSeg = 256 * kLoads;
    // a block takes 8 consecutive rows (one per warp) of one segment, so that the scale words of a word column,
    // which are contiguous over rows, leave the block as whole 32-byte sectors
    constexpr uint32_t kWordsPerWarp = kGran == 128 ? kLoads / 2 : 2 * kLoads;
    __shared__ uint32_t words[kWordsPerWarp][8];
    const uint32_t lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const uint32_t segs_per_row = (p.k + kSeg - 1) / kSeg;
    const uint32_t seg = blockIdx.x % segs_per_row, row0 = (blockIdx.x / segs_per_row) * 8;
    if (p.live_rows != nullptr && row0 >= __ldg(p.live_rows)) return;   // the same for the whole block
    const uint32_t row = row0 + warp;
    const bool live = row < p.rows;
    const uint16_t* src_row = p.src + static_cast<size_t>(live ? row : 0) * p.src_ld;

    uint4 raw[kLoads], raw_up[kSiluMul ? kLoads : 1];
    uint32_t k0[kLoads];
    #pragma unroll
    for (uint32_t h = 0; h < kLoads; ++h) {
        k0[h] = seg * kSeg + h * 256 + lane * 8;
        raw[h] = (live && k0[h] < p.k) ? __ldg(reinterpret_cast<const uint4*>(src_row + k0[h])) : make_uint4(0, 0, 0, 0);
        if constexpr (kSiluMul)
            raw_up[h] = (live && k0[h] < p.k) ? __ldg(reinterpret_cast<const uint4*>(src_row + p.k + k0[h])) : make_uint4(0, 0, 0, 0);
    }
    uint32_t exps[kLoads];
    #pragma unroll
    for (uint32_t h = 0; h < kLoads; ++h) {
        float v[8] = {bf16_lo(raw[h].x), bf16_hi(raw[h].x), bf16_lo(raw[h].y), bf16_hi(raw[h].y),
                      bf16_lo(raw[h].z), bf16_hi(raw[h].z), bf16_lo(raw[h].w), bf16_hi(raw[h].w)};
        if constexpr (kSiluMul) {
            const float u[8] = {bf16_lo(raw_up[h].x), bf16_hi(raw_up[h].x), bf16_lo(raw_up[h].y), bf16_hi(raw_up[h].y),
                                bf16_lo(raw_up[h].z), bf16_hi(raw_up[h].z), bf16_lo(raw_up[h].w), bf16_hi(raw_up[h].w)};
            #pragma unroll
            for (uint32_t i = 0; i < 8; i += 2) {
                const float2 a = silu_mul_bf16x2(make_float2(v[i], v[i + 1]), make_float2(u[i], u[i + 1]));
                v[i] = a.x;
                v[i + 1] = a.y;
            }
        }
        float amax = 0.0f;
        #pragma unroll
        for (uint32_t i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        // maximum over the lanes that share a scale (16 for per-128, 4 for per-32 scales); a shuffle ladder: warp reductions over
        // part of a warp run one lane group at a time and measured slower
        #pragma unroll
        for (uint32_t d = kGran / 16; d >= 1; d /= 2) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
        uint32_t e;
        float inv;
        if constexpr (kFp4) {
            e = sf_exp_e2m1(amax, p.rule);
            // rule 0 divides by 2^(e - 127) like the CPU rule: 2^(127 - e) is a normal number down to e = 253, the subnormal
            // 2^-127 for e = 254, and 1 / inf = 0 for e = 255 (a block maximum beyond 1.5 * 2^127)
            inv = __uint_as_float(e <= 253u ? (254u - e) << 23 : (e == 254u ? 0x00400000u : 0u));
        } else {
            e = sf_exp_e4m3(amax);
            inv = __uint_as_float((254u - e) << 23);
        }
        exps[h] = e;
        if (live && k0[h] < p.k) {
            if constexpr (kFp4) {
                float s[8];
                #pragma unroll
                for (uint32_t i = 0; i < 8; ++i) s[i] = v[i] * inv;
                *reinterpret_cast<uint32_t*>(p.dst + static_cast<size_t>(row) * (p.k / 2) + k0[h] / 2) = cvt_e2m1x8(s);
            } else {
                uint2 out;
                out.x = cvt_e4m3x4(scale_pos_zero(v[0], inv), scale_pos_zero(v[1], inv), scale_pos_zero(v[2], inv), scale_pos_zero(v[3], inv));
                out.y = cvt_e4m3x4(scale_pos_zero(v[4], inv), scale_pos_zero(v[5], inv), scale_pos_zero(v[6], inv), scale_pos_zero(v[7], inv));
                *reinterpret_cast<uint2*>(p.dst + static_cast<size_t>(row) * p.k + k0[h]) = out;
            }
        }
    }
    // assemble scale words: exps[h] on lane l belongs to K block (seg*1024 + h*256 + l*8) / kGran.  The first lane of every
    // scale block puts its exponent at the block's byte position and an OR over the lanes of a word collects the four bytes.
    if constexpr (kGran == 128) {
        // word w of this segment covers loads 2w and 2w+1, two 128-element blocks (half-warps) each
        #pragma unroll
        for (uint32_t w = 0; w < kLoads / 2; ++w) {
            uint32_t mine = 0;
            if (lane % 16 == 0) {
                if (k0[2 * w] < p.k) mine |= exps[2 * w] << (8 * (lane / 16));
                if (k0[2 * w + 1] < p.k) mine |= exps[2 * w + 1] << (16 + 8 * (lane / 16));
            }
            const uint32_t word = __reduce_or_sync(0xFFFFFFFFu, mine);
            if (lane == w) words[w][warp] = word;
        }
    } else {
        // load h holds eight 32-element blocks, four lanes each: words 2h (lanes 0..15) and 2h+1 (lanes 16..31)
        #pragma unroll
        for (uint32_t h = 0; h < kLoads; ++h) {
            uint32_t word = (lane % 4 == 0 && k0[h] < p.k) ? exps[h] << (8 * ((lane / 4) % 4)) : 0u;
            word |= __shfl_xor_sync(0xFFFFFFFFu, word, 4);
            word |= __shfl_xor_sync(0xFFFFFFFFu, word, 8);
            if (lane % 16 == 0) words[2 * h + lane / 16][warp] = word;
        }
    }
    __syncthreads();
    // thread t writes word column t / 8 of row t % 8: eight consecutive rows of a column are 32 contiguous bytes
    if (threadIdx.x < kWordsPerWarp * 8) {
        const uint32_t c = threadIdx.x / 8, r = row0 + threadIdx.x % 8;
        const uint32_t col = seg * kWordsPerWarp + c;
        if (r < p.rows && col < p.sf_cols) {
            const uint32_t g = r / p.group_rows, lr = r - g * p.group_rows;
            p.sf[(static_cast<size_t>(g) * p.sf_cols + col) * p.sf_stride + lr] = words[c][threadIdx.x % 8];
        }
    }
}

// f32 power-of-two scales -> packed UE8M0 words (exponent byte, mantissa dropped, K tail = 127).
//   mode 0: src (rows, src_ld) one scale per row per K block
//   mode 1: src (ceil(rows/128), src_ld) one scale per 128x128 tile, expanded per row
//   mode 2: src (groups * k_blocks, src_ld = align4(group_rows)) rows contiguous (transposed form)
struct SfPackParams {
    const float* src;
    uint32_t* dst;
    uint32_t src_ld, rows, group_rows, k_blocks, cols, dst_stride, mode;
};
__global__ void __launch_bounds__(256) dg_sf_pack_kernel(const SfPackParams p) {
    // consecutive threads take consecutive rows of one word column: the writes coalesce
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<uint64_t>(p.rows) * p.cols) return;
    const uint32_t col = static_cast<uint32_t>(idx / p.rows), row = static_cast<uint32_t>(idx % p.rows);
    const uint32_t group = row / p.group_rows, local_row = row - group * p.group_rows;
    uint32_t w = 0;
    #pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
        const uint32_t kc = col * 4 + j;
        uint32_t bits = 0x3F800000u;
        if (kc < p.k_blocks) {
            if (p.mode == 0) bits = __float_as_uint(__ldg(p.src + static_cast<size_t>(row) * p.src_ld + kc));
            else if (p.mode == 1) bits = __float_as_uint(__ldg(p.src + static_cast<size_t>(row / 128) * p.src_ld + kc));
            else bits = __float_as_uint(__ldg(p.src + (static_cast<size_t>(group) * p.k_blocks + kc) * p.src_ld + local_row));
        }
        w |= ((bits >> 23) & 0xFFu) << (8 * j);
    }
    p.dst[(static_cast<size_t>(group) * p.cols + col) * p.dst_stride + local_row] = w;
}

// (batches, mn, sf_k) f32 -> (batches * sf_k, align4(mn)) f32, padding columns zero.
// 32x32 tiles through shared memory so both the reads and the writes coalesce.
__global__ void __launch_bounds__(256) dg_transpose_sf_kernel(const float* __restrict__ src, float* __restrict__ dst, uint32_t mn,
                                                              uint32_t sf_k, uint32_t aligned_mn) {
    __shared__ float tile[32][33];
    const uint32_t b = blockIdx.z, r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const uint32_t tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    for (uint32_t i = ty; i < 32; i += 8) {
        const uint32_t r = r0 + i, c = c0 + tx;
        tile[i][tx] = (r < mn && c < sf_k) ? src[(static_cast<size_t>(b) * mn + r) * sf_k + c] : 0.0f;
    }
    __syncthreads();
    for (uint32_t i = ty; i < 32; i += 8) {
        const uint32_t c = c0 + i, r = r0 + tx;
        if (c < sf_k && r < aligned_mn) dst[(static_cast<size_t>(b) * sf_k + c) * aligned_mn + r] = tile[tx][i];
    }
}

// Group-end table of the contiguous layout: ends[g] = 1 + last row whose m_indices == g.
// Step 1 (grid): atomicMax per row.  Step 2 (one block): running maximum, so a group without
// rows inherits the previous end and the scheduler's prefix walk stays monotone.
__global__ void __launch_bounds__(256) dg_group_ends_kernel(const int32_t* __restrict__ m_indices, uint32_t* ends, uint32_t groups,
                                                            uint32_t m) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= m) return;
    const int32_t g = __ldg(m_indices + i);
    if (g < 0 || static_cast<uint32_t>(g) >= groups) return;
    // only the last row of a run needs to publish
    if (i + 1 < m && __ldg(m_indices + i + 1) == g) return;
    atomicMax(ends + g, static_cast<uint32_t>(i) + 1);
}
__global__ void __launch_bounds__(1024) dg_group_ends_scan_kernel(uint32_t* ends, uint32_t groups) {
    // inclusive running maximum over `groups` entries, 1024 threads, any length
    __shared__ uint32_t warp_max[32];
    __shared__ uint32_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (uint32_t base = 0; base < groups; base += 1024) {
        const uint32_t i = base + threadIdx.x;
        uint32_t v = i < groups ? ends[i] : 0u;
        #pragma unroll
        for (uint32_t d = 1; d < 32; d *= 2) {
            const uint32_t o = __shfl_up_sync(0xFFFFFFFFu, v, d);
            if (threadIdx.x % 32 >= d) v = max(v, o);
        }
        if (threadIdx.x % 32 == 31) warp_max[threadIdx.x / 32] = v;
        __syncthreads();
        uint32_t prefix = carry;
        for (uint32_t w = 0; w < threadIdx.x / 32; ++w) prefix = max(prefix, warp_max[w]);
        v = max(v, prefix);
        if (i < groups) ends[i] = v;
        __syncthreads();
        if (threadIdx.x == 1023) carry = v;
        __syncthreads();
    }
}

// Sum of the f32 partial products of a K-split GEMM: out[m, n] = alpha * sum_s partial[s, m, n], added in order
// s = 0, 1, ... (deterministic), written as bf16 or f32.  One thread owns 4 columns (16-byte loads).
template <bool kBf16>
__global__ void __launch_bounds__(256) dg_splitk_reduce_kernel(const float* __restrict__ partial, uint32_t splits, uint32_t m, uint32_t n,
                                                               uint32_t pitch, float alpha, void* __restrict__ out, uint32_t out_ld) {
    griddep_wait();                // launched beside the tail of the GEMM that writes the partials
    griddep_launch_dependents();
    const uint32_t chunks = (n + 3) / 4;
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<uint64_t>(m) * chunks) return;
    const uint32_t row = static_cast<uint32_t>(i / chunks), c = static_cast<uint32_t>(i % chunks) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* first = partial + static_cast<size_t>(row) * pitch + c;
    const size_t plane = static_cast<size_t>(m) * pitch;
    // four planes' loads in flight before the first add (the planes mostly sit in L2: latency, not bandwidth, is the cost);
    // the adds keep the order s = 0, 1, ...
    for (uint32_t s = 0; s < splits; s += 4) {
        float4 v[4];
        #pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
            v[u] = s + u < splits ? __ldg(reinterpret_cast<const float4*>(first + (s + u) * plane)) : make_float4(0.f, 0.f, 0.f, 0.f);
        #pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
            if (s + u < splits) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
        }
    }
    acc.x *= alpha; acc.y *= alpha; acc.z *= alpha; acc.w *= alpha;
    const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
    if constexpr (kBf16) {
        uint16_t* o = static_cast<uint16_t*>(out) + static_cast<size_t>(row) * out_ld + c;
        if (c + 4 <= n && (reinterpret_cast<uintptr_t>(o) & 7) == 0) {
            *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16x2(vals[0], vals[1]), pack_bf16x2(vals[2], vals[3]));
        } else {
            for (uint32_t j = 0; j < 4 && c + j < n; ++j) o[j] = static_cast<uint16_t>(pack_bf16x2(vals[j], 0.f) & 0xFFFF);
        }
    } else {
        float* o = static_cast<float*>(out) + static_cast<size_t>(row) * out_ld + c;
        for (uint32_t j = 0; j < 4 && c + j < n; ++j) o[j] = vals[j];
    }
}

// Self-test of the bounded wait every kernel of this library uses: one warp waits on a barrier nothing will ever
// arrive on, with a short limit.  The wait must give up, record (code, block, site) in the status block and let the
// kernel finish normally, leaving the context usable.
__global__ void dg_expire_wait_kernel(Status* status, uint64_t limit_ns) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    mbar_wait(&bar, 0, &abort_flag, status, 0x700, limit_ns);
}

// Packed e2m1 -> one code per byte (low nibble), 16 bytes in, 32 bytes out per thread.
__global__ void __launch_bounds__(256) dg_unpack_fp4_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t packed_len) {
    const uint64_t i = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 16;
    if (i + 16 <= packed_len) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
        #pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
            // byte b of w -> two output bytes (low nibble, high nibble)
            const uint32_t lo = w[q] & 0x0F0F0F0Fu, hi = (w[q] >> 4) & 0x0F0F0F0Fu;
            o[2 * q] = __byte_perm(lo, hi, 0x5140);
            o[2 * q + 1] = __byte_perm(lo, hi, 0x7362);
        }
        uint4* out = reinterpret_cast<uint4*>(dst + 2 * i);
        out[0] = make_uint4(o[0], o[1], o[2], o[3]);
        out[1] = make_uint4(o[4], o[5], o[6], o[7]);
    } else {
        for (uint64_t j = i; j < packed_len; ++j) {
            dst[2 * j] = src[j] & 0x0F;
            dst[2 * j + 1] = src[j] >> 4;
        }
    }
}

}  // namespace dg
