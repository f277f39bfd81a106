// Row movers either side of the expert-sharded grouped GEMM: they pack quantised token rows and
// their scale words into all-to-all send rows, unpack received rows into the group-contiguous
// arena (data + packed scale layout), gather result rows for the way back and reduce a token's
// expert outputs.  Byte movers: 16-byte loads/stores, one warp per row.
#pragma once
#include "dg_ptx.cuh"

namespace dg {

// dst row i = src row idx[i] (row_bytes, a multiple of 16); idx[i] < 0 writes zeros.
__global__ void __launch_bounds__(256) dg_gather_rows_kernel(const uint8_t* __restrict__ src, size_t src_pitch, const int32_t* __restrict__ idx,
                                                             uint32_t n_dst, uint32_t row_bytes, uint8_t* __restrict__ dst, size_t dst_pitch) {
    const uint32_t lane = threadIdx.x % 32;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= n_dst) return;
    const int32_t s = __ldg(idx + row);
    uint4* d = reinterpret_cast<uint4*>(dst + row * dst_pitch);
    if (s < 0) {
        for (uint32_t c = lane; c < row_bytes / 16; c += 32) d[c] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* p = reinterpret_cast<const uint4*>(src + static_cast<size_t>(s) * src_pitch);
    for (uint32_t c = lane; c < row_bytes / 16; c += 32) d[c] = __ldg(p + c);
}

// Send row i = [k data bytes of token idx[i] | its sf_cols scale words | zero padding up to out_pitch].
// Scale words come from the packed layout sf[c * sf_stride + token].
__global__ void __launch_bounds__(256) dg_moe_pack_rows_kernel(const uint8_t* __restrict__ data, uint32_t k, const uint32_t* __restrict__ sf,
                                                               uint32_t sf_stride, uint32_t sf_cols, const int32_t* __restrict__ idx, uint32_t n,
                                                               uint8_t* __restrict__ out, size_t out_pitch) {
    const uint32_t lane = threadIdx.x % 32;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= n) return;
    const uint32_t tok = static_cast<uint32_t>(__ldg(idx + row));
    const uint4* p = reinterpret_cast<const uint4*>(data + static_cast<size_t>(tok) * k);
    uint4* d = reinterpret_cast<uint4*>(out + row * out_pitch);
    for (uint32_t c = lane; c < k / 16; c += 32) d[c] = __ldg(p + c);
    uint32_t* tail = reinterpret_cast<uint32_t*>(out + row * out_pitch + k);
    const uint32_t tail_words = static_cast<uint32_t>((out_pitch - k) / 4);
    for (uint32_t c = lane; c < tail_words; c += 32) tail[c] = c < sf_cols ? __ldg(sf + static_cast<size_t>(c) * sf_stride + tok) : 0u;
}

// Arena row i takes received row idx[i]: data bytes to dst_data, scale words to the packed layout
// dst_sf[c * dst_sf_stride + i].  idx[i] < 0 (alignment padding) writes zero data and zero scales.
__global__ void __launch_bounds__(256) dg_moe_unpack_rows_kernel(const uint8_t* __restrict__ in, size_t in_pitch, uint32_t k, uint32_t sf_cols,
                                                                 const int32_t* __restrict__ idx, uint32_t n_dst, uint8_t* __restrict__ dst_data,
                                                                 uint32_t* __restrict__ dst_sf, uint32_t dst_sf_stride) {
    const uint32_t lane = threadIdx.x % 32;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= n_dst) return;
    const int32_t s = __ldg(idx + row);
    uint4* d = reinterpret_cast<uint4*>(dst_data + row * k);
    if (s < 0) {
        for (uint32_t c = lane; c < k / 16; c += 32) d[c] = make_uint4(0, 0, 0, 0);
        for (uint32_t c = lane; c < sf_cols; c += 32) dst_sf[static_cast<size_t>(c) * dst_sf_stride + row] = 0u;
        return;
    }
    const uint8_t* src = in + static_cast<size_t>(s) * in_pitch;
    const uint4* p = reinterpret_cast<const uint4*>(src);
    for (uint32_t c = lane; c < k / 16; c += 32) d[c] = __ldg(p + c);
    const uint32_t* tail = reinterpret_cast<const uint32_t*>(src + k);
    for (uint32_t c = lane; c < sf_cols; c += 32) dst_sf[static_cast<size_t>(c) * dst_sf_stride + row] = __ldg(tail + c);
}

// out[t, :] = bf16( sum_j w[t, j] * rows[pos[t, j], :] ), f32 accumulation in order j = 0..topk-1
// with one fused multiply-add per term; pos < 0 skips the term.  One thread owns 8 columns.
__global__ void __launch_bounds__(256) dg_moe_combine_kernel(const uint16_t* __restrict__ rows, size_t pitch, const int32_t* __restrict__ pos,
                                                             const float* __restrict__ w, uint32_t tokens, uint32_t topk, uint32_t n,
                                                             uint16_t* __restrict__ out, size_t out_pitch) {
    const uint32_t chunks = n / 8;
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<uint64_t>(tokens) * chunks) return;
    const uint32_t t = static_cast<uint32_t>(i / chunks), c = static_cast<uint32_t>(i % chunks);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t j = 0; j < topk; ++j) {
        const int32_t p = __ldg(pos + static_cast<size_t>(t) * topk + j);
        if (p < 0) continue;
        const float wj = __ldg(w + static_cast<size_t>(t) * topk + j);
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(rows + static_cast<size_t>(p) * pitch) + c);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        #pragma unroll
        for (uint32_t q = 0; q < 4; ++q) {
            acc[2 * q] = fmaf(wj, __uint_as_float(u[q] << 16), acc[2 * q]);
            acc[2 * q + 1] = fmaf(wj, __uint_as_float(u[q] & 0xFFFF0000u), acc[2 * q + 1]);
        }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * out_pitch)[c] = o;
}

}  // namespace dg
