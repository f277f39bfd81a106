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

// ---------------------------------------------------------------------------------------------
// Expert-parallel exchange over peer memory.  Every rank owns num_experts / world consecutive
// experts and exposes three buffers to its peers: the group-contiguous arena (e4m3 rows), the
// arena's packed scale words, and the result rows of its last grouped GEMM.  A step:
//   rank pairs    stable position of every (token, j) pair among this rank's pairs for its expert
//   block scan    per-expert totals of this rank (exchanged with a small all-gather)
//   layout        from all ranks' totals: where each expert's group starts on its owner, where this
//                 rank's rows go inside it, and the owner's group-end table for the grouped GEMM
//   dispatch      every pair's row and scale words are written straight to their arena row on the
//                 owner (plain stores to peer memory; no send buffer, no unpack pass)
//   combine       every token reads its topk result rows from the owners' result buffers and
//                 reduces them (plain loads from peer memory; no gather pass, no receive buffer)
// Cross-rank ordering (arena complete before the GEMM reads it, results complete before the
// combine reads them) is the host's job: a collective on the same stream between the steps.
// None of these kernels waits on another rank.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kEpChunk = 256;   // pairs per block of the ranking kernel

// local_rank[p] = number of earlier pairs of the same chunk with the same expert;
// block_hist[b * num_experts + e] = pairs of chunk b routed to expert e.  Expert ids outside
// [0, num_experts) are dropped (rank -1): such a pair is neither sent nor reduced.
__global__ void __launch_bounds__(kEpChunk) dg_ep_rank_pairs_kernel(const int32_t* __restrict__ expert_of_pair, uint32_t pairs, uint32_t num_experts,
                                                                    int32_t* __restrict__ local_rank, uint32_t* __restrict__ block_hist) {
    extern __shared__ uint32_t ep_hist[];
    __shared__ int32_t ids[kEpChunk];
    const uint32_t tid = threadIdx.x, p = blockIdx.x * kEpChunk + tid;
    int32_t e = p < pairs ? __ldg(expert_of_pair + p) : -1;
    if (e < 0 || static_cast<uint32_t>(e) >= num_experts) e = -1;
    ids[tid] = e;
    for (uint32_t i = tid; i < num_experts; i += kEpChunk) ep_hist[i] = 0;
    __syncthreads();
    int32_t rank = 0;
    for (uint32_t j = 0; j < tid; ++j) rank += ids[j] == e ? 1 : 0;
    if (e >= 0) atomicAdd(&ep_hist[e], 1u);
    if (p < pairs) local_rank[p] = e >= 0 ? rank : -1;
    __syncthreads();
    for (uint32_t i = tid; i < num_experts; i += kEpChunk) block_hist[static_cast<size_t>(blockIdx.x) * num_experts + i] = ep_hist[i];
}

// Exclusive scan over chunks, per expert, in place; counts[e] = this rank's pairs for expert e.  One warp per expert:
// 32 chunks per round (independent loads, shuffle scan), so a scan over hundreds of chunks costs a handful of memory
// round trips instead of one per chunk.
__global__ void __launch_bounds__(256) dg_ep_block_scan_kernel(uint32_t* __restrict__ block_hist, uint32_t num_blocks, uint32_t num_experts,
                                                               uint32_t* __restrict__ counts) {
    const uint32_t lane = threadIdx.x % 32;
    const uint32_t e = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (e >= num_experts) return;
    uint32_t running = 0;
    for (uint32_t b0 = 0; b0 < num_blocks; b0 += 32) {
        const uint32_t b = b0 + lane;
        const size_t at = static_cast<size_t>(b) * num_experts + e;
        const uint32_t v = b < num_blocks ? block_hist[at] : 0u;
        uint32_t inc = v;                                     // inclusive scan over the 32 lanes
        #pragma unroll
        for (uint32_t d = 1; d < 32; d *= 2) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, d);
            if (lane >= d) inc += up;
        }
        if (b < num_blocks) block_hist[at] = running + inc - v;
        running += __shfl_sync(0xFFFFFFFFu, inc, 31);
    }
    if (lane == 0) counts[e] = running;
}

// all_counts: (world, num_experts) pairs per source rank and expert.  One block.
//   pair_base[e]   arena row (on the owner of e) of this rank's first pair for expert e
//   group_ends[l]  one past the last valid arena row of local expert l (the grouped GEMM's table)
//   totals[0..3]   arena rows in use on this rank (groups padded to `alignment`), valid rows on this
//                  rank, 1 if any owner's arena would exceed `capacity` rows (dispatch then drops the
//                  rows that do not fit), largest arena in use on any rank
// slot_rows != 0 selects the masked layout instead: local expert l owns the fixed slot of rows [l * slot_rows,
// (l + 1) * slot_rows), group_ends[l] is then its valid row count (the masked GEMM's masked_m), and the overflow flag is
// raised when some expert receives more than slot_rows rows (or the slots exceed `capacity`).
__global__ void __launch_bounds__(1024) dg_ep_layout_kernel(const uint32_t* __restrict__ all_counts, uint32_t world, uint32_t rank, uint32_t num_experts,
                                                            uint32_t alignment, uint32_t capacity, uint32_t slot_rows, uint32_t* __restrict__ pair_base,
                                                            uint32_t* __restrict__ group_ends, uint32_t* __restrict__ totals) {
    extern __shared__ uint32_t ep_smem[];
    uint32_t* rows_of = ep_smem;                  // [num_experts] rows of the expert over all source ranks
    uint32_t* before_me = ep_smem + num_experts;  // [num_experts] rows from lower source ranks
    uint32_t* start_of = ep_smem + 2 * num_experts;
    __shared__ uint32_t arena_rows[1024];
    const uint32_t local = num_experts / world;
    for (uint32_t e = threadIdx.x; e < num_experts; e += blockDim.x) {
        uint32_t total = 0, before = 0;
        for (uint32_t s = 0; s < world; ++s) {
            const uint32_t c = __ldg(all_counts + static_cast<size_t>(s) * num_experts + e);
            if (s < rank) before += c;
            total += c;
        }
        rows_of[e] = total;
        before_me[e] = before;
    }
    __syncthreads();
    __shared__ uint32_t slot_overflow;
    if (threadIdx.x == 0) slot_overflow = 0;
    __syncthreads();
    // one warp per owner: padded group sizes scanned 32 experts at a time
    const uint32_t lane = threadIdx.x % 32;
    for (uint32_t owner = threadIdx.x / 32; owner < world; owner += blockDim.x / 32) {
        uint32_t running = 0, valid = 0;
        for (uint32_t l0 = 0; l0 < local; l0 += 32) {
            const uint32_t l = l0 + lane, e = owner * local + l;
            const uint32_t r = l < local ? rows_of[e] : 0u;
            const uint32_t padded = slot_rows ? (l < local ? slot_rows : 0u) : (r + alignment - 1) / alignment * alignment;
            if (slot_rows && r > slot_rows) slot_overflow = 1;
            uint32_t inc = padded, sum_r = r;
            #pragma unroll
            for (uint32_t d = 1; d < 32; d *= 2) {
                const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, d);
                if (lane >= d) inc += up;
                sum_r += __shfl_xor_sync(0xFFFFFFFFu, sum_r, d);
            }
            if (l < local) {
                const uint32_t start = running + inc - padded;
                start_of[e] = start;
                if (owner == rank) group_ends[l] = slot_rows ? r : start + r;
            }
            running += __shfl_sync(0xFFFFFFFFu, inc, 31);
            valid += sum_r;
        }
        if (lane == 0) {
            arena_rows[owner] = running;
            if (owner == rank) { totals[0] = running; totals[1] = valid; }
        }
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < num_experts; e += blockDim.x) pair_base[e] = start_of[e] + before_me[e];
    if (threadIdx.x == 0) {
        uint32_t largest = 0;
        for (uint32_t s = 0; s < world; ++s) largest = arena_rows[s] > largest ? arena_rows[s] : largest;
        totals[2] = (largest > capacity || slot_overflow) ? 1u : 0u;
        totals[3] = largest;
    }
}

struct EpDispatchParams;
DG_DEVICE void ep_dispatch_pair(const EpDispatchParams& p, uint64_t pair, uint32_t lane);

struct EpDispatchParams {
    const int32_t* expert_of_pair;   // (pairs)
    const int32_t* local_rank;       // (pairs)
    const uint32_t* block_base;      // (chunks, num_experts) exclusive scan of the chunk histograms
    const uint32_t* pair_base;       // (num_experts)
    const uint8_t* data;             // (tokens, k) e4m3 rows of this rank's tokens
    const uint32_t* sf;              // packed scale words sf[c * sf_stride + token]
    uint8_t* const* peer_data;       // [world] arena of each rank, (capacity, k)
    uint32_t* const* peer_sf;        // [world] arena scale words, sf[c * peer_sf_stride + row]
    int32_t* pos_of_pair;            // (pairs) arena row on the owner, -1 if dropped
    uint32_t pairs, topk, k, sf_cols, sf_stride, peer_sf_stride, num_experts, experts_per_rank, capacity;
    uint32_t slot_rows;              // masked layout: rows per expert slot (0: contiguous layout); the arena's scale words are then
                                     // laid out per slot, sf[(slot * sf_cols + c) * peer_sf_stride + row in slot]
};

DG_DEVICE void ep_dispatch_pair(const EpDispatchParams& p, uint64_t pair, uint32_t lane) {
    const int32_t lr = __ldg(p.local_rank + pair);
    if (lr < 0) { if (lane == 0) p.pos_of_pair[pair] = -1; return; }
    const uint32_t e = static_cast<uint32_t>(__ldg(p.expert_of_pair + pair));
    const uint32_t row = __ldg(p.pair_base + e) + __ldg(p.block_base + (pair / kEpChunk) * p.num_experts + e) + static_cast<uint32_t>(lr);
    const uint32_t owner = e / p.experts_per_rank, slot = e - owner * p.experts_per_rank;
    const uint32_t in_slot = row - slot * p.slot_rows;      // masked layout only
    if (row >= p.capacity || (p.slot_rows != 0 && in_slot >= p.slot_rows)) { if (lane == 0) p.pos_of_pair[pair] = -1; return; }
    if (lane == 0) p.pos_of_pair[pair] = static_cast<int32_t>(row);
    const uint32_t tok = static_cast<uint32_t>(pair / p.topk);
    const uint4* src = reinterpret_cast<const uint4*>(p.data + static_cast<size_t>(tok) * p.k);
    uint4* dst = reinterpret_cast<uint4*>(p.peer_data[owner] + static_cast<size_t>(row) * p.k);
    const uint32_t vecs = p.k / 16;
    uint32_t c = lane;
    constexpr uint32_t kDeep = 8;          // loads in flight per lane before the first store (4 KB per warp)
    for (; c + 32 * (kDeep - 1) < vecs; c += 32 * kDeep) {
        uint4 v[kDeep];
        #pragma unroll
        for (uint32_t i = 0; i < kDeep; ++i) v[i] = __ldg(src + c + 32 * i);
        #pragma unroll
        for (uint32_t i = 0; i < kDeep; ++i) dst[c + 32 * i] = v[i];
    }
    for (; c + 96 < vecs; c += 128) {
        const uint4 v0 = __ldg(src + c), v1 = __ldg(src + c + 32), v2 = __ldg(src + c + 64), v3 = __ldg(src + c + 96);
        dst[c] = v0; dst[c + 32] = v1; dst[c + 64] = v2; dst[c + 96] = v3;
    }
    for (; c < vecs; c += 32) dst[c] = __ldg(src + c);
    uint32_t* dsf = p.peer_sf[owner];
    const size_t sf_base = p.slot_rows ? static_cast<size_t>(slot) * p.sf_cols * p.peer_sf_stride + in_slot : row;
    for (uint32_t w = lane; w < p.sf_cols; w += 32)
        dsf[sf_base + static_cast<size_t>(w) * p.peer_sf_stride] = __ldg(p.sf + static_cast<size_t>(w) * p.sf_stride + tok);
}


// One warp per (token, j) pair; the grid may be smaller than the pair count (warps stride over the pairs), which
// lets a caller leave room on every SM for a kernel running beside this one.
__global__ void __launch_bounds__(256) dg_ep_dispatch_kernel(const EpDispatchParams p) {
    const uint32_t lane = threadIdx.x % 32;
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x / 32);
    for (uint64_t pair = static_cast<uint64_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32; pair < p.pairs; pair += warps)
        ep_dispatch_pair(p, pair, lane);
}

struct EpCombineParams {
    const int32_t* expert_of_pair;    // (tokens, topk)
    const int32_t* pos_of_pair;       // (tokens, topk) result row on the owner, < 0 skips the term
    const float* weights;             // (tokens, topk)
    const uint16_t* const* peer_rows; // [world] bf16 result rows of each rank, (capacity, pitch)
    uint16_t* out;                    // (tokens, out_pitch) bf16
    size_t pitch, out_pitch;
    uint32_t tokens, topk, n, experts_per_rank;
};

// out[t, :] = bf16( sum_j w[t, j] * rows_of_owner(t, j)[pos[t, j], :] ): the same ordered fused multiply-add
// chain as dg_moe_combine_kernel, reading each term from the rank that computed it.  One thread owns 8 columns.
__global__ void __launch_bounds__(256) dg_ep_combine_kernel(const EpCombineParams p) {
    const uint32_t chunks = p.n / 8;
    // tokens x chunks fits 32 bits (checked by the host): 32-bit division instead of the 64-bit sequence
    const uint32_t total = p.tokens * chunks, stride = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const uint32_t t = i / chunks, c = i - t * chunks;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    constexpr uint32_t kDeep = 8;
    for (uint32_t j0 = 0; j0 < p.topk; j0 += kDeep) {
        // up to eight independent peer loads in flight before the first use
        uint4 v[kDeep];
        float wj[kDeep];
        bool live[kDeep];
        #pragma unroll
        for (uint32_t u = 0; u < kDeep; ++u) {
            const uint32_t j = j0 + u;
            live[u] = false;
            if (j < p.topk) {
                const size_t at = static_cast<size_t>(t) * p.topk + j;
                const int32_t row = __ldg(p.pos_of_pair + at);
                if (row >= 0) {
                    const uint32_t owner = static_cast<uint32_t>(__ldg(p.expert_of_pair + at)) / p.experts_per_rank;
                    live[u] = true;
                    wj[u] = __ldg(p.weights + at);
                    v[u] = *(reinterpret_cast<const uint4*>(p.peer_rows[owner] + static_cast<size_t>(row) * p.pitch) + c);
                }
            }
        }
        #pragma unroll
        for (uint32_t u = 0; u < kDeep; ++u) {
            if (!live[u]) continue;
            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
            #pragma unroll
            for (uint32_t q = 0; q < 4; ++q) {
                acc[2 * q] = fmaf(wj[u], __uint_as_float(w[q] << 16), acc[2 * q]);
                acc[2 * q + 1] = fmaf(wj[u], __uint_as_float(w[q] & 0xFFFF0000u), acc[2 * q + 1]);
            }
        }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(p.out + static_cast<size_t>(t) * p.out_pitch)[c] = o;
    }
}

}  // namespace dg
