// FP8 GEMM with f32 scale factors applied exactly (the reference's older "1d2d" contract):
//
//   D[g][m, n] = sum over 128-wide K blocks kb of ( sum_{k in kb} A[m, k] B[n, k] ) * sfa[m, kb] * sfb[n / 128, kb]
//
// which is what deepgemm/src/reference.rs:85-114 (and :133-208 for the grouped layouts) computes.  The tensor core's block
// scaling only takes power-of-two (UE8M0) scales, so an f32 scale with a mantissa cannot ride the UMMA: here every K block
// is multiplied on its own (tcgen05.mma kind::f8f6f4 into one of two TMEM buffers, starting from zero) and the epilogue
// warps fold it into f32 accumulators they keep in registers: acc += (block * sfa) * sfb, the reference's order of
// operations.  One 384-thread CTA per SM, 128 x 128 tiles: warp 0 loads A / B k-blocks with TMA, warp 1 issues the UMMAs, and
// eight epilogue warps (4-11) each own 32 accumulator rows x 64 columns (a warp reads the TMEM lanes of its quadrant, warp % 4;
// warps 4-7 take columns 0-63, warps 8-11 columns 64-127), read every K block's partial tile (tcgen05.ld), scale and add it,
// and at the end store bf16 through swizzled staging and TMA.  Reading a partial tile out of TMEM per 128 of K costs more
// than that block's tensor time even with eight warps, so this path stays well below the block-scaled kernel's rate: it
// exists for exactness with arbitrary scales, the UE8M0 path for speed.
#pragma once
#include "dg_gemm_kernel.cuh"

namespace dg {

constexpr uint32_t kF32BlockN = 128;
constexpr uint32_t kF32Threads = 384;      // producer, UMMA issuer, two idle warps, eight epilogue warps
constexpr uint32_t kF32ColsPerWarp = 64;   // accumulator columns an epilogue warp keeps in registers

struct F32ScaleParams {
    GemmParams g;              // shape, layout, scheduler inputs (block_n = tile_n = 128, block_k_elems = 128)
    const float* sfa_t;        // activation scales, transposed: [(group * k_blocks + kb) * sfa_stride + row]
    const float* sfb;          // weight scales: [(group * n_blocks128 + n / 128) * k_blocks + kb]
    uint32_t sfa_stride;       // align4(rows per group)
    uint32_t k_blocks, n_blocks128;
};

// kind::f8f6f4 instruction descriptor, e4m3 operands, f32 accumulate, both K-major:
//   [4,6) D format (1 = f32), [7,10) A format (0 = e4m3), [10,13) B format, [17,23) N >> 3, [24,29) M >> 4.
DG_DEVICE uint32_t make_idesc_f8(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }

DG_DEVICE void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(kF32Threads, 1)
dg_gemm_f32scale_kernel(const __grid_constant__ F32ScaleParams q, const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_d) {
    const GemmParams& p = q.g;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    constexpr uint32_t kTile = kBlockM * kBlockKBytes;        // 16 KB per operand and k-block
    constexpr uint32_t kEpiBuf = 2048;                        // 32 rows x 64 bytes of bf16 per staging buffer
    const uint32_t num_stages = p.num_stages;

    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem_a + num_stages * kTile;
    uint8_t* smem_epi = smem_b + num_stages * kTile;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + 16 * kEpiBuf);
    uint64_t* bar_full = bars;
    uint64_t* bar_empty = bars + kMaxStages;
    uint64_t* bar_tmem_full = bars + 2 * kMaxStages;         // a K block's partial tile is complete in TMEM buffer e
    uint64_t* bar_tmem_empty = bars + 2 * kMaxStages + 2;    // the epilogue warps have read buffer e
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < num_stages; ++s) {
            mbar_init(bar_full + s, 1);
            mbar_init(bar_empty + s, 1);
        }
        for (uint32_t e = 0; e < 2; ++e) {
            mbar_init(bar_tmem_full + e, 1);
            mbar_init(bar_tmem_empty + e, 8);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_d);
    }
    if (warp == 1) {
        tmem_alloc<1>(tmem_slot, 2 * kF32BlockN);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_wait();
    griddep_launch_dependents();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t total_kb = q.k_blocks;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        Scheduler sched(p, 1);
        Tile t;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        while (ok && sched.next(t)) {
            for (uint32_t kb = 0; kb < total_kb; ++kb) {
                if (!mbar_wait_warp(bar_empty + stage, phase ^ 1, abort_flag, p.status, 0x100 + stage)) { ok = false; break; }
                if (elect_one()) {
                    mbar_arrive_expect_tx(bar_full + stage, 2 * kTile);
                    const int32_t kx = static_cast<int32_t>(kb * kBlockKBytes);
                    tma_load_3d(smem_a + stage * kTile, &tmap_a, bar_full + stage, kx, static_cast<int32_t>(t.m0), static_cast<int32_t>(t.ga));
                    tma_load_3d(smem_b + stage * kTile, &tmap_b, bar_full + stage, kx, static_cast<int32_t>(t.n0), static_cast<int32_t>(t.gb));
                }
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- UMMA issuer
        Scheduler sched(p, 1);
        Tile t;
        uint32_t stage = 0, phase = 0, block = 0;
        const uint32_t idesc = make_idesc_f8(kBlockM, kF32BlockN);
        bool ok = true;
        while (ok && sched.next(t)) {
            for (uint32_t kb = 0; kb < total_kb; ++kb, ++block) {
                const uint32_t e = block & 1, buf_phase = (block >> 1) & 1;
                if (!mbar_wait_warp(bar_tmem_empty + e, buf_phase ^ 1, abort_flag, p.status, 0x200 + e)) { ok = false; break; }
                if (!mbar_wait_warp(bar_full + stage, phase, abort_flag, p.status, 0x300 + stage)) { ok = false; break; }
                tc_fence_after();
                const uint64_t a_desc = make_smem_desc(smem_u32(smem_a + stage * kTile), 0, 1024, 2);
                const uint64_t b_desc = make_smem_desc(smem_u32(smem_b + stage * kTile), 0, 1024, 2);
                if (elect_one()) {
                    #pragma unroll
                    for (uint32_t k = 0; k < kBlockKBytes / kUmmaKBytes; ++k)
                        umma_f8(tmem_base + e * kF32BlockN, a_desc + k * (kUmmaKBytes >> 4), b_desc + k * (kUmmaKBytes >> 4), idesc, k != 0 ? 1u : 0u);
                    umma_commit(bar_empty + stage);
                    umma_commit(bar_tmem_full + e);
                }
                __syncwarp();
                if (++stage == num_stages) { stage = 0; phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue
        const uint32_t ew = warp % 4, col_half = (warp - 4) / 4;       // TMEM lane quadrant; which 64 of the tile's 128 columns
        uint8_t* buf0 = smem_epi + (warp - 4) * 2 * kEpiBuf;
        Scheduler sched(p, 1);
        Tile t;
        uint32_t block = 0, buf_idx = 0;
        bool ok = true;
        while (ok && sched.next(t)) {
            const uint32_t row0 = t.m0 + ew * 32, row = row0 + lane;
            const bool row_ok = row < t.m_end;
            // the activation scale of this thread's row for K block kb, and the weight scale of the tile's 128 columns
            const float* sfa_row = q.sfa_t + static_cast<size_t>(t.ga) * total_kb * q.sfa_stride + row;
            const float* sfb_tile = q.sfb + (static_cast<size_t>(t.gb) * q.n_blocks128 + t.n0 / 128) * total_kb;
            float acc[kF32ColsPerWarp];
            #pragma unroll
            for (uint32_t i = 0; i < kF32ColsPerWarp; ++i) acc[i] = 0.0f;
            for (uint32_t kb = 0; kb < total_kb; ++kb, ++block) {
                const uint32_t e = block & 1, buf_phase = (block >> 1) & 1;
                const float sa = row_ok ? __ldg(sfa_row + static_cast<size_t>(kb) * q.sfa_stride) : 0.0f;
                const float sb = __ldg(sfb_tile + kb);
                if (!mbar_wait(bar_tmem_full + e, buf_phase, abort_flag, p.status, 0x600 + e)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((ew * 32) << 16) + e * kF32BlockN + col_half * kF32ColsPerWarp;
                #pragma unroll
                for (uint32_t c = 0; c < kF32ColsPerWarp / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, v);
                    tmem_ld_wait_x32(v);
                    if (c + 1 == kF32ColsPerWarp / 32) {
                        // the buffer is in registers: hand it back to the UMMA warp
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tmem_empty + e);
                    }
                    // two elements per instruction (packed f32x2: the same IEEE operations, half the issue slots)
                    const float2 sa2 = make_float2(sa, sa), sb2 = make_float2(sb, sb);
                    #pragma unroll
                    for (uint32_t i = 0; i < 32; i += 2) {
                        const float2 x = __fmul2_rn(__fmul2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sa2), sb2);
                        const float2 r = __fadd2_rn(make_float2(acc[c * 32 + i], acc[c * 32 + i + 1]), x);
                        acc[c * 32 + i] = r.x;
                        acc[c * 32 + i + 1] = r.y;
                    }
                }
            }
            if (!ok) break;
            // bf16 rows through 64-byte-swizzled staging, one TMA store per 32 columns (rows past the group's end are cut off by
            // the store's 32-row granularity exactly as in the block-scaled kernel)
            #pragma unroll
            for (uint32_t c = 0; c < kF32ColsPerWarp / 32; ++c) {
                uint8_t* buf = buf0 + buf_idx * kEpiBuf;
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
                const uint32_t row_addr = smem_u32(buf) + lane * 64;
                #pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    const uint32_t chunk = j ^ ((lane >> 1) & 3);
                    st_shared_v4(row_addr + chunk * 16, pack_bf16x2(acc[c * 32 + 8 * j + 0], acc[c * 32 + 8 * j + 1]),
                                 pack_bf16x2(acc[c * 32 + 8 * j + 2], acc[c * 32 + 8 * j + 3]), pack_bf16x2(acc[c * 32 + 8 * j + 4], acc[c * 32 + 8 * j + 5]),
                                 pack_bf16x2(acc[c * 32 + 8 * j + 6], acc[c * 32 + 8 * j + 7]));
                }
                fence_proxy_async_smem();
                __syncwarp();
                const uint32_t col0 = t.n0 + col_half * kF32ColsPerWarp + c * 32;
                if (lane == 0) {
                    if (col0 < p.n && row0 < t.m_end) tma_store_3d(&tmap_d, buf, static_cast<int32_t>(col0), static_cast<int32_t>(row0), static_cast<int32_t>(t.gd));
                    tma_store_commit();
                }
                buf_idx ^= 1;
            }
        }
        if (lane == 0) tma_store_wait<0>();
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, 2 * kF32BlockN);
    }
}

inline uint32_t f32scale_smem_bytes(uint32_t stages) { return 1024 + stages * 2 * kBlockM * kBlockKBytes + 16 * 2048 + (2 * kMaxStages + 4) * 8 + 16; }

}  // namespace dg
