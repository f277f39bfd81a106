// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05
// (TMEM allocation, UMMA issue, commit, TMEM loads), proxy fences.  Every wait is
// bounded: a wait that runs out records where it gave up and returns false so the
// kernel can tear down instead of hanging the device.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dg {

#define DG_DEVICE __device__ __forceinline__

DG_DEVICE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
DG_DEVICE uint32_t lane_id() { uint32_t l; asm volatile("mov.u32 %0, %%laneid;" : "=r"(l)); return l; }
DG_DEVICE uint64_t global_ns() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

DG_DEVICE bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
DG_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
DG_DEVICE void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
DG_DEVICE void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DG_DEVICE void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Arrive on the same-offset barrier of CTA `cta` of the cluster.
DG_DEVICE void mbar_arrive_remote(uint64_t* bar, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}\n" ::"r"(smem_u32(bar)),
        "r"(cta)
        : "memory");
}
DG_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Device-visible record of a wait that ran out.  word[0] = code (0 = fine),
// word[1] = block, word[2] = role/site tag, word[3] = extra.
struct Status {
    uint32_t code, block, site, extra;
};
constexpr uint32_t kStatusTimeout = 1;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s: far above any legal wait of these kernels

// Bounded wait.  `abort_flag` is a shared-memory word any role sets when it gives
// up; the others see it within a few hundred polls and leave as well.
DG_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, Status* status, uint32_t site,
                         uint64_t limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    uint32_t polls = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++polls & 0xFF) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                if (status != nullptr && atomicCAS(&status->code, 0u, kStatusTimeout) == 0u) {
                    status->block = blockIdx.x;
                    status->site = site;
                    status->extra = parity;
                    __threadfence();
                }
                return false;
            }
        }
    }
}

// Whole-warp flavour: every lane polls, the verdict is combined with a vote so the branch that
// follows is warp-uniform (the compiler then keeps loop state, addresses and descriptors in
// uniform registers, which the TMA and tcgen05 issue paths read directly).
DG_DEVICE bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, Status* status, uint32_t site) {
    const bool ok = mbar_wait(bar, parity, abort_flag, status, site);
    return __all_sync(0xFFFFFFFFu, ok);
}

// -------------------------------------------------------------------- fences
DG_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
DG_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DG_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
DG_DEVICE void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
DG_DEVICE void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
DG_DEVICE void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
DG_DEVICE void cluster_sync() { cluster_arrive(); cluster_wait(); }
DG_DEVICE uint32_t cluster_cta_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }

// ----------------------------------------------------------------------- TMA
DG_DEVICE void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2-D / 3-D tiled loads into this CTA's shared memory, completion on `bar`.
// x is the innermost coordinate and must keep x * elem_size a multiple of 16 bytes.
DG_DEVICE void tma_load_2d(void* smem, const void* tmap, uint64_t* bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
DG_DEVICE void tma_load_3d(void* smem, const void* tmap, uint64_t* bar, int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// Same loads issued from a CTA pair: the completion bytes are signalled on the
// barrier at the given (possibly peer-CTA) shared::cluster address.
DG_DEVICE void tma_load_3d_2cta(void* smem, const void* tmap, uint32_t bar_cluster_addr, int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
        : "memory");
}
DG_DEVICE void tma_load_2d_2cta(void* smem, const void* tmap, uint32_t bar_cluster_addr, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
// 4-D forms: the K-major operand seen as (128 bytes, rows, K slabs, groups), so that one instruction brings both K slabs
// of a two-slab stage (x is always 0; slab and row coordinates have no alignment rule).
DG_DEVICE void tma_load_4d(void* smem, const void* tmap, uint64_t* bar, int32_t x, int32_t y, int32_t z, int32_t w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
DG_DEVICE void tma_load_4d_2cta(void* smem, const void* tmap, uint32_t bar_cluster_addr, int32_t x, int32_t y, int32_t z, int32_t w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
// The same loads with an L2 eviction hint.  evict_first marks lines that will not be read again (an operand streamed
// from DRAM exactly once): they leave L2 before anything else does, instead of pushing out lines that are still needed or
// forcing write-backs of dirty ones; measured on B200, a streamed operand arrives 7-25 % faster with the hint.
DG_DEVICE uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
DG_DEVICE void tma_load_3d_hint(void* smem, const void* tmap, uint64_t* bar, int32_t x, int32_t y, int32_t z, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}
DG_DEVICE void tma_load_3d_2cta_hint(void* smem, const void* tmap, uint32_t bar_cluster_addr, int32_t x, int32_t y, int32_t z, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(
            smem_u32(smem)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}
DG_DEVICE void tma_store_3d(const void* tmap, const void* smem, int32_t x, int32_t y, int32_t z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(smem_u32(smem)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
// Same tile, added to what global memory holds (element type of the tensor map: f32 or bf16).
DG_DEVICE void tma_reduce_add_3d(const void* tmap, const void* smem, int32_t x, int32_t y, int32_t z) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(smem_u32(smem)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
DG_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
DG_DEVICE void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
DG_DEVICE void tma_store_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

DG_DEVICE uint32_t mapa_u32(uint32_t smem_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
    return r;
}

// ------------------------------------------------------------------- tcgen05
template <int CTAS>
DG_DEVICE void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    if constexpr (CTAS == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
template <int CTAS>
DG_DEVICE void tmem_relinquish() {
    if constexpr (CTAS == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTAS>
DG_DEVICE void tmem_dealloc(uint32_t addr, uint32_t cols) {
    if constexpr (CTAS == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

// Shared-memory matrix descriptor (K-major operand rows of 128/64/32 swizzled bytes,
// or an unswizzled 8x16-byte core-matrix layout for the scale-factor copy).
//   [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte
//   offset >> 4, [46,48) version = 1, [61,64) swizzle: 0 none, 2 128B, 4 64B, 6 32B.
DG_DEVICE uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    d |= static_cast<uint64_t>(layout & 7) << 61;
    return d;
}

// Block-scaled instruction descriptor (UE8M0 scales, f32 accumulate):
//   [4,6) B scale id, [7,10) A format, [10,13) B format, [15] A MN-major, [16] B MN-major,
//   [17,23) N >> 3, [23] scale format (1 = UE8M0), [24,29) M >> 4, [29,31) A scale id.
// Formats: 0 = e4m3, 5 = e2m1 (kind::mxf8f6f4); 1 = e2m1 (kind::mxf4).
DG_DEVICE uint32_t make_idesc_block_scaled(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt) {
    return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}
// kind::f16 instruction descriptor, bf16 operands, f32 accumulate, both K-major:
//   [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format, [17,23) N >> 3, [24,29) M >> 4.
DG_DEVICE uint32_t make_idesc_bf16(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
DG_DEVICE uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_id, uint32_t b_id) {
    return idesc | (b_id << 4) | (a_id << 29);
}

template <int CTAS, bool MXF4>
DG_DEVICE void umma_block_scaled(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                 uint32_t sfb_tmem, uint32_t accumulate) {
    if constexpr (!MXF4) {
        if constexpr (CTAS == 1)
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(d_tmem),
                "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
                : "memory");
        else
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(d_tmem),
                "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
                : "memory");
    } else {
        if constexpr (CTAS == 1)
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(d_tmem),
                "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
                : "memory");
        else
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(d_tmem),
                "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
                : "memory");
    }
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may start while the
// kernel before it in the stream is still running; griddep_wait() returns once that kernel has completed and its
// memory is visible, so everything before the call (barrier set-up, TMEM allocation, descriptor prefetch) overlaps the
// predecessor's tail and nothing after it can race with it.  griddep_launch_dependents() lets the next kernel in the
// stream do the same with this one.  Both are no-ops for a kernel launched without the attribute.
DG_DEVICE void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
DG_DEVICE void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Plain (not block-scaled) 16-bit UMMA: K = 16 elements = 32 bytes per instruction.
template <int CTAS>
DG_DEVICE void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (CTAS == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// Scale-factor copy shared memory -> TMEM: 32 rows x 16 bytes replicated to the four
// 32-lane quadrants.
template <int CTAS>
DG_DEVICE void utccp_32x128b_warpx4(uint32_t tmem_col, uint64_t smem_desc) {
    if constexpr (CTAS == 1) asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(smem_desc) : "memory");
    else asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(smem_desc) : "memory");
}

// Make `bar` complete once every tcgen05 operation this thread issued so far is done.
DG_DEVICE void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// CTA-pair form: signals the same-offset barrier in every CTA of `cta_mask`
// (an mbarrier arrive, not a data load).
DG_DEVICE void umma_commit_2cta(uint64_t* bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"(cta_mask)
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread.
DG_DEVICE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
DG_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Wait for outstanding TMEM loads and tie the 32 loaded registers to the wait, so no use of
// them can be scheduled ahead of it.
DG_DEVICE void tmem_ld_wait_x32(uint32_t* r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                   "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                   "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// ------------------------------------------------------------------ numerics
DG_DEVICE uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
DG_DEVICE uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return static_cast<uint32_t>(r);
}
DG_DEVICE uint32_t cvt_e4m3x4(float v0, float v1, float v2, float v3) {
    return cvt_e4m3x2(v0, v1) | (cvt_e4m3x2(v2, v3) << 16);
}
// Eight floats -> eight e2m1 codes in one word (element 0 in the low nibble of byte 0).
DG_DEVICE uint32_t cvt_e2m1x8(const float* v) {
    uint32_t r;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}\n"
        : "=r"(r)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return r;
}
// v * inv rounded to f32, with a product of -0.0 (exact or underflowed) turned into +0.0: the CPU
// encoder takes the sign from (v < 0) after the multiply, the hardware conversion keeps the sign bit.
// Separate rounded multiply and add on purpose: a fused multiply-add would keep the sign of an
// underflowing product.
DG_DEVICE float scale_pos_zero(float v, float inv) { return __fadd_rn(__fmul_rn(v, inv), 0.0f); }
// Store to the shared memory of a CTA of this cluster (address from mapa_u32).
DG_DEVICE void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
DG_DEVICE void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace dg
