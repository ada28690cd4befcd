// ptx.cuh — thin inline-PTX wrappers for the sm_100a features the kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc, MMA, commit, ld)
// and the descriptor encodings tcgen05.mma takes.  Device-only, header-only.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

// ----------------------------------------------------------------- addresses
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Non-blocking test (try_wait may suspend the thread for a while; a thread that polls several barriers in turn
// must not).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Wait with a wall-clock limit.  Every spin in these kernels goes through
// here: when the limit passes the caller records an error word and unwinds
// instead of spinning for ever on a barrier nobody will complete.
#ifndef AXB_WAIT_LIMIT_NS
#define AXB_WAIT_LIMIT_NS 2000000000ull  // 2 s
#endif
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > AXB_WAIT_LIMIT_NS) return false;
    }
}

// Whole-warp wait for warps that wait long (epilogue warps wait a whole K loop): only lane 0
// polls, with a sleep between polls, so the waiters do not compete with the MMA-issuing
// thread for the barrier unit; the outcome is broadcast to the warp.
__device__ __forceinline__ bool mbar_wait_warp_bounded(uint32_t bar, uint32_t parity)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        if (!mbar_try_wait(bar, parity)) {
            const uint64_t t0 = global_timer_ns();
            for (;;) {
                __nanosleep(200);
                if (mbar_try_wait(bar, parity)) break;
                if (global_timer_ns() - t0 > AXB_WAIT_LIMIT_NS) { ok = 0; break; }
            }
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

// ----------------------------------------------------------------------- TMA
// 2-D tiled load global -> this CTA's shared memory, completion counted in
// bytes on an mbarrier of the same CTA.  crd0 is the innermost (contiguous)
// coordinate: crd0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, uint32_t bar,
                                            int32_t crd0, int32_t crd1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"(tmap), "r"(bar), "r"(crd0), "r"(crd1)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ------------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// mbarrier arrive once every tcgen05.mma issued so far by this thread has
// finished reading shared memory and writing TMEM.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

enum MmaKind { KIND_TF32 = 0, KIND_BF16 = 1, KIND_I8 = 2 };

// D[tmem] (+)= A[smem] . B[smem]^T, one thread issues for the whole CTA.
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate)
{
    if constexpr (KIND == KIND_TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
    } else if constexpr (KIND == KIND_BF16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
    }
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives
// row (lane base + t), registers r[0..31] = columns col..col+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// The same for 4 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x32_x4(uint32_t taddr, uint32_t (&r)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}

// The same for 8 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x32_x8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// --------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of
// `swizzle_bytes` (128 or 64) bytes with the matching TMA swizzle; groups of 8
// rows are contiguous (stride-byte-offset = 8 * swizzle_bytes).
//   [0,14) start address >> 4      [16,30) leading byte offset >> 4 (unused: 1)
//   [32,46) stride byte offset >> 4   [46,48) descriptor version = 1
//   [61,64) layout: 2 = 128-byte swizzle, 4 = 64-byte swizzle
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t addr, int swizzle_bytes)
{
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8u * (uint32_t)swizzle_bytes) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(swizzle_bytes == 128 ? 2 : 4) << 61;
    return d;
}

// Instruction descriptor for kind::tf32 / kind::f16 / kind::i8, both operands
// K-major, dense, no negate:
//   [4,6) D format (1 = f32, 2 = s32)   [7,10) A format   [10,13) B format
//   [17,23) N >> 3   [24,29) M >> 4
template <int KIND>
__host__ __device__ constexpr uint32_t make_idesc(int m, int n)
{
    const uint32_t cfmt = KIND == KIND_I8 ? 2u : 1u;
    const uint32_t abfmt = KIND == KIND_TF32 ? 2u : 1u;  // tf32 = 2, bf16 = 1, s8 = 1
    return (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// 3-D tiled load (innermost coordinate first); same alignment rule as the 2-D form.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *tmap, uint32_t bar, int32_t crd0,
                                            int32_t crd1, int32_t crd2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        :
        : "r"(dst), "l"(tmap), "r"(bar), "r"(crd0), "r"(crd1), "r"(crd2)
        : "memory");
}

// 4-D tiled load (innermost coordinate first); same alignment rule as the 2-D form.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *tmap, uint32_t bar, int32_t crd0,
                                            int32_t crd1, int32_t crd2, int32_t crd3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :
        : "r"(dst), "l"(tmap), "r"(bar), "r"(crd0), "r"(crd1), "r"(crd2), "r"(crd3)
        : "memory");
}

// 2-D tiled store shared memory -> global (bulk async-group completion).  The part of the box outside the tensor
// is clipped by the hardware; crd0 * element size must be a multiple of 16 bytes and no coordinate negative.
__device__ __forceinline__ void tma_store_2d(const void *tmap, uint32_t src, int32_t crd0, int32_t crd1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src),
                 "r"(crd0), "r"(crd1)
                 : "memory");
}

// The same box ADDED to what global memory holds (one rounded fp32 addition per element, done by the memory system:
// nothing is read back into the SM).  Same coordinate rules as the store.
__device__ __forceinline__ void tma_reduce_add_2d(const void *tmap, uint32_t src, int32_t crd0, int32_t crd1)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
                 "r"(src), "r"(crd0), "r"(crd1)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// all committed bulk stores of this thread have finished READING shared memory (the source may be reused)
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ... have completed altogether (required before the CTA exits)
__device__ __forceinline__ void tma_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// generic-proxy writes to shared memory become visible to the async proxy (TMA, tcgen05)
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Ask for a tile to be brought into L2 (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_3d(const void *tmap, int32_t crd0, int32_t crd1, int32_t crd2)
{
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];" ::"l"(tmap), "r"(crd0), "r"(crd1),
                 "r"(crd2)
                 : "memory");
}

// D[tmem] (+)= A[tmem] . B[smem]: the A operand is read from tensor memory (128 lanes = rows,
// consecutive 32-bit columns = K), B through a shared-memory descriptor.  kind::tf32.
__device__ __forceinline__ void tc_mma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate));
}

// registers -> tensor memory, the mirror image of tmem_ld_32x32
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory descriptor for an MN-major tf32 operand tile: rows of 128 bytes run along M/N (32 elements),
// consecutive K indices are consecutive rows, and the 128-byte swizzle moves 32-byte chunks by (row % 4) — the
// only layout an MN-major 32-bit operand may have (TMA: the 128B swizzle with 32-byte atoms).  A swizzle atom is
// 4 rows.  lbo_bytes: distance between 128-byte column groups along M/N; sbo_bytes: distance between 4-row K
// groups.  Layout type 1 in bits [61,64).
__device__ __forceinline__ uint64_t smem_desc_mnmajor_sw128_32b(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float tf32_rna(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

}  // namespace axb

// ---------------------------------------------------------------------------
// CTA-pair (cta_group::2) forms: two CTAs of a cluster share one MMA of M = 256.
// The leader (cluster rank 0) issues the MMA; each CTA stages its own half of
// both operands and owns the 128 accumulator rows in its own TMEM.
namespace axb {

// Programmatic dependent launch: a kernel launched with the programmatic-serialisation attribute may start while
// the kernel before it on the stream still runs; grid_dep_wait() blocks until that kernel has finished and its
// writes are visible, grid_dep_launch() (called by the earlier kernel) lets the dependent start early.
__device__ __forceinline__ void grid_dep_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_dep_launch()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cluster address of `local_addr` (a shared::cta address of this CTA) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Arrive on the barrier at the same offset in every CTA named by cta_mask once all MMAs
// issued so far by this thread have completed (a commit, not a load: no data moves).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate)
{
    if constexpr (KIND == KIND_TF32) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
    } else if constexpr (KIND == KIND_BF16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            :
            : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate));
    }
}

// TMA tile load issued by either CTA of a pair into ITS OWN shared memory; the byte
// count is credited to `bar`, a shared::cluster address that may name the leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void *tmap, uint32_t bar, int32_t crd0,
                                                 int32_t crd1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"(tmap), "r"(bar), "r"(crd0), "r"(crd1)
        : "memory");
}

// the 4-D form (the image windows of an implicit convolution), same completion rule
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const void *tmap, uint32_t bar, int32_t crd0, int32_t crd1,
                                                 int32_t crd2, int32_t crd3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :
        : "r"(dst), "l"(tmap), "r"(bar), "r"(crd0), "r"(crd1), "r"(crd2), "r"(crd3)
        : "memory");
}

}  // namespace axb
