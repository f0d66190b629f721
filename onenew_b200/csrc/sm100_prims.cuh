// sm100_prims.cuh -- thin inline-PTX wrappers for the Blackwell (sm_100a) features the
// contraction kernels use: mbarriers, TMA tensor loads (tiled and im2col mode), tensor memory
// (TMEM) allocation, tcgen05.mma / commit / ld, and the shared-memory matrix descriptor and
// instruction descriptor encodings.  Every wait is bounded: a wait that runs out records
// where it gave up and returns false so the kernel can unwind instead of hanging.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace one {

// Status word bits written by kernels (read back by one_cuda_status()).
enum : unsigned int {
    ST_TIMEOUT_PRODUCER = 1u << 0,   // TMA producer gave up waiting for a free stage
    ST_TIMEOUT_MMA = 1u << 1,        // MMA issuer gave up waiting for operand bytes
    ST_TIMEOUT_EPILOGUE = 1u << 2,   // epilogue gave up waiting for the accumulator
    ST_TIMEOUT_DRAIN = 1u << 3,      // teardown gave up waiting for copies in flight
    ST_RANGE_F16 = 1u << 4,          // a value written as fp16 was larger than the format's largest finite value
};

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  try_wait itself suspends the thread in hardware until the phase completes or a
// system time limit passes, so the loop body runs rarely; the clock and the abort flag are
// looked at only every 256 failed attempts to keep the waiting warps off the issue ports and the
// shared-memory pipe that the working warps need.  Gives up after ~2^31 clocks (about a second)
// or once another role of the CTA has raised *abort_flag.  Returns false when it gave up.
#ifndef ONE_WAIT_CLOCKS
#define ONE_WAIT_CLOCKS (1ll << 31)
#endif
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long limit_clocks = ONE_WAIT_CLOCKS)
{
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    const uint32_t check_mask = limit_clocks < (1ll << 28) ? 0u : 255u;   // a short limit (self test) looks at the clock every time
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & check_mask) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_clocks) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------- programmatic dependent launch
// wait: returns once the kernel this one was launched behind (programmatic stream serialisation) has
// completed and its memory operations are visible; returns at once for an ordinary launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel on the stream be scheduled as SMs free up.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- TMA loads
// Plain (single-CTA) tensor loads only: each CTA fetches its own tiles from this GPU's memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *tmap, uint32_t bar, int x, int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// im2col-mode load of a 4-D (C, W, H, N) tensor: the coordinates name the first base pixel
// (which may lie in the padding, i.e. be negative), offs are the filter tap (kw, kh).
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const void *tmap, uint32_t bar, int c,
                                                   int w, int h, int n, uint16_t off_w, uint16_t off_h)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w),
        "h"(off_h)
        : "memory");
}
// TMA stores (shared -> global); completion is tracked per thread with bulk groups.
__device__ __forceinline__ void tma_store_2d(const void *tmap, uint32_t src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void *tmap, uint32_t src, int x, int y, int z)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until the bulk stores this thread committed have finished READING shared memory.
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... all but the most recent one of them.
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// Make generic-proxy writes to shared memory visible to the async proxy (TMA).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---------------------------------------------------------------- CTA pairs (clusters of two)
// A pair of CTAs on the two SMs of one TPC shares a 256-row tile: tcgen05.mma.cta_group::2, issued by
// the even CTA alone, multiplies each CTA's own 128 rows of A by the two halves of B held by the two CTAs
// and accumulates into each CTA's own tensor memory.  Every CTA loads only half of B, which is what
// lifts the L2 -> SM operand rate that bounds a single-CTA tile.
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of both CTAs.  The wait has no bound of its own: it is only placed where every thread of
// the peer gets to by bounded waits.
__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address, in the cluster's shared window, of the same shared-memory location in CTA `rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Loads of a pair: plain per-CTA tensor loads (each CTA fetches its own bytes from this GPU's memory) whose bytes
// are counted on the EVEN CTA's barrier: in the cluster window the two CTAs' addresses differ in bit 24,
// so clearing it names the even CTA's copy of the barrier.
constexpr uint32_t PAIR_LEADER_MASK = 0xFEFFFFFFu;
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void *tmap, uint32_t bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar & PAIR_LEADER_MASK), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d_pair(uint32_t dst, const void *tmap, uint32_t bar, int c, int w, int h, int n,
                                                        uint16_t off_w, uint16_t off_h)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar & PAIR_LEADER_MASK), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on a barrier (cluster-window address: this CTA's or the peer's) once every MMA of the pair issued
// so far has completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

// ---------------------------------------------------------------- TMEM + tcgen05
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
// Arrive on an mbarrier once every tcgen05.mma this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// KIND_F16 is a host-side name: the kernels have one 16-bit instantiation (KIND_BF16, kind::f16) whose operand
// format -- bf16 or fp16 -- is a field of the instruction descriptor, set at run time.
enum MmaKind { KIND_TF32 = 0, KIND_BF16 = 1, KIND_I8 = 2, KIND_F16 = 3 };

// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate == 0 overwrites D.
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate)
{
    if constexpr (KIND == KIND_TF32) {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else if constexpr (KIND == KIND_BF16) {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// The pair form: D of both CTAs (+)= [A of CTA 0; A of CTA 1] * [B half of CTA 0; B half of CTA 1]^T.
template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (KIND == KIND_TF32) {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else if constexpr (KIND == KIND_BF16) {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
            " tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Instruction descriptor (32 bit): c_format [4,6) (1 = F32, 2 = S32); a_format [7,10) and
// b_format [10,13) (kind::f16: 0 = F16, 1 = BF16; kind::tf32: 2 = TF32; kind::i8: 1 = signed 8 bit);
// a_major bit 15 and b_major bit 16 (0 = K-major); N>>3 in [17,23); M>>4 in [24,29).
template <int KIND>
__host__ __device__ constexpr uint32_t make_idesc(int m, int n)
{
    uint32_t cfmt = (KIND == KIND_I8) ? 2u : 1u;
    uint32_t abfmt = (KIND == KIND_TF32) ? 2u : 1u;
    return (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are `row_bytes`
// (32, 64 or 128) wide and stored with the matching TMA swizzle: start address >> 4 in
// [0,14); leading byte offset (unused for swizzled K-major, encoded 1) in [16,30); stride byte
// offset = 8 rows * row_bytes, >> 4, in [32,46); descriptor version 1 at bit 46; swizzle mode
// in [61,64): 2 = 128 B, 4 = 64 B, 6 = 32 B.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t row_bytes)
{
    const uint64_t layout = (row_bytes == 128) ? 2ull : (row_bytes == 64) ? 4ull : 6ull;
    uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8u * row_bytes) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= layout << 61;
    return d;
}

// 32 lanes x 32 columns of 32-bit TMEM cells: thread i of the warp gets lane (base+i), r[j] =
// column (base+j).  A warp may only touch the lane quarter 32*(warp_id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace one
