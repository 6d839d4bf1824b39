// Thin inline-PTX wrappers for the sm_100a features the decode kernel uses:
// mbarrier, cp.async, proxy fences, tensor memory (TMEM) management and
// tcgen05.mma / tcgen05.ld.  Nothing here is generic; each wrapper is the exact
// instruction form the kernel needs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sharedkv {
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// One arrival that also announces `bytes` of asynchronous (TMA) traffic to the current phase.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while its
// predecessor in the stream is still running.  wait: blocks until the predecessor has completed and
// its memory operations are visible (returns at once for a normal launch).  launch_dependents: lets
// the successor's CTAs be scheduled as soon as every CTA of this grid has said so or exited.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- release / acquire on global memory
// Fetch-and-add that publishes every write ordered before it (this thread's, and those of other
// threads it has synchronised with) to the GPU, and orders later reads behind the value it returns.
__device__ __forceinline__ uint32_t atomic_add_acq_rel(uint32_t *address, uint32_t value)
{
    uint32_t old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(address), "r"(value) : "memory");
    return old;
}

// ---------------------------------------------------------------- cp.async (16-byte, L2 only)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- TMA row gather
// Four rows (any row indices) x one 128-byte column block of a 2-D tensor into four consecutive
// 128-byte rows of shared memory; completion is counted in bytes on `bar`.  Rows outside the
// tensor are filled with zeros.  The tensor map's box is {128 bytes, 1 row}, 128-byte swizzle.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void *tensor_map, int32_t x, int32_t r0, int32_t r1,
                                            int32_t r2, int32_t r3, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(tensor_map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar)
        : "memory");
}
// One box {128 bytes, 32 rows, 1 page} of a 3-D [512 B, 32 rows, pages] view: a whole page's
// 128-channel segment (4 KB) per instruction.
__device__ __forceinline__ void tma_page_segment(uint32_t dst, const void *tensor_map, int32_t x, int32_t page, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(tensor_map), "r"(x), "r"(0), "r"(page), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const void *tensor_map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// Make generic-proxy shared-memory writes visible to the async proxy (tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns)
                 : "memory");
}
// Register file re-partitioning between warpgroups (four consecutive warps, all of which must
// execute the instruction): a kernel launched with N registers per thread lets roles that need few
// give registers up (dec) so that roles that need many can take them (inc, which waits until
// they are free).  Counts are multiples of 8 in [24, 256].
template <uint32_t COUNT>
__device__ __forceinline__ void registers_release()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(COUNT));
}
template <uint32_t COUNT>
__device__ __forceinline__ void registers_acquire()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(COUNT));
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp receives lane (base + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}

// One lane of a fully converged warp.  The compiler keeps code predicated on this (unlike on a
// lane-id comparison) on the warp-uniform datapath.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// D[tmem] (+)= A[smem desc] * B[smem desc], INT8 x INT8 -> INT32, one CTA.
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor (64 bit): start address, leading / stride byte offsets
// (all >> 4), descriptor version 1, swizzle mode in bits 61-63.
constexpr uint64_t kSwizzleNone = 0, kSwizzle128 = 2;
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t swizzle)
{
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (swizzle << 61);
}
// Instruction descriptor for kind::i8: signed A and B, INT32 accumulator, M x N tile,
// operand majors (0 = K-major, 1 = MN-major).
__host__ __device__ constexpr uint32_t idesc_i8(uint32_t m, uint32_t n, uint32_t a_mn_major, uint32_t b_mn_major)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
           ((m >> 4) << 24);
}

}  // namespace ptx
}  // namespace sharedkv
