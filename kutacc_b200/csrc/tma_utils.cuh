// mbarrier and TMA (cp.async.bulk.tensor) helpers for sm_100a, plus the host-side tensor-map encoder.
// Every wait is bounded: after about two seconds without progress a wait gives up, records a code in
// the host-visible error word and returns false so that the kernel can unwind instead of hanging.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kutacc {
namespace dev {

// ---- host: tensor maps ---------------------------------------------------------------------------
// rank-3 bf16 tensor [d2][d1][d0] (d0 innermost, contiguous), strides in ELEMENTS for d1 and d2,
// box [box2][box1][box0]. swizzle_bytes in {0, 32, 64, 128} must equal box0 * 2 when non-zero.
bool make_tensor_map_bf16_3d(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                             uint64_t stride1, uint64_t stride2, uint32_t box0, uint32_t box1, int swizzle_bytes,
                             uint32_t box2 = 1);

// rank-2 tensor [d1][d0] of 2-byte (bf16) or 4-byte (fp32, raw bits) elements, row stride in ELEMENTS, box [box1][box0]
bool make_tensor_map_2d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t stride1,
                        uint32_t box0, uint32_t box1, int swizzle_bytes);

// Host-visible error word written by kernels whose bounded waits ran out (0 = none). The pointer is a
// device-accessible alias of pinned host memory; the host reads *host after synchronising.
struct KernelErrorWord {
    int *host = nullptr;
    int *device = nullptr;
};
KernelErrorWord &kernel_error_word();

#ifdef __CUDACC__
// ---- device: mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same test with a suspend-time hint: the thread may sleep in hardware for up to `ns` nanoseconds (or until the
// phase completes) instead of returning at once, so a waiting warp re-issues the instruction rarely and leaves the
// issue slots and the memory-instruction queue to the warps that have work.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait. `code` identifies the wait site in the error word; `limit` is in SM clocks.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, int *err, int code, long long limit)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait_suspend(bar, parity, 0x989680u)) {
        if (clock64() - t0 > limit) {
            if (err) atomicCAS(err, 0, code);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *err, int code)
{
    return mbar_wait_limit(bar, parity, err, code, 4000000000LL);  // ~2 s at 1.9 GHz
}

// The same wait for a whole warp. Lanes can leave the polling loop at different iterations; the vote at
// the end brings the warp back together (instructions such as tcgen05.ld, ldmatrix and mma.sync are
// .aligned and must be issued by a converged warp) and makes the result uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int *err, int code)
{
    const bool ok = mbar_wait(bar, parity, err, code);
    return __all_sync(0xffffffffu, ok);
}

// ---- device: thread-block clusters and distributed shared memory --------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_shared_rank(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_shared_cluster_f32(uint32_t addr, float v)
{
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
// fire-and-forget store of one word into another CTA's shared memory; the destination CTA's mbarrier
// receives 4 transaction bytes when the word has landed (it must expect them: mbar_arrive_expect_tx)
__device__ __forceinline__ void st_async_cluster_f32(uint32_t remote_addr, float v, uint32_t remote_bar)
{
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];\n" ::"r"(remote_addr),
                 "r"(__float_as_uint(v)), "r"(remote_bar)
                 : "memory");
}
__device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;\n" ::: "memory"); }
// arrive on an mbarrier that lives in another CTA of the cluster; releases this thread's earlier writes
__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier that CTAs of the whole cluster arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int *err, int code)
{
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait_cluster(bar, parity)) {
        if (clock64() - t0 > 4000000000LL) {
            if (err) atomicCAS(err, 0, code);
            return false;
        }
    }
    return true;
}
// Hardware barrier over every thread of the cluster. Only used where all threads are known to arrive.
__device__ __forceinline__ void cluster_barrier_all()
{
    asm volatile("barrier.cluster.arrive.release;\nbarrier.cluster.wait.acquire;\n" ::: "memory");
}

// ---- device: TMA -----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// global -> shared tile load of a rank-3 tensor; completion is signalled on `bar` in bytes
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// shared -> global tile store (bulk async group)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];\n" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait()
{
    asm volatile("cp.async.bulk.wait_group %0;\n" ::"n"(N) : "memory");
}
#endif  // __CUDACC__

}  // namespace dev
}  // namespace kutacc
