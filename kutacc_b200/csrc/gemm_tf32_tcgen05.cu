// fp32 projections on the fifth-generation tensor cores with fp32-level accuracy.
//
//   C[m, n] = sum_k A[m, k] * W[n, k] (+ bias[n])         A [M, K] fp32, W [N, K] fp32 (W[out][in]), C fp32
//
// tcgen05.mma has no fp32 input type; its tf32 kind keeps 11 significant bits of each operand. Every operand is
// therefore split beforehand (split_tf32_kernel) into a tf32 head and a tail, x = hi + lo with |lo| <= 2^-11 |x|,
// stored side by side as one row [hi(0..K) | lo(0..K)] of 2K floats, and the product is taken as
//   lo(A).hi(W) + hi(A).lo(W) + hi(A).hi(W)        (small terms first; lo.lo, about 2^-22 of the result, is dropped)
// accumulated in fp32 in tensor memory. With the operands laid out like that the three products are ONE K-loop of
// 3 * K / 32 slab pairs whose TMA column coordinates pick the head or the tail, so the kernel has the plain GEMM's
// structure: persistent CTAs (two per SM) walk 128 x 128 output tiles;
//   warp 0      producer: TMA loads of 128 x 32 fp32 slabs of A' and W' (128-byte swizzle) into a 3-stage ring
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma kind::tf32 (M = 128, N = 128, K = 8) four times per
//               slab pair into one of two 128-column TMEM accumulators and commits to mbarriers
//   warps 2-9   epilogue: each warp owns 32 TMEM lanes x 64 columns: tcgen05.ld, bias add, 16-byte global stores
//               (a thread writes 256 contiguous bytes of its own output row)
// Up to four weight matrices share one pass over A (the fused Q/K/V/gate projection of the fp32 attention).
//
// Replaces addmm -> kutacc_core_bgemm_ex of the reference for fp32 tensors
// (src/attention/gating_attention.cpp:47-66,152-157; src/linear/mm.cpp:46-86).
//
// All mbarrier waits are bounded; on a timeout the roles fall through to the common tail, the TMEM allocation is
// released and the host-visible error word carries the site.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"
#include "tcgen05_utils.cuh"
#include "tma_utils.cuh"

#include <algorithm>

namespace kutacc {
namespace dev {

namespace {

constexpr int BM = 128, BN = 128, BK = 32;              // BK floats = one 128-byte swizzle row
constexpr int NSTAGE = 3;
constexpr int ACC_STAGES = 2;
constexpr int SLAB_BYTES = BM * BK * 4;                 // 16 KB, A' and W' slabs alike
constexpr int STAGE_BYTES = 2 * SLAB_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int BAR_OFF = NSTAGE * STAGE_BYTES;
constexpr int NBARS = 2 * NSTAGE + 2 * ACC_STAGES;
constexpr int SMEM_BYTES = BAR_OFF + NBARS * 8 + 16 + 1024;
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = ACC_STAGES * BN;              // 256: half of the SM's tensor memory (two CTAs per SM)

struct alignas(64) Tf32Maps {
    CUtensorMap a;        // A' [M][2K] fp32, box [32, 128], 128-byte swizzle
    CUtensorMap w[4];     // W' [N][2K] fp32 per segment, box [32, 128], 128-byte swizzle
};

struct Tf32Params {
    const float *bias[4];   // per segment, may be null
    float *out[4];          // per segment, [M][ldo]
    int64_t ldo;
    int M, N, K, nseg;
    int *err;
};

// instruction descriptor of tcgen05.mma kind::tf32: D fp32, A and B tf32, both K-major, N = 128, M = 128
constexpr uint32_t kInstrDescTf32 =
    (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(THREADS, 2) gemm_tf32x3_tc_kernel(const __grid_constant__ Tf32Maps maps, const Tf32Params p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem + BAR_OFF;
    auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(NSTAGE + s); };
    auto acc_full = [&](int a) { return bar_base + 8u * (uint32_t)(2 * NSTAGE + a); };
    auto acc_empty = [&](int a) { return bar_base + 8u * (uint32_t)(2 * NSTAGE + ACC_STAGES + a); };
    const uint32_t tmem_slot = bar_base + 8u * NBARS;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.M + BM - 1) / BM;
    const int n_tiles_seg = p.N / BN;
    const int n_tiles = n_tiles_seg * p.nseg;
    const int num_tiles = m_tiles * n_tiles;
    const int nk = p.K / BK;
    const int niter = 3 * nk;                           // slab pairs per tile: lo.hi, hi.lo, hi.hi

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), EPI_WARPS);
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(tmem_base) : "r"(tmem_slot));

    if (warp == 0) {
        // ================= producer =================
        if (lane == 0) {
            tma_prefetch_desc(&maps.a);
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / n_tiles) * BM, n_tile = tile % n_tiles;
                const int seg = n_tile / n_tiles_seg, n0 = (n_tile % n_tiles_seg) * BN;
                const CUtensorMap *wmap = &maps.w[seg];
                for (int j = 0; j < niter; ++j, ++it) {
                    const int s = it % NSTAGE;
                    if (it >= NSTAGE && !mbar_wait(empty_bar(s), (uint32_t)((it / NSTAGE - 1) & 1), p.err, 41)) {
                        ok = false;
                        break;
                    }
                    const int prod = j / nk, kc = (j % nk) * BK;
                    const int a_col = (prod == 0 ? p.K : 0) + kc;        // product 0 reads the tail of A
                    const int w_col = (prod == 1 ? p.K : 0) + kc;        // product 1 reads the tail of W
                    const uint32_t st = smem + (uint32_t)s * STAGE_BYTES;
                    mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
                    tma_load_2d(st, &maps.a, full_bar(s), a_col, m0);
                    tma_load_2d(st + SLAB_BYTES, wmap, full_bar(s), w_col, n0);
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        int it = 0, tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
            const int a = tcount % ACC_STAGES;
            if (tcount >= ACC_STAGES && !mbar_wait_warp(acc_empty(a), (uint32_t)((tcount / ACC_STAGES - 1) & 1), p.err, 42)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
            for (int j = 0; j < niter; ++j, ++it) {
                const int s = it % NSTAGE;
                if (!mbar_wait_warp(full_bar(s), (uint32_t)((it / NSTAGE) & 1), p.err, 43)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t st = smem + (uint32_t)s * STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 8; ++k) {               // 8 tf32 = 32 bytes per instruction
                        const uint64_t adesc = make_smem_desc_kmajor(st + k * 32, 128);
                        const uint64_t bdesc = make_smem_desc_kmajor(st + SLAB_BYTES + k * 32, 128);
                        tc_mma_tf32(d_tmem, adesc, bdesc, kInstrDescTf32, (j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));                 // slab pair may be overwritten once these MMAs retire
                    if (j == niter - 1) tc_commit(acc_full(a));
                }
                __syncwarp();
            }
        }
    } else {
        // ================= epilogue =================
        const int quad = warp & 3;                            // TMEM lanes 32*quad .. 32*quad+31
        const int half = (warp - 2) >> 2;                     // which 64 columns of the 128-column tile
        int tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
            const int m0 = (tile / n_tiles) * BM, n_tile = tile % n_tiles;
            const int seg = n_tile / n_tiles_seg, n0 = (n_tile % n_tiles_seg) * BN;
            const int a = tcount % ACC_STAGES;
            if (!mbar_wait_warp(acc_full(a), (uint32_t)((tcount / ACC_STAGES) & 1), p.err, 44)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const float *bias = p.bias[seg];
            const int m = m0 + quad * 32 + lane;
            float *orow = p.out[seg] + (int64_t)(m < p.M ? m : 0) * p.ldo + n0 + half * 64;
            const uint32_t tcol = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * BN + half * 64);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tcol + c * 32, r);
                tmem_ld_wait();
                if (c == 1) {
                    // both halves are in registers: the accumulator may be overwritten by the tile after next
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(a));
                }
                if (m < p.M) {
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        float4 v = make_float4(__uint_as_float(r[4 * j4]), __uint_as_float(r[4 * j4 + 1]),
                                               __uint_as_float(r[4 * j4 + 2]), __uint_as_float(r[4 * j4 + 3]));
                        if (bias) {
                            const float4 bv = __ldg(reinterpret_cast<const float4 *>(bias + n0 + half * 64 + c * 32) + j4);
                            v.x += bv.x;
                            v.y += bv.y;
                            v.z += bv.z;
                            v.w += bv.w;
                        }
                        reinterpret_cast<float4 *>(orow + c * 32)[j4] = v;
                    }
                }
            }
        }
    }

    // ================= common tail =================
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// up to eight matrices of the same shape per launch (blockIdx.y picks one): the five weights of an attention call
struct SplitArgs {
    const float *src[8];
    float *dst[8];
};

// dst[r, 0..K) = tf32 head of src[r, :], dst[r, K..2K) = src - head (fp32, at most 12 significant bits)
__global__ void __launch_bounds__(256) split_tf32_kernel(const SplitArgs args, int64_t src_ld, int64_t rows, int K)
{
    const float *__restrict__ src = args.src[blockIdx.y];
    float *__restrict__ dst = args.dst[blockIdx.y];
    const int kv = K / 4;
    const int64_t total = rows * kv;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / kv;
        const int c = (int)(i % kv) * 4;
        const float4 v = __ldg(reinterpret_cast<const float4 *>(src + r * src_ld + c));
        float4 hi, lo;
        const float x[4] = {v.x, v.y, v.z, v.w};
        float h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            uint32_t t;
            asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(t) : "f"(x[e]));
            h[e] = __uint_as_float(t);
            l[e] = x[e] - h[e];
        }
        hi = make_float4(h[0], h[1], h[2], h[3]);
        lo = make_float4(l[0], l[1], l[2], l[3]);
        float *d = dst + r * 2 * K;
        *reinterpret_cast<float4 *>(d + c) = hi;
        *reinterpret_cast<float4 *>(d + K + c) = lo;
    }
}

int sm_count_tf32()
{
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

}  // namespace

bool launch_split_tf32_many(cudaStream_t stream, int count, const void *const *src, int64_t src_ld, void *const *dst,
                            int64_t rows, int K)
{
    if (count < 1 || count > 8 || rows <= 0 || K <= 0 || K % 4 != 0 || src_ld % 4 != 0) return false;
    SplitArgs a;
    for (int i = 0; i < 8; ++i) {
        const int j = i < count ? i : 0;
        if ((((uintptr_t)src[j] | (uintptr_t)dst[j]) & 15u) != 0) return false;
        a.src[i] = (const float *)src[j];
        a.dst[i] = (float *)dst[j];
    }
    const int64_t total = rows * (K / 4);
    const unsigned gx = (unsigned)std::min<int64_t>((total + 255) / 256, (int64_t)sm_count_tf32() * 16);
    KernelTimer timer__("split_tf32", stream);
    split_tf32_kernel<<<dim3(gx, (unsigned)count), 256, 0, stream>>>(a, src_ld, rows, K);
    count_launch();
    return true;
}

bool launch_split_tf32(cudaStream_t stream, const void *src, int64_t src_ld, void *dst, int64_t rows, int K)
{
    return launch_split_tf32_many(stream, 1, &src, src_ld, &dst, rows, K);
}

bool tcgen05_gemm_tf32x3(cudaStream_t stream, const void *a_split, const void *const *w_split, const float *const *bias,
                         void *const *out, int64_t ldo, int64_t M, int N, int K, int nseg)
{
    if (nseg < 1 || nseg > 4 || M <= 0 || M > INT32_MAX / 2 || N % BN != 0 || K % BK != 0 || K <= 0 || ldo % 4 != 0 ||
        ldo < N || (((uintptr_t)a_split) & 15u))
        return false;
    for (int i = 0; i < nseg; ++i)
        if ((((uintptr_t)w_split[i] | (uintptr_t)out[i] | (uintptr_t)bias[i]) & 15u) != 0) return false;
    KernelErrorWord &ew = kernel_error_word();
    if (ew.device == nullptr) return false;
    Tf32Maps maps;
    if (!make_tensor_map_2d(&maps.a, a_split, /*elem_bytes=*/4, (uint64_t)2 * K, (uint64_t)M, (uint64_t)2 * K, BK, BM, 128))
        return false;
    for (int i = 0; i < 4; ++i) {
        const int j = i < nseg ? i : 0;
        if (!make_tensor_map_2d(&maps.w[i], w_split[j], 4, (uint64_t)2 * K, (uint64_t)N, (uint64_t)2 * K, BK, BN, 128))
            return false;
    }
    Tf32Params p;
    for (int i = 0; i < 4; ++i) {
        const int j = i < nseg ? i : 0;
        p.bias[i] = bias[j];
        p.out[i] = (float *)out[j];
    }
    p.ldo = ldo;
    p.M = (int)M;
    p.N = N;
    p.K = K;
    p.nseg = nseg;
    p.err = ew.device;
    static bool configured = false;
    if (!configured) {
        KUTACC_CUDA(cudaFuncSetAttribute(gemm_tf32x3_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured = true;
    }
    const int64_t tiles = ((M + BM - 1) / BM) * (int64_t)(N / BN) * nseg;
    const unsigned grid = (unsigned)std::min<int64_t>(tiles, 2 * std::max(1, sm_count_tf32() - runtime().sm_margin));
    KernelTimer timer__("gemm_tf32x3_tc", stream);
    gemm_tf32x3_tc_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(maps, p);
    count_launch();
    return true;
}

}  // namespace dev
}  // namespace kutacc
