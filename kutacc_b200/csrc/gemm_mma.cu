// Projection GEMMs on the warp-level tensor-core path (mma.sync m16n8k16, bf16 in, fp32 accumulate).
//
//   C[m, n] = sum_k A[m, k] * W[n, k]      A [M, K] row-major, W [N, K] row-major (W[out][in])
//
// One CTA computes a 128 x BN tile; K is walked in 64-wide slabs through a 3-stage cp.async ring in
// shared memory (16-byte chunks XOR-swizzled so that ldmatrix is bank-conflict free). Eight warps
// are laid out 4 (rows) x 2 (columns). The epilogue is a functor, which is where the four fused
// projections scatter into the attention kernel's [B, H, S, D] layout, add the gate bias and fold
// the 1/sqrt(D) scale into q.
//
// These GEMMs replace addmm -> kutacc_core_bgemm_ex on the reference's path
// (src/attention/gating_attention.cpp:47-66,152-157; src/linear/mm.cpp:46-86).
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

namespace kutacc {
namespace dev {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int NSTAGE = 3;
constexpr int GEMM_THREADS = 256;

struct WeightSegs {
    const __nv_bfloat16 *w[4];
    int seg_n;  // output channels per segment; N = nseg * seg_n
};

template <int BN>
constexpr int gemm_smem_bytes()
{
    return NSTAGE * (BM + BN) * BK * 2;
}

template <int BN, class Epi>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_bf16_tn_kernel(const __nv_bfloat16 *__restrict__ A, int64_t lda,
                                                                    WeightSegs ws, int64_t M, int K, Epi epi)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16 *sA = reinterpret_cast<__nv_bfloat16 *>(smem_raw);
    __nv_bfloat16 *sW = sA + NSTAGE * BM * BK;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int warp_m = warp & 3, warp_n = warp >> 2;
    constexpr int WN = BN / 2;
    constexpr int NT = WN / 8;

    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;
    const int seg = n0 / ws.seg_n;
    const __nv_bfloat16 *wsel = seg == 0 ? ws.w[0] : (seg == 1 ? ws.w[1] : (seg == 2 ? ws.w[2] : ws.w[3]));
    const __nv_bfloat16 *__restrict__ W = wsel + (int64_t)(n0 - seg * ws.seg_n) * K;

    const int nk = K / BK;

    auto load_stage = [&](int stage, int kc) {
        __nv_bfloat16 *a_dst = sA + stage * BM * BK;
        __nv_bfloat16 *w_dst = sW + stage * BN * BK;
#pragma unroll
        for (int i = 0; i < (BM * 8) / GEMM_THREADS; ++i) {
            const int idx = tid + i * GEMM_THREADS;
            const int r = idx >> 3, c = idx & 7;
            const int64_t gm = m0 + r;
            const bool ok = gm < M;
            const __nv_bfloat16 *src = A + (ok ? gm : 0) * lda + kc * BK + c * 8;
            cp_async16(smem_u32(a_dst + r * BK + swz8(r, c) * 8), src, ok ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < (BN * 8) / GEMM_THREADS; ++i) {
            const int idx = tid + i * GEMM_THREADS;
            const int r = idx >> 3, c = idx & 7;
            const __nv_bfloat16 *src = W + (int64_t)r * K + kc * BK + c * 8;
            cp_async16(smem_u32(w_dst + r * BK + swz8(r, c) * 8), src, 16);
        }
    };

    float acc[2][NT][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < NSTAGE - 1; ++s) {
        if (s < nk) load_stage(s, s);
        cp_async_commit();
    }

    for (int kc = 0; kc < nk; ++kc) {
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        {
            const int nxt = kc + NSTAGE - 1;
            if (nxt < nk) load_stage(nxt % NSTAGE, nxt);
            cp_async_commit();
        }
        const __nv_bfloat16 *a_s = sA + (kc % NSTAGE) * BM * BK;
        const __nv_bfloat16 *w_s = sW + (kc % NSTAGE) * BN * BK;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            uint32_t af[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                const int r = warp_m * 32 + mt * 16 + (lane & 15);
                const int c = ks * 2 + (lane >> 4);
                ldmatrix_x4(af[mt][0], af[mt][1], af[mt][2], af[mt][3], smem_u32(a_s + r * BK + swz8(r, c) * 8));
            }
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                const int r = warp_n * WN + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int c = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(b0, b1, b2, b3, smem_u32(w_s + r * BK + swz8(r, c) * 8));
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    mma_bf16_16816(acc[mt][np * 2], af[mt], b0, b1);
                    mma_bf16_16816(acc[mt][np * 2 + 1], af[mt], b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int64_t m = m0 + warp_m * 32 + mt * 16 + half * 8 + g;
            if (m >= M) continue;
            const auto row = epi.row(m);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int n = n0 + warp_n * WN + nt * 8 + 2 * t;
                epi.store(row, n, acc[mt][nt][half * 2], acc[mt][nt][half * 2 + 1]);
            }
        }
    }
}

// ---- epilogues -----------------------------------------------------------------------------------
struct EpiQKVG {
    static const char *name() { return "proj_qkvg"; }
    __nv_bfloat16 *q, *k, *v, *g;
    const float *bg;
    int S, H, D, C;
    float q_scale;
    struct Row {
        int64_t m;
        int64_t bh0;  // b * H
        int s;
    };
    __device__ __forceinline__ Row row(int64_t m) const
    {
        const int64_t b = m / S;
        return Row{m, b * H, (int)(m - b * S)};
    }
    __device__ __forceinline__ void store(const Row &r, int n, float v0, float v1) const
    {
        const int seg = n / C;
        const int c = n - seg * C;
        if (seg == 3) {
            *reinterpret_cast<uint32_t *>(g + r.m * C + c) = pack_bf16x2(v0 + __ldg(bg + c), v1 + __ldg(bg + c + 1));
            return;
        }
        const int h = c / D, d = c - h * D;
        __nv_bfloat16 *dst = seg == 0 ? q : (seg == 1 ? k : v);
        if (seg == 0) {
            v0 *= q_scale;
            v1 *= q_scale;
        }
        *reinterpret_cast<uint32_t *>(dst + ((r.bh0 + h) * S + r.s) * D + d) = pack_bf16x2(v0, v1);
    }
};

struct EpiBias {
    static const char *name() { return "linear_bias"; }
    __nv_bfloat16 *out;
    int64_t ldo;
    const float *bias;
    struct Row {
        __nv_bfloat16 *p;
    };
    __device__ __forceinline__ Row row(int64_t m) const { return Row{out + m * ldo}; }
    __device__ __forceinline__ void store(const Row &r, int n, float v0, float v1) const
    {
        if (bias) {
            v0 += __ldg(bias + n);
            v1 += __ldg(bias + n + 1);
        }
        *reinterpret_cast<uint32_t *>(r.p + n) = pack_bf16x2(v0, v1);
    }
};

template <int BN, class Epi>
bool launch_gemm(cudaStream_t stream, const void *A, int64_t lda, const WeightSegs &ws, int64_t M, int N, int K,
                 const Epi &epi)
{
    static bool configured = false;
    constexpr int smem = gemm_smem_bytes<BN>();
    if (!configured) {
        KUTACC_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel<BN, Epi>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)(N / BN));
    KernelTimer timer__(Epi::name(), stream);
    gemm_bf16_tn_kernel<BN, Epi><<<grid, GEMM_THREADS, smem, stream>>>((const __nv_bfloat16 *)A, lda, ws, M, K, epi);
    count_launch();
    return true;
}

}  // namespace

bool launch_proj_qkvg_bf16(cudaStream_t stream, const void *x, const void *wq, const void *wk, const void *wv,
                           const void *wg, const float *bg, void *q, void *k, void *v, void *gate, int B, int S,
                           int H, int D, float q_scale)
{
    const int C = H * D;
    if (C % 64 != 0 || (D & 1)) return false;
    WeightSegs ws;
    ws.w[0] = (const __nv_bfloat16 *)wq;
    ws.w[1] = (const __nv_bfloat16 *)wk;
    ws.w[2] = (const __nv_bfloat16 *)wv;
    ws.w[3] = (const __nv_bfloat16 *)wg;
    ws.seg_n = C;
    EpiQKVG epi{(__nv_bfloat16 *)q, (__nv_bfloat16 *)k, (__nv_bfloat16 *)v, (__nv_bfloat16 *)gate, bg, S, H, D, C, q_scale};
    const int64_t M = (int64_t)B * S;
    if (C % 128 == 0) return launch_gemm<128>(stream, x, C, ws, M, 4 * C, C, epi);
    return launch_gemm<64>(stream, x, C, ws, M, 4 * C, C, epi);
}

bool launch_linear_bias_bf16(cudaStream_t stream, const void *a, int64_t lda, const void *w, const float *bias,
                             void *out, int64_t ldo, int64_t M, int N, int K)
{
    if (K % 64 != 0 || N % 64 != 0 || (lda % 8) != 0 || (ldo & 1)) return false;
    WeightSegs ws;
    ws.w[0] = ws.w[1] = ws.w[2] = ws.w[3] = (const __nv_bfloat16 *)w;
    ws.seg_n = N;
    EpiBias epi{(__nv_bfloat16 *)out, ldo, bias};
    if (N % 128 == 0) return launch_gemm<128>(stream, a, lda, ws, M, N, K, epi);
    return launch_gemm<64>(stream, a, lda, ws, M, N, K, epi);
}

}  // namespace dev
}  // namespace kutacc
