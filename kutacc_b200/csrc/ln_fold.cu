// LayerNorm folded into the projections that follow it.
//
// The reference's callers normalise the activations (src/normalization/layernorm_kernel.h:22-53) and hand the
// normalised bf16 tensor to the attention operator, which costs a read and a write of the whole tensor before the
// projections read it again. Here the normalisation is carried by the projection itself. With the row statistics
// mean and rstd, a weight row w (one output channel) and g = gamma * w taken element by element,
//
//   sum_k ((x_k - mean) * rstd * gamma_k + beta_k) * w_k  =  rstd * sum_k x_k * (g_k - gbar)  +  sum_k beta_k * w_k
//
// because sum_k (x_k - mean) = 0 makes the constant gbar = mean_k(g_k) drop out. Centring the folded weight row keeps
// the product free of the cancellation a large mean would cause. The centred row is rounded to bf16 for the tensor
// cores, which breaks its zero sum by a rounding residue s = sum_k bf16(g_k - gbar); the epilogue removes exactly that
// term:  y = rstd * (acc - mean * s) + t,  acc = sum_k x_k * bf16(g_k - gbar),  t = sum_k beta_k * w_k (+ the layer's
// own bias). What is left of the rounding is rstd * sum_k (x_k - mean) * delta_k, a relative 2^-9 whatever the mean.
//
//   ln_stats_kernel : mean and rstd of every row (one read of x; the reference's shifted-data sums)
//   ln_fold_kernel  : folded weights, s and t for up to four weight matrices (a few hundred KB, once per call)
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

#include <algorithm>

namespace kutacc {
namespace dev {

namespace {

// Sums of one 16-byte vector (8 bf16) of shifted data
__device__ __forceinline__ void stats_acc(const uint4 &raw, float delta, float &sum, float &sum2)
{
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float a = bf16lo_to_f32(w[e]) - delta, b = bf16hi_to_f32(w[e]) - delta;
        sum += a;
        sum2 = fmaf(a, a, sum2);
        sum += b;
        sum2 = fmaf(b, b, sum2);
    }
}

// Rows of 16-byte vectors: a group of G lanes (the smallest power of two that covers a row, 4 to 32) per row, so a
// warp works on 32 / G rows at once, and every group keeps NR rows in flight. The shift (the reference sums the
// data minus the row's first element) comes out of the first vector by a shuffle instead of a load of its own.
constexpr int NR = 4;
template <int G>
__global__ void __launch_bounds__(256) ln_stats_vec_kernel(const __nv_bfloat16 *__restrict__ x, int64_t rows, int size,
                                                           int64_t x_stride, float eps, float2 *__restrict__ stats)
{
    constexpr int R = 32 / G;                                    // rows per warp and pass
    const int lane = threadIdx.x & 31, l = lane % G, gi = lane / G;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t step = (int64_t)gridDim.x * (blockDim.x >> 5) * R;
    const int nvec = size / 8;
    const float inv_n = 1.0f / (float)size;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // a warp's lanes stay together (the shuffles below are warp-wide): the loop runs while ANY group has a row
    for (int64_t base = warp * R; base < rows; base += NR * step) {
        int64_t row[NR];
        const uint4 *p[NR];
        uint4 a[NR];
        float d[NR], s[NR], q[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            row[r] = base + r * step + gi;
            p[r] = reinterpret_cast<const uint4 *>(x + (row[r] < rows ? row[r] : 0) * x_stride);
            a[r] = l < nvec ? __ldg(p[r] + l) : zero;
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            d[r] = bf16lo_to_f32(__shfl_sync(0xffffffffu, a[r].x, gi * G));
            s[r] = q[r] = 0.f;
        }
        for (int v = l; v < nvec; v += G) {
            uint4 b[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) b[r] = v + G < nvec ? __ldg(p[r] + v + G) : zero;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                stats_acc(a[r], d[r], s[r], q[r]);
                a[r] = b[r];
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) {
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                s[r] += __shfl_xor_sync(0xffffffffu, s[r], o);
                q[r] += __shfl_xor_sync(0xffffffffu, q[r], o);
            }
        }
        if (l == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
                if (row[r] < rows) {
                    // a reciprocal of n taken once and the hardware reciprocal square root (2 ulp): IEEE divisions
                    // and a square root per row made this kernel instruction-bound at twice its memory time
                    const float var = fmaxf((q[r] - s[r] * s[r] * inv_n) * inv_n, 0.f);
                    stats[row[r]] = make_float2(fmaf(s[r], inv_n, d[r]), rsqrtf(var + eps));
                }
        }
    }
}

// any row length and alignment: one warp per row, element loads
__global__ void __launch_bounds__(256) ln_stats_kernel(const __nv_bfloat16 *__restrict__ x, int64_t rows, int size,
                                                       int64_t x_stride, float eps, float2 *__restrict__ stats)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const float n = (float)size;
    for (int64_t row = warp; row < rows; row += nwarps) {
        const __nv_bfloat16 *xr = x + row * x_stride;
        const float delta = __bfloat162float(xr[0]);            // shifted data, as the reference sums it
        float sum = 0.f, sum2 = 0.f;
        for (int i = lane; i < size; i += 32) {
            const float a = __bfloat162float(xr[i]) - delta;
            sum += a;
            sum2 = fmaf(a, a, sum2);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
        }
        if (lane == 0) {
            const float mean = sum / n + delta;
            const float var = fmaxf((sum2 - sum * sum / n) / n, 0.f);
            stats[row] = make_float2(mean, 1.0f / sqrtf(var + eps));
        }
    }
}

struct FoldArgs {
    const __nv_bfloat16 *w[4];     // [N, K] each
    const float *bias[4];          // [N] or null
    __nv_bfloat16 *w2[4];          // folded, centred, bf16
    float *s[4], *t[4];
};

// one warp per weight row (output channel) of every matrix
__global__ void __launch_bounds__(256) ln_fold_kernel(const FoldArgs a, const float *__restrict__ gamma,
                                                      const float *__restrict__ beta, int N, int K, int nmat)
{
    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (warp >= N * nmat) return;
    const int mat = warp / N, n = warp % N;
    const __nv_bfloat16 *wr = a.w[mat] + (int64_t)n * K;
    float gsum = 0.f, tsum = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float w = __bfloat162float(wr[k]);
        gsum = fmaf(gamma[k], w, gsum);
        tsum = fmaf(beta[k], w, tsum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        gsum += __shfl_xor_sync(0xffffffffu, gsum, o);
        tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
    }
    const float gbar = gsum / (float)K;
    float ssum = 0.f;
    __nv_bfloat16 *w2 = a.w2[mat] + (int64_t)n * K;
    for (int k = lane; k < K; k += 32) {
        const __nv_bfloat16 v = __float2bfloat16_rn(fmaf(gamma[k], __bfloat162float(wr[k]), -gbar));
        w2[k] = v;
        ssum += __bfloat162float(v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
    if (lane == 0) {
        a.s[mat][n] = ssum;
        a.t[mat][n] = tsum + (a.bias[mat] ? a.bias[mat][n] : 0.f);
    }
}

}  // namespace

bool launch_ln_stats(cudaStream_t stream, const void *x, int64_t rows, int64_t size, int64_t x_stride, float eps, void *stats)
{
    if (rows <= 0 || size <= 0 || size > INT32_MAX) return false;
    const bool vec = (size % 8 == 0) && (x_stride % 8 == 0) && (((uintptr_t)x & 15u) == 0);
    const __nv_bfloat16 *xp = (const __nv_bfloat16 *)x;
    float2 *sp = (float2 *)stats;
    KernelTimer timer__("ln_stats", stream);
    if (vec) {
        const int64_t nvec = size / 8;
        const int g = nvec <= 4 ? 4 : nvec <= 8 ? 8 : nvec <= 16 ? 16 : 32;
        const int64_t rows_per_block = 8 * (32 / g) * NR;                   // 8 warps, NR rows in flight per group
        const unsigned grid = (unsigned)std::min<int64_t>((rows + rows_per_block - 1) / rows_per_block, 148 * 8);
        if (g == 4)
            ln_stats_vec_kernel<4><<<grid, 256, 0, stream>>>(xp, rows, (int)size, x_stride, eps, sp);
        else if (g == 8)
            ln_stats_vec_kernel<8><<<grid, 256, 0, stream>>>(xp, rows, (int)size, x_stride, eps, sp);
        else if (g == 16)
            ln_stats_vec_kernel<16><<<grid, 256, 0, stream>>>(xp, rows, (int)size, x_stride, eps, sp);
        else
            ln_stats_vec_kernel<32><<<grid, 256, 0, stream>>>(xp, rows, (int)size, x_stride, eps, sp);
    } else {
        const unsigned grid = (unsigned)std::min<int64_t>((rows + 7) / 8, 148 * 16);
        ln_stats_kernel<<<grid, 256, 0, stream>>>(xp, rows, (int)size, x_stride, eps, sp);
    }
    count_launch();
    return true;
}

bool launch_ln_fold(cudaStream_t stream, int nmat, const void *const *w, const float *const *bias, const float *gamma,
                    const float *beta, void *const *w2, float *const *s, float *const *t, int N, int K)
{
    if (nmat < 1 || nmat > 4 || N <= 0 || K <= 0) return false;
    FoldArgs a;
    for (int i = 0; i < 4; ++i) {
        const int j = i < nmat ? i : 0;
        a.w[i] = (const __nv_bfloat16 *)w[j];
        a.bias[i] = bias[j];
        a.w2[i] = (__nv_bfloat16 *)w2[j];
        a.s[i] = s[j];
        a.t[i] = t[j];
    }
    const int warps = N * nmat;
    KernelTimer timer__("ln_fold", stream);
    ln_fold_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(a, gamma, beta, N, K, nmat);
    count_launch();
    return true;
}

}  // namespace dev
}  // namespace kutacc
