// Row LayerNorm in front of the attention operators (bf16 in and out, fp32 gamma and beta).
//
// Reference: src/normalization/layernorm_kernel.h:22-53 normalises ONE row of `size` channels per call
// (kutacc_af2_layernorm, include/kutacc.h:334); its callers loop over the rows. On a GPU a launch per row is
// useless, so besides that entry point (rows = 1) the library exports kutacc_b200_layernorm_rows, which
// runs the same arithmetic over every row of a [rows, size] matrix in one launch: a warp (or a half or quarter warp for
// short rows) per row, the row held in registers between the statistics pass and the normalising pass, 128-bit loads and stores.
//
// Arithmetic kept from the reference: the sums are taken of (x - x[0]) ("shifted data"), mean = sum / n +
// x[0], var = max((sum2 - sum * sum / n) / n, 0), rstd = 1 / sqrt(var + eps), then two fused multiply-adds
// y = fma(fma(x, rstd, -rstd * mean), gamma, beta) and one bf16 rounding. The order in which the fp32
// partial sums are added differs (SVE lanes there, warp lanes here).
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

#include <algorithm>

namespace kutacc {
namespace dev {

namespace {

constexpr int LN_MAX_VEC = 4;          // 16-byte vectors per lane: rows of up to 32 * 8 * 4 = 1024 channels in registers

// LPR lanes share a row (32 / LPR rows per warp and step), each lane holds NVEC 16-byte vectors of it.
template <int LPR, int NVEC>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const __nv_bfloat16 *__restrict__ x,
                                                             const float *__restrict__ gamma,
                                                             const float *__restrict__ beta,
                                                             __nv_bfloat16 *__restrict__ out, int64_t rows, int size,
                                                             int64_t x_stride, int64_t out_stride, float eps)
{
    constexpr int RPW = 32 / LPR;                              // rows per warp and step
    const int lane = threadIdx.x & 31, sub = lane / LPR, l = lane % LPR;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int nv = size >> 3;                                  // 16-byte vectors per row
    const float inv_n = 1.0f / (float)size;
    // the loop bound depends on the warp only, so that all lanes reach the shuffles together; U rows per lane
    // group and step keep 2 x 16 x NVEC bytes per lane in flight
    constexpr int U = 2;
    for (int64_t row0 = warp * RPW * U; row0 < rows; row0 += nwarps * RPW * U) {
        int64_t row[U];
        bool live[U];
        float delta[U], sum[U], sum2[U];
        uint4 raw[U][NVEC];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            row[u] = row0 + u * RPW + sub;
            live[u] = row[u] < rows;
            const __nv_bfloat16 *xr = x + (live[u] ? row[u] : 0) * x_stride;
#pragma unroll
            for (int i = 0; i < NVEC; ++i) {
                const int v = l + LPR * i;
                raw[u][i] = v < nv ? __ldg(reinterpret_cast<const uint4 *>(xr) + v) : make_uint4(0, 0, 0, 0);
            }
            delta[u] = __bfloat162float(xr[0]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            sum[u] = sum2[u] = 0.f;
#pragma unroll
            for (int i = 0; i < NVEC; ++i) {
                if (l + LPR * i < nv) {
                    const uint32_t w[4] = {raw[u][i].x, raw[u][i].y, raw[u][i].z, raw[u][i].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = bf16lo_to_f32(w[e]) - delta[u], b = bf16hi_to_f32(w[e]) - delta[u];
                        sum[u] += a;
                        sum2[u] = fmaf(a, a, sum2[u]);
                        sum[u] += b;
                        sum2[u] = fmaf(b, b, sum2[u]);
                    }
                }
            }
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) {
                sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], o);
                sum2[u] += __shfl_xor_sync(0xffffffffu, sum2[u], o);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            // reciprocal of n taken once, hardware reciprocal square root (2 ulp, far below the bf16 step of the
            // output): the IEEE divisions and square root cost more instructions per row than its 128 channels
            const float mean = fmaf(sum[u], inv_n, delta[u]);
            const float var = fmaxf((sum2[u] - sum[u] * sum[u] * inv_n) * inv_n, 0.f);
            const float rstd = rsqrtf(var + eps);
            const float shift = -rstd * mean;
            __nv_bfloat16 *orow = out + row[u] * out_stride;
#pragma unroll
            for (int i = 0; i < NVEC; ++i) {
                const int v = l + LPR * i;
                if (live[u] && v < nv) {
                    const uint32_t w[4] = {raw[u][i].x, raw[u][i].y, raw[u][i].z, raw[u][i].w};
                    const float4 g0 = __ldg(reinterpret_cast<const float4 *>(gamma) + 2 * v),
                                 g1 = __ldg(reinterpret_cast<const float4 *>(gamma) + 2 * v + 1);
                    const float4 b0 = __ldg(reinterpret_cast<const float4 *>(beta) + 2 * v),
                                 b1 = __ldg(reinterpret_cast<const float4 *>(beta) + 2 * v + 1);
                    const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                    const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float y0 = fmaf(fmaf(bf16lo_to_f32(w[e]), rstd, shift), gs[2 * e], bs[2 * e]);
                        const float y1 = fmaf(fmaf(bf16hi_to_f32(w[e]), rstd, shift), gs[2 * e + 1], bs[2 * e + 1]);
                        o[e] = pack_bf16x2(y0, y1);
                    }
                    reinterpret_cast<uint4 *>(orow)[v] = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        }
    }
}

// any size / alignment: one warp per row, scalar accesses, the row is read twice
__global__ void __launch_bounds__(256) layernorm_rows_generic_kernel(const __nv_bfloat16 *__restrict__ x,
                                                                     const float *__restrict__ gamma,
                                                                     const float *__restrict__ beta,
                                                                     __nv_bfloat16 *__restrict__ out, int64_t rows,
                                                                     int64_t size, int64_t x_stride, int64_t out_stride,
                                                                     float eps)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t row = warp; row < rows; row += nwarps) {
        const __nv_bfloat16 *xr = x + row * x_stride;
        const float delta = __bfloat162float(xr[0]);
        float sum = 0.f, sum2 = 0.f;
        for (int64_t i = lane; i < size; i += 32) {
            const float a = __bfloat162float(xr[i]) - delta;
            sum += a;
            sum2 = fmaf(a, a, sum2);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
        }
        const float n = (float)size;
        const float mean = sum / n + delta;
        const float var = fmaxf((sum2 - sum * sum / n) / n, 0.f);
        const float rstd = 1.0f / sqrtf(var + eps);
        const float shift = -rstd * mean;
        __nv_bfloat16 *orow = out + row * out_stride;
        for (int64_t i = lane; i < size; i += 32)
            orow[i] = __float2bfloat16_rn(fmaf(fmaf(__bfloat162float(xr[i]), rstd, shift), gamma[i], beta[i]));
    }
}

}  // namespace

bool launch_layernorm_rows(cudaStream_t stream, const void *x, const float *gamma, const float *beta, void *out,
                           int64_t rows, int64_t size, int64_t x_stride, int64_t out_stride, float eps)
{
    if (rows <= 0 || size <= 0) return false;
    KernelTimer timer__("layernorm", stream);
    const int64_t blocks_needed = (rows + 7) / 8;
    const unsigned grid = (unsigned)std::min<int64_t>(blocks_needed, 148 * 16);
    const bool vec = (size % 8) == 0 && size <= 32 * 8 * LN_MAX_VEC && (x_stride % 8) == 0 && (out_stride % 8) == 0 &&
                     (((uintptr_t)x | (uintptr_t)out | (uintptr_t)gamma | (uintptr_t)beta) & 15u) == 0;
    const __nv_bfloat16 *xp = (const __nv_bfloat16 *)x;
    __nv_bfloat16 *op = (__nv_bfloat16 *)out;
    if (vec) {
        const int nv = (int)(size / 8);
#define KUTACC_LN_LAUNCH(LPR, NVEC)                                                                                   \
    layernorm_rows_kernel<LPR, NVEC><<<grid, 256, 0, stream>>>(xp, gamma, beta, op, rows, (int)size, x_stride, out_stride, eps)
        if (nv <= 8)
            KUTACC_LN_LAUNCH(8, 1);
        else if (nv <= 16)
            KUTACC_LN_LAUNCH(16, 1);
        else if (nv <= 32)
            KUTACC_LN_LAUNCH(32, 1);
        else if (nv <= 64)
            KUTACC_LN_LAUNCH(32, 2);
        else
            KUTACC_LN_LAUNCH(32, 4);
#undef KUTACC_LN_LAUNCH
    } else {
        layernorm_rows_generic_kernel<<<grid, 256, 0, stream>>>(xp, gamma, beta, op, rows, size, x_stride, out_stride, eps);
    }
    count_launch();
    return true;
}

}  // namespace dev
}  // namespace kutacc
