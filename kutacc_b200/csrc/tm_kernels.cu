// Element-wise steps of the triangle multiplication and its CUDA-core fallbacks.
// Replaces the SVE loops of src/attention/triangle_multiplication.cpp:51-69 (mask and gate of the projections)
// and :138-158 (the final gate); the matrix products themselves run on the tcgen05 GEMM (gemm_tcgen05.cu) where
// the shape allows it and on the plain kernels below otherwise.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

#include <algorithm>

namespace kutacc {
namespace dev {

namespace {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float sigmoidf_fast(float g) { return 1.0f / (1.0f + ex2_approx(-g * kLog2e)); }

// one thread per 8 consecutive positions of one (channel, batch row) line when `vec`, else per position
template <bool VEC>
__global__ void tm_mask_gate_kernel(__nv_bfloat16 *__restrict__ proj, const __nv_bfloat16 *__restrict__ gate,
                                    const __nv_bfloat16 *__restrict__ mask, int64_t c_i, int64_t n_res, int64_t n_gather,
                                    int64_t p_s0, int64_t p_s1, int64_t g_s0, int64_t g_s1, int64_t m_s0)
{
    const int64_t per_line = VEC ? n_gather / 8 : n_gather;
    const int64_t total = c_i * n_res * per_line;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = (t % per_line) * (VEC ? 8 : 1), line = t / per_line, b = line % n_res, c = line / n_res;
        __nv_bfloat16 *pp = proj + c * p_s0 + b * p_s1 + i;
        const __nv_bfloat16 *gp = gate + c * g_s0 + b * g_s1 + i, *mp = mask + b * m_s0 + i;
        if (VEC) {
            const uint4 pv = *reinterpret_cast<const uint4 *>(pp), gv = *reinterpret_cast<const uint4 *>(gp),
                        mv = *reinterpret_cast<const uint4 *>(mp);
            const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w}, mw[4] = {mv.x, mv.y, mv.z, mv.w};
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // (proj * mask) * sigmoid(gate), in this order (triangle_multiplication.cpp:60-64)
                const float lo = (bf16lo_to_f32(pw[j]) * bf16lo_to_f32(mw[j])) * sigmoidf_fast(bf16lo_to_f32(gw[j]));
                const float hi = (bf16hi_to_f32(pw[j]) * bf16hi_to_f32(mw[j])) * sigmoidf_fast(bf16hi_to_f32(gw[j]));
                ow[j] = pack_bf16x2(lo, hi);
            }
            *reinterpret_cast<uint4 *>(pp) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        } else {
            const float v = (__bfloat162float(*pp) * __bfloat162float(*mp)) * sigmoidf_fast(__bfloat162float(*gp));
            *pp = __float2bfloat16_rn(v);
        }
    }
}

// both projections of one (position, channel) per thread: dot products of length c_o on CUDA cores
__global__ void tm_proj_generic_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ w0,
                                       const float *__restrict__ b0, const __nv_bfloat16 *__restrict__ w1,
                                       const float *__restrict__ b1, __nv_bfloat16 *__restrict__ out0,
                                       __nv_bfloat16 *__restrict__ out1, int64_t p_s0, int64_t p_s1, int64_t g_s0,
                                       int64_t g_s1, int64_t n_res, int64_t n_gather, int64_t c_o, int64_t c_i)
{
    const int64_t total = n_res * n_gather * c_i;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = t % n_gather, b = (t / n_gather) % n_res, c = t / (n_gather * n_res);
        const __nv_bfloat16 *xr = x + (b * n_gather + i) * c_o, *wr0 = w0 + c * c_o, *wr1 = w1 + c * c_o;
        float a0 = 0.f, a1 = 0.f;
        for (int64_t k = 0; k < c_o; ++k) {
            const float xv = __bfloat162float(xr[k]);
            a0 += xv * __bfloat162float(wr0[k]);
            a1 += xv * __bfloat162float(wr1[k]);
        }
        out0[c * p_s0 + b * p_s1 + i] = __float2bfloat16_rn(a0 + b0[c]);
        out1[c * g_s0 + b * g_s1 + i] = __float2bfloat16_rn(a1 + b1[c]);
    }
}

// one output element per thread
__global__ void tm_equation_generic_kernel(const __nv_bfloat16 *__restrict__ left, int64_t l_s0, int64_t l_s1,
                                           const __nv_bfloat16 *__restrict__ right, int64_t r_s0, int64_t r_s1,
                                           __nv_bfloat16 *__restrict__ center, int64_t c_s0, int64_t c_s1, int64_t c_i,
                                           int64_t n, int incoming)
{
    const int64_t total = c_i * n * n;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = t % n, a = (t / n) % n, c = t / (n * n);
        const __nv_bfloat16 *L = left + c * l_s0, *R = right + c * r_s0;
        float acc = 0.f;
        if (!incoming)
            for (int64_t k = 0; k < n; ++k) acc += __bfloat162float(L[a * l_s1 + k]) * __bfloat162float(R[b * r_s1 + k]);
        else
            for (int64_t k = 0; k < n; ++k) acc += __bfloat162float(R[k * r_s1 + a]) * __bfloat162float(L[k * l_s1 + b]);
        center[c * c_s0 + a * c_s1 + b] = __float2bfloat16_rn(acc);
    }
}

// 32 x 32 tiles through shared memory: dst[c, a, k] = src[c, k, a]
__global__ void tm_transpose_kernel(const __nv_bfloat16 *__restrict__ src, int64_t s_s0, int64_t s_s1,
                                    __nv_bfloat16 *__restrict__ dst, int64_t d_pitch, int64_t n)
{
    __shared__ __nv_bfloat16 tile[32][33];
    const int64_t c = blockIdx.z, k0 = (int64_t)blockIdx.y * 32, a0 = (int64_t)blockIdx.x * 32;
    const __nv_bfloat16 *s = src + c * s_s0;
    __nv_bfloat16 *d = dst + c * n * d_pitch;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int64_t k = k0 + r, a = a0 + threadIdx.x;
        tile[r][threadIdx.x] = (k < n && a < n) ? s[k * s_s1 + a] : __float2bfloat16_rn(0.f);
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int64_t a = a0 + r, k = k0 + threadIdx.x;
        if (a < n && k < n) d[a * d_pitch + k] = tile[threadIdx.x][r];
    }
}

template <bool VEC>
__global__ void tm_last_kernel(__nv_bfloat16 *__restrict__ out, int64_t o_rs, const __nv_bfloat16 *__restrict__ gate,
                               int64_t g_rs, int64_t rows, int64_t c_o)
{
    const int64_t per_row = VEC ? c_o / 8 : c_o;
    const int64_t total = rows * per_row;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / per_row, i = (t % per_row) * (VEC ? 8 : 1);
        __nv_bfloat16 *op = out + r * o_rs + i;
        const __nv_bfloat16 *gp = gate + r * g_rs + i;
        if (VEC) {
            const uint4 ov = *reinterpret_cast<const uint4 *>(op), gv = *reinterpret_cast<const uint4 *>(gp);
            const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
            uint32_t rw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                rw[j] = pack_bf16x2(bf16lo_to_f32(ow[j]) * sigmoidf_fast(bf16lo_to_f32(gw[j])),
                                    bf16hi_to_f32(ow[j]) * sigmoidf_fast(bf16hi_to_f32(gw[j])));
            *reinterpret_cast<uint4 *>(op) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
        } else {
            *op = __float2bfloat16_rn(__bfloat162float(*op) * sigmoidf_fast(__bfloat162float(*gp)));
        }
    }
}

unsigned grid_for(int64_t work_items, int block)
{
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>((work_items + block - 1) / block, 148 * 16));
}

}  // namespace

bool launch_tm_mask_gate(cudaStream_t stream, void *proj, const void *gate, const void *mask, int64_t c_i, int64_t n_res,
                         int64_t n_gather, int64_t p_s0, int64_t p_s1, int64_t g_s0, int64_t g_s1, int64_t m_s0)
{
    const bool vec = n_gather % 8 == 0 && ((p_s0 | p_s1 | g_s0 | g_s1 | m_s0) % 8 == 0) &&
                     ((((uintptr_t)proj | (uintptr_t)gate | (uintptr_t)mask) & 15u) == 0);
    KernelTimer timer__("tm_mask_gate", stream);
    if (vec)
        tm_mask_gate_kernel<true><<<grid_for(c_i * n_res * n_gather / 8, 256), 256, 0, stream>>>(
            (__nv_bfloat16 *)proj, (const __nv_bfloat16 *)gate, (const __nv_bfloat16 *)mask, c_i, n_res, n_gather, p_s0, p_s1,
            g_s0, g_s1, m_s0);
    else
        tm_mask_gate_kernel<false><<<grid_for(c_i * n_res * n_gather, 256), 256, 0, stream>>>(
            (__nv_bfloat16 *)proj, (const __nv_bfloat16 *)gate, (const __nv_bfloat16 *)mask, c_i, n_res, n_gather, p_s0, p_s1,
            g_s0, g_s1, m_s0);
    count_launch();
    return true;
}

bool launch_tm_proj_generic(cudaStream_t stream, const void *x, const void *w0, const float *b0, const void *w1,
                            const float *b1, void *out0, void *out1, int64_t p_s0, int64_t p_s1, int64_t g_s0,
                            int64_t g_s1, int64_t n_res, int64_t n_gather, int64_t c_o, int64_t c_i)
{
    KernelTimer timer__("tm_proj_generic", stream);
    tm_proj_generic_kernel<<<grid_for(n_res * n_gather * c_i, 256), 256, 0, stream>>>(
        (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)w0, b0, (const __nv_bfloat16 *)w1, b1, (__nv_bfloat16 *)out0,
        (__nv_bfloat16 *)out1, p_s0, p_s1, g_s0, g_s1, n_res, n_gather, c_o, c_i);
    count_launch();
    return true;
}

bool launch_tm_equation_generic(cudaStream_t stream, const void *left, int64_t l_s0, int64_t l_s1, const void *right,
                                int64_t r_s0, int64_t r_s1, void *center, int64_t c_s0, int64_t c_s1, int64_t c_i,
                                int64_t n, bool incoming)
{
    KernelTimer timer__("tm_equation_generic", stream);
    tm_equation_generic_kernel<<<grid_for(c_i * n * n, 256), 256, 0, stream>>>(
        (const __nv_bfloat16 *)left, l_s0, l_s1, (const __nv_bfloat16 *)right, r_s0, r_s1, (__nv_bfloat16 *)center, c_s0, c_s1,
        c_i, n, incoming ? 1 : 0);
    count_launch();
    return true;
}

bool launch_tm_transpose(cudaStream_t stream, const void *src, int64_t s_s0, int64_t s_s1, void *dst, int64_t d_pitch,
                         int64_t c_i, int64_t n)
{
    const int64_t tiles = (n + 31) / 32;
    if (c_i > 65535 || tiles > 65535) return false;
    KernelTimer timer__("tm_transpose", stream);
    dim3 grid((unsigned)tiles, (unsigned)tiles, (unsigned)c_i), block(32, 8);
    tm_transpose_kernel<<<grid, block, 0, stream>>>((const __nv_bfloat16 *)src, s_s0, s_s1, (__nv_bfloat16 *)dst, d_pitch, n);
    count_launch();
    return true;
}

bool launch_tm_last(cudaStream_t stream, void *out, int64_t o_rs, const void *gate, int64_t g_rs, int64_t rows, int64_t c_o)
{
    const bool vec = c_o % 8 == 0 && o_rs % 8 == 0 && g_rs % 8 == 0 && ((((uintptr_t)out | (uintptr_t)gate) & 15u) == 0);
    KernelTimer timer__("tm_last", stream);
    if (vec)
        tm_last_kernel<true><<<grid_for(rows * c_o / 8, 256), 256, 0, stream>>>((__nv_bfloat16 *)out, o_rs,
                                                                                  (const __nv_bfloat16 *)gate, g_rs, rows, c_o);
    else
        tm_last_kernel<false><<<grid_for(rows * c_o, 256), 256, 0, stream>>>((__nv_bfloat16 *)out, o_rs,
                                                                               (const __nv_bfloat16 *)gate, g_rs, rows, c_o);
    count_launch();
    return true;
}

}  // namespace dev
}  // namespace kutacc
