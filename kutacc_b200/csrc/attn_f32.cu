// fp32 gated-attention core on tensor cores (head size 32), for callers that keep fp32 activations.
//
// The reference has no fp32 path (its only tensor type is bf16, include/kutacc.h:467-471); this kernel
// computes the same operator (src/attention/gating_attention.cpp:73-151) without any bf16 rounding, to
// fp32 accuracy: both products use error-compensated tf32 ("3xTF32": every operand is split into a tf32
// head and a tf32 tail, the product is hi*hi + hi*lo + lo*hi accumulated in fp32), the softmax is an
// online softmax in fp32.
//
// A CTA of 8 warps handles 128 queries of one (batch row, head); each warp owns 16 of them (with 4 warps and 64
// queries the split of every K/V tile was shared by half as many queries: 0.290 against 0.263 ms on the MSA-row shape). Keys are walked
// in tiles of 64: the CTA splits the K and V tiles into head/tail images in shared memory once (the next
// tile's global loads are in flight meanwhile), each warp forms S = Q.K^T (16 x 64), adds the biases,
// updates its running max and sum, and accumulates O += P.V. The probabilities never leave registers: an
// accumulator fragment holds columns (2t, 2t+1) of an 8-key group, and the next product simply reads the V
// rows in that order (k index t <-> key 2t, k index t+4 <-> key 2t+1), which is legal because the sum over
// keys does not care about their order.
//
// q, k, v, gate, avg: [B, S, H*32] fp32; bias [B, S] (row stride bias_stride0); pair bias [H, S, S] with
// strides (nb_stride_h, nb_stride_q, 1) or null.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

namespace kutacc {
namespace dev {

namespace {

constexpr int AD = 32;                 // head size
constexpr int AQ = 128;                // queries per CTA (8 warps: the K/V split of a tile is shared by twice the queries)
constexpr int AK = 64;                 // keys per tile
constexpr int ALD = 36;                // row pitch (floats) of the K and V images: fragment loads hit 32 banks
constexpr int A_THREADS = 256;
constexpr int A_FETCH = AK * 8 / A_THREADS;   // 16-byte vectors of a K (or V) tile per thread

__device__ __forceinline__ uint32_t tf32_hi(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct F32Smem {
    uint32_t khi[AK * ALD], klo[AK * ALD];
    uint32_t vhi[AK * ALD], vlo[AK * ALD];
    float bias[AK];
};

__global__ void __launch_bounds__(A_THREADS, 2) attn_f32_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                                             const float *__restrict__ v, const float *__restrict__ gate,
                                                             const float *__restrict__ bias, int64_t bias_stride0,
                                                             const float *__restrict__ nb, int64_t nb_stride_h,
                                                             int64_t nb_stride_q, float *__restrict__ avg, int S, int H,
                                                             int n_qt, float scale, float *__restrict__ avg_split)
{
    __shared__ F32Smem sm;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int item = blockIdx.x;
    const int qt = item % n_qt, h = (item / n_qt) % H, b = item / (n_qt * H);
    const int C = H * AD;
    const int q0 = qt * AQ + warp * 16;                       // first query of this warp
    const float *qb = q + (int64_t)b * S * C + h * AD;
    const float *kb = k + (int64_t)b * S * C + h * AD;
    const float *vb = v + (int64_t)b * S * C + h * AD;
    const float *brow = bias + (int64_t)b * bias_stride0;
    const int r0 = q0 + g, r1 = q0 + g + 8;                   // the two query rows of this thread's fragments
    const int r0c = min(r0, S - 1), r1c = min(r1, S - 1);     // clamped for loads

    // Q fragments of the four k8 steps, split once
    uint32_t qhi[4][4], qlo[4][4];
#pragma unroll
    for (int k8 = 0; k8 < 4; ++k8) {
        const float x[4] = {qb[(int64_t)r0c * C + k8 * 8 + t], qb[(int64_t)r1c * C + k8 * 8 + t],
                            qb[(int64_t)r0c * C + k8 * 8 + t + 4], qb[(int64_t)r1c * C + k8 * 8 + t + 4]};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            qhi[k8][e] = tf32_hi(x[e]);
            qlo[k8][e] = tf32_hi(x[e] - __uint_as_float(qhi[k8][e]));
        }
    }
    const float *nb0 = nb ? nb + (int64_t)h * nb_stride_h + (int64_t)r0c * nb_stride_q : nullptr;
    const float *nb1 = nb ? nb + (int64_t)h * nb_stride_h + (int64_t)r1c * nb_stride_q : nullptr;

    float o[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // the tile's K and V rows this thread fetches: 64 rows x 8 float4 per matrix, A_FETCH float4 per thread each
    const int nkt = (S + AK - 1) / AK;
    float4 kreg[A_FETCH], vreg[A_FETCH];
    auto fetch = [&](int kt) {
#pragma unroll
        for (int i = 0; i < A_FETCH; ++i) {
            const int idx = tid + i * A_THREADS, r = idx >> 3, c = idx & 7;
            const int key = kt * AK + r;
            if (key < S) {
                kreg[i] = __ldg(reinterpret_cast<const float4 *>(kb + (int64_t)key * C) + c);
                vreg[i] = __ldg(reinterpret_cast<const float4 *>(vb + (int64_t)key * C) + c);
            } else {
                kreg[i] = vreg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    };
    fetch(0);
    for (int kt = 0; kt < nkt; ++kt) {
        __syncthreads();                                       // every warp is done with the previous images
#pragma unroll
        for (int i = 0; i < A_FETCH; ++i) {
            const int idx = tid + i * A_THREADS, r = idx >> 3, c = idx & 7;
            const float kx[4] = {kreg[i].x, kreg[i].y, kreg[i].z, kreg[i].w}, vx[4] = {vreg[i].x, vreg[i].y, vreg[i].z, vreg[i].w};
            uint32_t kh[4], kl[4], vh[4], vl[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                kh[e] = tf32_hi(kx[e]);
                kl[e] = tf32_hi(kx[e] - __uint_as_float(kh[e]));
                vh[e] = tf32_hi(vx[e]);
                vl[e] = tf32_hi(vx[e] - __uint_as_float(vh[e]));
            }
            *reinterpret_cast<uint4 *>(&sm.khi[r * ALD + c * 4]) = make_uint4(kh[0], kh[1], kh[2], kh[3]);
            *reinterpret_cast<uint4 *>(&sm.klo[r * ALD + c * 4]) = make_uint4(kl[0], kl[1], kl[2], kl[3]);
            *reinterpret_cast<uint4 *>(&sm.vhi[r * ALD + c * 4]) = make_uint4(vh[0], vh[1], vh[2], vh[3]);
            *reinterpret_cast<uint4 *>(&sm.vlo[r * ALD + c * 4]) = make_uint4(vl[0], vl[1], vl[2], vl[3]);
        }
        if (tid < AK) {
            const int key = kt * AK + tid;
            sm.bias[tid] = key < S ? brow[key] : -INFINITY;    // keys past the end never win the max, exp gives 0
        }
        __syncthreads();
        if (kt + 1 < nkt) fetch(kt + 1);                       // in flight during the products below

        // S = Q . K^T for this warp's 16 queries and the tile's 64 keys
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
            for (int k8 = 0; k8 < 4; ++k8) {
                const int off = (nt * 8 + g) * ALD + k8 * 8 + t;
                const uint32_t bh0 = sm.khi[off], bh1 = sm.khi[off + 4], bl0 = sm.klo[off], bl1 = sm.klo[off + 4];
                mma_tf32(s[nt], qlo[k8], bh0, bh1);            // small terms first
                mma_tf32(s[nt], qhi[k8], bl0, bl1);
                mma_tf32(s[nt], qhi[k8], bh0, bh1);
            }
        }
        // x = s * scale + bias (+ pair bias); fragment columns are keys nt*8 + 2t, + 1
        float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int kc = nt * 8 + 2 * t, key = kt * AK + kc;
            const float b0 = sm.bias[kc], b1 = sm.bias[kc + 1];
            float n00 = 0.f, n01 = 0.f, n10 = 0.f, n11 = 0.f;
            if (nb0) {
                if (key < S) {
                    n00 = __ldg(nb0 + key);
                    n10 = __ldg(nb1 + key);
                }
                if (key + 1 < S) {
                    n01 = __ldg(nb0 + key + 1);
                    n11 = __ldg(nb1 + key + 1);
                }
            }
            s[nt][0] = (s[nt][0] * scale + b0) + n00;
            s[nt][1] = (s[nt][1] * scale + b1) + n01;
            s[nt][2] = (s[nt][2] * scale + b0) + n10;
            s[nt][3] = (s[nt][3] * scale + b1) + n11;
            tm0 = fmaxf(tm0, fmaxf(s[nt][0], s[nt][1]));
            tm1 = fmaxf(tm1, fmaxf(s[nt][2], s[nt][3]));
        }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        const float mn0 = fmaxf(m0, tm0), mn1 = fmaxf(m1, tm1);    // finite: every tile holds at least one real key
        const float c0 = __expf(m0 - mn0), c1 = __expf(m1 - mn1);  // first tile: exp(-inf) = 0
        m0 = mn0;
        m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s[nt][0] = __expf(s[nt][0] - mn0);
            s[nt][1] = __expf(s[nt][1] - mn0);
            s[nt][2] = __expf(s[nt][2] - mn1);
            s[nt][3] = __expf(s[nt][3] - mn1);
            ps0 += s[nt][0] + s[nt][1];
            ps1 += s[nt][2] + s[nt][3];
        }
        l0 = l0 * c0 + ps0;
        l1 = l1 * c1 + ps1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[i][0] *= c0;
            o[i][1] *= c0;
            o[i][2] *= c1;
            o[i][3] *= c1;
        }
        // O += P . V: the 8 keys of group nt are one k8 step, in the order (2t, 2t + 1)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            // A fragment: a0 (row g, k t) a1 (row g+8, k t) a2 (row g, k t+4) a3 (row g+8, k t+4)
            const float pv[4] = {s[nt][0], s[nt][2], s[nt][1], s[nt][3]};
            uint32_t phi[4], plo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                phi[e] = tf32_hi(pv[e]);
                plo[e] = tf32_hi(pv[e] - __uint_as_float(phi[e]));
            }
#pragma unroll
            for (int ct = 0; ct < 4; ++ct) {
                const int off0 = (nt * 8 + 2 * t) * ALD + ct * 8 + g, off1 = off0 + ALD;
                const uint32_t bh0 = sm.vhi[off0], bh1 = sm.vhi[off1], bl0 = sm.vlo[off0], bl1 = sm.vlo[off1];
                mma_tf32(o[ct], plo, bh0, bh1);
                mma_tf32(o[ct], phi, bl0, bl1);
                mma_tf32(o[ct], phi, bh0, bh1);
            }
        }
    }
    // row sums across the quad, normalise, sigmoid gate, store
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    // With avg_split the gated average goes out as the operand of the output projection's tensor-memory GEMM: rows
    // of 2C floats, [tf32 head | tail] (what launch_split_tf32 would make of avg), and avg itself is not written.
    auto store_result = [&](int64_t off, int64_t row, int ch, float2 res) {
        if (avg_split == nullptr) {
            *reinterpret_cast<float2 *>(avg + off) = res;
            return;
        }
        const float hx = __uint_as_float(tf32_hi(res.x)), hy = __uint_as_float(tf32_hi(res.y));
        float *dst = avg_split + row * 2 * C + ch;
        *reinterpret_cast<float2 *>(dst) = make_float2(hx, hy);
        *reinterpret_cast<float2 *>(dst + C) = make_float2(res.x - hx, res.y - hy);
    };
#pragma unroll
    for (int ct = 0; ct < 4; ++ct) {
        const int ch = h * AD + ct * 8 + 2 * t;
        if (r0 < S) {
            const int64_t off = ((int64_t)b * S + r0) * C + ch;
            const float2 gv = *reinterpret_cast<const float2 *>(gate + off);
            float2 res;
            res.x = o[ct][0] * i0 * (1.0f / (1.0f + __expf(-gv.x)));
            res.y = o[ct][1] * i0 * (1.0f / (1.0f + __expf(-gv.y)));
            store_result(off, ((int64_t)b * S + r0), ch, res);
        }
        if (r1 < S) {
            const int64_t off = ((int64_t)b * S + r1) * C + ch;
            const float2 gv = *reinterpret_cast<const float2 *>(gate + off);
            float2 res;
            res.x = o[ct][2] * i1 * (1.0f / (1.0f + __expf(-gv.x)));
            res.y = o[ct][3] * i1 * (1.0f / (1.0f + __expf(-gv.y)));
            store_result(off, ((int64_t)b * S + r1), ch, res);
        }
    }
}

}  // namespace

// fp32, head size 32 only; returns false for anything else (the caller falls back to the generic kernel).
bool launch_attn_f32(cudaStream_t stream, const void *q, const void *k, const void *v, const void *gate, const void *bias,
                     int64_t bias_stride0, const void *nb, int64_t nb_stride_h, int64_t nb_stride_q, void *avg, int B,
                     int S, int H, int D, float scale, void *avg_split)
{
    if (D != AD || B < 1 || S < 1 || H < 1) return false;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)gate | (uintptr_t)avg | (uintptr_t)avg_split) & 15u) != 0) return false;
    const int n_qt = (S + AQ - 1) / AQ;
    const int64_t items = (int64_t)B * H * n_qt;
    if (items > 0x7fffffff) return false;
    KernelTimer timer__("attn_f32", stream);
    attn_f32_kernel<<<(unsigned)items, A_THREADS, 0, stream>>>(
        (const float *)q, (const float *)k, (const float *)v, (const float *)gate, (const float *)bias, bias_stride0,
        (const float *)nb, nb_stride_h, nb_stride_q, (float *)avg, S, H, n_qt, scale, (float *)avg_split);
    count_launch();
    return true;
}

}  // namespace dev
}  // namespace kutacc
