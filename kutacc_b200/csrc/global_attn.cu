// Extra-MSA global column attention (nchannels = 64), bandwidth-bound.
//
// Reference path: src/attention/global_attention.cpp:30-164 makes five passes over the [B, S, 64]
// activations (pool, K, V, gate, output) and materialises k, v and gate. Here each batch column is
// handled by three kernels that stream the activations with 128-bit loads and keep every
// intermediate on chip:
//   pool : partial masked sums of x over a slice of the rows                      (:44-75)
//   core : q = q_avg.Wq^T; per row k = x.Wk^T, v = x.Wv^T, logits for all heads, online softmax,
//          partial weighted sums of v                                              (:76-89, :96-133)
//   out  : gate = x.Wg^T + bg; out = (sigmoid(gate) * wa).Wo^T + bo on tensor cores (:90-94, :134-163)
// The batch is processed in groups whose activations fit in L2, so that the second and third read
// of x are L2 hits and HBM sees one read of x and one write of out.
//
// bf16 rounding points of the reference that are kept: q_avg, q, k, v, logits, wa, gate, gated
// gate, out. Probabilities are kept in fp32 (the reference rounds them to bf16 after normalising).
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

#include <algorithm>
#include <climits>

namespace kutacc {
namespace dev {

namespace {

constexpr int GC = 64;            // channels
constexpr int POOL_THREADS = 256;
constexpr int CORE_THREADS = 256;
constexpr int OUT_ROWS = 128;     // rows per CTA of the output kernel (8 warps x 16 rows)

__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// scratch layout per batch column b (all fp32):
//   pool  : [nsplit][GC + 1]   partial sums and partial mask sum
//   core  : [nsplit][H][2 + D] running max, running sum, partial weighted v
struct Scratch {
    float *pool;
    float *core;
    int nsplit;
};

// ---- pool ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(POOL_THREADS) global_pool_kernel(const __nv_bfloat16 *__restrict__ x,
                                                                   const __nv_bfloat16 *__restrict__ mask,
                                                                   Scratch sc, int b0, int S, int rows_per_split)
{
    const int b = b0 + blockIdx.y, split = blockIdx.x;
    const int s_begin = split * rows_per_split, s_end = min(S, s_begin + rows_per_split);
    const int sub = threadIdx.x & 7, rgrp = threadIdx.x >> 3;  // 8 lanes x 8 channels per row, 32 rows in flight
    float acc[8] = {};
    float msum = 0.f;
    const __nv_bfloat16 *xb = x + (int64_t)b * S * GC;
    const __nv_bfloat16 *mb = mask + (int64_t)b * S;
    for (int s = s_begin + rgrp; s < s_end; s += POOL_THREADS / 8) {
        const float mv = __bfloat162float(mb[s]);
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(xb + (int64_t)s * GC) + sub);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] = fmaf(bf16lo_to_f32(w[i]), mv, acc[2 * i]);
            acc[2 * i + 1] = fmaf(bf16hi_to_f32(w[i]), mv, acc[2 * i + 1]);
        }
        if (sub == 0) msum += mv;
    }
    __shared__ float red[POOL_THREADS / 8][GC + 1];
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rgrp][sub * 8 + i] = acc[i];
    if (sub == 0) red[rgrp][GC] = msum;
    __syncthreads();
    if (threadIdx.x <= GC) {
        float t = 0.f;
        for (int r = 0; r < POOL_THREADS / 8; ++r) t += red[r][threadIdx.x];
        sc.pool[((int64_t)b * sc.nsplit + split) * (GC + 1) + threadIdx.x] = t;
    }
}

// ---- core ----------------------------------------------------------------------------------------
template <int H, int D>
__global__ void __launch_bounds__(CORE_THREADS) global_core_kernel(const __nv_bfloat16 *__restrict__ x,
                                                                   const __nv_bfloat16 *__restrict__ mask,
                                                                   const __nv_bfloat16 *__restrict__ wq,
                                                                   const __nv_bfloat16 *__restrict__ wk,
                                                                   const __nv_bfloat16 *__restrict__ wv, Scratch sc,
                                                                   int b0, int S, int rows_per_split)
{
    static_assert(H * D == GC, "global attention is specialised to 64 channels");
    __shared__ float s_qa[GC];
    __shared__ float s_q[GC];
    __shared__ float s_wk[D][GC];
    __shared__ float s_wv[D][GC];
    __shared__ float s_m[CORE_THREADS / 32][H];
    __shared__ float s_part[CORE_THREADS / 32][H][1 + D];

    const int b = b0 + blockIdx.y, split = blockIdx.x;
    const int tid = threadIdx.x;
    for (int i = tid; i < D * GC; i += CORE_THREADS) {
        s_wk[i / GC][i % GC] = __bfloat162float(wk[i]);
        s_wv[i / GC][i % GC] = __bfloat162float(wv[i]);
    }
    if (tid < GC) {
        float t = 0.f, ms = 0.f;
        for (int sp = 0; sp < sc.nsplit; ++sp) {
            const float *pp = sc.pool + ((int64_t)b * sc.nsplit + sp) * (GC + 1);
            t += pp[tid];
            ms += pp[GC];
        }
        s_qa[tid] = rbf(t * (1.0f / (ms + 1e-10f)));
    }
    __syncthreads();
    if (tid < GC) {
        float t = 0.f;
        for (int c = 0; c < GC; ++c) t = fmaf(s_qa[c], __bfloat162float(wq[tid * GC + c]), t);
        s_q[tid] = rbf(t);
    }
    __syncthreads();

    const float scale = 1.0f / sqrtf((float)D);
    float m_run[H], l_run[H], acc[H][D];
#pragma unroll
    for (int h = 0; h < H; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
#pragma unroll
        for (int d = 0; d < D; ++d) acc[h][d] = 0.f;
    }
    const int s_begin = split * rows_per_split, s_end = min(S, s_begin + rows_per_split);
    const __nv_bfloat16 *xb = x + (int64_t)b * S * GC;
    const __nv_bfloat16 *mb = mask + (int64_t)b * S;
    for (int s = s_begin + tid; s < s_end; s += CORE_THREADS) {
        float kk[D], vv[D];
#pragma unroll
        for (int d = 0; d < D; ++d) kk[d] = vv[d] = 0.f;
        const uint4 *xr = reinterpret_cast<const uint4 *>(xb + (int64_t)s * GC);
#pragma unroll
        for (int ch = 0; ch < GC / 8; ++ch) {
            const uint4 raw = __ldg(xr + ch);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x0 = bf16lo_to_f32(w[i]), x1 = bf16hi_to_f32(w[i]);
                const int c = ch * 8 + 2 * i;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    kk[d] = fmaf(x0, s_wk[d][c], kk[d]);
                    kk[d] = fmaf(x1, s_wk[d][c + 1], kk[d]);
                    vv[d] = fmaf(x0, s_wv[d][c], vv[d]);
                    vv[d] = fmaf(x1, s_wv[d][c + 1], vv[d]);
                }
            }
        }
#pragma unroll
        for (int d = 0; d < D; ++d) {
            kk[d] = rbf(kk[d]);
            vv[d] = rbf(vv[d]);
        }
        const float mbias = fmaf(__bfloat162float(mb[s]), 1e9f, -1e9f);
#pragma unroll
        for (int h = 0; h < H; ++h) {
            float l = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) l = fmaf(s_q[h * D + d], kk[d], l);
            const float xv = rbf(l) * scale + mbias;
            if (xv > m_run[h]) {
                const float corr = __expf(m_run[h] - xv);
                l_run[h] *= corr;
#pragma unroll
                for (int d = 0; d < D; ++d) acc[h][d] *= corr;
                m_run[h] = xv;
            }
            const float pv = __expf(xv - m_run[h]);
            l_run[h] += pv;
#pragma unroll
            for (int d = 0; d < D; ++d) acc[h][d] = fmaf(pv, vv[d], acc[h][d]);
        }
    }

    // merge the per-thread softmax states: block max per head, then rescaled sums
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int h = 0; h < H; ++h) {
        float mx = m_run[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) s_m[warp][h] = mx;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < H; ++h) {
        float mx = s_m[0][h];
        for (int w = 1; w < CORE_THREADS / 32; ++w) mx = fmaxf(mx, s_m[w][h]);
        const float f = (m_run[h] == -INFINITY) ? 0.f : __expf(m_run[h] - mx);
        float lv = l_run[h] * f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lv += __shfl_xor_sync(0xffffffffu, lv, o);
        if (lane == 0) s_part[warp][h][0] = lv;
#pragma unroll
        for (int d = 0; d < D; ++d) {
            float av = acc[h][d] * f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) av += __shfl_xor_sync(0xffffffffu, av, o);
            if (lane == 0) s_part[warp][h][1 + d] = av;
        }
    }
    __syncthreads();
    float *dst = sc.core + ((int64_t)b * sc.nsplit + split) * H * (2 + D);
    for (int i = tid; i < H * (1 + D); i += CORE_THREADS) {
        const int h = i / (1 + D), j = i % (1 + D);
        float t = 0.f;
        for (int w = 0; w < CORE_THREADS / 32; ++w) t += s_part[w][h][j];
        dst[h * (2 + D) + 1 + j] = t;
        if (j == 0) {
            float mx = s_m[0][h];
            for (int w = 1; w < CORE_THREADS / 32; ++w) mx = fmaxf(mx, s_m[w][h]);
            dst[h * (2 + D)] = mx;
        }
    }
}

// ---- core on tensor cores (8 heads x 8 channels) -----------------------------------------------------
// Each warp walks 16-row tiles of x (double-buffered cp.async into its own shared-memory slab) and chains
// four small products through registers, using the fact that an mma.sync accumulator fragment (row g,
// columns 2t, 2t+1) has the layout of an A fragment of the next product and, read "transposed", of a B
// fragment:
//   k   [16 rows x 8]   = x . Wk^T                 m16n8k16 x 4   (A = x tile, B = Wk in registers)
//   v^T [8 x 16 rows]   = Wv . x^T                 m16n8k16 x 8   (A = Wv in registers, B = the same x fragments)
//   L^T [8 heads x 16]  = q . k^T                  m16n8k8  x 2   (B = bf16(k) accumulators)
//   wa  [8 heads x 8]  += P^T . v                  m16n8k16 x 1   (A = bf16(P), B = bf16(v^T) accumulators)
// Thread (g, t) therefore owns head g: its running max is shared by the quad (two shuffles per tile).
__device__ __forceinline__ void mma_bf16_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

__global__ void __launch_bounds__(CORE_THREADS) global_core_mma_kernel(const __nv_bfloat16 *__restrict__ x,
                                                                       const __nv_bfloat16 *__restrict__ mask,
                                                                       const __nv_bfloat16 *__restrict__ wq,
                                                                       const __nv_bfloat16 *__restrict__ wk,
                                                                       const __nv_bfloat16 *__restrict__ wv, Scratch sc,
                                                                       int b0, int S, int rows_per_split)
{
    constexpr int H = 8, D = 8, NW = CORE_THREADS / 32;
    __shared__ float s_qa[GC];
    __shared__ float s_q[GC];
    __shared__ __align__(128) __nv_bfloat16 s_x[NW][2][16 * GC];
    __shared__ float s_m[NW][H];
    __shared__ float s_part[NW][H][1 + D];

    const int b = b0 + blockIdx.y, split = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    if (tid < GC) {
        float acc = 0.f, ms = 0.f;
        for (int sp = 0; sp < sc.nsplit; ++sp) {
            const float *pp = sc.pool + ((int64_t)b * sc.nsplit + sp) * (GC + 1);
            acc += pp[tid];
            ms += pp[GC];
        }
        s_qa[tid] = rbf(acc * (1.0f / (ms + 1e-10f)));
    }
    __syncthreads();
    if (tid < GC) {
        float acc = 0.f;
        for (int c = 0; c < GC; ++c) acc = fmaf(s_qa[c], __bfloat162float(wq[tid * GC + c]), acc);
        s_q[tid] = rbf(acc);
    }
    __syncthreads();

    // operands that stay in registers: Wk as B fragments, Wv as A fragments (rows 8..15 zero), q as A fragment
    uint32_t bk[4][2], av[4][2];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        bk[ks][0] = *reinterpret_cast<const uint32_t *>(wk + g * GC + 16 * ks + 2 * t);
        bk[ks][1] = *reinterpret_cast<const uint32_t *>(wk + g * GC + 16 * ks + 8 + 2 * t);
        av[ks][0] = *reinterpret_cast<const uint32_t *>(wv + g * GC + 16 * ks + 2 * t);
        av[ks][1] = *reinterpret_cast<const uint32_t *>(wv + g * GC + 16 * ks + 8 + 2 * t);
    }
    const uint32_t aq = pack_bf16x2(s_q[g * D + 2 * t], s_q[g * D + 2 * t + 1]);
    const float scale = 1.0f / sqrtf((float)D);

    const int s_begin = split * rows_per_split, s_end = min(S, s_begin + rows_per_split);
    const int ntile = (s_end - s_begin + 15) / 16;
    const __nv_bfloat16 *xb = x + (int64_t)b * S * GC;
    const __nv_bfloat16 *mb = mask + (int64_t)b * S;

    auto load_tile = [&](int tile, int buf) {
        const int r0 = s_begin + tile * 16;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = lane + 32 * i, r = idx >> 3, c = idx & 7;
            const bool ok = r0 + r < s_end;
            cp_async16(smem_u32(&s_x[warp][buf][r * GC + swz8(r, c) * 8]), xb + (int64_t)(ok ? r0 + r : s_begin) * GC + c * 8,
                       ok ? 16 : 0);
        }
    };

    float m_run = -INFINITY, l_run = 0.f, wa[4] = {0.f, 0.f, 0.f, 0.f};
    int it = 0;
    if (warp < ntile) load_tile(warp, 0);
    cp_async_commit();
    for (int tile = warp; tile < ntile; tile += NW, ++it) {
        const int buf = it & 1;
        if (tile + NW < ntile) load_tile(tile + NW, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();

        float kacc[4] = {0.f, 0.f, 0.f, 0.f}, v0[4] = {0.f, 0.f, 0.f, 0.f}, v1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t a[4];
            const int r = lane & 15, c = ks * 2 + (lane >> 4);
            ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(&s_x[warp][buf][r * GC + swz8(r, c) * 8]));
            mma_bf16_16816(kacc, a, bk[ks][0], bk[ks][1]);
            const uint32_t wvf[4] = {av[ks][0], 0u, av[ks][1], 0u};
            mma_bf16_16816(v0, wvf, a[0], a[2]);       // rows 0..7 of the tile
            mma_bf16_16816(v1, wvf, a[1], a[3]);       // rows 8..15
        }
        // logits of head g for rows 2t, 2t+1 (l0) and 8+2t, 9+2t (l1); k is stored as bf16 by the reference
        float l0[4] = {0.f, 0.f, 0.f, 0.f}, l1[4] = {0.f, 0.f, 0.f, 0.f};
        mma_bf16_1688(l0, aq, 0u, pack_bf16x2(kacc[0], kacc[1]));
        mma_bf16_1688(l1, aq, 0u, pack_bf16x2(kacc[2], kacc[3]));
        const int r0 = s_begin + tile * 16;
        const int rows[4] = {r0 + 2 * t, r0 + 2 * t + 1, r0 + 8 + 2 * t, r0 + 9 + 2 * t};
        const float lg[4] = {l0[0], l0[1], l1[0], l1[1]};
        float xv[4];
        float tmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool ok = rows[i] < s_end;
            const float mbias = ok ? fmaf(__bfloat162float(mb[ok ? rows[i] : s_begin]), 1e9f, -1e9f) : -INFINITY;
            xv[i] = rbf(lg[i]) * scale + mbias;
            tmax = fmaxf(tmax, xv[i]);
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m_run, tmax);
        const float corr = __expf(m_run - m_new);      // first tile: exp(-inf) = 0
        m_run = m_new;
        float pv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pv[i] = __expf(xv[i] - m_new);
        l_run = l_run * corr + (pv[0] + pv[1] + pv[2] + pv[3]);
        wa[0] *= corr;
        wa[1] *= corr;
        const uint32_t pa[4] = {pack_bf16x2(pv[0], pv[1]), 0u, pack_bf16x2(pv[2], pv[3]), 0u};
        mma_bf16_16816(wa, pa, pack_bf16x2(v0[0], v0[1]), pack_bf16x2(v1[0], v1[1]));
        __syncwarp();
    }
    cp_async_wait<0>();

    // merge: row sums across the quad, then the per-warp states across the block
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (t == 0) {
        s_m[warp][g] = m_run;
        s_part[warp][g][0] = l_run;
    }
    s_part[warp][g][1 + 2 * t] = wa[0];
    s_part[warp][g][2 + 2 * t] = wa[1];
    __syncthreads();
    float *dst = sc.core + ((int64_t)b * sc.nsplit + split) * H * (2 + D);
    for (int i = tid; i < H * (1 + D); i += CORE_THREADS) {
        const int h = i / (1 + D), j = i % (1 + D);
        float mx = s_m[0][h];
        for (int w = 1; w < NW; ++w) mx = fmaxf(mx, s_m[w][h]);
        float acc = 0.f;
        for (int w = 0; w < NW; ++w) {
            const float f = (s_m[w][h] == -INFINITY) ? 0.f : __expf(s_m[w][h] - mx);
            acc += s_part[w][h][j] * f;
        }
        dst[h * (2 + D) + 1 + j] = acc;
        if (j == 0) dst[h * (2 + D)] = mx;
    }
}

// ---- out -----------------------------------------------------------------------------------------
struct OutSmem {
    __nv_bfloat16 x[OUT_ROWS * GC];   // activations tile, later reused to stage the output tile
    __nv_bfloat16 wg[GC * GC];
    __nv_bfloat16 wo[GC * GC];
    float wa[GC];
    float bg[GC];
    float bo[GC];
};

template <int H, int D>
__global__ void __launch_bounds__(256) global_out_kernel(const __nv_bfloat16 *__restrict__ x,
                                                         const __nv_bfloat16 *__restrict__ wg,
                                                         const float *__restrict__ bg,
                                                         const __nv_bfloat16 *__restrict__ wo,
                                                         const float *__restrict__ bo, __nv_bfloat16 *__restrict__ out,
                                                         int64_t out_row_stride, Scratch sc, int b0, int S)
{
    __shared__ __align__(128) OutSmem sm;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = b0 + blockIdx.y;
    const int ntiles = (S + OUT_ROWS - 1) / OUT_ROWS;

    for (int idx = tid; idx < GC * 8; idx += 256) {
        const int r = idx >> 3, c = idx & 7;
        cp_async16(smem_u32(&sm.wg[r * GC + swz8(r, c) * 8]), wg + r * GC + c * 8, 16);
        cp_async16(smem_u32(&sm.wo[r * GC + swz8(r, c) * 8]), wo + r * GC + c * 8, 16);
    }
    cp_async_commit();
    if (tid < GC) {
        // combine the split softmax states of this column into wa (bf16-rounded, as the reference stores it)
        const int h = tid / D, d = tid % D;
        float mx = -INFINITY;
        for (int sp = 0; sp < sc.nsplit; ++sp)
            mx = fmaxf(mx, sc.core[(((int64_t)b * sc.nsplit + sp) * H + h) * (2 + D)]);
        float l = 0.f, a = 0.f;
        for (int sp = 0; sp < sc.nsplit; ++sp) {
            const float *pp = sc.core + (((int64_t)b * sc.nsplit + sp) * H + h) * (2 + D);
            const float f = (pp[0] == -INFINITY) ? 0.f : __expf(pp[0] - mx);
            l += pp[1] * f;
            a += pp[2 + d] * f;
        }
        sm.wa[tid] = rbf(a / l);
        sm.bg[tid] = bg[tid];
        sm.bo[tid] = bo[tid];
    }
    const int g = lane >> 2, t = lane & 3;
    // the weights and wa stay resident; the CTA walks several 128-row tiles of this column
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int s0 = tile * OUT_ROWS;
    const __nv_bfloat16 *xb = x + ((int64_t)b * S + s0) * GC;
    for (int idx = tid; idx < OUT_ROWS * 8; idx += 256) {
        const int r = idx >> 3, c = idx & 7;
        const bool ok = s0 + r < S;
        cp_async16(smem_u32(&sm.x[r * GC + swz8(r, c) * 8]), xb + (int64_t)(ok ? r : 0) * GC + c * 8, ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // gate = x . Wg^T : 16 rows x 64 per warp
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4];
        {
            const int r = warp * 16 + (lane & 15), c = ks * 2 + (lane >> 4);
            ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(&sm.x[r * GC + swz8(r, c) * 8]));
        }
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            uint32_t b0r, b1r, b2r, b3r;
            const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3), c = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b0r, b1r, b2r, b3r, smem_u32(&sm.wg[r * GC + swz8(r, c) * 8]));
            mma_bf16_16816(acc[np * 2], a, b0r, b1r);
            mma_bf16_16816(acc[np * 2 + 1], a, b2r, b3r);
        }
    }
    // gated = bf16(sigmoid(bf16(gate + bg)) * wa), packed as the A operand of the output product
    uint32_t pf[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const int c = nt * 8 + 2 * t;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int cc = c + (e & 1);
            const float gate = rbf(acc[nt][e] + sm.bg[cc]);
            v[e] = (1.0f / (1.0f + __expf(-gate))) * sm.wa[cc];
        }
        pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(v[0], v[1]);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(v[2], v[3]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            uint32_t b0r, b1r, b2r, b3r;
            const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3), c = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b0r, b1r, b2r, b3r, smem_u32(&sm.wo[r * GC + swz8(r, c) * 8]));
            mma_bf16_16816(acc[np * 2], pf[ks], b0r, b1r);
            mma_bf16_16816(acc[np * 2 + 1], pf[ks], b2r, b3r);
        }
    }
    // stage the 16 x 64 result of this warp in its own rows of the x tile, then store 16-byte rows
    __syncwarp();
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const int c = nt * 8 + 2 * t;
        const int r0 = warp * 16 + g, r1 = r0 + 8;
        *reinterpret_cast<uint32_t *>(&sm.x[r0 * GC + swz8(r0, nt) * 8 + 2 * t]) =
            pack_bf16x2(acc[nt][0] + sm.bo[c], acc[nt][1] + sm.bo[c + 1]);
        *reinterpret_cast<uint32_t *>(&sm.x[r1 * GC + swz8(r1, nt) * 8 + 2 * t]) =
            pack_bf16x2(acc[nt][2] + sm.bo[c], acc[nt][3] + sm.bo[c + 1]);
    }
    __syncwarp();
    __nv_bfloat16 *ob = out + ((int64_t)b * S + s0) * out_row_stride;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = lane + i * 32;
        const int r = warp * 16 + (idx >> 3), c = idx & 7;
        if (s0 + r < S) {
            const uint4 val = *reinterpret_cast<const uint4 *>(&sm.x[r * GC + swz8(r, c) * 8]);
            *reinterpret_cast<uint4 *>(ob + (int64_t)r * out_row_stride + c * 8) = val;
        }
    }
    __syncthreads();   // the tile buffer is reloaded in the next iteration
    }
}

struct Plan {
    int group;      // batch columns per L2-resident group
    int nsplit;     // row slices per column in pool/core
    int rows_per_split;
};

Plan make_plan(int B, int S)
{
    Plan p;
    const int64_t col_bytes = (int64_t)S * GC * 2;
    const int64_t l2_budget = (int64_t)32 << 20;
    p.group = (int)std::max<int64_t>(1, std::min<int64_t>(B, l2_budget / std::max<int64_t>(col_bytes, 1)));
    // The row slices of a column depend on S alone, so a column's partial sums are formed and
    // merged in the same order whatever the batch it arrives in.
    const int ns = std::max(1, std::min(32, S / 384));
    p.nsplit = ns;
    p.rows_per_split = (S + ns - 1) / ns;
    return p;
}

template <int H, int D>
void run_global(cudaStream_t stream, const void *x, const void *mask, const void *wq, const void *wk, const void *wv,
                const void *wg, const float *bg, const void *wo, const float *bo, void *out, int64_t out_row_stride,
                void *scratch, int B, int S)
{
    const Plan pl = make_plan(B, S);
    Scratch sc;
    sc.nsplit = pl.nsplit;
    sc.pool = (float *)scratch;
    sc.core = sc.pool + (int64_t)B * pl.nsplit * (GC + 1);
    for (int b0 = 0; b0 < B; b0 += pl.group) {
        const int nb = std::min(pl.group, B - b0);
        dim3 g1((unsigned)pl.nsplit, (unsigned)nb);
        {
            KernelTimer timer__("global_pool", stream);
        global_pool_kernel<<<g1, POOL_THREADS, 0, stream>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)mask, sc,
                                                            b0, S, pl.rows_per_split);
        }
        {
            KernelTimer timer__("global_core", stream);
        if (H == 8 && D == 8)
            global_core_mma_kernel<<<g1, CORE_THREADS, 0, stream>>>(
                (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)mask, (const __nv_bfloat16 *)wq,
                (const __nv_bfloat16 *)wk, (const __nv_bfloat16 *)wv, sc, b0, S, pl.rows_per_split);
        else
            global_core_kernel<H, D><<<g1, CORE_THREADS, 0, stream>>>(
                (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)mask, (const __nv_bfloat16 *)wq,
                (const __nv_bfloat16 *)wk, (const __nv_bfloat16 *)wv, sc, b0, S, pl.rows_per_split);
        }
        const int out_tiles = (S + OUT_ROWS - 1) / OUT_ROWS;
        dim3 g3((unsigned)((out_tiles + 3) / 4), (unsigned)nb);
        {
            KernelTimer timer__("global_out", stream);
        global_out_kernel<H, D><<<g3, 256, 0, stream>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)wg, bg,
                                                        (const __nv_bfloat16 *)wo, bo, (__nv_bfloat16 *)out,
                                                        out_row_stride, sc, b0, S);
        }
        count_launch(3);
    }
}

}  // namespace

size_t global_attention_scratch_bytes(int B, int S, int H, int D)
{
    const Plan pl = make_plan(B, S);
    return ((size_t)B * pl.nsplit * (GC + 1) + (size_t)B * pl.nsplit * H * (2 + D)) * sizeof(float);
}

bool launch_global_attention_bf16(cudaStream_t stream, const void *x, const void *mask, const void *wq,
                                  const void *wk, const void *wv, const void *wg, const float *bg, const void *wo,
                                  const float *bo, void *out, int64_t out_row_stride, void *scratch, int B, int S,
                                  int H, int D)
{
    if (H * D != GC || (out_row_stride % 8) != 0 || B > 65535) return false;
#define KUTACC_GLOBAL_CASE(HH, DD)                                                                              \
    if (H == HH && D == DD) {                                                                                   \
        run_global<HH, DD>(stream, x, mask, wq, wk, wv, wg, bg, wo, bo, out, out_row_stride, scratch, B, S);   \
        return true;                                                                                            \
    }
    KUTACC_GLOBAL_CASE(8, 8)
    KUTACC_GLOBAL_CASE(4, 16)
    KUTACC_GLOBAL_CASE(16, 4)
    KUTACC_GLOBAL_CASE(2, 32)
    KUTACC_GLOBAL_CASE(1, 64)
#undef KUTACC_GLOBAL_CASE
    return false;
}

}  // namespace dev
}  // namespace kutacc

// ---------------------------------------------------------------------------------------------------
// Global attention without any allocation.
//
// Some hosts of this library may not allocate device memory when they call an operator: an inference
// server that handed all of HBM to its own pool at start-up (cudaMalloc then fails or fragments the
// pool), a latency-critical loop that cannot accept the device-wide synchronisation cudaMalloc and
// cudaFree imply, or a process running under a fixed memory quota. For them this entry point runs the
// same three kernels as kutacc_af2_global_attention with the split-softmax scratch placed in a
// file-scope device array instead of the library's grow-only workspace. Inputs and outputs are plain
// device pointers supplied by the caller; nothing is staged, and no CUDA allocation routine is called.
//
// The array is part of the library image: every GPU that loads the library holds
// KUTACC_B200_NOALLOC_SCRATCH_BYTES (4 MiB) of it until the process exits. The first call on each
// device resolves the array's device address (cudaGetSymbolAddress); make that first call outside of
// any stream capture. All calls share the one array and it keeps whatever the previous call left, so
// two calls that overlap on the GPU (different streams, or different host threads) race; every slot a
// call reads is written earlier in that same call, so nothing has to be cleared between calls.
// ---------------------------------------------------------------------------------------------------
#define KUTACC_B200_NOALLOC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char g_noalloc_scratch[KUTACC_B200_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void *g_noalloc_scratch_addr[kMaxDevices] = {};

// In host code the array's name is only a handle for the runtime, not an address a kernel could use:
// the device address has to be asked for, once per device, with that device current.
void *noalloc_scratch_for_current_device()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (g_noalloc_scratch_addr[dev] == nullptr) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        KUTACC_CHECK(e == cudaSuccess, "cudaGetSymbolAddress(static scratch): ", cudaGetErrorString(e));
        if (e != cudaSuccess) return nullptr;
        g_noalloc_scratch_addr[dev] = ptr;
    }
    return g_noalloc_scratch_addr[dev];
}
}  // namespace

extern "C" int kutacc_b200_global_attention_noalloc(const void *q_data, const void *q_mask, const void *query_w,
                                                    const void *key_w, const void *value_w, const void *gating_w,
                                                    const float *gating_b, const void *output_w,
                                                    const float *output_b, void *out, int64_t out_row_stride,
                                                    int64_t batch, int64_t seq_len, int64_t nheads, int64_t head_size,
                                                    void *cuda_stream)
{
    using namespace kutacc;
    if (kutacc_check_err_set) return -1;
    KUTACC_CHECK(q_data && q_mask && query_w && key_w && value_w && gating_w && gating_b && output_w && output_b && out,
                 "kutacc_b200_global_attention_noalloc: nullptr error");
    KUTACC_CHECK(batch > 0 && seq_len > 0 && nheads > 0 && head_size > 0 && nheads * head_size == 64 &&
                     batch <= 65535 && seq_len <= INT32_MAX / 64 && out_row_stride >= 64 && out_row_stride % 8 == 0,
                 "kutacc_b200_global_attention_noalloc: invalid size (64 channels, batch <= 65535, out row stride a "
                 "multiple of 8 required)");
    if (kutacc_check_err_set) return -1;
    // the kernels read activations and weights with 4- to 16-byte vector loads
    KUTACC_CHECK((((uintptr_t)q_data | (uintptr_t)out | (uintptr_t)gating_w | (uintptr_t)output_w | (uintptr_t)query_w |
                   (uintptr_t)key_w | (uintptr_t)value_w) & 15u) == 0 &&
                     (((uintptr_t)gating_b | (uintptr_t)output_b) & 3u) == 0 && ((uintptr_t)q_mask & 1u) == 0,
                 "kutacc_b200_global_attention_noalloc: q_data, out and the five weights must be 16-byte aligned");
    const size_t need = dev::global_attention_scratch_bytes((int)batch, (int)seq_len, (int)nheads, (int)head_size);
    KUTACC_CHECK(need <= KUTACC_B200_NOALLOC_SCRATCH_BYTES, "kutacc_b200_global_attention_noalloc: this shape needs ",
                 need, " bytes of scratch, the static scratch holds ", (size_t)KUTACC_B200_NOALLOC_SCRATCH_BYTES,
                 " (use kutacc_af2_global_attention for larger batches)");
    if (kutacc_check_err_set) return -1;
    void *scratch = noalloc_scratch_for_current_device();
    if (scratch == nullptr) {
        KUTACC_CHECK(false, "kutacc_b200_global_attention_noalloc: static scratch is not available on this device");
        return -1;
    }
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const bool ok = dev::launch_global_attention_bf16(stream, q_data, q_mask, query_w, key_w, value_w, gating_w,
                                                      gating_b, output_w, output_b, out, out_row_stride, scratch,
                                                      (int)batch, (int)seq_len, (int)nheads, (int)head_size);
    KUTACC_CHECK(ok, "kutacc_b200_global_attention_noalloc: no kernel for nheads=", nheads, " head_size=", head_size);
    const cudaError_t e = cudaGetLastError();
    KUTACC_CHECK(e == cudaSuccess, "kernel launch failed: ", cudaGetErrorString(e));
    return kutacc_check_err_set ? -1 : 0;
}
