// Shape-agnostic kernels: any channel count, head size and sequence length, bf16 or fp32 storage,
// fp32 arithmetic on the CUDA cores. They cover what the tensor-core kernels do not (fp32 tensors,
// head sizes other than 16/32/64, channel counts that are not multiples of 64, unaligned pair-bias
// strides) so that every shape the reference accepts has a device path.
//
// Same math as src/attention/gating_attention.cpp:47-157 with the rounding points of the storage
// type (none for fp32).
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

#include <algorithm>

namespace kutacc {
namespace dev {

namespace {

template <typename T>
__device__ __forceinline__ float ld(const T *p);
template <>
__device__ __forceinline__ float ld<float>(const float *p)
{
    return *p;
}
template <>
__device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16 *p)
{
    return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void st(T *p, float v);
template <>
__device__ __forceinline__ void st<float>(float *p, float v)
{
    *p = v;
}
template <>
__device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16 *p, float v)
{
    *p = __float2bfloat16_rn(v);
}
template <typename T>
__device__ __forceinline__ float round_store(float v);
template <>
__device__ __forceinline__ float round_store<float>(float v)
{
    return v;
}
template <>
__device__ __forceinline__ float round_store<__nv_bfloat16>(float v)
{
    return __bfloat162float(__float2bfloat16_rn(v));
}

// ---- GEMM: 64 x 64 tile, 16-wide K slabs, 4 x 4 outputs per thread ------------------------------
constexpr int GT = 64, GK = 16;

template <typename T>
__global__ void __launch_bounds__(256) gemm_generic_kernel(const T *__restrict__ a, int64_t lda,
                                                           const T *__restrict__ w, int64_t ldw,
                                                           const float *__restrict__ bias, float beta, T *c,
                                                           int64_t ldc, int64_t M, int64_t N, int64_t K)
{
    __shared__ float sa[GK][GT + 1];
    __shared__ float sw[GK][GT + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t m0 = (int64_t)blockIdx.x * GT, n0 = (int64_t)blockIdx.y * GT;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < K; k0 += GK) {
        for (int i = threadIdx.x; i < GT * GK; i += 256) {
            const int r = i / GK, kk = i % GK;
            const int64_t gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            sa[kk][r] = (gm < M && gk < K) ? ld(a + gm * lda + gk) : 0.f;
            sw[kk][r] = (gn < N && gk < K) ? ld(w + gn * ldw + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = sa[kk][ty * 4 + i];
                wv[i] = sw[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (beta != 0.f) v += beta * ld(c + m * ldc + n);
            if (bias) v += bias[n];
            st(c + m * ldc + n, v);
        }
    }
}

// ---- fp32 GEMM on tensor cores with error compensation ("3xTF32") -------------------------------------
// Each fp32 operand is split into a tf32 head and a tf32 tail (x = hi + lo, |lo| <= 2^-11 |x|); the product
// is accumulated as hi*hi + hi*lo + lo*hi in fp32 (the lo*lo term, 2^-22 relative, is dropped), which keeps
// the result within a few fp32 ulps of a plain fp32 GEMM at a third of the tf32 tensor rate.
// 128 x 128 x 32 tiles, 8 warps (4 x 2), cp.async double buffering, rows padded to 36 floats so that the
// fragment loads (row g, column t) touch 32 different banks.
constexpr int TM = 128, TN = 128, TK = 32, TPAD = 36;
constexpr int T_STAGE_FLOATS = (TM + TN) * TPAD;
constexpr int T_SMEM_BYTES = 2 * T_STAGE_FLOATS * 4;

__device__ __forceinline__ uint32_t to_tf32(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32_1688(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256) gemm_tf32x3_kernel(const float *__restrict__ a, int64_t lda,
                                                          const float *__restrict__ w, int64_t ldw,
                                                          const float *__restrict__ bias, float *__restrict__ c,
                                                          int64_t ldc, int64_t M, int64_t N, int64_t K)
{
    extern __shared__ __align__(16) float t_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp >> 1, wn = warp & 1;                   // warp tile: rows wm*32.., columns wn*64..
    const int64_t m0 = (int64_t)blockIdx.x * TM, n0 = (int64_t)blockIdx.y * TN;
    const uint32_t smem0 = smem_u32(t_smem);
    auto load_stage = [&](int stage, int64_t k0) {
        const uint32_t sa = smem0 + stage * T_STAGE_FLOATS * 4, sw = sa + TM * TPAD * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256, r = idx >> 3, ch = idx & 7;
            const bool oka = m0 + r < M, okw = n0 + r < N;
            cp_async16(sa + (r * TPAD + ch * 4) * 4, a + (oka ? m0 + r : 0) * lda + k0 + ch * 4, oka ? 16 : 0);
            cp_async16(sw + (r * TPAD + ch * 4) * 4, w + (okw ? n0 + r : 0) * ldw + k0 + ch * 4, okw ? 16 : 0);
        }
        cp_async_commit();
    };
    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
    const int nk = (int)(K / TK);
    load_stage(0, 0);
    for (int kc = 0; kc < nk; ++kc) {
        if (kc + 1 < nk) load_stage((kc + 1) & 1, (int64_t)(kc + 1) * TK);
        else cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const float *sa = t_smem + (kc & 1) * T_STAGE_FLOATS, *sw = sa + TM * TPAD;
#pragma unroll
        for (int k8 = 0; k8 < TK / 8; ++k8) {
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                const float *p0 = sa + (wm * 32 + mt * 16 + g) * TPAD + k8 * 8 + t;
                const float v[4] = {p0[0], p0[8 * TPAD], p0[4], p0[8 * TPAD + 4]};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    ahi[mt][e] = to_tf32(v[e]);
                    alo[mt][e] = to_tf32(v[e] - __uint_as_float(ahi[mt][e]));
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float *q0 = sw + (wn * 64 + nt * 8 + g) * TPAD + k8 * 8 + t;
                const float b0 = q0[0], b1 = q0[4];
                const uint32_t bh0 = to_tf32(b0), bh1 = to_tf32(b1);
                const uint32_t bl0 = to_tf32(b0 - __uint_as_float(bh0)), bl1 = to_tf32(b1 - __uint_as_float(bh1));
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    mma_tf32_1688(acc[mt][nt], alo[mt], bh0, bh1);     // small terms first
                    mma_tf32_1688(acc[mt][nt], ahi[mt], bl0, bl1);
                    mma_tf32_1688(acc[mt][nt], ahi[mt], bh0, bh1);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int64_t n = n0 + wn * 64 + nt * 8 + 2 * t;
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int64_t m = m0 + wm * 32 + mt * 16 + g + 8 * hrow;
                if (m >= M) continue;
#pragma unroll
                for (int e = 0; e < 2; ++e)
                    if (n + e < N) c[m * ldc + n + e] = acc[mt][nt][2 * hrow + e] + (bias ? bias[n + e] : 0.f);
            }
        }
}

// ---- attention: one warp per (b, h, query) --------------------------------------------------------
// Lanes split the keys for the logits (each lane a dot product over D) and split the head
// channels for P.V. Online softmax across 32-key chunks.
template <typename T, int DMAX>
__global__ void __launch_bounds__(128) attn_generic_kernel(const T *__restrict__ q, const T *__restrict__ k,
                                                           const T *__restrict__ v, const T *__restrict__ gate,
                                                           const T *__restrict__ bias, int64_t bias_stride0,
                                                           const T *__restrict__ nb, int64_t nb_stride_h,
                                                           int64_t nb_stride_q, T *__restrict__ avg, int B, int S,
                                                           int H, int D, float scale)
{
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (int64_t)B * H * S) return;
    const int i = (int)(row % S);
    const int h = (int)((row / S) % H);
    const int b = (int)(row / ((int64_t)S * H));
    const int C = H * D;
    const T *qi = q + ((int64_t)b * S + i) * C + h * D;
    const T *kb = k + (int64_t)b * S * C + h * D;
    const T *vb = v + (int64_t)b * S * C + h * D;
    const T *brow = bias + (int64_t)b * bias_stride0;
    const T *nbrow = nb ? nb + (int64_t)h * nb_stride_h + (int64_t)i * nb_stride_q : nullptr;

    constexpr int ND = DMAX / 32;  // output channels per lane
    float qreg[DMAX];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) qreg[d] = d < D ? ld(qi + d) : 0.f;
    float o[ND];
#pragma unroll
    for (int j = 0; j < ND; ++j) o[j] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    for (int j0 = 0; j0 < S; j0 += 32) {
        const int j = j0 + lane;
        float x = -INFINITY;
        if (j < S) {
            const T *kj = kb + (int64_t)j * C;
            float acc = 0.f;
#pragma unroll
            for (int d = 0; d < DMAX; ++d)
                if (d < D) acc = fmaf(qreg[d], ld(kj + d), acc);
            acc = round_store<T>(acc);                       // logits are stored in the tensor type
            x = acc * scale + ld(brow + j);
            if (nbrow) x = x + ld(nbrow + j);
        }
        float mx = x;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        const float m_new = fmaxf(m_run, mx);
        const float corr = __expf(m_run - m_new);
        const float pj = (j < S) ? __expf(x - m_new) : 0.f;
        float ps = pj;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, s);
        l_run = l_run * corr + ps;
        m_run = m_new;
#pragma unroll
        for (int jj = 0; jj < ND; ++jj) o[jj] *= corr;
        const int lim = min(32, S - j0);
        for (int kk = 0; kk < lim; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pj, kk);
            const T *vj = vb + (int64_t)(j0 + kk) * C;
#pragma unroll
            for (int jj = 0; jj < ND; ++jj) {
                const int d = jj * 32 + lane;
                if (d < D) o[jj] = fmaf(pk, ld(vj + d), o[jj]);
            }
        }
    }
    const float inv = 1.0f / l_run;
    const T *gi = gate + ((int64_t)b * S + i) * C + h * D;
    T *ai = avg + ((int64_t)b * S + i) * C + h * D;
#pragma unroll
    for (int jj = 0; jj < ND; ++jj) {
        const int d = jj * 32 + lane;
        if (d < D) {
            const float wa = round_store<T>(o[jj] * inv);
            const float sg = 1.0f / (1.0f + __expf(-ld(gi + d)));
            st(ai + d, wa * sg);
        }
    }
}

// ---- pair-bias projection -------------------------------------------------------------------------
// One warp per (row, key) pair reads z[r, k, :] with 16-byte loads where possible and reduces the
// H dot products with shuffles; writes nb[h, r, k]. Bandwidth bound: reads R*Nk*Cz elements once.
template <typename T, int HMAX>
__global__ void __launch_bounds__(256) pair_bias_kernel(const T *__restrict__ z, const T *__restrict__ wb,
                                                        T *__restrict__ nb, int64_t nb_head_stride, int64_t pos_stride,
                                                        int64_t R, int64_t Nk, int Cz, int H)
{
    extern __shared__ float swb[];  // [H][Cz]
    for (int i = threadIdx.x; i < H * Cz; i += blockDim.x) swb[i] = ld(wb + i);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t pos = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); pos < R * Nk; pos += nwarps) {
        const T *zr = z + pos * Cz;
        float acc[HMAX];
#pragma unroll
        for (int hh = 0; hh < HMAX; ++hh) acc[hh] = 0.f;
        for (int c = lane; c < Cz; c += 32) {
            const float zv = ld(zr + c);
#pragma unroll
            for (int hh = 0; hh < HMAX; ++hh)
                if (hh < H) acc[hh] = fmaf(zv, swb[hh * Cz + c], acc[hh]);
        }
#pragma unroll
        for (int hh = 0; hh < HMAX; ++hh) {
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) acc[hh] += __shfl_xor_sync(0xffffffffu, acc[hh], s);
        }
        if (lane == 0) {
            const int64_t r = pos / Nk, kk = pos % Nk;
#pragma unroll
            for (int hh = 0; hh < HMAX; ++hh)
                if (hh < H) st(nb + hh * nb_head_stride + (r * Nk + kk) * pos_stride, acc[hh]);
        }
    }
}

// bf16 fast variant: Cz/8 lanes share one (row, key) position, each lane fetches 8 channels with one
// 128-bit load; partial dot products are combined with xor shuffles inside the lane group.
template <int HMAX>
__global__ void __launch_bounds__(256) pair_bias_vec_kernel(const __nv_bfloat16 *__restrict__ z,
                                                            const __nv_bfloat16 *__restrict__ wb,
                                                            __nv_bfloat16 *__restrict__ nb, int64_t nb_head_stride,
                                                            int64_t pos_stride, int64_t R, int64_t Nk, int Cz, int H,
                                                            int lanes_per_pos)
{
    const int sub = threadIdx.x % lanes_per_pos;
    // this lane's 8 channels of every head's weight row stay in registers for the whole kernel
    float wreg[HMAX][8];
#pragma unroll
    for (int hh = 0; hh < HMAX; ++hh)
#pragma unroll
        for (int i = 0; i < 8; ++i) wreg[hh][i] = hh < H ? __bfloat162float(wb[hh * Cz + sub * 8 + i]) : 0.f;
    const int64_t pos_per_block = blockDim.x / lanes_per_pos;
    const int64_t total = R * Nk;
    // the loop bound depends on the block only, so whole warps stay together for the shuffles
    for (int64_t base = (int64_t)blockIdx.x * pos_per_block; base < total; base += (int64_t)gridDim.x * pos_per_block) {
        const int64_t pos = base + threadIdx.x / lanes_per_pos;
        const bool live = pos < total;
        float acc[HMAX];
#pragma unroll
        for (int hh = 0; hh < HMAX; ++hh) acc[hh] = 0.f;
        if (live) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(z + pos * Cz) + sub);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            float zv[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                zv[2 * i] = bf16lo_to_f32(w[i]);
                zv[2 * i + 1] = bf16hi_to_f32(w[i]);
            }
#pragma unroll
            for (int hh = 0; hh < HMAX; ++hh) {
                if (hh < H) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[hh] = fmaf(zv[i], wreg[hh][i], acc[hh]);
                }
            }
        }
#pragma unroll
        for (int hh = 0; hh < HMAX; ++hh) {
            for (int s = lanes_per_pos >> 1; s > 0; s >>= 1) acc[hh] += __shfl_xor_sync(0xffffffffu, acc[hh], s);
        }
        if (live && sub == 0) {
#pragma unroll
            for (int hh = 0; hh < HMAX; ++hh)
                if (hh < H) nb[hh * nb_head_stride + pos * pos_stride] = __float2bfloat16_rn(acc[hh]);
        }
    }
}

// bf16 pair bias on tensor cores: a CTA streams 128-position tiles of z through a cp.async ring (16-byte
// chunks, swizzled by row), each warp multiplies its 16 positions by Wb^T (heads padded to 8) with
// mma.sync m16n8k16 and writes nb[h, pos]. Bandwidth bound: z is read once, 128-bit loads.
// With LN the weights are LayerNorm-folded (ln_fold.cu) and a position's result is rstd * (acc - mean * s[h]) + t[h].
template <int CZ, bool LN>
__global__ void __launch_bounds__(256) pair_bias_mma_kernel(const __nv_bfloat16 *__restrict__ z,
                                                            const __nv_bfloat16 *__restrict__ wb,
                                                            __nv_bfloat16 *__restrict__ nb, int64_t nb_head_stride,
                                                            int64_t total, int H, const float2 *__restrict__ stats,
                                                            const float *__restrict__ ln_s, const float *__restrict__ ln_t,
                                                            int64_t nk, int64_t nb_row_stride)
{
    constexpr int ROWB = CZ * 2, CHUNKS = ROWB / 16, TP = 128, STAGES = 3, STAGE_BYTES = TP * ROWB;
    extern __shared__ __align__(128) unsigned char pb_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    uint32_t bf[CZ / 16][2];
#pragma unroll
    for (int ks = 0; ks < CZ / 16; ++ks) {
        bf[ks][0] = g < H ? *reinterpret_cast<const uint32_t *>(wb + g * CZ + ks * 16 + 2 * t) : 0u;
        bf[ks][1] = g < H ? *reinterpret_cast<const uint32_t *>(wb + g * CZ + ks * 16 + 8 + 2 * t) : 0u;
    }
    const int64_t ntiles = (total + TP - 1) / TP;
    const uint32_t smem0 = smem_u32(pb_smem);
    auto load_tile = [&](int64_t tile, int stage) {
        if (tile < ntiles) {
#pragma unroll
            for (int i = 0; i < TP * CHUNKS / 256; ++i) {
                const int idx = tid + i * 256, r = idx / CHUNKS, c = idx % CHUNKS;
                const int64_t pos = tile * TP + r;
                const bool ok = pos < total;
                cp_async16(smem0 + stage * STAGE_BYTES + r * ROWB + ((c ^ (r & 7)) << 4), z + (ok ? pos : 0) * CZ + c * 8,
                           ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };
    int64_t tile = blockIdx.x;
    for (int st = 0; st < STAGES - 1; ++st) load_tile(tile + (int64_t)st * gridDim.x, st);
    for (int it = 0; tile < ntiles; tile += gridDim.x, ++it) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                       // tile `it` has landed; the stage refilled below is no longer read
        load_tile(tile + (int64_t)(STAGES - 1) * gridDim.x, (it + STAGES - 1) % STAGES);
        const uint32_t base = smem0 + (it % STAGES) * STAGE_BYTES + warp * 16 * ROWB;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < CZ / 16; ++ks) {
            uint32_t a[4];
            const int r = lane & 15, c = ks * 2 + (lane >> 4);
            ldmatrix_x4(a[0], a[1], a[2], a[3], base + r * ROWB + ((c ^ (r & 7)) << 4));
            mma_bf16_16816(acc, a, bf[ks][0], bf[ks][1]);
        }
        const int64_t p0 = tile * TP + warp * 16 + g, p1 = p0 + 8;
        const int h0 = 2 * t, h1 = 2 * t + 1;
        if (LN) {
            const float s0 = h0 < H ? ln_s[h0] : 0.f, s1 = h1 < H ? ln_s[h1] : 0.f;
            const float t0 = h0 < H ? ln_t[h0] : 0.f, t1 = h1 < H ? ln_t[h1] : 0.f;
            const float2 st0 = stats[p0 < total ? p0 : 0], st1 = stats[p1 < total ? p1 : 0];
            acc[0] = fmaf(st0.y, acc[0] - st0.x * s0, t0);
            acc[1] = fmaf(st0.y, acc[1] - st0.x * s1, t1);
            acc[2] = fmaf(st1.y, acc[2] - st1.x * s0, t0);
            acc[3] = fmaf(st1.y, acc[3] - st1.x * s1, t1);
        }
        // position p = row * nk + key is stored at row * nb_row_stride + key (rows of the output may be further apart
        // than nk: a layout with the heads of a row next to each other, [rows, H, keys], for instance)
        const int64_t o0 = nb_row_stride == nk ? p0 : (p0 / nk) * nb_row_stride + p0 % nk;
        const int64_t o1 = nb_row_stride == nk ? p1 : (p1 / nk) * nb_row_stride + p1 % nk;
        if (p0 < total) {
            if (h0 < H) nb[h0 * nb_head_stride + o0] = __float2bfloat16_rn(acc[0]);
            if (h1 < H) nb[h1 * nb_head_stride + o0] = __float2bfloat16_rn(acc[1]);
        }
        if (p1 < total) {
            if (h0 < H) nb[h0 * nb_head_stride + o1] = __float2bfloat16_rn(acc[2]);
            if (h1 < H) nb[h1 * nb_head_stride + o1] = __float2bfloat16_rn(acc[3]);
        }
    }
    cp_async_wait<0>();
}

template <int CZ, bool LN = false>
bool launch_pair_bias_mma(cudaStream_t stream, const void *z, const void *wb, void *nb, int64_t nb_head_stride,
                          int64_t total, int H, const void *stats = nullptr, const float *ln_s = nullptr,
                          const float *ln_t = nullptr, int64_t nk = 1, int64_t nb_row_stride = 1)
{
    constexpr int SMEM = 3 * 128 * CZ * 2;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(pair_bias_mma_kernel<CZ, LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        configured = true;
    }
    const int64_t ntiles = (total + 127) / 128;
    const unsigned grid = (unsigned)std::min<int64_t>(ntiles, 148 * 2);
    pair_bias_mma_kernel<CZ, LN><<<grid, 256, SMEM, stream>>>((const __nv_bfloat16 *)z, (const __nv_bfloat16 *)wb,
                                                              (__nv_bfloat16 *)nb, nb_head_stride, total, H,
                                                              (const float2 *)stats, ln_s, ln_t, nk, nb_row_stride);
    return true;
}

__global__ void relu_bf16_kernel(__nv_bfloat16 *x, int64_t n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        if (__bfloat162float(x[i]) < 0.f) x[i] = __float2bfloat16_rn(0.f);
}

}  // namespace

// max(0, .) over a dense bf16 buffer (fallback of the transition operator when the fused epilogue is not available)
bool launch_relu_bf16(cudaStream_t stream, void *x, int64_t n)
{
    if (n <= 0) return true;
    relu_bf16_kernel<<<(unsigned)std::min<int64_t>((n + 255) / 256, 148 * 16), 256, 0, stream>>>((__nv_bfloat16 *)x, n);
    count_launch();
    return true;
}

bool launch_gemm_generic(cudaStream_t stream, ElemType t, const void *a, int64_t lda, const void *w, int64_t ldw,
                         const float *bias, float beta, void *c, int64_t ldc, int64_t M, int64_t N, int64_t K)
{
    if (t == kElemF32 && beta == 0.f && K % TK == 0 && lda % 4 == 0 && ldw % 4 == 0 &&
        (((uintptr_t)a | (uintptr_t)w) & 15u) == 0 && (N + TN - 1) / TN <= 65535) {
        static bool configured = false;
        if (!configured) {
            configured = cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM_BYTES) ==
                         cudaSuccess;
            cudaGetLastError();
        }
        if (configured) {
            KernelTimer timer__("gemm_tf32x3", stream);
            dim3 gridt((unsigned)((M + TM - 1) / TM), (unsigned)((N + TN - 1) / TN));
            gemm_tf32x3_kernel<<<gridt, 256, T_SMEM_BYTES, stream>>>((const float *)a, lda, (const float *)w, ldw, bias,
                                                                      (float *)c, ldc, M, N, K);
            count_launch();
            return true;
        }
    }
    dim3 grid((unsigned)((M + GT - 1) / GT), (unsigned)((N + GT - 1) / GT));
    if (grid.y > 65535) return false;
    KernelTimer timer__("gemm_generic", stream);
    if (t == kElemF32)
        gemm_generic_kernel<float><<<grid, 256, 0, stream>>>((const float *)a, lda, (const float *)w, ldw, bias, beta,
                                                            (float *)c, ldc, M, N, K);
    else
        gemm_generic_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16 *)a, lda,
                                                                    (const __nv_bfloat16 *)w, ldw, bias, beta,
                                                                    (__nv_bfloat16 *)c, ldc, M, N, K);
    count_launch();
    return true;
}

template <typename T>
static bool launch_attn_generic_t(cudaStream_t stream, const void *q, const void *k, const void *v, const void *gate,
                                  const void *bias, int64_t bias_stride0, const void *nb, int64_t nb_stride_h,
                                  int64_t nb_stride_q, void *avg, int B, int S, int H, int D, float scale)
{
    const int64_t rows = (int64_t)B * H * S;
    const unsigned grid = (unsigned)((rows + 3) / 4);
    KernelTimer timer__("attn_generic", stream);
#define KUTACC_ATTN_GENERIC(DMAX)                                                                                  \
    attn_generic_kernel<T, DMAX><<<grid, 128, 0, stream>>>((const T *)q, (const T *)k, (const T *)v, (const T *)gate, \
                                                           (const T *)bias, bias_stride0, (const T *)nb, nb_stride_h, \
                                                           nb_stride_q, (T *)avg, B, S, H, D, scale)
    if (D <= 32)
        KUTACC_ATTN_GENERIC(32);
    else if (D <= 64)
        KUTACC_ATTN_GENERIC(64);
    else if (D <= 128)
        KUTACC_ATTN_GENERIC(128);
    else
        return false;
#undef KUTACC_ATTN_GENERIC
    count_launch();
    return true;
}

bool launch_attn_generic(cudaStream_t stream, ElemType t, const void *q, const void *k, const void *v,
                         const void *gate, const void *bias, int64_t bias_stride0, const void *nb,
                         int64_t nb_stride_h, int64_t nb_stride_q, void *avg, int B, int S, int H, int D, float scale)
{
    if (t == kElemF32)
        return launch_attn_generic_t<float>(stream, q, k, v, gate, bias, bias_stride0, nb, nb_stride_h, nb_stride_q,
                                            avg, B, S, H, D, scale);
    return launch_attn_generic_t<__nv_bfloat16>(stream, q, k, v, gate, bias, bias_stride0, nb, nb_stride_h,
                                                nb_stride_q, avg, B, S, H, D, scale);
}

bool launch_pair_bias_ln(cudaStream_t stream, const void *z, const void *wb_folded, const void *stats, const float *ln_s,
                         const float *ln_t, void *nb, int64_t nb_head_stride, int64_t R, int64_t Nk, int Cz, int H)
{
    if (H > 8 || (Cz != 128 && Cz != 64) || ((uintptr_t)z % 16) != 0 || ((uintptr_t)wb_folded % 4) != 0) return false;
    KernelTimer timer__("pair_bias_ln", stream);
    const bool ok = Cz == 128 ? launch_pair_bias_mma<128, true>(stream, z, wb_folded, nb, nb_head_stride, R * Nk, H, stats, ln_s, ln_t)
                              : launch_pair_bias_mma<64, true>(stream, z, wb_folded, nb, nb_head_stride, R * Nk, H, stats, ln_s, ln_t);
    if (ok) count_launch();
    return ok;
}

bool launch_pair_bias(cudaStream_t stream, ElemType t, const void *z, const void *wb, void *nb,
                      int64_t nb_head_stride, int64_t pos_stride, int64_t R, int64_t Nk, int Cz, int H, int64_t nb_row_stride)
{
    if (nb_row_stride <= 0) nb_row_stride = Nk;
    if (H > 16 || (size_t)H * Cz * 4 > 48 * 1024) return false;
    KernelTimer timer__("pair_bias", stream);
    const int64_t pos = R * Nk;
    const unsigned grid = (unsigned)std::min<int64_t>((pos + 7) / 8, 148 * 16);
    const size_t smem = (size_t)H * Cz * 4;
    const int lanes = Cz / 8;
    const bool pow2 = lanes > 0 && (lanes & (lanes - 1)) == 0 && lanes <= 32 && Cz % 8 == 0;
    if (t == kElemBF16 && H <= 8 && pos_stride == 1 && ((uintptr_t)z % 16) == 0 && ((uintptr_t)wb % 4) == 0 &&
        (Cz == 128 || Cz == 64)) {
        const bool ok = Cz == 128 ? launch_pair_bias_mma<128>(stream, z, wb, nb, nb_head_stride, pos, H, nullptr, nullptr,
                                                              nullptr, Nk, nb_row_stride)
                                  : launch_pair_bias_mma<64>(stream, z, wb, nb, nb_head_stride, pos, H, nullptr, nullptr,
                                                             nullptr, Nk, nb_row_stride);
        if (ok) {
            count_launch();
            return true;
        }
    }
    if (nb_row_stride != Nk) return false;                   // only the tensor-core kernel writes rows that are apart
    if (t == kElemBF16 && pow2 && H <= 8 && ((uintptr_t)z % 16) == 0) {
        const int64_t ppb = 256 / lanes;
        const unsigned gridv = (unsigned)std::min<int64_t>((pos + ppb - 1) / ppb, 148 * 32);
        pair_bias_vec_kernel<8><<<gridv, 256, 0, stream>>>((const __nv_bfloat16 *)z, (const __nv_bfloat16 *)wb,
                                                              (__nv_bfloat16 *)nb, nb_head_stride, pos_stride, R, Nk, Cz, H, lanes);
        count_launch();
        return true;
    }
    if (t == kElemF32) {
        if (H <= 8)
            pair_bias_kernel<float, 8><<<grid, 256, smem, stream>>>((const float *)z, (const float *)wb, (float *)nb,
                                                                    nb_head_stride, pos_stride, R, Nk, Cz, H);
        else
            pair_bias_kernel<float, 16><<<grid, 256, smem, stream>>>((const float *)z, (const float *)wb, (float *)nb,
                                                                     nb_head_stride, pos_stride, R, Nk, Cz, H);
    } else {
        if (H <= 8)
            pair_bias_kernel<__nv_bfloat16, 8><<<grid, 256, smem, stream>>>(
                (const __nv_bfloat16 *)z, (const __nv_bfloat16 *)wb, (__nv_bfloat16 *)nb, nb_head_stride, pos_stride, R, Nk, Cz, H);
        else
            pair_bias_kernel<__nv_bfloat16, 16><<<grid, 256, smem, stream>>>(
                (const __nv_bfloat16 *)z, (const __nv_bfloat16 *)wb, (__nv_bfloat16 *)nb, nb_head_stride, pos_stride, R, Nk, Cz, H);
    }
    count_launch();
    return true;
}

}  // namespace dev
}  // namespace kutacc
