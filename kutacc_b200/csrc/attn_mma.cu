// Fused gated-attention core: logits, mask bias, pair bias, online softmax, P.V, sigmoid gate.
// The S x S logits never leave the SM.
//
// One CTA owns (batch row b, head h, a tile of NWARPS*16 queries). Each warp owns 16 query rows and
// walks the keys in tiles of 64: Q.K^T with mma.sync m16n8k16 into fp32 registers, biases added in
// the accumulator layout, running max / sum kept per row with quad shuffles, P re-packed in
// registers as the A operand of the P.V product. K, V, the pair-bias tile and the mask-bias slice
// of the next key tile are prefetched with cp.async while the current one is consumed.
//
// Arithmetic is done in the base-2 domain: q arrives pre-multiplied by log2(e)/sqrt(D) (folded
// into the projection epilogue), both biases are multiplied by log2(e) on the fly, and exp becomes a
// single ex2. This computes the same function as the reference loop
// (src/attention/gating_attention.cpp:97-147, src/softmax/softmax.h:22-43) without its bf16 round
// trips of the logits and probabilities through memory.
//
// A fully masked row (every key carries -1e9) stays uniform as in the reference: the fp32 sum
// logit + bias absorbs the logit, every entry equals the row max, and every probability is 1/S.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"

namespace kutacc {
namespace dev {

namespace {

constexpr int BN = 64;  // keys per tile
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
    const __nv_bfloat16 *q, *k, *v;   // [B, H, S, D]
    const __nv_bfloat16 *gate;        // [B, S, H*D]
    const __nv_bfloat16 *bias;        // [B, S] (row stride bias_stride0)
    const __nv_bfloat16 *nb;          // [H, S, S] or null
    __nv_bfloat16 *avg;               // [B, S, H*D]
    int64_t bias_stride0, nb_stride_h, nb_stride_q;
    int S, H;
};

// chunk swizzle for tiles whose rows hold CPR 16-byte chunks (CPR = 2, 4 or 8)
template <int CPR>
__device__ __forceinline__ int swz(int row, int chunk)
{
    constexpr int SH = CPR == 8 ? 0 : (CPR == 4 ? 1 : 2);
    return chunk ^ ((row >> SH) & (CPR - 1));
}

template <int D, int NWARPS>
struct Smem {
    static constexpr int BM = NWARPS * 16;
    __nv_bfloat16 q[BM * D];
    __nv_bfloat16 k[2][BN * D];
    __nv_bfloat16 v[2][BN * D];
    __nv_bfloat16 nb[2][BM * BN];
    float mb[2][BN];
};

template <int D, int NWARPS, bool HAS_NB>
__global__ void __launch_bounds__(NWARPS * 32) attn_core_kernel(const AttnParams p)
{
    constexpr int BM = NWARPS * 16;
    constexpr int CPR = D / 8;       // 16-byte chunks per q/k/v row
    constexpr int KS = D / 16;       // k16 steps of Q.K^T
    constexpr int NT_S = BN / 8;     // n8 tiles of the logits
    constexpr int NT_O = D / 8;      // n8 tiles of the output
    constexpr int THREADS = NWARPS * 32;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem<D, NWARPS> &sm = *reinterpret_cast<Smem<D, NWARPS> *>(smem_raw);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int S = p.S;
    const int q0 = blockIdx.x * BM;
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int64_t bh = (int64_t)b * p.H + h;
    const __nv_bfloat16 *__restrict__ qg = p.q + bh * S * D;
    const __nv_bfloat16 *__restrict__ kg = p.k + bh * S * D;
    const __nv_bfloat16 *__restrict__ vg = p.v + bh * S * D;
    const __nv_bfloat16 *__restrict__ biasg = p.bias + (int64_t)b * p.bias_stride0;
    const __nv_bfloat16 *__restrict__ nbg = HAS_NB ? p.nb + (int64_t)h * p.nb_stride_h : nullptr;

    auto load_tile = [&](int stage, int kt) {
        const int k0 = kt * BN;
        for (int idx = tid; idx < BN * CPR; idx += THREADS) {
            const int r = idx / CPR, c = idx % CPR;
            const bool ok = (k0 + r) < S;
            const int64_t off = (int64_t)(ok ? k0 + r : 0) * D + c * 8;
            const int so = r * D + swz<CPR>(r, c) * 8;
            cp_async16(smem_u32(&sm.k[stage][so]), kg + off, ok ? 16 : 0);
            cp_async16(smem_u32(&sm.v[stage][so]), vg + off, ok ? 16 : 0);
        }
        if (HAS_NB) {
            for (int idx = tid; idx < BM * 8; idx += THREADS) {
                const int r = idx >> 3, c = idx & 7;
                const int col = k0 + c * 8;
                int bytes = (q0 + r < S) ? (S - col) * 2 : 0;
                bytes = bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes);
                const __nv_bfloat16 *src = nbg + (int64_t)(bytes ? q0 + r : 0) * p.nb_stride_q + (bytes ? col : 0);
                cp_async16(smem_u32(&sm.nb[stage][r * BN + swz8(r, c) * 8]), src, bytes);
            }
        }
        for (int j = tid; j < BN; j += THREADS) {
            const int key = k0 + j;
            sm.mb[stage][j] = key < S ? __bfloat162float(biasg[key]) * kLog2e : -INFINITY;
        }
    };

    // prologue: Q tile and key tile 0
    for (int idx = tid; idx < BM * CPR; idx += THREADS) {
        const int r = idx / CPR, c = idx % CPR;
        const bool ok = (q0 + r) < S;
        cp_async16(smem_u32(&sm.q[r * D + swz<CPR>(r, c) * 8]), qg + (int64_t)(ok ? q0 + r : 0) * D + c * 8, ok ? 16 : 0);
    }
    load_tile(0, 0);
    cp_async_commit();

    const int nkt = (S + BN - 1) / BN;
    uint32_t qf[KS][4];
    float oacc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};

    for (int kt = 0; kt < nkt; ++kt) {
        const int st = kt & 1;
        if (kt + 1 < nkt) {
            load_tile(st ^ 1, kt + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        if (kt == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int r = warp * 16 + (lane & 15);
                const int c = ks * 2 + (lane >> 4);
                ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], smem_u32(&sm.q[r * D + swz<CPR>(r, c) * 8]));
            }
        }

        // ---- logits: 16 x 64 per warp ----
        float sacc[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < NT_S / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int c = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(b0, b1, b2, b3, smem_u32(&sm.k[st][r * D + swz<CPR>(r, c) * 8]));
                mma_bf16_16816(sacc[np * 2], qf[ks], b0, b1);
                mma_bf16_16816(sacc[np * 2 + 1], qf[ks], b2, b3);
            }
        }

        // ---- biases (base-2 domain) and tile max ----
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
            const float2 mb = *reinterpret_cast<const float2 *>(&sm.mb[st][nt * 8 + 2 * t]);
            if (HAS_NB) {
                const int r0 = warp * 16 + g;
                const uint32_t n0 = *reinterpret_cast<const uint32_t *>(&sm.nb[st][r0 * BN + swz8(r0, nt) * 8 + 2 * t]);
                const uint32_t n1 =
                    *reinterpret_cast<const uint32_t *>(&sm.nb[st][(r0 + 8) * BN + swz8(r0 + 8, nt) * 8 + 2 * t]);
                sacc[nt][0] = fmaf(bf16lo_to_f32(n0), kLog2e, sacc[nt][0]) + mb.x;
                sacc[nt][1] = fmaf(bf16hi_to_f32(n0), kLog2e, sacc[nt][1]) + mb.y;
                sacc[nt][2] = fmaf(bf16lo_to_f32(n1), kLog2e, sacc[nt][2]) + mb.x;
                sacc[nt][3] = fmaf(bf16hi_to_f32(n1), kLog2e, sacc[nt][3]) + mb.y;
            } else {
                sacc[nt][0] += mb.x;
                sacc[nt][1] += mb.y;
                sacc[nt][2] += mb.x;
                sacc[nt][3] += mb.y;
            }
            tmax[0] = fmaxf(tmax[0], fmaxf(sacc[nt][0], sacc[nt][1]));
            tmax[1] = fmaxf(tmax[1], fmaxf(sacc[nt][2], sacc[nt][3]));
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
            const float m_new = fmaxf(m_run[r], tmax[r]);
            corr[r] = ex2_approx(m_run[r] - m_new);   // first tile: ex2(-inf) = 0
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            oacc[i][0] *= corr[0];
            oacc[i][1] *= corr[0];
            oacc[i][2] *= corr[1];
            oacc[i][3] *= corr[1];
        }

        // ---- probabilities, packed straight into A fragments ----
        uint32_t pf[NT_S / 2][4];
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
            const float p0 = ex2_approx(sacc[nt][0] - m_run[0]);
            const float p1 = ex2_approx(sacc[nt][1] - m_run[0]);
            const float p2 = ex2_approx(sacc[nt][2] - m_run[1]);
            const float p3 = ex2_approx(sacc[nt][3] - m_run[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(p0, p1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
        }

        // ---- O += P . V ----
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < NT_O / 2; ++dp) {
                uint32_t b0, b1, b2, b3;
                const int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int c = dp * 2 + (lane >> 4);
                ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(&sm.v[st][r * D + swz<CPR>(r, c) * 8]));
                mma_bf16_16816(oacc[dp * 2], pf[kk], b0, b1);
                mma_bf16_16816(oacc[dp * 2 + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();
    }

    // ---- epilogue: normalise, round, gate, store ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const int C = p.H * D;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qi = q0 + warp * 16 + g + r * 8;
        if (qi >= S) continue;
        const float inv = 1.0f / l_run[r];
        const int64_t base = ((int64_t)b * S + qi) * C + h * D;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + 2 * t;
            const uint32_t gv = *reinterpret_cast<const uint32_t *>(p.gate + base + d);
            // weighted average is stored as bf16 before gating in the reference (:128-133)
            const uint32_t wa = pack_bf16x2(oacc[nt][r * 2] * inv, oacc[nt][r * 2 + 1] * inv);
            const float s0 = 1.0f / (1.0f + ex2_approx(-bf16lo_to_f32(gv) * kLog2e));
            const float s1 = 1.0f / (1.0f + ex2_approx(-bf16hi_to_f32(gv) * kLog2e));
            *reinterpret_cast<uint32_t *>(p.avg + base + d) = pack_bf16x2(bf16lo_to_f32(wa) * s0, bf16hi_to_f32(wa) * s1);
        }
    }
}

template <int D, int NWARPS, bool HAS_NB>
bool launch_one(cudaStream_t stream, const AttnParams &p, int B)
{
    constexpr int smem = (int)sizeof(Smem<D, NWARPS>);
    static bool configured = false;
    if (!configured) {
        KUTACC_CUDA(cudaFuncSetAttribute(attn_core_kernel<D, NWARPS, HAS_NB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    constexpr int BM = NWARPS * 16;
    dim3 grid((unsigned)((p.S + BM - 1) / BM), (unsigned)p.H, (unsigned)B);
    KernelTimer timer__("attn_core");
    attn_core_kernel<D, NWARPS, HAS_NB><<<grid, NWARPS * 32, smem, stream>>>(p);
    count_launch();
    return true;
}

template <int D>
bool launch_d(cudaStream_t stream, const AttnParams &p, int B)
{
    if (p.nb) return launch_one<D, 8, true>(stream, p, B);
    return launch_one<D, 8, false>(stream, p, B);
}

}  // namespace

bool launch_attn_core_bf16(cudaStream_t stream, const void *q, const void *k, const void *v, const void *gate,
                           const void *bias, int64_t bias_stride0, const void *nb, int64_t nb_stride_h,
                           int64_t nb_stride_q, void *avg, int B, int S, int H, int D)
{
    if (B > 65535 || H > 65535) return false;
    if (nb && ((nb_stride_h % 8) || (nb_stride_q % 8) || ((uintptr_t)nb % 16))) return false;
    AttnParams p;
    p.q = (const __nv_bfloat16 *)q;
    p.k = (const __nv_bfloat16 *)k;
    p.v = (const __nv_bfloat16 *)v;
    p.gate = (const __nv_bfloat16 *)gate;
    p.bias = (const __nv_bfloat16 *)bias;
    p.nb = (const __nv_bfloat16 *)nb;
    p.avg = (__nv_bfloat16 *)avg;
    p.bias_stride0 = bias_stride0;
    p.nb_stride_h = nb_stride_h;
    p.nb_stride_q = nb_stride_q;
    p.S = S;
    p.H = H;
    switch (D) {
        case 16: return launch_d<16>(stream, p, B);
        case 32: return launch_d<32>(stream, p, B);
        case 64: return launch_d<64>(stream, p, B);
        default: return false;
    }
}

}  // namespace dev
}  // namespace kutacc
