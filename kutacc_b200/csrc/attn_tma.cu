// Fused gated-attention core: logits, mask bias, pair bias, online softmax, P.V, sigmoid gate.
// The S x S logits never leave the SM.
//
// Work split. One CTA owns (batch row b, head h, 128 queries). Eight consumer warps own 16 query rows
// each; a ninth warp is the producer. Keys are walked in tiles of 64 through a ring of shared-memory
// stages: the producer's elected lane issues TMA tile loads (cp.async.bulk.tensor, hardware swizzle)
// of K, V and the 128 x 64 pair-bias tile, all lanes of the producer convert the 64 mask-bias values
// to fp32, and mbarriers hand full stages to the consumers and empty stages back. No __syncthreads in
// the main loop, no per-thread address arithmetic for loads.
//
// Math per tile and warp: Q.K^T with mma.sync m16n8k16 (bf16 in, fp32 accumulate); the raw logit is
// rounded to bf16 exactly where the reference stores its logits scratch
// (src/attention/gating_attention.cpp:97-101), then x = logit*scale + bias + pair_bias in fp32 in the
// reference's operation order (:112-117); online softmax with quad shuffles; P re-packed in registers
// as the A operand of P.V; epilogue divides by the row sum, rounds to bf16 (:128-133), applies the
// sigmoid gate (:134-147) and stores bf16. The pair-bias tile is fetched with ldmatrix, whose register
// distribution is exactly the accumulator layout of the logits, and the producer stores the mask-bias
// values pre-permuted so that each thread reads its 16 values with four 128-bit loads.
//
// A fully masked row (every key carries -1e9) stays uniform as in the reference: fp32 absorbs the
// logit into the bias, every entry equals the row max, every probability is equal.
//
// Every mbarrier wait is bounded; a wait that runs out records a code in the host-visible error word
// and the warp leaves the kernel.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"
#include "tma_utils.cuh"

namespace kutacc {
namespace dev {

namespace {

constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct Cfg {
    static constexpr int NCW = 8;              // consumer warps
    static constexpr int BM = NCW * 16;        // queries per CTA
    static constexpr int BN = 64;              // keys per tile
    static constexpr int NST = 3;              // ring depth
    static constexpr int THREADS = (NCW + 1) * 32;
    static constexpr int KV_BYTES = BN * D * 2;
    static constexpr int NB_BYTES = BM * BN * 2;
    static constexpr int MB_BYTES = 1024;      // 64 floats, padded so that every tile stays 1024-byte aligned
    static constexpr int STAGE_BYTES = NB_BYTES + 2 * KV_BYTES + MB_BYTES;
    static constexpr int Q_BYTES = BM * D * 2;
    static constexpr int BAR_OFF = NST * STAGE_BYTES + Q_BYTES;
    static constexpr int SMEM_BYTES = BAR_OFF + 128 + 1024;   // barriers + slack for manual 1024-byte alignment
    static constexpr int CPR = D / 8;          // 16-byte chunks per q/k/v row
    static constexpr int KS = D / 16;          // k16 steps of Q.K^T; also pairs of output n-tiles
    static constexpr int SWZ_SHIFT = CPR == 8 ? 0 : (CPR == 4 ? 1 : 2);
};

struct AttnParams {
    const __nv_bfloat16 *gate;        // [B, S, H*D]
    const __nv_bfloat16 *bias;        // [B, S] (row stride bias_stride0)
    __nv_bfloat16 *avg;               // [B, S, H*D]
    int64_t bias_stride0;
    int *err;
    int S, H;
    float scale;
};

// physical 16-byte chunk of logical chunk c in row r of a TMA-swizzled tile with CPR chunks per row
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk)
{
    using C = Cfg<D>;
    return (uint32_t)(row * (D * 2) + ((chunk ^ ((row >> C::SWZ_SHIFT) & (C::CPR - 1))) << 4));
}

template <int D, bool HAS_NB>
__global__ void __launch_bounds__(Cfg<D>::THREADS, 2)
attn_core_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_nb,
                 const AttnParams p)
{
    using C = Cfg<D>;
    constexpr int NT_S = C::BN / 8;
    constexpr int NT_O = D / 8;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_base = smem + C::NST * C::STAGE_BYTES;
    const uint32_t bar_base = smem + C::BAR_OFF;
    auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(C::NST + s); };
    const uint32_t q_bar = bar_base + 8u * (2 * C::NST);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.S;
    const int q0 = blockIdx.x * C::BM;
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int bh = b * p.H + h;
    const int nkt = (S + C::BN - 1) / C::BN;

    if (tid == 0) {
        for (int s = 0; s < C::NST; ++s) {
            mbar_init(full_bar(s), 33);          // 32 producer lanes + the expect_tx arrival
            mbar_init(empty_bar(s), C::NCW);     // one elected lane per consumer warp
        }
        mbar_init(q_bar, 1);
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == C::NCW) {
        // ================= producer =================
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            if (HAS_NB) tma_prefetch_desc(&tm_nb);
            mbar_arrive_expect_tx(q_bar, C::Q_BYTES);
            tma_load_3d(q_base, &tm_q, q_bar, 0, q0, bh);
        }
        const __nv_bfloat16 *__restrict__ biasg = p.bias + (int64_t)b * p.bias_stride0;
        for (int kt = 0; kt < nkt; ++kt) {
            const int s = kt % C::NST;
            if (kt >= C::NST) {
                if (!mbar_wait_warp(empty_bar(s), (uint32_t)((kt / C::NST - 1) & 1), p.err, 1)) return;
            }
            const uint32_t st = smem + (uint32_t)s * C::STAGE_BYTES;
            const int k0 = kt * C::BN;
            float *mb = reinterpret_cast<float *>(smem_raw + (st - smem_u32(smem_raw)) + C::NB_BYTES + 2 * C::KV_BYTES);
            // key j = 8*nt + 2*t + e of the tile is stored at 16*t + 2*nt + e: thread t of a consumer quad
            // then finds the mask bias of all its accumulator columns in 64 consecutive bytes
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int kj = lane + 32 * j;
                const int key = k0 + kj;
                const int pos = (((kj >> 1) & 3) << 4) + ((kj >> 3) << 1) + (kj & 1);
                mb[pos] = key < S ? __bfloat162float(biasg[key]) : -INFINITY;
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(full_bar(s), (HAS_NB ? C::NB_BYTES : 0) + 2 * C::KV_BYTES);
                if (HAS_NB) tma_load_3d(st, &tm_nb, full_bar(s), k0, q0, h);
                tma_load_3d(st + C::NB_BYTES, &tm_k, full_bar(s), 0, k0, bh);
                tma_load_3d(st + C::NB_BYTES + C::KV_BYTES, &tm_v, full_bar(s), 0, k0, bh);
            }
            mbar_arrive(full_bar(s));
        }
        return;
    }

    // ================= consumers =================
    const int g = lane >> 2, t = lane & 3;

    // per-lane shared-memory offsets relative to the tile bases
    uint32_t k_off[4][C::KS];   // [pair of key n-tiles][k16 step over D]
    uint32_t v_off[4][C::KS];   // [k16 step over keys][pair of d n-tiles]
    uint32_t nb_off[4];         // [pair of key n-tiles]: rows g / g+8 of this warp's 16 x 64 slab
#pragma unroll
    for (int np = 0; np < 4; ++np) {
#pragma unroll
        for (int ks = 0; ks < C::KS; ++ks) {
            k_off[np][ks] = tile_off<D>(np * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1));
            v_off[np][ks] = tile_off<D>(np * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), ks * 2 + (lane >> 4));
        }
        const int nrow = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        nb_off[np] = (uint32_t)(nrow * 128 + (((2 * np + (lane >> 4)) ^ (nrow & 7)) << 4));
    }
    const uint32_t mb_off = (uint32_t)(C::NB_BYTES + 2 * C::KV_BYTES + t * 64);

    if (!mbar_wait_warp(q_bar, 0, p.err, 2)) return;
    uint32_t qf[C::KS][4];
#pragma unroll
    for (int ks = 0; ks < C::KS; ++ks)
        ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                    q_base + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));

    float oacc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    const float scale = p.scale;

    for (int kt0 = 0; kt0 < nkt; kt0 += C::NST) {
#pragma unroll
        for (int s = 0; s < C::NST; ++s) {
            const int kt = kt0 + s;
            if (kt >= nkt) break;
            if (!mbar_wait_warp(full_bar(s), (uint32_t)((kt0 / C::NST) & 1), p.err, 3)) return;
            const uint32_t st = smem + (uint32_t)s * C::STAGE_BYTES;
            const uint32_t k_base = st + C::NB_BYTES, v_base = k_base + C::KV_BYTES;

            // ---- raw logits: 16 x 64 per warp ----
            float sacc[NT_S][4];
#pragma unroll
            for (int i = 0; i < NT_S; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < C::KS; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, k_base + k_off[np][ks]);
                    mma_bf16_16816(sacc[np * 2], qf[ks], b0, b1);
                    mma_bf16_16816(sacc[np * 2 + 1], qf[ks], b2, b3);
                }
            }

            // ---- operands of the bias add ----
            float mbv[16];
            {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 v4 = lds128_f32(st + mb_off + 16 * i);
                    mbv[4 * i] = v4.x;
                    mbv[4 * i + 1] = v4.y;
                    mbv[4 * i + 2] = v4.z;
                    mbv[4 * i + 3] = v4.w;
                }
            }
            uint32_t nbw[NT_S][2];   // [key n-tile][row g / g+8]: packed pair-bias of columns 2t, 2t+1
            if (HAS_NB) {
#pragma unroll
                for (int np = 0; np < 4; ++np)
                    ldmatrix_x4(nbw[2 * np][0], nbw[2 * np][1], nbw[2 * np + 1][0], nbw[2 * np + 1][1], st + nb_off[np]);
            }

            // ---- x = bf16(logit)*scale + bias (+ pair bias), tile max ----
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < NT_S; ++nt) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t pr = pack_bf16x2(sacc[nt][2 * r], sacc[nt][2 * r + 1]);   // logits scratch is bf16
                    float x0 = fmaf(bf16lo_to_f32(pr), scale, mbv[2 * nt]);
                    float x1 = fmaf(bf16hi_to_f32(pr), scale, mbv[2 * nt + 1]);
                    if (HAS_NB) {
                        x0 += bf16lo_to_f32(nbw[nt][r]);
                        x1 += bf16hi_to_f32(nbw[nt][r]);
                    }
                    sacc[nt][2 * r] = x0;
                    sacc[nt][2 * r + 1] = x1;
                    tmax[r] = fmaxf(tmax[r], fmaxf(x0, x1));
                }
            }
            float mneg[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
                const float m_new = fmaxf(m_run[r], tmax[r]);
                const float corr = ex2_approx((m_run[r] - m_new) * kLog2e);   // first tile: ex2(-inf) = 0
                m_run[r] = m_new;
                mneg[r] = -m_new * kLog2e;
                l_run[r] *= corr;
#pragma unroll
                for (int i = 0; i < NT_O; ++i) {
                    oacc[i][2 * r] *= corr;
                    oacc[i][2 * r + 1] *= corr;
                }
            }

            // ---- probabilities, packed straight into A fragments ----
            uint32_t pf[NT_S / 2][4];
#pragma unroll
            for (int nt = 0; nt < NT_S; ++nt) {
                const float p0 = ex2_approx(fmaf(sacc[nt][0], kLog2e, mneg[0]));
                const float p1 = ex2_approx(fmaf(sacc[nt][1], kLog2e, mneg[0]));
                const float p2 = ex2_approx(fmaf(sacc[nt][2], kLog2e, mneg[1]));
                const float p3 = ex2_approx(fmaf(sacc[nt][3], kLog2e, mneg[1]));
                l_run[0] += p0 + p1;
                l_run[1] += p2 + p3;
                pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(p0, p1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
            }

            // ---- O += P . V ----
#pragma unroll
            for (int kk = 0; kk < C::BN / 16; ++kk) {
#pragma unroll
                for (int dp = 0; dp < C::KS; ++dp) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, v_base + v_off[kk][dp]);
                    mma_bf16_16816(oacc[dp * 2], pf[kk], b0, b1);
                    mma_bf16_16816(oacc[dp * 2 + 1], pf[kk], b2, b3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
        }
    }

    // ---- epilogue: normalise, round, gate, store ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const int Cn = p.H * D;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qi = q0 + warp * 16 + g + r * 8;
        if (qi >= S) continue;
        const float inv = 1.0f / l_run[r];
        const int64_t base = ((int64_t)b * S + qi) * Cn + h * D;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + 2 * t;
            const uint32_t gv = *reinterpret_cast<const uint32_t *>(p.gate + base + d);
            // the weighted average is stored as bf16 before gating in the reference (:128-133)
            const uint32_t wa = pack_bf16x2(oacc[nt][r * 2] * inv, oacc[nt][r * 2 + 1] * inv);
            const float s0 = 1.0f / (1.0f + ex2_approx(-bf16lo_to_f32(gv) * kLog2e));
            const float s1 = 1.0f / (1.0f + ex2_approx(-bf16hi_to_f32(gv) * kLog2e));
            *reinterpret_cast<uint32_t *>(p.avg + base + d) = pack_bf16x2(bf16lo_to_f32(wa) * s0, bf16hi_to_f32(wa) * s1);
        }
    }
}

template <int D, bool HAS_NB>
bool launch_one(cudaStream_t stream, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                const CUtensorMap &tnb, const AttnParams &p, int B)
{
    using C = Cfg<D>;
    static bool configured = false;
    if (!configured) {
        KUTACC_CUDA(cudaFuncSetAttribute(attn_core_kernel<D, HAS_NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES));
        configured = true;
    }
    dim3 grid((unsigned)((p.S + C::BM - 1) / C::BM), (unsigned)p.H, (unsigned)B);
    KernelTimer timer__("attn_core", stream);
    attn_core_kernel<D, HAS_NB><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, tnb, p);
    count_launch();
    return true;
}

template <int D>
bool launch_d(cudaStream_t stream, const void *q, const void *k, const void *v, const void *nb, int64_t nb_stride_h,
              int64_t nb_stride_q, AttnParams &p, int B)
{
    using C = Cfg<D>;
    const uint64_t S = (uint64_t)p.S, BH = (uint64_t)B * p.H;
    CUtensorMap tq, tk, tv, tnb;
    constexpr int swz = D * 2;   // 32, 64 or 128 bytes per row
    if (!make_tensor_map_bf16_3d(&tq, q, D, S, BH, D, S * D, D, C::BM, swz)) return false;
    if (!make_tensor_map_bf16_3d(&tk, k, D, S, BH, D, S * D, D, C::BN, swz)) return false;
    if (!make_tensor_map_bf16_3d(&tv, v, D, S, BH, D, S * D, D, C::BN, swz)) return false;
    if (nb) {
        if (!make_tensor_map_bf16_3d(&tnb, nb, S, S, (uint64_t)p.H, (uint64_t)nb_stride_q, (uint64_t)nb_stride_h,
                                     C::BN, C::BM, 128))
            return false;
        return launch_one<D, true>(stream, tq, tk, tv, tnb, p, B);
    }
    tnb = tk;
    return launch_one<D, false>(stream, tq, tk, tv, tnb, p, B);
}

}  // namespace

bool launch_attn_core_bf16(cudaStream_t stream, const void *q, const void *k, const void *v, const void *gate,
                           const void *bias, int64_t bias_stride0, const void *nb, int64_t nb_stride_h,
                           int64_t nb_stride_q, void *avg, int B, int S, int H, int D, float scale)
{
    if (B > 65535 || H > 65535) return false;
    if (nb && ((nb_stride_h % 8) || (nb_stride_q % 8) || ((uintptr_t)nb % 16))) return false;
    if (nb && nb_stride_h < nb_stride_q) return false;     // heads inside rows: only the tcgen05 core and the generic kernel
    KernelErrorWord &ew = kernel_error_word();
    if (ew.device == nullptr) return false;
    AttnParams p;
    p.gate = (const __nv_bfloat16 *)gate;
    p.bias = (const __nv_bfloat16 *)bias;
    p.avg = (__nv_bfloat16 *)avg;
    p.bias_stride0 = bias_stride0;
    p.err = ew.device;
    p.S = S;
    p.H = H;
    p.scale = scale;
    switch (D) {
        case 16: return launch_d<16>(stream, q, k, v, nb, nb_stride_h, nb_stride_q, p, B);
        case 32: return launch_d<32>(stream, q, k, v, nb, nb_stride_h, nb_stride_q, p, B);
        case 64: return launch_d<64>(stream, q, k, v, nb, nb_stride_h, nb_stride_q, p, B);
        default: return false;
    }
}

}  // namespace dev
}  // namespace kutacc
