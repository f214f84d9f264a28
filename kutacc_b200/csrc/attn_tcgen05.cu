// Fused gated-attention core on the fifth-generation tensor cores (head size 32).
//
// A work item is (pair of batch rows b0, b0+1; head h; 128 queries). The two batch rows of an item share the
// pair-bias tile nb[h, q, k], so a thread unpacks each pair-bias value once and adds it to the logits of both
// rows. The kernel is persistent: one CTA per SM walks a strided list of items, and every pipeline below keeps
// running across item boundaries, so the loads and the first Q.K^T of the next item overlap the epilogue of the
// current one. Both matrix products run on tcgen05.mma with accumulators in tensor memory, issued by one elected
// lane; the softmax runs on the logits read back with tcgen05.ld. The S x S logits never leave the SM.
//
//   warp 0      producer: TMA tile loads (hardware swizzle) of Q for both rows (double-buffered across items)
//               and, per 64-key step, K [64 x 32] and V^T [32 x 64] of both rows plus the one 128 x 64 pair-bias
//               tile into a ring; its lanes also convert the step's 2 x 64 mask-bias values to fp32
//   warp 1      MMA issuer: S_r = Q_r.K_r^T (M 128, N 64, K 32) into TMEM columns 64r..64r+63; then, per row r
//               and 16-key quarter c, O_rc += P_r[:, 16c..16c+15] . V_r^T[:, 16c..16c+15]^T (M 128, N 48, K 16)
//               into eight separate TMEM accumulators. Row 32 of the V^T operand is all ones, so column 32 of
//               each accumulator collects the row sum of the bf16 probabilities for free
//   warps 2-17  softmax: four threads per query row, one per 16-key quarter of every step (split-key online
//               softmax: each quarter keeps its own running max and its own accumulator, merged once per item).
//               A thread pulls its 2 x 16 logits out of TMEM (S is free for the next Q.K^T once all have done
//               so), rounds each raw logit to bf16 as the reference's logits scratch does
//               (src/attention/gating_attention.cpp:97-101), forms x = logit*scale + bias + pair_bias in fp32 in
//               the reference's order (:112-117), and writes P = exp2(x*log2e - max) as bf16 (the packed
//               ex2.approx.ftz.bf16x2 was measured: it issues as two MUFU operations plus a permute, one
//               instruction more per pair than two ex2.f32 and a pack): row 0's probabilities over the pair-bias values it has just consumed
//               (same row, same swizzled chunks), row 1's into a tile of their own; both are A operands of
//               P.V^T. After the first step of an item P is formed against the running max chunk by chunk; an
//               accumulator is rescaled in TMEM and the step redone only when the max grows by more than 2^8 (a
//               stale max cancels in the final division). Item epilogue: each thread merges the four quarters for
//               8 of the 32 channels of both rows straight from TMEM (only the running maxima cross through
//               shared memory), O / rowsum, bf16 (:128-133), gate (:134-147; the projection kernel has already
//               applied the sigmoid when gate_is_sigmoid is set), 16-byte row stores.
//
// Fully masked rows stay uniform as in the reference (fp32 absorption of the logit by the -1e9 bias).
//
// mbarrier phases. A parity wait names "the current or the preceding phase", so every barrier here is
// awaited by each of its waiters once per completion, in order; the one exception (pv_done on the rare
// rescale path) is safe because that waiter is provably at most one phase behind. All waits are bounded;
// on a timeout the roles fall through to the common tail, tensor memory is released, and the host-visible
// error word carries the site.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"
#include "tcgen05_utils.cuh"
#include "tma_utils.cuh"

#include <algorithm>
#include <climits>

namespace kutacc {
namespace dev {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int D = 32;                 // head size
constexpr int BM = 128;               // queries per item
constexpr int BN = 64;                // keys per step
constexpr int NR = 2;                 // batch rows per item
constexpr int NQ = 4;                 // key quarters per step (16 keys each)
#ifndef KUTACC_ATTN_NST
#define KUTACC_ATTN_NST 3
#endif
constexpr int NST = KUTACC_ATTN_NST;  // ring depth
constexpr int VT_ROWS = 48;           // 32 channels + the ones row + zero padding to a multiple of 16
constexpr int Q_BYTES = BM * D * 2;           // 8 KB per row, 64-byte rows, 64-byte swizzle
constexpr int K_BYTES = BN * D * 2;           // 4 KB per row, 64-byte rows
constexpr int VT_BYTES = VT_ROWS * BN * 2;    // 6 KB per row, 128-byte rows (TMA fills the first 32)
constexpr int NB_BYTES = BM * BN * 2;         // 16 KB, 128-byte rows: pair bias in, probabilities of row 0 out (in place)
constexpr int MB_BYTES = 1024;                // 2 x 64 floats, padded
constexpr int OFF_K = 0, OFF_VT = NR * K_BYTES, OFF_NB = OFF_VT + NR * VT_BYTES, OFF_P1 = OFF_NB + NB_BYTES,
              OFF_MB = OFF_P1 + NB_BYTES;
constexpr int STAGE_BYTES = OFF_MB + MB_BYTES;
static_assert(OFF_NB % 1024 == 0 && OFF_VT % 1024 == 0 && (OFF_VT + VT_BYTES) % 1024 == 0 && STAGE_BYTES % 1024 == 0,
              "swizzled tiles must start on 1024-byte boundaries");
constexpr int OFF_STAGE = 2 * NR * Q_BYTES;                 // Q: two item parities x two rows
constexpr int OFF_XCH = OFF_STAGE + NST * STAGE_BYTES;      // running maxima: [item parity][row][quarter][query]
constexpr int XCH_BYTES = 2 * NR * NQ * BM * 4;
constexpr int OFF_BAR = OFF_XCH + XCH_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int SOFTMAX_WARPS = 16;
constexpr int THREADS = (2 + SOFTMAX_WARPS) * 32;
constexpr int TMEM_COLS = 512;
constexpr int S_COL = 0, O_COL = NR * BN, O_STRIDE = VT_ROWS;   // O_rc at 128 + (4r + c) * 48
static_assert(O_COL + NR * NQ * O_STRIDE <= TMEM_COLS, "accumulators exceed tensor memory");
constexpr float kRescaleThreshold = 8.0f;     // log2 units

struct AttnParams {
    const __nv_bfloat16 *gate;        // [B, S, H*D]
    const __nv_bfloat16 *bias;        // [B, S] (row stride bias_stride0)
    __nv_bfloat16 *avg;               // [B, S, H*D]
    int64_t bias_stride0;
    int *err;
    int S, H, B;
    int n_qt;                         // query tiles per (b, h)
    int n_items;                      // ceil(B / 2) * H * n_qt
    int gate_is_sigmoid;              // gate already holds bf16(sigmoid(bf16(x.Wg + bg)))
    float scale;
};

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

template <bool HAS_NB>
__global__ void __launch_bounds__(THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_vt, const __grid_constant__ CUtensorMap tm_nb,
               const AttnParams p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *smem_gen = smem_raw + (smem - smem_u32(smem_raw));
    auto q_buf = [&](int i, int r) { return smem + (uint32_t)((i & 1) * NR + r) * Q_BYTES; };
    auto stage_base = [&](int s) { return smem + OFF_STAGE + (uint32_t)s * STAGE_BYTES; };
    const uint32_t bar = smem + OFF_BAR;
    auto kv_full = [&](int s) { return bar + 8u * (uint32_t)s; };
    auto kv_empty = [&](int s) { return bar + 8u * (uint32_t)(NST + s); };
    auto p_full = [&](int s) { return bar + 8u * (uint32_t)(2 * NST + s); };
    auto q_full = [&](int i) { return bar + 8u * (uint32_t)(3 * NST + (i & 1)); };
    auto q_empty = [&](int i) { return bar + 8u * (uint32_t)(3 * NST + 2 + (i & 1)); };
    const uint32_t s_full = bar + 8u * (3 * NST + 4), s_free = s_full + 8, pv_done = s_full + 16, o_final = s_full + 24,
                   o_free = s_full + 32, x_full = s_full + 40, tmem_slot = s_full + 48;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.S;
    const int nkt = (S + BN - 1) / BN;
    // items of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
    const int my_items = ((int)blockIdx.x < p.n_items) ? (p.n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    // item -> first query, head, the two batch rows (the second repeats the first when B is odd and this is the
    // last pair: it is computed and not stored)
    auto decode = [&](int i, int &q0, int &h, int &b0, int &b1) {
        const int w = (int)blockIdx.x + i * (int)gridDim.x;
        const int qt = w % p.n_qt, hb = w / p.n_qt;
        q0 = qt * BM;
        h = hb % p.H;
        b0 = 2 * (hb / p.H);
        b1 = b0 + 1 < p.B ? b0 + 1 : b0;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(kv_full(s), 33);      // 32 producer lanes (mask bias) + the expect_tx arrival
            mbar_init(kv_empty(s), 1);      // the commit that follows P.V^T (P lives in the stage)
            mbar_init(p_full(s), SOFTMAX_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full(i), 1);
            mbar_init(q_empty(i), 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_free, SOFTMAX_WARPS);
        mbar_init(pv_done, 1);
        mbar_init(o_final, 1);
        mbar_init(o_free, SOFTMAX_WARPS);
        mbar_init(x_full, SOFTMAX_WARPS);
        fence_barrier_init();
    }
    // static rows 32..47 of every V^T tile: row 32 = 1.0 (row-sum column of O), rows 33..47 = 0
    for (int i = threadIdx.x; i < NST * NR * 16 * (BN * 2 / 16); i += THREADS) {
        const int t = i / (16 * 8), rem = i % (16 * 8), row = 32 + rem / 8, ch = rem % 8;
        const int s = t / NR, r = t % NR;
        const uint32_t v = row == 32 ? 0x3F803F80u : 0u;
        uint4 *dst = reinterpret_cast<uint4 *>(smem_gen + OFF_STAGE + s * STAGE_BYTES + OFF_VT + r * VT_BYTES + row * 128 + ch * 16);
        *dst = make_uint4(v, v, v, v);
    }
    fence_proxy_async();
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
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_vt);
            if (HAS_NB) tma_prefetch_desc(&tm_nb);
        }
        int g = 0;                                      // steps issued so far (all items)
        bool ok = true;
        // The step's 2 x 64 mask-bias values are read from global memory by the lanes (two keys of each row per
        // lane) one step ahead and kept in registers, so that neither the wait for a free stage nor the TMA issue
        // ever sits behind the latency of those loads.
        float mbreg[NR][2];
        auto fetch_mask_bias = [&](int i, int kt) {
            if (i >= my_items) return;
            int q0, h, b0, b1;
            decode(i, q0, h, b0, b1);
            const int bb[NR] = {b0, b1};
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int key = kt * BN + lane + 32 * j;
                    mbreg[r][j] = key < S ? __bfloat162float(p.bias[(int64_t)bb[r] * p.bias_stride0 + key]) : -INFINITY;
                }
        };
        fetch_mask_bias(0, 0);
        for (int i = 0; i < my_items && ok; ++i) {
            int q0, h, b0, b1;
            decode(i, q0, h, b0, b1);
            const int bh[NR] = {b0 * p.H + h, b1 * p.H + h};
            if (i >= 2 && !mbar_wait_warp(q_empty(i), (uint32_t)(((i >> 1) - 1) & 1), p.err, 20)) break;
            if (lane == 0) {
                mbar_arrive_expect_tx(q_full(i), NR * Q_BYTES);
#pragma unroll
                for (int r = 0; r < NR; ++r) tma_load_3d(q_buf(i, r), &tm_q, q_full(i), 0, q0, bh[r]);
            }
            for (int kt = 0; kt < nkt; ++kt, ++g) {
                const int s = g % NST;
                if (g >= NST && !mbar_wait_warp(kv_empty(s), (uint32_t)((g / NST - 1) & 1), p.err, 21)) {
                    ok = false;
                    break;
                }
                const uint32_t st = stage_base(s);
                const int k0 = kt * BN;
                if (lane == 0) {
                    mbar_arrive_expect_tx(kv_full(s), NR * (K_BYTES + BN * D * 2) + (HAS_NB ? NB_BYTES : 0));
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        tma_load_3d(st + OFF_K + r * K_BYTES, &tm_k, kv_full(s), 0, k0, bh[r]);
                        tma_load_3d(st + OFF_VT + r * VT_BYTES, &tm_vt, kv_full(s), k0, 0, bh[r]);
                    }
                    if (HAS_NB) tma_load_3d(st + OFF_NB, &tm_nb, kv_full(s), k0, q0, h);
                }
                float *mb = reinterpret_cast<float *>(smem_gen + OFF_STAGE + s * STAGE_BYTES + OFF_MB);
#pragma unroll
                for (int r = 0; r < NR; ++r)
#pragma unroll
                    for (int j = 0; j < 2; ++j) mb[r * BN + lane + 32 * j] = mbreg[r][j];
                mbar_arrive(kv_full(s));
                // the next step's values (possibly the first step of the next item): in flight during the next wait
                if (kt + 1 < nkt)
                    fetch_mask_bias(i, kt + 1);
                else
                    fetch_mask_bias(i + 1, 0);
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        constexpr uint32_t idesc_s = make_instr_desc_bf16(BM, BN);
        constexpr uint32_t idesc_o = make_instr_desc_bf16(BM, VT_ROWS);
        const int total = my_items * nkt;               // steps of this CTA, all items
        // S_r = Q_r . K_r^T for step g of item i, both rows
        auto issue_qk = [&](int g, int i, bool first_of_item) -> bool {
            const int s = g % NST;
            if (first_of_item && !mbar_wait_warp(q_full(i), (uint32_t)((i >> 1) & 1), p.err, 22)) return false;
            if (!mbar_wait_warp(kv_full(s), (uint32_t)((g / NST) & 1), p.err, 23)) return false;
            if (g > 0 && !mbar_wait_warp(s_free, (uint32_t)((g - 1) & 1), p.err, 24)) return false;
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t kb = stage_base(s) + OFF_K + r * K_BYTES, qb = q_buf(i, r);
#pragma unroll
                    for (int k = 0; k < D / 16; ++k)
                        tc_mma_bf16(tmem_base + S_COL + r * BN, make_smem_desc_kmajor(qb + k * 32, 64),
                                    make_smem_desc_kmajor(kb + k * 32, 64), idesc_s, k > 0 ? 1u : 0u);
                }
                tc_commit(s_full);
            }
            __syncwarp();
            return true;
        };
        bool ok = total > 0 ? issue_qk(0, 0, true) : true;
        int g = 0;
        for (int i = 0; i < my_items && ok; ++i) {
            for (int kt = 0; kt < nkt && ok; ++kt, ++g) {
                const int s = g % NST;
                // look one step ahead in the stream (possibly the first step of the next item): its Q.K^T
                // overlaps the softmax of step g
                if (g + 1 < total) ok = issue_qk(g + 1, kt + 1 < nkt ? i : i + 1, kt + 1 == nkt);
                if (!ok) break;
                if (!mbar_wait_warp(p_full(s), (uint32_t)((g / NST) & 1), p.err, 25)) {
                    ok = false;
                    break;
                }
                // the first P.V^T of an item overwrites O: the previous item's epilogue must have read it
                if (kt == 0 && i > 0 && !mbar_wait_warp(o_free, (uint32_t)((i - 1) & 1), p.err, 30)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        const uint32_t vb = stage_base(s) + OFF_VT + r * VT_BYTES;
                        const uint32_t pb = stage_base(s) + (r == 0 ? OFF_NB : OFF_P1);
#pragma unroll
                        for (int c = 0; c < NQ; ++c)      // one k16 step per quarter, each into its own accumulator
                            tc_mma_bf16(tmem_base + O_COL + (r * NQ + c) * O_STRIDE, make_smem_desc_kmajor(pb + c * 32, 128),
                                        make_smem_desc_kmajor(vb + c * 32, 128), idesc_o, kt > 0 ? 1u : 0u);
                    }
                    tc_commit(pv_done);
                    tc_commit(kv_empty(s));
                    if (kt == nkt - 1) {
                        tc_commit(o_final);
                        tc_commit(q_empty(i));
                    }
                }
                __syncwarp();
            }
        }
    } else {
        // ================= softmax / epilogue =================
        const int quad = warp & 3;                       // TMEM lanes 32*quad .. 32*quad+31
        const int qtr = (warp - 2) >> 2;                 // which 16 keys of every step this thread owns
        const int row = quad * 32 + lane;                // query row inside the tile
        const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
        const float scale = p.scale;
        const uint64_t scale2 = pack_f32x2(scale, scale), log2e2 = pack_f32x2(kLog2e, kLog2e);
        bool ok = true;
        // per-thread shared-memory addresses of stage 0; other stages add a multiple of STAGE_BYTES
        const uint32_t st0 = smem + OFF_STAGE;
        uint32_t nb_addr[2];                             // this row's 2 swizzled 16-byte chunks (pair bias in, P_0 out)
#pragma unroll
        for (int c = 0; c < 2; ++c)
            nb_addr[c] = st0 + OFF_NB + (uint32_t)row * 128 + (uint32_t)(((qtr * 2 + c) ^ (row & 7)) << 4);
        const uint32_t mb_addr = st0 + OFF_MB + qtr * 64;
        float *xch = reinterpret_cast<float *>(smem_gen + OFF_XCH);      // [item parity][row r][quarter][query]
        float m2[NR] = {-INFINITY, -INFINITY};           // running (possibly stale) maxima of this quarter, log2 units

        // one step of the softmax: global step g, step kt of its item
        auto do_tile = [&](const int g, const int kt) -> bool {
            const int s = g % NST;
            const uint32_t soff = (uint32_t)s * STAGE_BYTES;
            if (!mbar_wait_warp(s_full, (uint32_t)(g & 1), p.err, 26)) return false;
            tc_fence_after();
            uint32_t sr[NR][16];
            tmem_ld_32x16(t_lane + S_COL + qtr * 16, sr[0]);
            tmem_ld_32x16(t_lane + S_COL + BN + qtr * 16, sr[1]);
            // the test of kv_full (pair bias and mask bias of this step have landed; a barrier test costs about a
            // hundred cycles even when it succeeds at once) runs while the tensor-memory loads are in flight
            const bool landed = mbar_wait_warp(kv_full(s), (uint32_t)((g / NST) & 1), p.err, 27);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free);
            if (!landed) return false;

            float tmax[NR] = {-INFINITY, -INFINITY};
            // x = bf16(logit)*scale + bias (+ pair bias) for 8 keys of both rows; keeps x in sr and tracks the maxima
            auto x_chunk = [&](const int c) {
                uint64_t nb2[4];
                if (HAS_NB) {
                    uint32_t nbw[4];
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(nbw[0]), "=r"(nbw[1]), "=r"(nbw[2]), "=r"(nbw[3])
                                 : "r"(nb_addr[c] + soff));
#pragma unroll
                    for (int j = 0; j < 4; ++j) nb2[j] = pack_f32x2(bf16lo_to_f32(nbw[j]), bf16hi_to_f32(nbw[j]));
                }
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t ma = mb_addr + soff + r * (BN * 4) + c * 32;
                    const float4 mb0 = lds128_f32(ma), mb1 = lds128_f32(ma + 16);
                    const float mbv[8] = {mb0.x, mb0.y, mb0.z, mb0.w, mb1.x, mb1.y, mb1.z, mb1.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int i0 = c * 8 + 2 * j;
                        // the raw logit is stored as bf16 by the reference: one cvt gives its fp32 image. The two
                        // keys of a pair go through the packed fp32 pipe (one issue slot for both).
                        uint64_t x2 = fma_f32x2(pack_f32x2(round_to_bf16_f32(__uint_as_float(sr[r][i0])),
                                                           round_to_bf16_f32(__uint_as_float(sr[r][i0 + 1]))),
                                                scale2, pack_f32x2(mbv[2 * j], mbv[2 * j + 1]));
                        if (HAS_NB) x2 = add_f32x2(x2, nb2[j]);
                        float x0, x1;
                        unpack_f32x2(x2, x0, x1);
                        sr[r][i0] = __float_as_uint(x0);
                        sr[r][i0 + 1] = __float_as_uint(x1);
                        tmax[r] = fmax3(tmax[r], x0, x1);
                    }
                }
            };
            // P = exp2(x*log2e - m2) for 8 keys of row r -> bf16 -> A operand of P.V^T
            auto p_chunk = [&](const int c, const int r, const float mneg) {
                uint32_t w[4];
                const uint64_t mneg2 = pack_f32x2(mneg, mneg);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i0 = c * 8 + 2 * j;
                    float e0, e1;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[r][i0]), __uint_as_float(sr[r][i0 + 1])), log2e2,
                                           mneg2), e0, e1);
                    w[j] = pack_bf16x2(ex2_approx(e0), ex2_approx(e1));
                }
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(nb_addr[c] + soff + (r ? (uint32_t)(OFF_P1 - OFF_NB) : 0u)),
                             "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                             : "memory");
            };

            // The same two steps for 8 keys of BOTH rows, written stage by stage over the 8 independent key pairs (all
            // loads, all roundings, all scale-and-bias, ... all exponentials, all packs) instead of pair by pair: the
            // instruction stream of a warp then has eight independent chains in flight at every point, which is what
            // hides the arithmetic and MUFU latencies at four softmax warps per scheduler.
            auto xp_chunk = [&](const int c) {
                uint32_t nbw[4] = {0, 0, 0, 0};
                if (HAS_NB)
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(nbw[0]), "=r"(nbw[1]), "=r"(nbw[2]), "=r"(nbw[3])
                                 : "r"(nb_addr[c] + soff));
                float4 mbq[NR][2];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t ma = mb_addr + soff + r * (BN * 4) + c * 32;
                    mbq[r][0] = lds128_f32(ma);
                    mbq[r][1] = lds128_f32(ma + 16);
                }
                float lr[NR][8];
#pragma unroll
                for (int r = 0; r < NR; ++r)
#pragma unroll
                    for (int i = 0; i < 8; ++i) lr[r][i] = round_to_bf16_f32(__uint_as_float(sr[r][c * 8 + i]));
                uint64_t x2[NR][4];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const float mbv[8] = {mbq[r][0].x, mbq[r][0].y, mbq[r][0].z, mbq[r][0].w,
                                          mbq[r][1].x, mbq[r][1].y, mbq[r][1].z, mbq[r][1].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        x2[r][j] = fma_f32x2(pack_f32x2(lr[r][2 * j], lr[r][2 * j + 1]), scale2, pack_f32x2(mbv[2 * j], mbv[2 * j + 1]));
                }
                if (HAS_NB) {
                    uint64_t nb2[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) nb2[j] = pack_f32x2(bf16lo_to_f32(nbw[j]), bf16hi_to_f32(nbw[j]));
#pragma unroll
                    for (int r = 0; r < NR; ++r)
#pragma unroll
                        for (int j = 0; j < 4; ++j) x2[r][j] = add_f32x2(x2[r][j], nb2[j]);
                }
                uint64_t t2[NR][4];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint64_t mneg2 = pack_f32x2(-m2[r], -m2[r]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) t2[r][j] = fma_f32x2(x2[r][j], log2e2, mneg2);
                }
#pragma unroll
                for (int r = 0; r < NR; ++r)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float x0, x1;
                        unpack_f32x2(x2[r][j], x0, x1);
                        sr[r][c * 8 + 2 * j] = __float_as_uint(x0);          // kept for the rare redo against a new max
                        sr[r][c * 8 + 2 * j + 1] = __float_as_uint(x1);
                        tmax[r] = fmax3(tmax[r], x0, x1);
                    }
                float e[NR][8];
#pragma unroll
                for (int r = 0; r < NR; ++r)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float a, b;
                        unpack_f32x2(t2[r][j], a, b);
                        e[r][2 * j] = ex2_approx(a);
                        e[r][2 * j + 1] = ex2_approx(b);
                    }
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) w[j] = pack_bf16x2(e[r][2 * j], e[r][2 * j + 1]);
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(nb_addr[c] + soff + (r ? (uint32_t)(OFF_P1 - OFF_NB) : 0u)),
                                 "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                                 : "memory");
                }
            };

            if (kt == 0) {
                // first step of an item: the maxima must be known before any probability is formed
#pragma unroll
                for (int c = 0; c < 2; ++c) x_chunk(c);
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    // a quarter whose keys all lie beyond S has no max yet: park it on a finite floor
                    m2[r] = tmax[r] > -INFINITY ? tmax[r] * kLog2e : -1e30f;
#pragma unroll
                    for (int c = 0; c < 2; ++c) p_chunk(c, r, -m2[r]);
                }
            } else {
                // later steps: form the probabilities against the running maxima straight away, chunk by chunk,
                // so that the exp (XU pipe) of one chunk overlaps the arithmetic of the next; a running max
                // may be stale by up to 2^8, which cancels in the final division
#pragma unroll
                for (int c = 0; c < 2; ++c) xp_chunk(c);
                bool grow[NR];
                float t2[NR];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    t2[r] = tmax[r] > -INFINITY ? tmax[r] * kLog2e : -1e30f;
                    grow[r] = t2[r] > m2[r] + kRescaleThreshold;
                }
                if (__any_sync(0xffffffffu, grow[0] || grow[1])) {
                    // rare: the max of some row grew past the threshold. Rescale those rows of this quarter's
                    // accumulators (and their row-sum column) and redo this step's probabilities against the new
                    // max. The previous step's P.V^T must have retired first (this warp is at most one phase behind
                    // pv_done here: s_full(g) implies that the product of step g-2 has retired).
                    if (!mbar_wait_warp(pv_done, (uint32_t)((g - 1) & 1), p.err, 28)) return false;
                    tc_fence_after();
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        if (!__any_sync(0xffffffffu, grow[r])) continue;
                        const uint32_t o_col = t_lane + O_COL + (r * NQ + qtr) * O_STRIDE;
                        const float f = grow[r] ? ex2_approx(m2[r] - t2[r]) : 1.0f;
                        uint32_t o[32];
                        tmem_ld_32x32(o_col, o);
                        uint32_t osum = tmem_ld_32x1(o_col + 32);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        osum = __float_as_uint(__uint_as_float(osum) * f);
                        tmem_st_32x32(o_col, o);
                        tmem_st_32x1(o_col + 32, osum);
                        tmem_st_wait();
                        if (grow[r]) m2[r] = t2[r];
#pragma unroll
                        for (int c = 0; c < 2; ++c) p_chunk(c, r, -m2[r]);
                    }
                    tc_fence_before();
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(s));
            return true;
        };

        int g = 0;
        for (int i = 0; i < my_items && ok; ++i) {
            int q0, h, b0, b1;
            decode(i, q0, h, b0, b1);
            for (int kt = 0; kt < nkt && ok; ++kt, ++g) ok = do_tile(g, kt);
            if (!ok) break;

            // ---- item epilogue: this thread finishes channels [8*qtr, 8*qtr + 8) of its query for both rows ----
            const int qi = q0 + row;
            const int Cn = p.H * D;
            const int bb[NR] = {b0, b1};
            int64_t base[NR];
            uint4 gv[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                base[r] = ((int64_t)bb[r] * S + (qi < S ? qi : 0)) * Cn + h * D + qtr * 8;
                gv[r] = __ldg(reinterpret_cast<const uint4 *>(p.gate + base[r]));   // in flight while the last product retires
            }
            float *xw = xch + (i & 1) * (NR * NQ * BM);
#pragma unroll
            for (int r = 0; r < NR; ++r) xw[(r * NQ + qtr) * BM + row] = m2[r];
            __syncwarp();
            if (lane == 0) mbar_arrive(x_full);                      // this warp's maxima are written
            if (!mbar_wait_warp(o_final, (uint32_t)(i & 1), p.err, 29) ||
                !mbar_wait_warp(x_full, (uint32_t)(i & 1), p.err, 31)) {     // maxima of all quarters visible
                ok = false;
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                uint32_t oa[NQ][8], la[NQ];
#pragma unroll
                for (int c = 0; c < NQ; ++c) {
                    const uint32_t col = t_lane + O_COL + (r * NQ + c) * O_STRIDE;
                    tmem_ld_32x8(col + qtr * 8, oa[c]);
                    la[c] = tmem_ld_32x1(col + 32);
                }
                tmem_ld_wait();
                if (r == NR - 1) {
                    // every accumulator of this item has been read by this warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(o_free);
                }
                float mq[NQ], mm = -INFINITY;
#pragma unroll
                for (int c = 0; c < NQ; ++c) {
                    mq[c] = xw[(r * NQ + c) * BM + row];
                    mm = fmaxf(mm, mq[c]);
                }
                float fq[NQ], den = 0.f;
#pragma unroll
                for (int c = 0; c < NQ; ++c) {
                    fq[c] = ex2_approx(mq[c] - mm);
                    den += __uint_as_float(la[c]) * fq[c];
                }
                const float inv = 1.0f / den;
#pragma unroll
                for (int c = 0; c < NQ; ++c) fq[c] *= inv;
                if (qi < S && (r == 0 || b1 != b0)) {
                    const uint32_t gw[4] = {gv[r].x, gv[r].y, gv[r].z, gv[r].w};
                    uint32_t ow[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float a0 = 0.f, a1 = 0.f;
#pragma unroll
                        for (int c = 0; c < NQ; ++c) {
                            a0 += __uint_as_float(oa[c][2 * j]) * fq[c];
                            a1 += __uint_as_float(oa[c][2 * j + 1]) * fq[c];
                        }
                        // the weighted average is stored as bf16 before gating in the reference (:128-133)
                        const uint32_t wa = pack_bf16x2(a0, a1);
                        float s0 = bf16lo_to_f32(gw[j]), s1 = bf16hi_to_f32(gw[j]);
                        if (!p.gate_is_sigmoid) {
                            s0 = 1.0f / (1.0f + ex2_approx(-s0 * kLog2e));
                            s1 = 1.0f / (1.0f + ex2_approx(-s1 * kLog2e));
                        }
                        ow[j] = pack_bf16x2(bf16lo_to_f32(wa) * s0, bf16hi_to_f32(wa) * s1);
                    }
                    *reinterpret_cast<uint4 *>(p.avg + base[r]) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
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

int sm_count_attn()
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

template <bool HAS_NB>
bool launch_one(cudaStream_t stream, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tvt,
                const CUtensorMap &tnb, const AttnParams &p)
{
    static bool configured = false;
    if (!configured) {
        KUTACC_CUDA(cudaFuncSetAttribute(attn_tc_kernel<HAS_NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured = true;
    }
    const unsigned grid = (unsigned)std::min<int64_t>(p.n_items, std::max(1, sm_count_attn() - runtime().sm_margin));
    KernelTimer timer__("attn_core", stream);
    attn_tc_kernel<HAS_NB><<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tvt, tnb, p);
    count_launch();
    return true;
}

}  // namespace

bool tcgen05_attn_core_bf16(cudaStream_t stream, const void *q, const void *k, const void *vt, int64_t vt_pitch,
                            const void *gate, const void *bias, int64_t bias_stride0, const void *nb,
                            int64_t nb_stride_h, int64_t nb_stride_q, void *avg, int B, int S, int H, int Dh,
                            float scale, bool gate_is_sigmoid)
{
    if (Dh != D || vt_pitch % 8 != 0) return false;
    if (nb && ((nb_stride_h % 8) || (nb_stride_q % 8) || ((uintptr_t)nb % 16))) return false;
    if ((((uintptr_t)gate | (uintptr_t)avg) & 15u) != 0) return false;
    const int64_t n_qt = (S + BM - 1) / BM, n_items = n_qt * H * ((B + NR - 1) / NR);
    if (n_items > INT32_MAX / 64) return false;
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
    p.B = B;
    p.n_qt = (int)n_qt;
    p.n_items = (int)n_items;
    p.scale = scale;
    p.gate_is_sigmoid = gate_is_sigmoid ? 1 : 0;
    const uint64_t Su = (uint64_t)S, BH = (uint64_t)B * H;
    CUtensorMap tq, tk, tvt, tnb;
    if (!make_tensor_map_bf16_3d(&tq, q, D, Su, BH, D, Su * D, D, BM, 64)) return false;
    if (!make_tensor_map_bf16_3d(&tk, k, D, Su, BH, D, Su * D, D, BN, 64)) return false;
    if (!make_tensor_map_bf16_3d(&tvt, vt, Su, D, BH, (uint64_t)vt_pitch, (uint64_t)D * vt_pitch, BN, D, 128)) return false;
    if (nb) {
        if (!make_tensor_map_bf16_3d(&tnb, nb, Su, Su, (uint64_t)H, (uint64_t)nb_stride_q, (uint64_t)nb_stride_h, BN, BM,
                                     128))
            return false;
        return launch_one<true>(stream, tq, tk, tvt, tnb, p);
    }
    tnb = tk;
    return launch_one<false>(stream, tq, tk, tvt, tnb, p);
}

}  // namespace dev
}  // namespace kutacc
