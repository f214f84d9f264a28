// Fused gated-attention core on the fifth-generation tensor cores (head size 32).
//
// A work item is (batch row b, head h, 128 queries). The kernel is persistent: two CTAs per SM each take
// items from an atomic counter until the list is exhausted (a CTA whose SM was busy at launch takes fewer
// items instead of finishing late), and every pipeline below keeps running across item boundaries, so the
// loads and the first Q.K^T of the next item overlap the epilogue of the current one. Both matrix products run
// on tcgen05.mma with accumulators in tensor memory, issued by one elected lane; the softmax runs on the
// logits read back with tcgen05.ld. The S x S logits never leave the SM.
//
//   warp 0     producer: takes the next item number and publishes it to the other roles; TMA tile loads
//              (hardware swizzle) of Q (double-buffered across items) and, per
//              64-key tile, K [64 x 32], V^T [32 x 64] and the 128 x 64 pair-bias tile into a 3-stage ring;
//              its lanes also convert the tile's 64 mask-bias values to fp32
//   warp 1     MMA issuer: S = Q.K^T (M 128, N 64, K 32) into TMEM columns 0..63; then two products
//              O_h += P[:, 32h..32h+31] . V^T[:, 32h..32h+31]^T (M 128, N 48, K 32), h = 0, 1, into two
//              separate TMEM accumulators. Row 32 of the V^T operand is all ones, so column 32 of each O_h
//              accumulates the row sum of the bf16 probabilities for free
//   warps 2-9  softmax: two threads per query row, one per 32-key half of every tile (split-key online
//              softmax: each half keeps its own running max and its own accumulator, merged once per item).
//              A thread pulls its 32 logits out of TMEM (S is free for the next Q.K^T once all have done
//              so), rounds each raw logit to bf16 as the reference's logits scratch does
//              (src/attention/gating_attention.cpp:97-101), forms x = logit*scale + bias + pair_bias in
//              fp32 in the reference's order (:112-117), and writes P = exp(x - max) as bf16 over the
//              pair-bias values it has just consumed (same row, same swizzled chunks), which is the A
//              operand of P.V^T. After the first tile of an item P is formed against the running max
//              chunk by chunk, so exp (XU pipe) overlaps the arithmetic; O_h is rescaled in TMEM and the
//              tile redone only when the max grows by more than 2^8 (a stale max cancels in the final
//              division). Item epilogue: each thread merges both halves for 16 of the 32 channels straight
//              from TMEM (only the two running maxima cross through shared memory), O / rowsum, bf16
//              (:128-133), gate (:134-147; with gate_is_sigmoid the projection kernel has already applied the
//              sigmoid and this is one multiply), 32-byte row stores.
//
// A second design was built and measured against this one: one CTA per SM, two batch rows per work item sharing the
// pair-bias tile, four threads per query row, all 512 tensor-memory columns in use. It issues a quarter fewer
// instructions per logit and moves a third less data from L2, and runs 1 to 8 % slower on the benchmark shapes:
// the kernel is bound by instruction latency at 16 softmax warps per SM, which neither design changes.
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
constexpr int BN = 64;                // keys per tile
constexpr int NST = 3;                // ring depth
constexpr int VT_ROWS = 48;           // 32 channels + the ones row + zero padding to a multiple of 16
constexpr int Q_BYTES = BM * D * 2;           // 8 KB, 64-byte rows, 64-byte swizzle (two buffers)
constexpr int K_BYTES = BN * D * 2;           // 4 KB, 64-byte rows
constexpr int VT_BYTES = VT_ROWS * BN * 2;    // 6 KB, 128-byte rows (TMA fills the first 32)
constexpr int NB_BYTES = BM * BN * 2;         // 16 KB, 128-byte rows: pair bias in, probabilities out (in place)
constexpr int MB_BYTES = 1024;                // 64 floats, padded
constexpr int STAGE_BYTES = K_BYTES + VT_BYTES + NB_BYTES + MB_BYTES;
constexpr int OFF_STAGE = 2 * Q_BYTES;
constexpr int OFF_XCH = OFF_STAGE + NST * STAGE_BYTES;      // running maxima of both halves, two item parities
constexpr int XCH_BYTES = 2 * 2 * BM * 4;
constexpr int OFF_BAR = OFF_XCH + XCH_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int SOFTMAX_WARPS = 8;
constexpr int THREADS = (2 + SOFTMAX_WARPS) * 32;
constexpr int TMEM_COLS = 256;
constexpr int S_COL = 0, O_COL = 64, O_STRIDE = VT_ROWS;   // O_0 at 64..111, O_1 at 112..159
constexpr float kRescaleThreshold = 8.0f;     // log2 units

struct AttnParams {
    const __nv_bfloat16 *gate;        // [B, S, H*D]
    const __nv_bfloat16 *bias;        // [B, S] (row stride bias_stride0)
    __nv_bfloat16 *avg;               // [B, S, H*D]
    int64_t bias_stride0;
    int *err;
    int S, H, B;
    int n_qt;                         // query tiles per (b, h)
    int n_items;                      // B * H * n_qt
    int gate_is_sigmoid;              // gate already holds bf16(sigmoid(bf16(x.Wg + bg)))
    int nb_head_inner;                // pair-bias tensor map has the dimensions (key, head, query): the heads of a
                                      // query row lie closer together than the rows (a [S, H, S] storage)
    int *counter;                     // [0] next work item of this launch, [1] CTAs that have finished (both zero at
                                      // launch; the last CTA to finish zeroes them again)
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

template <bool HAS_NB>
__global__ void __launch_bounds__(THREADS, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_vt, const __grid_constant__ CUtensorMap tm_nb,
               const AttnParams p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *smem_gen = smem_raw + (smem - smem_u32(smem_raw));
    auto q_buf = [&](int i) { return smem + (uint32_t)(i & 1) * Q_BYTES; };
    auto stage_base = [&](int s) { return smem + OFF_STAGE + (uint32_t)s * STAGE_BYTES; };
    const uint32_t bar = smem + OFF_BAR;
    auto kv_full = [&](int s) { return bar + 8u * (uint32_t)s; };
    auto kv_empty = [&](int s) { return bar + 8u * (uint32_t)(NST + s); };
    auto p_full = [&](int s) { return bar + 8u * (uint32_t)(2 * NST + s); };
    auto q_full = [&](int i) { return bar + 8u * (uint32_t)(3 * NST + (i & 1)); };
    auto q_empty = [&](int i) { return bar + 8u * (uint32_t)(3 * NST + 2 + (i & 1)); };
    const uint32_t s_full = bar + 8u * (3 * NST + 4), s_free = s_full + 8, pv_done = s_full + 16, o_final = s_full + 24,
                   o_free = s_full + 32, x_full = s_full + 40, tmem_slot = s_full + 48;
    auto it_full = [&](int i) { return s_full + 56u + 8u * (uint32_t)(i & 3); };      // item id of item i has been written
    const uint32_t item_ring = s_full + 88;                                          // four ints

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.S;
    const int nkt = (S + BN - 1) / BN;
    // Work items are handed out through an atomic counter in global memory: the producer warp takes the next
    // item number, publishes it to the other roles through a ring of four shared-memory words (one mbarrier each),
    // and publishes -1 when the list is exhausted. A CTA that starts late (its SM was busy with another kernel, a
    // collective running beside this one for instance) simply takes fewer items instead of finishing late.
    // Ring depth: the producer writes slot i & 3 after its wait for Q buffer i & 1 to be free, i.e. after the MMA
    // role has finished item i - 2, by which time every role has long read the number of item i - 4.
    auto decode = [&](int w, int &q0, int &h, int &b) {
        const int qt = w % p.n_qt, hb = w / p.n_qt;
        q0 = qt * BM;
        h = hb % p.H;
        b = hb / p.H;
    };
    // item number of this CTA's i-th item, or -1 (bounded wait; -2 on a timeout)
    auto item_of = [&](int i, int code) -> int {
        if (!mbar_wait_warp(it_full(i), (uint32_t)((i >> 2) & 1), p.err, code)) return -2;
        int w;
        asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(w) : "r"(item_ring + 4u * (uint32_t)(i & 3)));
        return w;
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
        for (int i = 0; i < 4; ++i) mbar_init(it_full(i), 1);
        fence_barrier_init();
    }
    // static rows 32..47 of every V^T stage: row 32 = 1.0 (row-sum column of O), rows 33..47 = 0
    for (int i = threadIdx.x; i < NST * 16 * (BN * 2 / 16); i += THREADS) {
        const int s = i / (16 * 8), rem = i % (16 * 8), row = 32 + rem / 8, ch = rem % 8;
        const uint32_t v = row == 32 ? 0x3F803F80u : 0u;
        uint4 *dst = reinterpret_cast<uint4 *>(smem_gen + OFF_STAGE + s * STAGE_BYTES + K_BYTES + row * 128 + ch * 16);
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
        int g = 0;                                      // tiles issued so far (all items)
        bool ok = true;
        for (int i = 0; ok; ++i) {
            int w = 0;
            if (lane == 0) w = atomicAdd(p.counter, 1);
            w = __shfl_sync(0xffffffffu, w, 0);
            const bool have = w < p.n_items;
            if (i >= 2 && !mbar_wait_warp(q_empty(i), (uint32_t)(((i >> 1) - 1) & 1), p.err, 20)) break;
            if (lane == 0) {
                asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(item_ring + 4u * (uint32_t)(i & 3)), "r"(have ? w : -1) : "memory");
                mbar_arrive(it_full(i));                               // releases the store above
            }
            __syncwarp();
            if (!have) break;
            int q0, h, b;
            decode(w, q0, h, b);
            const int bh = b * p.H + h;
            if (lane == 0) {
                mbar_arrive_expect_tx(q_full(i), Q_BYTES);
                tma_load_3d(q_buf(i), &tm_q, q_full(i), 0, q0, bh);
            }
            const __nv_bfloat16 *__restrict__ biasg = p.bias + (int64_t)b * p.bias_stride0;
            for (int kt = 0; kt < nkt; ++kt, ++g) {
                const int s = g % NST;
                if (g >= NST && !mbar_wait_warp(kv_empty(s), (uint32_t)((g / NST - 1) & 1), p.err, 21)) {
                    ok = false;
                    break;
                }
                const uint32_t st = stage_base(s);
                const int k0 = kt * BN;
                if (lane == 0) {
                    mbar_arrive_expect_tx(kv_full(s), K_BYTES + BN * D * 2 + (HAS_NB ? NB_BYTES : 0));
                    tma_load_3d(st, &tm_k, kv_full(s), 0, k0, bh);
                    tma_load_3d(st + K_BYTES, &tm_vt, kv_full(s), k0, 0, bh);
                    if (HAS_NB) {
                        if (p.nb_head_inner)
                            tma_load_3d(st + K_BYTES + VT_BYTES, &tm_nb, kv_full(s), k0, h, q0);
                        else
                            tma_load_3d(st + K_BYTES + VT_BYTES, &tm_nb, kv_full(s), k0, q0, h);
                    }
                }
                float *mb = reinterpret_cast<float *>(smem_gen + OFF_STAGE + s * STAGE_BYTES + K_BYTES + VT_BYTES + NB_BYTES);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int key = k0 + lane + 32 * j;
                    mb[lane + 32 * j] = key < S ? __bfloat162float(biasg[key]) : -INFINITY;
                }
                mbar_arrive(kv_full(s));
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        constexpr uint32_t idesc_s = make_instr_desc_bf16(BM, BN);
        constexpr uint32_t idesc_o = make_instr_desc_bf16(BM, VT_ROWS);
        // S = Q_i . K_g^T for global tile g of item i
        auto issue_qk = [&](int g, int i, bool first_of_item) -> bool {
            const int s = g % NST;
            if (first_of_item && !mbar_wait_warp(q_full(i), (uint32_t)((i >> 1) & 1), p.err, 22)) return false;
            if (!mbar_wait_warp(kv_full(s), (uint32_t)((g / NST) & 1), p.err, 23)) return false;
            if (g > 0 && !mbar_wait_warp(s_free, (uint32_t)((g - 1) & 1), p.err, 24)) return false;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t kb = stage_base(s), qb = q_buf(i);
#pragma unroll
                for (int k = 0; k < D / 16; ++k)
                    tc_mma_bf16(tmem_base + S_COL, make_smem_desc_kmajor(qb + k * 32, 64),
                                make_smem_desc_kmajor(kb + k * 32, 64), idesc_s, k > 0 ? 1u : 0u);
                tc_commit(s_full);
            }
            __syncwarp();
            return true;
        };
        bool more = item_of(0, 32) >= 0;                 // this role needs only to know whether an item exists
        bool ok = more ? issue_qk(0, 0, true) : true;
        int g = 0;
        for (int i = 0; more && ok; ++i) {
            for (int kt = 0; kt < nkt && ok; ++kt, ++g) {
                const int s = g % NST;
                // look one tile ahead in the stream (possibly the first tile of the next item): its Q.K^T
                // overlaps the softmax of tile g
                if (kt + 1 < nkt) {
                    ok = issue_qk(g + 1, i, false);
                } else {
                    const int nxt = item_of(i + 1, 33);
                    more = nxt >= 0;
                    ok = nxt != -2 && (!more || issue_qk(g + 1, i + 1, true));
                }
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
                    const uint32_t vb = stage_base(s) + K_BYTES, pb = vb + VT_BYTES;
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k)    // k16 steps 0,1 -> O_0 (keys 0..31), 2,3 -> O_1 (keys 32..63)
                        tc_mma_bf16(tmem_base + O_COL + (k >> 1) * O_STRIDE, make_smem_desc_kmajor(pb + k * 32, 128),
                                    make_smem_desc_kmajor(vb + k * 32, 128), idesc_o, (kt > 0 || (k & 1)) ? 1u : 0u);
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
        const int half = (warp - 2) >> 2;                // which 32 keys of every tile this thread owns
        const int row = quad * 32 + lane;                // query row inside the tile
        const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t o_col = t_lane + O_COL + half * O_STRIDE;
        const float scale = p.scale;
        const uint64_t scale2 = pack_f32x2(scale, scale), log2e2 = pack_f32x2(kLog2e, kLog2e);
        bool ok = true;
        // per-thread shared-memory addresses of stage 0; other stages add a multiple of STAGE_BYTES
        const uint32_t st0 = smem + OFF_STAGE;
        uint32_t nb_addr[4];                             // this row's 4 swizzled 16-byte chunks (pair bias in, P out)
#pragma unroll
        for (int c = 0; c < 4; ++c)
            nb_addr[c] = st0 + K_BYTES + VT_BYTES + (uint32_t)row * 128 + (uint32_t)(((half * 4 + c) ^ (row & 7)) << 4);
        const uint32_t mb_addr = st0 + K_BYTES + VT_BYTES + NB_BYTES + half * 128;
        float *xch = reinterpret_cast<float *>(smem_gen + OFF_XCH);      // [item parity][half][row]
        float m2 = -INFINITY;                            // running (possibly stale) max of this half, log2 units

        // one tile of the softmax: global tile g, tile kt of its item
        auto do_tile = [&](const int g, const int kt) -> bool {
            const int s = g % NST;
            const uint32_t soff = (uint32_t)s * STAGE_BYTES;
            if (!mbar_wait_warp(s_full, (uint32_t)(g & 1), p.err, 26)) return false;
            tc_fence_after();
            uint32_t sr[32];
            tmem_ld_32x32(t_lane + S_COL + half * 32, sr);
            const bool landed = mbar_wait_warp(kv_full(s), (uint32_t)((g / NST) & 1), p.err, 27);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free);
            if (!landed) return false;

            // x = bf16(logit)*scale + bias (+ pair bias) for 8 keys; keeps x in sr and tracks the tile max
            float tmax = -INFINITY;
            auto x_chunk = [&](const int c) {
                const float4 mb0 = lds128_f32(mb_addr + soff + c * 32), mb1 = lds128_f32(mb_addr + soff + c * 32 + 16);
                const float mbv[8] = {mb0.x, mb0.y, mb0.z, mb0.w, mb1.x, mb1.y, mb1.z, mb1.w};
                uint32_t nbw[4] = {0, 0, 0, 0};
                if (HAS_NB) {
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(nbw[0]), "=r"(nbw[1]), "=r"(nbw[2]), "=r"(nbw[3])
                                 : "r"(nb_addr[c] + soff));
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i0 = c * 8 + 2 * j;
                    // the raw logit is stored as bf16 by the reference: one cvt gives its fp32 image. The two
                    // keys of a pair go through the packed fp32 pipe (one issue slot for both).
                    uint64_t x2 = fma_f32x2(pack_f32x2(round_to_bf16_f32(__uint_as_float(sr[i0])),
                                                       round_to_bf16_f32(__uint_as_float(sr[i0 + 1]))),
                                            scale2, pack_f32x2(mbv[2 * j], mbv[2 * j + 1]));
                    if (HAS_NB) x2 = add_f32x2(x2, pack_f32x2(bf16lo_to_f32(nbw[j]), bf16hi_to_f32(nbw[j])));
                    float x0, x1;
                    unpack_f32x2(x2, x0, x1);
                    sr[i0] = __float_as_uint(x0);
                    sr[i0 + 1] = __float_as_uint(x1);
                    tmax = fmax3(tmax, x0, x1);
                }
            };
            // P = exp2(x*log2e - m2) for 8 keys -> bf16 -> over this thread's pair-bias chunk (A operand of P.V^T)
            auto p_chunk = [&](const int c, const float mneg) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i0 = c * 8 + 2 * j;
                    float e0, e1;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[i0]), __uint_as_float(sr[i0 + 1])), log2e2,
                                           pack_f32x2(mneg, mneg)), e0, e1);
                    w[j] = pack_bf16x2(ex2_approx(e0), ex2_approx(e1));
                }
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(nb_addr[c] + soff), "r"(w[0]), "r"(w[1]),
                             "r"(w[2]), "r"(w[3])
                             : "memory");
            };

            if (kt == 0) {
                // first tile of an item: the max must be known before any probability is formed
#pragma unroll
                for (int c = 0; c < 4; ++c) x_chunk(c);
                // a half whose keys all lie beyond S has no max yet: park it on a finite floor
                m2 = tmax > -INFINITY ? tmax * kLog2e : -1e30f;
#pragma unroll
                for (int c = 0; c < 4; ++c) p_chunk(c, -m2);
            } else {
                // later tiles: form the probabilities against the running max straight away, chunk by chunk,
                // so that the exp (XU pipe) of one chunk overlaps the arithmetic of the next; the running max
                // may be stale by up to 2^8, which cancels in the final division
                const float mneg = -m2;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    x_chunk(c);
                    p_chunk(c, mneg);
                }
                const float t2 = tmax > -INFINITY ? tmax * kLog2e : -1e30f;
                const bool grow = t2 > m2 + kRescaleThreshold;
                if (__any_sync(0xffffffffu, grow)) {
                    // rare: the max of some row grew past the threshold. Rescale those rows of O_half (and
                    // their row-sum column) and redo this tile's probabilities against the new max. The
                    // previous tile's P.V^T must have retired first (this warp is at most one phase behind
                    // pv_done here: s_full(g) implies that the product of tile g-2 has retired).
                    if (!mbar_wait_warp(pv_done, (uint32_t)((g - 1) & 1), p.err, 28)) return false;
                    tc_fence_after();
                    const float f = grow ? ex2_approx(m2 - t2) : 1.0f;
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
                    tc_fence_before();
                    if (grow) m2 = t2;
#pragma unroll
                    for (int c = 0; c < 4; ++c) p_chunk(c, -m2);
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(s));
            return true;
        };

        int g = 0;
        for (int i = 0; ok; ++i) {
            const int w = item_of(i, 34);
            if (w < 0) break;
            int q0, h, b;
            decode(w, q0, h, b);
            for (int kt = 0; kt < nkt && ok; ++kt, ++g) ok = do_tile(g, kt);
            if (!ok) break;

            // ---- item epilogue: this thread finishes channels [16*half, 16*half + 16) of its row ----
            const int qi = q0 + row;
            const int Cn = p.H * D;
            const int64_t base = ((int64_t)b * S + (qi < S ? qi : 0)) * Cn + h * D + half * 16;
            const uint4 *gp = reinterpret_cast<const uint4 *>(p.gate + base);
            const uint4 gv0 = __ldg(gp), gv1 = __ldg(gp + 1);         // in flight while the last product retires
            float *xw = xch + (i & 1) * 2 * BM;
            xw[half * BM + row] = m2;
            __syncwarp();
            if (lane == 0) mbar_arrive(x_full);                      // this warp's maxima are written
            if (!mbar_wait_warp(o_final, (uint32_t)(i & 1), p.err, 29) ||
                !mbar_wait_warp(x_full, (uint32_t)(i & 1), p.err, 31)) {     // maxima of both halves visible (bounded wait)
                ok = false;
                break;
            }
            tc_fence_after();
            uint32_t oa[16], ob[16];
            tmem_ld_32x16(t_lane + O_COL + half * 16, oa);                       // O_0, this thread's channels
            tmem_ld_32x16(t_lane + O_COL + O_STRIDE + half * 16, ob);            // O_1
            const uint32_t la = tmem_ld_32x1(t_lane + O_COL + 32), lb = tmem_ld_32x1(t_lane + O_COL + O_STRIDE + 32);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free);                      // this warp has read its part of both accumulators
            const float mA = xw[row], mB = xw[BM + row];
            const float mm = fmaxf(mA, mB);
            const float fA = ex2_approx(mA - mm), fB = ex2_approx(mB - mm);
            const float inv = 1.0f / (__uint_as_float(la) * fA + __uint_as_float(lb) * fB);
            const float cA = fA * inv, cB = fB * inv;
            if (qi < S) {
                const uint32_t gw[8] = {gv0.x, gv0.y, gv0.z, gv0.w, gv1.x, gv1.y, gv1.z, gv1.w};
                uint32_t ow[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // the weighted average is stored as bf16 before gating in the reference (:128-133)
                    const uint32_t wa = pack_bf16x2(__uint_as_float(oa[2 * j]) * cA + __uint_as_float(ob[2 * j]) * cB,
                                                    __uint_as_float(oa[2 * j + 1]) * cA + __uint_as_float(ob[2 * j + 1]) * cB);
                    float s0 = bf16lo_to_f32(gw[j]), s1 = bf16hi_to_f32(gw[j]);
                    if (!p.gate_is_sigmoid) {
                        s0 = 1.0f / (1.0f + ex2_approx(-s0 * kLog2e));
                        s1 = 1.0f / (1.0f + ex2_approx(-s1 * kLog2e));
                    }
                    ow[j] = pack_bf16x2(bf16lo_to_f32(wa) * s0, bf16hi_to_f32(wa) * s1);
                }
                uint4 *op = reinterpret_cast<uint4 *>(p.avg + base);
                op[0] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                op[1] = make_uint4(ow[4], ow[5], ow[6], ow[7]);
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
    // The last CTA to get here puts the work counter back to zero for the launch that uses it next (every CTA has
    // taken its last item number by now: the producer's atomics precede the barrier above).
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.counter + 1, 1) == (int)gridDim.x - 1) {
            __threadfence();
            p.counter[0] = 0;
            p.counter[1] = 0;
            __threadfence();
        }
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
    const unsigned grid = (unsigned)std::min<int64_t>(p.n_items, 2 * std::max(1, sm_count_attn() - runtime().sm_margin));
    // One pair of counters per STREAM: launches on one stream run one after another, so they can share a pair (the
    // last CTA of a launch zeroes it again), while launches on different streams may overlap and must not. Up to 63
    // streams per device get a pair of their own; further streams share the last pair, which is only safe while they
    // do not run attention kernels at the same time.
    constexpr int kCounters = 64;
    static int *counters[64] = {};                       // per device
    static cudaStream_t owner[64][kCounters] = {};
    static int owners[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return false;
    if (counters[dev] == nullptr) {
        int *c = nullptr;
        KUTACC_CUDA(cudaMalloc(&c, 2 * kCounters * sizeof(int)));
        if (c == nullptr) return false;
        KUTACC_CUDA(cudaMemset(c, 0, 2 * kCounters * sizeof(int)));
        counters[dev] = c;
    }
    int slot = -1;
    for (int i = 0; i < owners[dev]; ++i)
        if (owner[dev][i] == stream) {
            slot = i;
            break;
        }
    if (slot < 0) {
        if (owners[dev] < kCounters - 1) {
            slot = owners[dev]++;
            owner[dev][slot] = stream;
        } else {
            slot = kCounters - 1;
        }
    }
    AttnParams q = p;
    q.counter = counters[dev] + 2 * slot;
    KernelTimer timer__("attn_core", stream);
    attn_tc_kernel<HAS_NB><<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tvt, tnb, q);
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
    const int64_t n_qt = (S + BM - 1) / BM, n_items = n_qt * H * B;
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
    p.counter = nullptr;
    const uint64_t Su = (uint64_t)S, BH = (uint64_t)B * H;
    CUtensorMap tq, tk, tvt, tnb;
    if (!make_tensor_map_bf16_3d(&tq, q, D, Su, BH, D, Su * D, D, BM, 64)) return false;
    if (!make_tensor_map_bf16_3d(&tk, k, D, Su, BH, D, Su * D, D, BN, 64)) return false;
    if (!make_tensor_map_bf16_3d(&tvt, vt, Su, D, BH, (uint64_t)vt_pitch, (uint64_t)D * vt_pitch, BN, D, 128)) return false;
    p.nb_head_inner = 0;
    if (nb) {
        if (nb_stride_h < nb_stride_q) {
            // heads closer together than query rows: dimensions in the order of their strides (key, head, query); the
            // box takes one head, so the tile in shared memory is the same 128 rows x 64 keys
            p.nb_head_inner = 1;
            if (!make_tensor_map_bf16_3d(&tnb, nb, Su, (uint64_t)H, Su, (uint64_t)nb_stride_h, (uint64_t)nb_stride_q, BN, 1,
                                         128, BM))
                return false;
        } else if (!make_tensor_map_bf16_3d(&tnb, nb, Su, Su, (uint64_t)H, (uint64_t)nb_stride_q, (uint64_t)nb_stride_h, BN,
                                            BM, 128)) {
            return false;
        }
        return launch_one<true>(stream, tq, tk, tvt, tnb, p);
    }
    tnb = tk;
    return launch_one<false>(stream, tq, tk, tvt, tnb, p);
}

}  // namespace dev
}  // namespace kutacc
