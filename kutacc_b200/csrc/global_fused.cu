// Extra-MSA global column attention in ONE pass over HBM (64 channels, 8 heads x 8).
//
// Reference path: src/attention/global_attention.cpp:30-164 reads the [B, S, 64] activations five times
// and materialises k, v and the gate. A batch column is 128 * S bytes (655 KB at S = 5120), which fits in
// the shared memory of a few SMs. Here a thread-block cluster owns one column at a time: each CTA of the
// cluster keeps a slab of the column's rows in its shared memory (loaded once by TMA), the three stages
// of the operator run out of that slab, and the result is written over the slab and stored by TMA:
//   pool : masked sum of the rows                                                   (:44-75)
//          -> the CTAs exchange their partial sums through distributed shared memory
//   core : q = q_avg.Wq^T; k, v, logits of all heads, online softmax, weighted v    (:76-89, :96-133)
//          -> the CTAs exchange their partial softmax states the same way
//   out  : gate = x.Wg^T + bg; out = (sigmoid(gate) * wa).Wo^T + bo                 (:90-94, :134-163)
// HBM sees one read of x and one write of out; no scratch in global memory is used.
//
// Shared memory is a ring of 16 KB slots (128 rows x 128 bytes, 128-byte TMA swizzle). A column uses
// `mych` consecutive slots in each CTA, the next column the slots after them; one thread of an extra
// warp issues every TMA load and store. A slot is reloaded as soon as the store out of it has been read,
// so the next column streams in while the current one is still being written out.
//
// bf16 rounding points of the reference that are kept: q_avg, q, k, v, logits, wa, gate, gated gate, out.
// Probabilities are rounded to bf16 un-normalised (they feed the tensor cores); the reference rounds
// them after normalising.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"
#include "tcgen05_utils.cuh"
#include "tma_utils.cuh"

#include <algorithm>

namespace kutacc {
namespace dev {

namespace {

constexpr int FC = 64;                 // channels
constexpr int FH = 8, FD = 8;          // heads x head size
constexpr int CH_ROWS = 128;           // rows per slot
constexpr int CH_BYTES = CH_ROWS * FC * 2;
constexpr int MAX_CTA = 8;             // portable cluster size limit
constexpr int CT = 1;                  // tiles per step of the core loop

// Two shapes of CTA:
//   Wide  : 16 computing warps, 11 slots, one CTA per SM. A column of up to 11 * 128 * 8 rows.
//   Half  : 8 computing warps, 5 slots, two CTAs per SM, so that the stages of two columns overlap on
//           every SM (the output stage is bound by the MUFU pipe, pooling and the softmax by latency).
//           A column of up to 5 * 128 * 8 = 5120 rows; Wq is read from global memory.
template <int NCW_, int NSLOT_, bool WQ_SMEM_, int MIN_CTAS_, int BOUND_THREADS_>
struct Cfg {
    static constexpr int NCW = NCW_;                    // computing warps
    static constexpr int NSLOT = NSLOT_;                // slots in the ring
    static constexpr int IO_WARP = NCW_, MMA_WARP = NCW_ + 1;
    static constexpr int NTHREADS = (NCW_ + 2) * 32;
    static constexpr int NPG = NCW_ / 8;                // groups of 8 warps in pool and core: group g takes chunks c = g (mod NPG)
    static constexpr int NGRP = NCW_ / 4;               // groups of 4 warps (128 rows) in the output stage
    static constexpr int NACC = 2 * NGRP;               // TMEM accumulators (128 lanes x 64 fp32 columns), two per group
    static constexpr int TMEM_COLS = NACC * FC;
    static constexpr int MAX_ROWS = NSLOT_ * CH_ROWS;
    static constexpr bool WQ_SMEM = WQ_SMEM_;
    static constexpr int MIN_CTAS = MIN_CTAS_;
    // thread count handed to __launch_bounds__: registers are split between the four schedulers of an SM by whole
    // warps, so two 10-warp CTAs need the register budget of two 12-warp CTAs (3 warps per scheduler each)
    static constexpr int BOUND_THREADS = BOUND_THREADS_;
};
using WideCfg = Cfg<16, 11, true, 1, 18 * 32>;
using HalfCfg = Cfg<8, 5, false, 2, 12 * 32>;

template <class K>
struct __align__(1024) FusedSmem {
    unsigned char slot[K::NSLOT][CH_BYTES];
    __nv_bfloat16 wg[FC * FC];         // 16-byte chunks swizzled by row: the K-major 128-byte-swizzle operand layout
    __nv_bfloat16 wo[FC * FC];
    __nv_bfloat16 wq[K::WQ_SMEM ? FC * FC : 8];
    __nv_bfloat16 wk[FD * FC];
    __nv_bfloat16 wv[FD * FC];
    unsigned short mask[2][K::MAX_ROWS];  // bf16 bits of this CTA's rows of the mask, double-buffered by column
    float pool_part[MAX_CTA][FC + 1];  // written by the CTA of that rank (remote stores)
    float core_part[MAX_CTA][FH][2 + FD];
    union {                            // pooling and the softmax merge never overlap in time
        float red[K::NCW][FC + 1];
        float s_part[K::NCW][FH][1 + FD];
    };
    float s_m[K::NCW][FH];
    __align__(16) float qa[FC], q[FC], hwa[FC], bg[FC], bo[FC];   // hwa = wa / 2
    uint64_t full[K::NSLOT], done[K::NSLOT], pool_bar, core_bar;
    uint64_t g1_done[K::NACC], p_ready[K::NACC], g2_done[K::NACC], d_free[K::NACC];
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(FusedSmem<WideCfg>) + 1024 <= 232448, "shared memory of one CTA");
static_assert(2 * (sizeof(FusedSmem<HalfCfg>) + 1024 + 1024) <= 233472, "two CTAs per SM");

struct FusedArgs {
    const __nv_bfloat16 *mask, *wq, *wk, *wv, *wg, *wo;
    const float *bg, *bo;
    int B, S;
    int ncta;        // CTAs per cluster
    int nch;         // slots (128-row chunks) per CTA and column
    int *err;
};

__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bits_to_f32(unsigned short b) { return __uint_as_float((uint32_t)b << 16); }
template <class K>
__device__ __forceinline__ void consumer_bar_t() { asm volatile("bar.sync 1, %0;\n" ::"n"(K::NCW * 32) : "memory"); }

// barrier over the consumer warps that also ORs a predicate across them
template <class K>
__device__ __forceinline__ bool consumer_bar_or_t(bool pred)
{
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %1, 0;\n"
        "bar.red.or.pred p, 1, %2, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r)
        : "r"((uint32_t)pred), "n"(K::NCW * 32)
        : "memory");
    return r != 0;
}

__device__ __forceinline__ void mma_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

// error codes of the bounded waits (reported through the host-visible error word)
constexpr int ERR_FULL = 0x4701, ERR_DONE = 0x4702, ERR_POOL = 0x4703, ERR_CORE = 0x4704, ERR_DRAIN = 0x4705,
              ERR_G1 = 0x4706, ERR_G2 = 0x4707, ERR_MMA = 0x4708;

// ---- the thread that moves data ----------------------------------------------------------------------
// Chunk `seq` (counted over all columns of this CTA) lives in slot seq % K::NSLOT. Loads run ahead of the
// consumers as far as free slots allow; a slot is free once the store out of it has been read.
template <class K>
__device__ __forceinline__ void io_thread(FusedSmem<K> &sm, const CUtensorMap *xmap, const CUtensorMap *omap,
                                          const FusedArgs &a, int cluster_id, int nclusters, int ncols, int mych,
                                          int row_base)
{
    const uint32_t slot0 = smem_u32(&sm.slot[0][0]);
    const int total = ncols * mych;
    int issued = 0, committed = 0, freed = 0;
    auto issue_loads = [&]() {
        while (issued < total && issued - K::NSLOT < freed) {
            const int j = issued / mych, c = issued - j * mych, s = issued % K::NSLOT;
            const uint32_t bar = smem_u32(&sm.full[s]);
            mbar_arrive_expect_tx(bar, CH_BYTES);
            tma_load_3d(slot0 + s * CH_BYTES, xmap, bar, 0, row_base + c * CH_ROWS, cluster_id + j * nclusters);
            ++issued;
        }
    };
    issue_loads();
    bool ok = true;
    for (int st = 0; st < total; ++st) {
        const int j = st / mych, c = st - j * mych, s = st % K::NSLOT;
        if (c == 0 && st > 0) {
            // between columns nothing else will free the last slots: wait for the stores in flight
            tma_store_wait_read<0>();
            freed = committed;
            issue_loads();
        }
        if (!mbar_wait(smem_u32(&sm.done[s]), (st / K::NSLOT) & 1, a.err, ERR_DONE)) {
            ok = false;
            break;
        }
        tma_store_3d(omap, slot0 + s * CH_BYTES, 0, row_base + c * CH_ROWS, cluster_id + j * nclusters);
        tma_store_commit();
        ++committed;
        tma_store_wait_read<2>();
        freed = max(freed, committed - 2);
        issue_loads();
    }
    if (!ok) {
        // unwind: no load may still be in flight into this CTA's shared memory when it exits
        sm.abort_flag = 1;
        for (int seq = max(0, issued - K::NSLOT); seq < issued; ++seq)
            mbar_wait(smem_u32(&sm.full[seq % K::NSLOT]), (seq / K::NSLOT) & 1, a.err, ERR_DRAIN);
    }
    tma_store_wait<0>();
}

// ---- the warps that compute --------------------------------------------------------------------------
template <class K>
__device__ __forceinline__ void consumer_warps(FusedSmem<K> &sm, const FusedArgs &a, int rank, int cluster_id,
                                               int nclusters, int ncols, int mych, int row_base)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = warp >> 3, w8 = warp & 7;
    const int g = lane >> 2, t = lane & 3;
    const int S = a.S;
    const float scale = 1.0f / sqrtf((float)FD);
    const uint32_t slot0 = smem_u32(&sm.slot[0][0]);
    const unsigned short *mask_bits = reinterpret_cast<const unsigned short *>(a.mask);
    volatile int *abort_flag = &sm.abort_flag;

    for (int j = 0; j < ncols; ++j) {
        if (consumer_bar_or_t<K>(*abort_flag != 0)) break;          // the same answer in every consumer thread
        const int b = cluster_id + j * nclusters;
        const int mb = j & 1;
        if (tid == 0) {
            mbar_arrive_expect_tx(smem_u32(&sm.pool_bar), (uint32_t)(a.ncta * (FC + 1) * 4));
            mbar_arrive_expect_tx(smem_u32(&sm.core_bar), (uint32_t)(a.ncta * FH * (2 + FD) * 4));
        }

        // the mask rows of the next column travel while this one is pooled
        unsigned short next_mask[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int r = tid + i * (K::NCW * 32);
            const bool ok = (j + 1 < ncols) && r < mych * CH_ROWS && row_base + r < S;
            next_mask[i] = ok ? __ldg(mask_bits + (int64_t)(b + nclusters) * S + row_base + r) : (unsigned short)0;
        }

        // ---- pool: masked column sums of this CTA's rows
        {
            float pacc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            float pms = 0.f;
            const int sub = lane & 7, r4 = lane >> 3;
            for (int c = grp; c < mych; c += K::NPG) {
                const int seq = j * mych + c, s = seq % K::NSLOT;
                if (!__any_sync(0xffffffffu, *abort_flag != 0) &&
                    !mbar_wait_warp(smem_u32(&sm.full[s]), (seq / K::NSLOT) & 1, a.err, ERR_FULL))
                    *abort_flag = 1;
                const uint32_t tile = slot0 + s * CH_BYTES + w8 * 16 * 128;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = r4 + 4 * i;
                    const float mv = bits_to_f32(sm.mask[mb][c * CH_ROWS + w8 * 16 + rr]);
                    uint32_t w[4];
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                                 : "r"(tile + rr * 128 + ((sub ^ (rr & 7)) << 4)));
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        pacc[2 * e] = fmaf(bf16lo_to_f32(w[e]), mv, pacc[2 * e]);
                        pacc[2 * e + 1] = fmaf(bf16hi_to_f32(w[e]), mv, pacc[2 * e + 1]);
                    }
                    if (sub == 0) pms += mv;
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                pacc[i] += __shfl_xor_sync(0xffffffffu, pacc[i], 8);
                pacc[i] += __shfl_xor_sync(0xffffffffu, pacc[i], 16);
            }
            pms += __shfl_xor_sync(0xffffffffu, pms, 8);
            pms += __shfl_xor_sync(0xffffffffu, pms, 16);
            if (lane < 8) {
#pragma unroll
                for (int i = 0; i < 8; ++i) sm.red[warp][lane * 8 + i] = pacc[i];
            }
            if (lane == 0) sm.red[warp][FC] = pms;
        }
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int r = tid + i * (K::NCW * 32);
            if (r < K::MAX_ROWS) sm.mask[mb ^ 1][r] = next_mask[i];
        }
        consumer_bar_t<K>();
        if (tid <= FC) {
            float tsum = 0.f;
#pragma unroll
            for (int w = 0; w < K::NCW; ++w) tsum += sm.red[w][tid];
            // asynchronous stores: each word credits 4 bytes to the destination CTA's barrier when it lands
            const uint32_t local = smem_u32(&sm.pool_part[rank][tid]), bar = smem_u32(&sm.pool_bar);
            for (int r = 0; r < a.ncta; ++r)
                st_async_cluster_f32(map_shared_rank(local, r), tsum, map_shared_rank(bar, r));
        }
        if (!*abort_flag && !mbar_wait(smem_u32(&sm.pool_bar), j & 1, a.err, ERR_POOL)) *abort_flag = 1;
        __syncwarp();

        // ---- q_avg and q (every CTA computes them for itself, in the same order)
        if (tid < FC) {
            float tsum = 0.f, ms = 0.f;
            for (int r = 0; r < a.ncta; ++r) {
                tsum += sm.pool_part[r][tid];
                ms += sm.pool_part[r][FC];
            }
            sm.qa[tid] = rbf(tsum * (1.0f / (ms + 1e-10f)));
        }
        consumer_bar_t<K>();
        for (int o = tid >> 3; o < FC; o += K::NCW * 4) {
            const int part = tid & 7;
            uint4 raw;
            if (K::WQ_SMEM)
                raw = *reinterpret_cast<const uint4 *>(&sm.wq[o * FC + ((part ^ (o & 7)) << 3)]);
            else
                raw = __ldg(reinterpret_cast<const uint4 *>(a.wq + o * FC) + part);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            float acc = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc = fmaf(sm.qa[part * 8 + 2 * e], bf16lo_to_f32(w[e]), acc);
                acc = fmaf(sm.qa[part * 8 + 2 * e + 1], bf16hi_to_f32(w[e]), acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (part == 0) sm.q[o] = rbf(acc);
        }
        consumer_bar_t<K>();

        // ---- core: thread (g, t) owns head g; four products chained through mma.sync fragments:
        //   k [16 x 8] = x.Wk^T, v^T [8 x 16] = Wv.x^T, logits^T [8 heads x 16] = q.k^T, wa [8 x 8] += P^T.v
        {
            uint32_t bk[4][2], av[4][2];
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                bk[ks][0] = *reinterpret_cast<const uint32_t *>(&sm.wk[g * FC + 16 * ks + 2 * t]);
                bk[ks][1] = *reinterpret_cast<const uint32_t *>(&sm.wk[g * FC + 16 * ks + 8 + 2 * t]);
                av[ks][0] = *reinterpret_cast<const uint32_t *>(&sm.wv[g * FC + 16 * ks + 2 * t]);
                av[ks][1] = *reinterpret_cast<const uint32_t *>(&sm.wv[g * FC + 16 * ks + 8 + 2 * t]);
            }
            const uint32_t aq = pack_bf16x2(sm.q[g * FD + 2 * t], sm.q[g * FD + 2 * t + 1]);
            float m_run = -INFINITY, l_run = 0.f, wa[4] = {0.f, 0.f, 0.f, 0.f};
            // CT tiles per step (independent chains of products in flight)
            for (int c = grp; c < mych; c += K::NPG * CT) {
                int loc0[CT];
                bool valid[CT];
                uint32_t tile[CT];
#pragma unroll
                for (int u = 0; u < CT; ++u) {
                    const int cu = c + K::NPG * u;
                    loc0[u] = cu * CH_ROWS + w8 * 16;            // first row of the tile within this CTA's slab
                    valid[u] = cu < mych && row_base + loc0[u] < S;
                    const int sq = j * mych + (valid[u] ? cu : c);
                    tile[u] = slot0 + (sq % K::NSLOT) * CH_BYTES + w8 * 16 * 128;
                }
                if (!valid[0]) continue;
                float kacc[CT][4], v0[CT][4], v1[CT][4];
#pragma unroll
                for (int u = 0; u < CT; ++u)
#pragma unroll
                    for (int e = 0; e < 4; ++e) kacc[u][e] = v0[u][e] = v1[u][e] = 0.f;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint32_t wvf[4] = {av[ks][0], 0u, av[ks][1], 0u};
#pragma unroll
                    for (int u = 0; u < CT; ++u) {
                        uint32_t af[4];
                        const int r = lane & 15, ci = ks * 2 + (lane >> 4);
                        ldmatrix_x4(af[0], af[1], af[2], af[3], tile[u] + r * 128 + ((ci ^ (r & 7)) << 4));
                        mma_bf16_16816(kacc[u], af, bk[ks][0], bk[ks][1]);
                        mma_bf16_16816(v0[u], wvf, af[0], af[2]);       // rows 0..7 of the tile
                        mma_bf16_16816(v1[u], wvf, af[1], af[3]);       // rows 8..15
                    }
                }
                float xv[CT][4];
                float tmax = -INFINITY;
#pragma unroll
                for (int u = 0; u < CT; ++u) {
                    float l0[4] = {0.f, 0.f, 0.f, 0.f}, l1[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_1688(l0, aq, 0u, pack_bf16x2(kacc[u][0], kacc[u][1]));
                    mma_1688(l1, aq, 0u, pack_bf16x2(kacc[u][2], kacc[u][3]));
                    const int rows[4] = {loc0[u] + 2 * t, loc0[u] + 2 * t + 1, loc0[u] + 8 + 2 * t, loc0[u] + 9 + 2 * t};
                    const float lg[4] = {l0[0], l0[1], l1[0], l1[1]};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const bool ok = valid[u] && row_base + rows[i] < S;
                        const float mbias = ok ? fmaf(bits_to_f32(sm.mask[mb][rows[i]]), 1e9f, -1e9f) : -INFINITY;
                        xv[u][i] = rbf(lg[i]) * scale + mbias;
                        tmax = fmaxf(tmax, xv[u][i]);
                    }
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run, tmax);
                const float corr = __expf(m_run - m_new);        // first step: exp(-inf) = 0
                m_run = m_new;
                float pv[CT][4];
                float psum = 0.f;
#pragma unroll
                for (int u = 0; u < CT; ++u)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        pv[u][i] = __expf(xv[u][i] - m_new);
                        psum += pv[u][i];
                    }
                l_run = l_run * corr + psum;
                wa[0] *= corr;
                wa[1] *= corr;
#pragma unroll
                for (int u = 0; u < CT; ++u) {
                    const uint32_t pa[4] = {pack_bf16x2(pv[u][0], pv[u][1]), 0u, pack_bf16x2(pv[u][2], pv[u][3]), 0u};
                    mma_bf16_16816(wa, pa, pack_bf16x2(v0[u][0], v0[u][1]), pack_bf16x2(v1[u][0], v1[u][1]));
                }
            }
            l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
            l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
            if (t == 0) {
                sm.s_m[warp][g] = m_run;
                sm.s_part[warp][g][0] = l_run;
            }
            sm.s_part[warp][g][1 + 2 * t] = wa[0];
            sm.s_part[warp][g][2 + 2 * t] = wa[1];
        }
        consumer_bar_t<K>();
        if (tid < FH * (1 + FD)) {
            const int h = tid / (1 + FD), jj = tid % (1 + FD);
            float mx = sm.s_m[0][h];
#pragma unroll
            for (int w = 1; w < K::NCW; ++w) mx = fmaxf(mx, sm.s_m[w][h]);
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < K::NCW; ++w) {
                const float f = (sm.s_m[w][h] == -INFINITY) ? 0.f : __expf(sm.s_m[w][h] - mx);
                acc += sm.s_part[w][h][jj] * f;
            }
            const uint32_t local = smem_u32(&sm.core_part[rank][h][0]);
            const uint32_t bar = smem_u32(&sm.core_bar);
            for (int r = 0; r < a.ncta; ++r) {
                const uint32_t dst = map_shared_rank(local, r), rbar = map_shared_rank(bar, r);
                st_async_cluster_f32(dst + 4 * (1 + jj), acc, rbar);
                if (jj == 0) st_async_cluster_f32(dst, mx, rbar);
            }
        }
        if (!*abort_flag && !mbar_wait(smem_u32(&sm.core_bar), j & 1, a.err, ERR_CORE)) *abort_flag = 1;
        __syncwarp();
        if (tid < FC) {
            const int h = tid >> 3, d = tid & 7;
            float mx = -INFINITY;
            for (int r = 0; r < a.ncta; ++r) mx = fmaxf(mx, sm.core_part[r][h][0]);
            float l = 0.f, av = 0.f;
            for (int r = 0; r < a.ncta; ++r) {
                const float pm = sm.core_part[r][h][0];
                const float f = (pm == -INFINITY) ? 0.f : __expf(pm - mx);
                l += sm.core_part[r][h][1] * f;
                av += sm.core_part[r][h][2 + d] * f;
            }
            sm.hwa[tid] = 0.5f * rbf(av / l);
        }
        consumer_bar_t<K>();

        // ---- out: both 64 x 64 products run on tcgen05 (issued by the MMA warp). Chunk `seq` uses TMEM
        // accumulator seq % 4 and is finished by the four warps of group seq % 4, one row per thread:
        //   D = x.Wg^T  -> gated = bf16(sigmoid(bf16(D + bg)) * wa) written over x in the slot (same
        //   K-major swizzled layout) -> D = gated.Wo^T -> out = bf16(D + bo) written over the slot -> TMA store
        {
            const int eg = warp >> 2, quarter = warp & 3;
            const int row = quarter * 32 + lane;
            const uint32_t tmem_lane = sm.tmem_base + ((uint32_t)(quarter * 32) << 16);
            // first half of a chunk's epilogue: gate -> gated rows, written over x
            auto gate_rows = [&](int seq) {
                const int k = seq & (K::NACC - 1), s = seq % K::NSLOT;
                const uint32_t par = (uint32_t)(seq / K::NACC) & 1u;
                const uint32_t rowaddr = slot0 + s * CH_BYTES + row * 128;
                const uint32_t taddr = tmem_lane + (uint32_t)(k * FC);
                if (!__any_sync(0xffffffffu, *abort_flag != 0) &&
                    !mbar_wait_warp(smem_u32(&sm.g1_done[k]), par, a.err, ERR_G1))
                    *abort_flag = 1;
                tc_fence_after();
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + half * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {          // 16-byte chunk = 8 channels
                        const int ch0 = half * 32 + q4 * 8;
                        uint32_t pk[4];
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const float4 bgv = *reinterpret_cast<const float4 *>(&sm.bg[ch0 + 4 * hh]);
                            const float4 hwv = *reinterpret_cast<const float4 *>(&sm.hwa[ch0 + 4 * hh]);
                            const float bgs[4] = {bgv.x, bgv.y, bgv.z, bgv.w}, hws[4] = {hwv.x, hwv.y, hwv.z, hwv.w};
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int i0 = q4 * 8 + hh * 4 + 2 * e;
                                float g0, g1, t0, t1, p0, p1;
                                unpack_f32x2(add_f32x2(pack_f32x2(__uint_as_float(v[i0]), __uint_as_float(v[i0 + 1])),
                                                       pack_f32x2(bgs[2 * e], bgs[2 * e + 1])), g0, g1);
                                // gate is a bf16 tensor in the reference; sigmoid(g) = 0.5 tanh(g / 2) + 0.5
                                unpack_f32x2(mul_f32x2(pack_f32x2(round_to_bf16_f32(g0), round_to_bf16_f32(g1)),
                                                       pack_f32x2(0.5f, 0.5f)), t0, t1);
                                const uint64_t hw2 = pack_f32x2(hws[2 * e], hws[2 * e + 1]);     // wa / 2
                                unpack_f32x2(fma_f32x2(pack_f32x2(tanh_approx(t0), tanh_approx(t1)), hw2, hw2), p0, p1);
                                pk[hh * 2 + e] = pack_bf16x2(p0, p1);
                            }
                        }
                        const int ci = half * 4 + q4;
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(rowaddr + ((ci ^ (row & 7)) << 4)),
                                     "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]));   // ordered by the fence below
                    }
                }
                fence_proxy_async();                 // the second product reads these rows through the async proxy
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm.p_ready[k]));
            };
            // second half: out rows, written over the gated rows, then handed to the TMA store
            auto out_rows = [&](int seq) {
                const int k = seq & (K::NACC - 1), s = seq % K::NSLOT;
                const uint32_t par = (uint32_t)(seq / K::NACC) & 1u;
                const uint32_t rowaddr = slot0 + s * CH_BYTES + row * 128;
                const uint32_t taddr = tmem_lane + (uint32_t)(k * FC);
                if (!__any_sync(0xffffffffu, *abort_flag != 0) &&
                    !mbar_wait_warp(smem_u32(&sm.g2_done[k]), par, a.err, ERR_G2))
                    *abort_flag = 1;
                tc_fence_after();
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + half * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const int ch0 = half * 32 + q4 * 8;
                        uint32_t pk[4];
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const float4 bov = *reinterpret_cast<const float4 *>(&sm.bo[ch0 + 4 * hh]);
                            const int i0 = q4 * 8 + hh * 4;
                            float o0, o1, o2, o3;
                            unpack_f32x2(add_f32x2(pack_f32x2(__uint_as_float(v[i0]), __uint_as_float(v[i0 + 1])),
                                                   pack_f32x2(bov.x, bov.y)), o0, o1);
                            unpack_f32x2(add_f32x2(pack_f32x2(__uint_as_float(v[i0 + 2]), __uint_as_float(v[i0 + 3])),
                                                   pack_f32x2(bov.z, bov.w)), o2, o3);
                            pk[hh * 2] = pack_bf16x2(o0, o1);
                            pk[hh * 2 + 1] = pack_bf16x2(o2, o3);
                        }
                        const int ci = half * 4 + q4;
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(rowaddr + ((ci ^ (row & 7)) << 4)),
                                     "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]));   // ordered by the fence below
                    }
                }
                fence_proxy_async();                 // the TMA store reads what these threads wrote
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&sm.d_free[k]));
                    mbar_arrive(smem_u32(&sm.done[s]));
                }
            };
            // this group's chunks of the column: seq = eg (mod 4). The gate of the next one is computed
            // while the tensor core forms the output product of the current one.
            const int seq0 = j * mych;
            int c = (eg - seq0) & (K::NGRP - 1);
            if (c < mych) gate_rows(seq0 + c);
            for (; c < mych; c += K::NGRP) {
                if (c + K::NGRP < mych) gate_rows(seq0 + c + K::NGRP);
                out_rows(seq0 + c);
            }
        }
    }
}

// ---- the thread that issues the tensor-core products of the output stage ---------------------------------
// In chunk order: D[seq % 4] = x.Wg^T as soon as the chunk has landed and the accumulator is free, then,
// three chunks behind, D[seq' % 4] = gated.Wo^T once the warps have written the gated rows.
template <class K>
__device__ __forceinline__ void mma_thread(FusedSmem<K> &sm, const FusedArgs &a, int ncols, int mych)
{
    const uint32_t slot0 = smem_u32(&sm.slot[0][0]);
    const uint32_t wg_addr = smem_u32(&sm.wg[0]), wo_addr = smem_u32(&sm.wo[0]);
    const uint32_t idesc = make_instr_desc_bf16(CH_ROWS, FC);
    const uint32_t tmem = sm.tmem_base;
    const int total = ncols * mych;
    int a_seq = 0, b_seq = 0;       // next chunk of the first and of the second product; both run in chunk order
    long long t0 = clock64();
    while (b_seq < total) {
        bool progress = false;
        if (a_seq < total) {
            const int k = a_seq & (K::NACC - 1), u = a_seq / K::NACC, s = a_seq % K::NSLOT;
            if ((u == 0 || mbar_try_wait(smem_u32(&sm.d_free[k]), (uint32_t)(u - 1) & 1u)) &&
                mbar_try_wait(smem_u32(&sm.full[s]), (uint32_t)(a_seq / K::NSLOT) & 1u)) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < FC / 16; ++ks)
                    tc_mma_bf16(tmem + k * FC, make_smem_desc_kmajor(slot0 + s * CH_BYTES + ks * 32, 128),
                                make_smem_desc_kmajor(wg_addr + ks * 32, 128), idesc, ks > 0 ? 1u : 0u);
                tc_commit(smem_u32(&sm.g1_done[k]));
                ++a_seq;
                progress = true;
            }
        }
        if (b_seq < a_seq) {
            const int k = b_seq & (K::NACC - 1), s = b_seq % K::NSLOT;
            if (mbar_try_wait(smem_u32(&sm.p_ready[k]), (uint32_t)(b_seq / K::NACC) & 1u)) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < FC / 16; ++ks)
                    tc_mma_bf16(tmem + k * FC, make_smem_desc_kmajor(slot0 + s * CH_BYTES + ks * 32, 128),
                                make_smem_desc_kmajor(wo_addr + ks * 32, 128), idesc, ks > 0 ? 1u : 0u);
                tc_commit(smem_u32(&sm.g2_done[k]));
                ++b_seq;
                progress = true;
            }
        }
        if (progress) {
            t0 = clock64();
        } else if (clock64() - t0 > 4000000000LL) {       // ~2 s without progress: give up
            if (a.err) atomicCAS(a.err, 0, ERR_MMA);
            sm.abort_flag = 1;
            break;
        }
    }
}

template <class K>
__global__ void __launch_bounds__(K::BOUND_THREADS, K::MIN_CTAS)
global_fused_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap omap,
                    const FusedArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    FusedSmem<K> &sm = *reinterpret_cast<FusedSmem<K> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rank = (int)cluster_cta_rank();
    const int cluster_id = blockIdx.x / a.ncta, nclusters = gridDim.x / a.ncta;
    const int row_base = rank * a.nch * CH_ROWS;
    const int mych = min(a.nch, max(0, (a.S - row_base + CH_ROWS - 1) / CH_ROWS));
    const int ncols = cluster_id < a.B ? (a.B - cluster_id + nclusters - 1) / nclusters : 0;

    if (tid == 0) {
        for (int s = 0; s < K::NSLOT; ++s) {
            mbar_init(smem_u32(&sm.full[s]), 1);
            mbar_init(smem_u32(&sm.done[s]), 4);
        }
        for (int k = 0; k < K::NACC; ++k) {
            mbar_init(smem_u32(&sm.g1_done[k]), 1);
            mbar_init(smem_u32(&sm.p_ready[k]), 4);
            mbar_init(smem_u32(&sm.g2_done[k]), 1);
            mbar_init(smem_u32(&sm.d_free[k]), 4);
        }
        mbar_init(smem_u32(&sm.pool_bar), 1);       // armed per column with the bytes the peers will send
        mbar_init(smem_u32(&sm.core_bar), 1);
        sm.abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&xmap);
        tma_prefetch_desc(&omap);
    }
    // weights, once per CTA: 16-byte chunks, swizzled by row for the three 64 x 64 matrices
    for (int idx = tid; idx < FC * 8; idx += K::NTHREADS) {
        const int r = idx >> 3, c = idx & 7;
        const int dst = r * FC + ((c ^ (r & 7)) << 3);
        *reinterpret_cast<uint4 *>(&sm.wg[dst]) = __ldg(reinterpret_cast<const uint4 *>(a.wg + r * FC) + c);
        *reinterpret_cast<uint4 *>(&sm.wo[dst]) = __ldg(reinterpret_cast<const uint4 *>(a.wo + r * FC) + c);
        if (K::WQ_SMEM) *reinterpret_cast<uint4 *>(&sm.wq[dst]) = __ldg(reinterpret_cast<const uint4 *>(a.wq + r * FC) + c);
    }
    for (int idx = tid; idx < FD * FC; idx += K::NTHREADS) {
        sm.wk[idx] = a.wk[idx];
        sm.wv[idx] = a.wv[idx];
    }
    if (tid < FC) {
        sm.bg[tid] = a.bg[tid];
        sm.bo[tid] = a.bo[tid];
    }
    if (ncols > 0) {
        const unsigned short *mask_bits = reinterpret_cast<const unsigned short *>(a.mask);
        for (int r = tid; r < K::MAX_ROWS; r += K::NTHREADS) {
            const bool ok = r < mych * CH_ROWS && row_base + r < a.S;
            sm.mask[0][r] = ok ? mask_bits[(int64_t)cluster_id * a.S + row_base + r] : (unsigned short)0;
        }
    }
    if (warp == K::MMA_WARP) {
        tmem_alloc(smem_u32(&sm.tmem_base), K::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    cluster_barrier_all();          // every CTA's barriers exist before a peer arrives on them

    if (warp == K::IO_WARP) {
        if (lane == 0) io_thread<K>(sm, &xmap, &omap, a, cluster_id, nclusters, ncols, mych, row_base);
    } else if (warp == K::MMA_WARP) {
        if (lane == 0) mma_thread<K>(sm, a, ncols, mych);
    } else {
        consumer_warps<K>(sm, a, rank, cluster_id, nclusters, ncols, mych, row_base);
    }
    tc_fence_before();
    __syncthreads();                // every tcgen05.ld and every product has been waited for by now
    if (warp == K::MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(sm.tmem_base, K::TMEM_COLS);
    }
    cluster_barrier_all();          // no CTA leaves while a peer may still write into its shared memory
}

// The occupancy calculator answers "one CTA per SM" for every kernel that allocates tensor memory, although
// two such CTAs do share an SM when their columns fit (measured). This empty kernel with the same block
// size, dynamic shared memory and residency bound stands in for the real one in the cluster-occupancy
// query; the real kernel's registers (at most 96 x 576 or 80 x 320 x 2 threads) fit the register file.
template <class K>
__global__ void __launch_bounds__(K::BOUND_THREADS, K::MIN_CTAS) occupancy_twin_kernel(int *p)
{
    extern __shared__ unsigned char twin_smem[];
    if (p) p[threadIdx.x] = twin_smem[threadIdx.x];
}

// Launch with configuration K; ncta CTAs per cluster, nch slots per CTA and column.
template <class K>
bool launch_fused(cudaStream_t stream, const void *x, const void *out, int64_t out_row_stride, FusedArgs a)
{
    const int smem_bytes = (int)sizeof(FusedSmem<K>) + 1024;
    static bool attr_set[64] = {};
    static int max_clusters[64][MAX_CTA + 1] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(global_fused_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) !=
            cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        // two CTAs of the Half shape fill the SM's shared memory exactly: ask for the largest carve-out
        cudaFuncSetAttribute(global_fused_kernel<K>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cudaGetLastError();
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)a.ncta;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(K::NTHREADS);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_clusters[dev][a.ncta] == 0) {
        cfg.gridDim = dim3((unsigned)(a.ncta * 64));
        int n = 0;
        if (cudaFuncSetAttribute(occupancy_twin_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) !=
                cudaSuccess ||
            cudaOccupancyMaxActiveClusters(&n, occupancy_twin_kernel<K>, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            max_clusters[dev][a.ncta] = -1;
        } else {
            max_clusters[dev][a.ncta] = n;
        }
    }
    if (max_clusters[dev][a.ncta] < 1) return false;
    const int nclusters = std::min(a.B, max_clusters[dev][a.ncta]);
    cfg.gridDim = dim3((unsigned)(nclusters * a.ncta));

    CUtensorMap xmap, omap;
    if (!make_tensor_map_bf16_3d(&xmap, x, FC, (uint64_t)a.S, (uint64_t)a.B, FC, (uint64_t)a.S * FC, FC, CH_ROWS, 128))
        return false;
    if (!make_tensor_map_bf16_3d(&omap, out, FC, (uint64_t)a.S, (uint64_t)a.B, (uint64_t)out_row_stride,
                                 (uint64_t)a.S * (uint64_t)out_row_stride, FC, CH_ROWS, 128))
        return false;
    {
        KernelTimer timer__("global_fused", stream);
        const cudaError_t e = cudaLaunchKernelEx(&cfg, global_fused_kernel<K>, xmap, omap, a);
        KUTACC_CHECK(e == cudaSuccess, "global_fused_kernel launch failed: ", cudaGetErrorString(e));
        if (e != cudaSuccess) return false;
    }
    count_launch(1);
    return true;
}

// smallest power-of-two cluster whose CTAs hold a column in at most `max_per` slots each
bool pick_cluster(int chunks, int max_per, int *ncta, int *nch)
{
    for (int n = 1; n <= MAX_CTA; n *= 2) {
        const int per = (chunks + n - 1) / n;
        if (per <= max_per) {
            *ncta = n;
            *nch = per;
            return true;
        }
    }
    return false;
}

}  // namespace

// H = 8, D = 8 only. Returns false when this shape or these pointers are not covered; the caller then
// takes the three-kernel path.
bool launch_global_fused_bf16(cudaStream_t stream, const void *x, const void *mask, const void *wq, const void *wk,
                              const void *wv, const void *wg, const float *bg, const void *wo, const float *bo,
                              void *out, int64_t out_row_stride, int B, int S, int H, int D)
{
    if (H != FH || D != FD || B < 1 || S < 1 || (out_row_stride % 8) != 0 || out_row_stride < FC) return false;
    if ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)wq | (uintptr_t)wg | (uintptr_t)wo) & 15u) != 0) return false;
    if ((((uintptr_t)wk | (uintptr_t)wv) & 3u) != 0) return false;
    FusedArgs a;
    a.mask = (const __nv_bfloat16 *)mask;
    a.wq = (const __nv_bfloat16 *)wq;
    a.wk = (const __nv_bfloat16 *)wk;
    a.wv = (const __nv_bfloat16 *)wv;
    a.wg = (const __nv_bfloat16 *)wg;
    a.wo = (const __nv_bfloat16 *)wo;
    a.bg = bg;
    a.bo = bo;
    a.B = B;
    a.S = S;
    a.err = kernel_error_word().device;
    // The cluster shape depends on S alone, so that a column is partitioned the same way in every batch.
    const int chunks = (S + CH_ROWS - 1) / CH_ROWS;
    if (pick_cluster(chunks, HalfCfg::NSLOT, &a.ncta, &a.nch))
        return launch_fused<HalfCfg>(stream, x, out, out_row_stride, a);
    if (pick_cluster(chunks, WideCfg::NSLOT, &a.ncta, &a.nch))
        return launch_fused<WideCfg>(stream, x, out, out_row_stride, a);
    return false;
}

}  // namespace dev
}  // namespace kutacc
