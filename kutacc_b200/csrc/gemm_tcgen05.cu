// Projection GEMMs on the fifth-generation tensor cores: tcgen05.mma with TMEM accumulators, operands
// staged in shared memory by TMA, results written back by TMA stores.
//
//   C[b, s, n] = sum_k X[b, s, k] * W[n, k] (+ bias[n])         X [B, S, K] bf16, W [N, K] bf16 (W[out][in])
//
// Persistent CTAs (two per SM) walk 128 x 128 output tiles; a row tile never crosses a batch row, so
// every TMA box lies inside one [S, *] slab and rows past S are zero-filled on load and clipped on
// store. Warp roles:
//   warp 0      producer: TMA loads of 128 x 64 slabs of X and W (128-byte swizzle) into a 2-stage ring
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (M = 128, N = 128, K = 16) four times per
//               slab into one of two 128-column TMEM accumulators and commits to mbarriers
//   warps 2-9   epilogue: each warp owns 32 TMEM lanes x 64 columns of the tile: two tcgen05.ld in flight,
//               bias add, bf16 rounding, swizzled 32 x 32 staging tiles in shared memory, TMA stores into
//               the destination layout
// The two accumulators let the epilogue of tile i overlap the MMAs of tile i+1; with K = 128 a tile is only
// eight MMAs, so what hides the rest of the per-tile chain (TMA in, tcgen05.ld, staging, TMA store) is the
// second CTA resident on the SM (99 KB of shared memory and half of the tensor memory each).
//
// For the fused Q/K/V/gate projection the four weights are four tensor maps and the destination maps
// scatter straight into the attention kernel's [B, H, S, D] layout (q, k, v) and into [B, S, C] (gate,
// with the gate bias added). The same kernel serves the output projection.
//
// Replaces addmm -> kutacc_core_bgemm_ex of the reference
// (src/attention/gating_attention.cpp:47-66,152-157; src/linear/mm.cpp:46-86).
//
// All mbarrier waits are bounded; on a timeout the roles fall through to the common tail, the TMEM
// allocation is released and the host-visible error word carries the site.
#include "common.h"
#include "kernels.h"
#include "ptx_utils.cuh"
#include "tcgen05_utils.cuh"
#include "tma_utils.cuh"

#include <algorithm>

namespace kutacc {
namespace dev {

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int NSTAGE = 2;
constexpr int ACC_STAGES = 2;
constexpr int SLAB_BYTES = BM * BK * 2;                 // 16 KB, A and W slabs alike
constexpr int STAGE_BYTES = 2 * SLAB_BYTES;
constexpr int EPI_WARPS = 8;                            // two per TMEM lane quarter, 64 columns each
constexpr int STG_BYTES = 32 * 32 * 2;                  // one 32 x 32 bf16 staging tile
constexpr int STG_PER_WARP = 2;
static_assert(STG_PER_WARP == 2, "the epilogue writes its two 32-column halves into staging tiles 0 and 1 of its warp");
constexpr int STG_OFF = NSTAGE * STAGE_BYTES;
constexpr int BAR_OFF = STG_OFF + EPI_WARPS * STG_PER_WARP * STG_BYTES;
constexpr int NBARS = 2 * NSTAGE + 2 * ACC_STAGES;
constexpr int SMEM_BYTES = BAR_OFF + NBARS * 8 + 16 + 1024;
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = ACC_STAGES * BN;              // 256: half of the SM's tensor memory (two CTAs per SM)

struct alignas(64) GemmMaps {
    CUtensorMap a;        // X  [B][S][K], box [64, 128, 1], 128-byte swizzle
    CUtensorMap w[4];     // W  [1][N_seg][K], box [64, 128, 1], 128-byte swizzle
    CUtensorMap out[4];   // destination per segment, box [32, 32, 1], 64-byte swizzle
};

struct GemmParams {
    const float *bias[4];   // per segment, may be null
    int seg_n;              // output channels per segment (multiple of 128)
    int nseg;
    int head_dim;           // > 0: segment output is [B*H][S][D] (coords d, s, b*H + h); 0: [B][S][N_seg]
    int head_layout_mask;   // bit i set: segment i uses the head layout
    int transposed_mask;    // bit i set: segment i is stored transposed, [B*H][D][S] (coords s, d, b*H + h)
    int chanmajor_mask;     // bit i set: segment i is stored transposed and channel-major, [N_seg][B][S] (coords s, b, n)
    int w_batched;          // non-zero: W is [B][N_seg][K], one matrix per batch row (coords k, n, b)
    int heads;
    int K;
    int S, B;
    int relu;               // non-zero: max(0, .) after the bias, before the bf16 rounding
    const float2 *ln_stats; // F_LN: (mean, rstd) of every row of X, [B * S]
    const float *ln_s[4];   // F_LN: rounding residue of the folded weight rows, per segment
    int rotate;             // non-zero: column tile of tile t is rotated by t / gridDim.x (see tile_of)
    int sigmoid_mask;       // bit i set: segment i stores bf16(sigmoid(bf16(y))) (the gate of the attention, whose
                            // reference rounds the gate to bf16 before the sigmoid: gating_attention.cpp:62-66,134-147)
    int *err;
};

// shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte swizzle, 8-row groups
// 1024 bytes apart; `addr` is the byte address of the (1024-aligned) slab plus the K offset inside the
// swizzle atom
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);         // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                          // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                          // 128-byte swizzle
    return d;
}
// instruction descriptor: D fp32, A and B bf16, both K-major, N = 128, M = 128
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// 1 / (1 + exp(-g)) of the bf16-rounded g as 0.5 * tanh(g / 2) + 0.5: one MUFU operation (relative error about
// 2^-11, below the bf16 step of the stored result) instead of an exponential and a division
__device__ __forceinline__ float sigmoid_of_bf16(float y)
{
    const float g = round_to_bf16_f32(y);
    return fmaf(0.5f, tanh_approx(0.5f * g), 0.5f);
}

// Compile-time feature sets, so that each use of the kernel carries only the epilogue code it needs
// (the sigmoid and the transposed staging cost registers that the plain linear layer would spill).
constexpr int F_SIGMOID = 1, F_TRANSPOSED = 2, F_RELU = 4, F_WBATCH = 8, F_LN = 16;

template <int FEAT>
__global__ void __launch_bounds__(THREADS, 2)
gemm_tcgen05_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem + BAR_OFF;
    auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(NSTAGE + s); };
    auto acc_full = [&](int a) { return bar_base + 8u * (uint32_t)(2 * NSTAGE + a); };
    auto acc_empty = [&](int a) { return bar_base + 8u * (uint32_t)(2 * NSTAGE + ACC_STAGES + a); };
    const uint32_t tmem_slot = bar_base + 8u * NBARS;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s_tiles = (p.S + BM - 1) / BM;
    const int n_tiles_seg = (p.seg_n + BN - 1) / BN;    // a ragged last tile is zero-filled on load and clipped on store
    const int n_tiles = n_tiles_seg * p.nseg;
    const int num_tiles = p.B * s_tiles * n_tiles;
    const int nk = (p.K + BK - 1) / BK;                 // columns past K are zero-filled by TMA
    // Tile t covers row tile t / n_tiles and column tile t % n_tiles. A CTA walks t = blockIdx.x + k * gridDim.x, so
    // when the grid size is a multiple of n_tiles it would meet the same column tile, i.e. the same segment, every
    // time, and the CTAs that only get the gate segment (a sigmoid per element) would finish long after the others.
    // With `rotate` the column tile is shifted by k, which is constant over the n_tiles tiles of a row tile (they
    // lie in one block of gridDim.x consecutive t), so the map stays one to one and every CTA meets every segment.
    auto tile_of = [&](int tile, int &m_tile, int &n_tile) {
        m_tile = tile / n_tiles;
        n_tile = tile % n_tiles;
        if (p.rotate) n_tile = (n_tile + tile / (int)gridDim.x) % n_tiles;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), EPI_WARPS);
        }
        fence_barrier_init();
    }
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
            tma_prefetch_desc(&maps.a);
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int m_tile, n_tile;
                tile_of(tile, m_tile, n_tile);
                const int b = m_tile / s_tiles, s0 = (m_tile % s_tiles) * BM;
                const int seg = n_tile / n_tiles_seg, n0 = (n_tile % n_tiles_seg) * BN;
                const CUtensorMap *wmap = &maps.w[seg];
                for (int kc = 0; kc < nk; ++kc, ++it) {
                    const int s = it % NSTAGE;
                    if (it >= NSTAGE && !mbar_wait(empty_bar(s), (uint32_t)((it / NSTAGE - 1) & 1), p.err, 11)) {
                        ok = false;
                        break;
                    }
                    const uint32_t st = smem + (uint32_t)s * STAGE_BYTES;
                    mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
                    tma_load_3d(st, &maps.a, full_bar(s), kc * BK, s0, b);
                    tma_load_3d(st + SLAB_BYTES, wmap, full_bar(s), kc * BK, n0, (FEAT & F_WBATCH) ? b : 0);
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        int it = 0, tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
            const int a = tcount % ACC_STAGES;
            if (tcount >= ACC_STAGES && !mbar_wait_warp(acc_empty(a), (uint32_t)((tcount / ACC_STAGES - 1) & 1), p.err, 12)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(a * BN);
            for (int kc = 0; kc < nk; ++kc, ++it) {
                const int s = it % NSTAGE;
                if (!mbar_wait_warp(full_bar(s), (uint32_t)((it / NSTAGE) & 1), p.err, 13)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t st = smem + (uint32_t)s * STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t adesc = make_smem_desc(st + k * 32);
                        const uint64_t bdesc = make_smem_desc(st + SLAB_BYTES + k * 32);
                        tc_mma_bf16(d_tmem, adesc, bdesc, kInstrDesc, (kc > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));                 // slab may be overwritten once these MMAs retire
                    if (kc == nk - 1) tc_commit(acc_full(a));
                }
                __syncwarp();
            }
        }
    } else {
        // ================= epilogue =================
        const int quad = warp & 3;                            // TMEM lanes 32*quad .. 32*quad+31
        const int ew = warp - 2;
        const int half = ew >> 2;                             // which 64 columns of the 128-column tile
        const uint32_t stg0 = smem + STG_OFF + (uint32_t)(ew * STG_PER_WARP) * STG_BYTES;
        int tcount = 0, nstore = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
            int m_tile, n_tile;
            tile_of(tile, m_tile, n_tile);
            const int b = m_tile / s_tiles, s0 = (m_tile % s_tiles) * BM;
            const int seg = n_tile / n_tiles_seg, n0 = (n_tile % n_tiles_seg) * BN;
            const int a = tcount % ACC_STAGES;
            if (!mbar_wait_warp(acc_full(a), (uint32_t)((tcount / ACC_STAGES) & 1), p.err, 14)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const float *bias = p.bias[seg];
            const bool head_layout = (p.head_layout_mask >> seg) & 1;
            const bool chanmajor = (FEAT & F_TRANSPOSED) && ((p.chanmajor_mask >> seg) & 1);
            const bool transposed = (FEAT & F_TRANSPOSED) && (((p.transposed_mask >> seg) & 1) || chanmajor);
            const bool sigmoid = (FEAT & F_SIGMOID) && ((p.sigmoid_mask >> seg) & 1);
            const bool relu = (FEAT & F_RELU) && p.relu;
            const CUtensorMap *omap = &maps.out[seg];
            const int row0 = s0 + quad * 32;                  // first row of this warp inside the batch row
            // LayerNorm-folded projection: y = rstd * (acc - mean * s[n]) + t[n] with this thread's row statistics
            float ln_a = 1.f, ln_b = 0.f;
            if (FEAT & F_LN) {
                const int rr = row0 + lane < p.S ? row0 + lane : p.S - 1;
                const float2 st = __ldg(p.ln_stats + (int64_t)b * p.S + rr);
                ln_a = st.y;
                ln_b = -st.y * st.x;
            }
            uint32_t r[2][32];
            const uint32_t tcol = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * BN + half * 64);
            tmem_ld_32x32(tcol, r[0]);
            tmem_ld_32x32(tcol + 32, r[1]);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int n = n0 + half * 64 + c * 32;
                uint32_t packed[16];
                if (bias) {
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        const float4 bv = __ldg(reinterpret_cast<const float4 *>(bias + n) + j4);
                        float y0, y1, y2, y3;
                        if (FEAT & F_LN) {
                            // two outputs per instruction on the packed fp32 pipe: y = ln_a * acc + (ln_b * s + t)
                            const float4 sv = __ldg(reinterpret_cast<const float4 *>(p.ln_s[seg] + n) + j4);
                            const uint64_t a2 = pack_f32x2(ln_a, ln_a), b2 = pack_f32x2(ln_b, ln_b);
                            const uint64_t w01 = fma_f32x2(pack_f32x2(sv.x, sv.y), b2, pack_f32x2(bv.x, bv.y));
                            const uint64_t w23 = fma_f32x2(pack_f32x2(sv.z, sv.w), b2, pack_f32x2(bv.z, bv.w));
                            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[c][4 * j4]), __uint_as_float(r[c][4 * j4 + 1])),
                                                   a2, w01), y0, y1);
                            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[c][4 * j4 + 2]),
                                                              __uint_as_float(r[c][4 * j4 + 3])), a2, w23), y2, y3);
                        } else {
                            y0 = __uint_as_float(r[c][4 * j4]) + bv.x;
                            y1 = __uint_as_float(r[c][4 * j4 + 1]) + bv.y;
                            y2 = __uint_as_float(r[c][4 * j4 + 2]) + bv.z;
                            y3 = __uint_as_float(r[c][4 * j4 + 3]) + bv.w;
                        }
                        if (relu) {
                            y0 = fmaxf(y0, 0.f);
                            y1 = fmaxf(y1, 0.f);
                            y2 = fmaxf(y2, 0.f);
                            y3 = fmaxf(y3, 0.f);
                        }
                        if (sigmoid) {
                            y0 = sigmoid_of_bf16(y0);
                            y1 = sigmoid_of_bf16(y1);
                            y2 = sigmoid_of_bf16(y2);
                            y3 = sigmoid_of_bf16(y3);
                        }
                        packed[2 * j4] = pack_bf16x2(y0, y1);
                        packed[2 * j4 + 1] = pack_bf16x2(y2, y3);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float y0 = __uint_as_float(r[c][2 * j]), y1 = __uint_as_float(r[c][2 * j + 1]);
                        if (relu) {
                            y0 = fmaxf(y0, 0.f);
                            y1 = fmaxf(y1, 0.f);
                        }
                        packed[j] = pack_bf16x2(y0, y1);
                    }
                }
                // staging tile: row = lane, 64 bytes per row, 16-byte chunks swizzled as the 64-byte TMA mode
                const uint32_t stg = stg0 + (uint32_t)c * STG_BYTES;
                if (nstore >= STG_PER_WARP) {
                    if (lane == 0) tma_store_wait_read<STG_PER_WARP - 1>();
                    __syncwarp();
                }
                if (transposed) {
                    // transposed staging tile: row = channel d, column = this lane's sequence position
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int d = 2 * j + e;
                            const uint32_t addr = stg + (uint32_t)(d * 64 + (((lane >> 3) ^ ((d >> 1) & 3)) << 4) + (lane & 7) * 2);
                            const uint16_t hv = (uint16_t)(e ? (packed[j] >> 16) : (packed[j] & 0xffffu));
                            asm volatile("st.shared.u16 [%0], %1;\n" ::"r"(addr), "h"(hv) : "memory");
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (chanmajor) {
                            tma_store_3d(omap, stg, row0, b, n);
                        } else {
                            const int hh = n / p.head_dim, d0 = n - hh * p.head_dim;
                            tma_store_3d(omap, stg, row0, d0, b * p.heads + hh);
                        }
                        tma_store_commit();
                    }
                    ++nstore;
                    continue;
                }
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const uint32_t addr = stg + (uint32_t)(lane * 64 + ((ch ^ ((lane >> 1) & 3)) << 4));
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(packed[4 * ch]),
                                 "r"(packed[4 * ch + 1]), "r"(packed[4 * ch + 2]), "r"(packed[4 * ch + 3])
                                 : "memory");
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    if (head_layout) {
                        const int hh = n / p.head_dim, d0 = n - hh * p.head_dim;
                        tma_store_3d(omap, stg, d0, row0, b * p.heads + hh);
                    } else {
                        tma_store_3d(omap, stg, n, row0, b);
                    }
                    tma_store_commit();
                }
                ++nstore;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(a));
        }
        if (lane == 0) tma_store_wait<0>();
    }

    // ================= common tail =================
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

int sm_count()
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

template <int FEAT>
bool launch(cudaStream_t stream, const GemmMaps &maps, const GemmParams &p, const char *name)
{
    static bool configured = false;
    if (!configured) {
        KUTACC_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<FEAT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured = true;
    }
    const int s_tiles = (p.S + BM - 1) / BM;
    const int64_t tiles = (int64_t)p.B * s_tiles * ((p.seg_n + BN - 1) / BN) * p.nseg;
    const unsigned grid = (unsigned)std::min<int64_t>(tiles, 2 * std::max(1, sm_count() - runtime().sm_margin));
    GemmParams q = p;
    const int n_tiles = ((p.seg_n + BN - 1) / BN) * p.nseg;
    q.rotate = (n_tiles > 1 && grid % (unsigned)n_tiles == 0) ? 1 : 0;
    KernelTimer timer__(name, stream);
    gemm_tcgen05_kernel<FEAT><<<grid, THREADS, SMEM_BYTES, stream>>>(maps, q);
    count_launch();
    return true;
}

}  // namespace

bool tcgen05_proj_qkvg_bf16(cudaStream_t stream, const void *x, const void *wq, const void *wk, const void *wv,
                            const void *wg, const float *bg, void *q, void *k, void *v, void *gate, int B, int S,
                            int H, int D, bool v_transposed, int64_t v_pitch, bool gate_sigmoid, const void *ln_stats,
                            const float *const *ln_s, const float *const *ln_t)
{
    const int C = H * D;
    if (C % 128 != 0 || (D != 32 && D != 64) || C > 256 * 64 || ((uintptr_t)bg & 15u)) return false;
    KernelErrorWord &ew = kernel_error_word();
    if (ew.device == nullptr) return false;
    GemmMaps maps;
    const void *w[4] = {wq, wk, wv, wg};
    void *o[3] = {q, k, v};
    if (!make_tensor_map_bf16_3d(&maps.a, x, C, S, B, C, (uint64_t)S * C, BK, BM, 128)) return false;
    for (int i = 0; i < 4; ++i)
        if (!make_tensor_map_bf16_3d(&maps.w[i], w[i], C, C, 1, C, (uint64_t)C * C, BK, BN, 128)) return false;
    for (int i = 0; i < 3; ++i) {
        if (i == 2 && v_transposed) {
            // v^T: [B*H][D][S] with row pitch v_pitch (a multiple of 8 elements)
            if (v_pitch % 8 != 0 || v_pitch < S) return false;
            if (!make_tensor_map_bf16_3d(&maps.out[i], o[i], S, D, (uint64_t)B * H, (uint64_t)v_pitch,
                                         (uint64_t)D * v_pitch, 32, 32, 64))
                return false;
            continue;
        }
        if (!make_tensor_map_bf16_3d(&maps.out[i], o[i], D, S, (uint64_t)B * H, D, (uint64_t)S * D, 32, 32, 64))
            return false;
    }
    if (!make_tensor_map_bf16_3d(&maps.out[3], gate, C, S, B, C, (uint64_t)S * C, 32, 32, 64)) return false;
    GemmParams p;
    p.bias[0] = p.bias[1] = p.bias[2] = nullptr;
    p.bias[3] = bg;
    p.ln_stats = (const float2 *)ln_stats;
    for (int i = 0; i < 4; ++i) {
        p.ln_s[i] = ln_stats ? ln_s[i] : nullptr;
        if (ln_stats) p.bias[i] = ln_t[i];
        if (ln_stats && ((((uintptr_t)ln_s[i] | (uintptr_t)ln_t[i]) & 15u) != 0)) return false;
    }
    p.seg_n = C;
    p.nseg = 4;
    p.head_dim = D;
    p.head_layout_mask = 0x7;
    p.transposed_mask = v_transposed ? 0x4 : 0;
    p.chanmajor_mask = 0;
    p.w_batched = 0;
    p.heads = H;
    p.K = C;
    p.S = S;
    p.B = B;
    p.relu = 0;
    p.sigmoid_mask = gate_sigmoid ? 0x8 : 0;
    p.err = ew.device;
    if (ln_stats)
        return v_transposed && gate_sigmoid ? launch<F_TRANSPOSED | F_SIGMOID | F_LN>(stream, maps, p, "proj_qkvg_ln") : false;
    if (v_transposed)
        return gate_sigmoid ? launch<F_TRANSPOSED | F_SIGMOID>(stream, maps, p, "proj_qkvg")
                            : launch<F_TRANSPOSED>(stream, maps, p, "proj_qkvg");
    return gate_sigmoid ? launch<F_SIGMOID>(stream, maps, p, "proj_qkvg") : launch<0>(stream, maps, p, "proj_qkvg");
}

bool tcgen05_linear_bias_bf16(cudaStream_t stream, const void *a, const void *w, const float *bias, void *out,
                              int64_t out_row_stride, int B, int S, int N, int K, bool relu, int64_t a_row_stride)
{
    if (a_row_stride <= 0) a_row_stride = K;
    if (N % 128 != 0 || K % 64 != 0 || out_row_stride % 8 != 0 || a_row_stride % 8 != 0 || a_row_stride < K ||
        ((uintptr_t)out & 15u) || ((uintptr_t)a & 15u) || ((uintptr_t)w & 15u) || ((uintptr_t)bias & 15u))
        return false;
    KernelErrorWord &ew = kernel_error_word();
    if (ew.device == nullptr) return false;
    GemmMaps maps;
    if (!make_tensor_map_bf16_3d(&maps.a, a, K, S, B, (uint64_t)a_row_stride, (uint64_t)S * a_row_stride, BK, BM, 128))
        return false;
    if (!make_tensor_map_bf16_3d(&maps.w[0], w, K, N, 1, K, (uint64_t)N * K, BK, BN, 128)) return false;
    if (!make_tensor_map_bf16_3d(&maps.out[0], out, N, S, B, (uint64_t)out_row_stride, (uint64_t)S * out_row_stride, 32,
                                 32, 64))
        return false;
    for (int i = 1; i < 4; ++i) {
        maps.w[i] = maps.w[0];
        maps.out[i] = maps.out[0];
    }
    GemmParams p;
    p.bias[0] = bias;
    p.bias[1] = p.bias[2] = p.bias[3] = nullptr;
    p.seg_n = N;
    p.nseg = 1;
    p.head_dim = 0;
    p.head_layout_mask = 0;
    p.transposed_mask = 0;
    p.chanmajor_mask = 0;
    p.w_batched = 0;
    p.heads = 1;
    p.K = K;
    p.S = S;
    p.B = B;
    p.relu = relu ? 1 : 0;
    p.ln_stats = nullptr;
    p.ln_s[0] = p.ln_s[1] = p.ln_s[2] = p.ln_s[3] = nullptr;
    p.sigmoid_mask = 0;
    p.err = ew.device;
    return relu ? launch<F_RELU>(stream, maps, p, "linear_bias_relu") : launch<0>(stream, maps, p, "linear_bias");
}

// Two projections of x [B, S, K] with row biases, both stored channel-major: out_i[n, b, s] = x[b, s, :] . w_i[n, :]
// + bias_i[n] (out strides in elements: out_c_stride between channels, out_b_stride between batch rows). The
// projection and gate products of the triangle multiplication (src/attention/triangle_multiplication.cpp:38-49).
bool tcgen05_proj2_chanmajor_bf16(cudaStream_t stream, const void *x, const void *w0, const float *bias0, const void *w1,
                                  const float *bias1, void *out0, void *out1, int64_t out_c_stride, int64_t out_b_stride,
                                  int B, int S, int N, int K)
{
    if (N % 128 != 0 || K % 64 != 0 || out_c_stride % 8 != 0 || out_b_stride % 8 != 0 || out_b_stride < S ||
        ((((uintptr_t)x | (uintptr_t)w0 | (uintptr_t)w1 | (uintptr_t)out0 | (uintptr_t)out1 | (uintptr_t)bias0 |
           (uintptr_t)bias1) & 15u) != 0))
        return false;
    KernelErrorWord &ew = kernel_error_word();
    if (ew.device == nullptr) return false;
    GemmMaps maps;
    const void *w[2] = {w0, w1};
    void *o[2] = {out0, out1};
    if (!make_tensor_map_bf16_3d(&maps.a, x, K, S, B, K, (uint64_t)S * K, BK, BM, 128)) return false;
    for (int i = 0; i < 2; ++i) {
        if (!make_tensor_map_bf16_3d(&maps.w[i], w[i], K, N, 1, K, (uint64_t)N * K, BK, BN, 128)) return false;
        // [N][B][S]: dims (s, b, n), one 32 (s) x 1 x 32 (n) box per staging tile
        if (!make_tensor_map_bf16_3d(&maps.out[i], o[i], S, B, N, (uint64_t)out_b_stride, (uint64_t)out_c_stride, 32, 1, 64, 32))
            return false;
    }
    for (int i = 2; i < 4; ++i) {
        maps.w[i] = maps.w[0];
        maps.out[i] = maps.out[0];
    }
    GemmParams p;
    p.bias[0] = bias0;
    p.bias[1] = bias1;
    p.bias[2] = p.bias[3] = nullptr;
    p.seg_n = N;
    p.nseg = 2;
    p.head_dim = 0;
    p.head_layout_mask = 0;
    p.transposed_mask = 0;
    p.chanmajor_mask = 0x3;
    p.w_batched = 0;
    p.heads = 1;
    p.K = K;
    p.S = S;
    p.B = B;
    p.relu = 0;
    p.ln_stats = nullptr;
    p.ln_s[0] = p.ln_s[1] = p.ln_s[2] = p.ln_s[3] = nullptr;
    p.sigmoid_mask = 0;
    p.err = ew.device;
    return launch<F_TRANSPOSED>(stream, maps, p, "tm_proj");
}

// Batched product with one right-hand matrix per batch: out[b, m, n] = sum_k a[b, m, k] * w[b, n, k]
// (a, w, out with row and batch strides in elements). The per-channel products of the triangle multiplication
// (src/attention/triangle_multiplication.cpp:75-104).
bool tcgen05_batched_nt_bf16(cudaStream_t stream, const void *a, int64_t a_row_stride, int64_t a_batch_stride,
                             const void *w, int64_t w_row_stride, int64_t w_batch_stride, void *out,
                             int64_t out_row_stride, int64_t out_batch_stride, int B, int M, int N, int K)
{
    if ((a_row_stride | a_batch_stride | w_row_stride | w_batch_stride | out_row_stride | out_batch_stride) % 8 != 0 ||
        a_row_stride < K || w_row_stride < K || out_row_stride < N ||
        ((((uintptr_t)a | (uintptr_t)w | (uintptr_t)out) & 15u) != 0))
        return false;
    KernelErrorWord &ew = kernel_error_word();
    if (ew.device == nullptr) return false;
    GemmMaps maps;
    if (!make_tensor_map_bf16_3d(&maps.a, a, K, M, B, (uint64_t)a_row_stride, (uint64_t)a_batch_stride, BK, BM, 128)) return false;
    if (!make_tensor_map_bf16_3d(&maps.w[0], w, K, N, B, (uint64_t)w_row_stride, (uint64_t)w_batch_stride, BK, BN, 128))
        return false;
    if (!make_tensor_map_bf16_3d(&maps.out[0], out, N, M, B, (uint64_t)out_row_stride, (uint64_t)out_batch_stride, 32, 32, 64))
        return false;
    for (int i = 1; i < 4; ++i) {
        maps.w[i] = maps.w[0];
        maps.out[i] = maps.out[0];
    }
    GemmParams p;
    p.bias[0] = p.bias[1] = p.bias[2] = p.bias[3] = nullptr;
    p.seg_n = N;
    p.nseg = 1;
    p.head_dim = 0;
    p.head_layout_mask = 0;
    p.transposed_mask = 0;
    p.chanmajor_mask = 0;
    p.w_batched = 1;
    p.heads = 1;
    p.K = K;
    p.S = M;
    p.B = B;
    p.relu = 0;
    p.ln_stats = nullptr;
    p.ln_s[0] = p.ln_s[1] = p.ln_s[2] = p.ln_s[3] = nullptr;
    p.sigmoid_mask = 0;
    p.err = ew.device;
    return launch<F_WBATCH>(stream, maps, p, "tm_equation");
}

}  // namespace dev
}  // namespace kutacc
