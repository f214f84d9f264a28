// CPU oracle for the gated-attention path of KuTACC.
//
// TEST INFRASTRUCTURE ONLY. This file is a CPU restatement of the reference's arithmetic; it is
// the checker for the CUDA library and the timed CPU baseline of the benchmark. Nothing in the
// shipped library links, loads or calls it.
//
// PARITY UNPINNED: the reference's own tests hold no numerical vector for gating or global
// attention (its attention tests only pass null or negative arguments), and its GEMM lives in a
// closed library (kutacc_core_bgemm_ex, src/utils/blas.cpp:53-91). The GEMM is restated here as
// "fp32 accumulate, fp32 bias add, one bf16 round-to-nearest-even on store". The all-gather
// restatement IS pinned by the byte grid of test/functest/comm/all_gather_test.cpp:29-67.
//
// Two arithmetic modes:
//   faithful : bf16 storage at every point where the reference stores bf16, exp through a bit-level
//              restatement of the SVE FEXPA path (src/math/fast_exp.h:21-27).
//   exact    : fp32 inputs, double accumulation, std::exp, no intermediate rounding.
//
// Build: g++ -O3 -march=x86-64-v3 -fopenmp -shared -fPIC (oracle/build.py).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- bf16 <-> fp32 ---------------------------------------------------------------------------
// Round to nearest even on narrowing (src/utils/collapse.h:21-24, src/wrapper/svcvt.h:23-31);
// widening is a 16-bit left shift (src/wrapper/svcvt.h:33-37).
inline uint16_t f2bf(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
    }
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
inline float bf2f(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline float rbf(float f) { return bf2f(f2bf(f)); }

// ---- FEXPA exp -------------------------------------------------------------------------------
// src/math/fast_exp.h:21-27: n = u32(round_half_away(min(x, ln FLT_MAX) * 64/ln2 + 127*64)),
// then FEXPA(n): exponent field = n[13:6], fraction = table[n[5:0]] = 23-bit fraction of 2^(i/64).
uint32_t g_fexpa_frac[64];
bool g_fexpa_ready = false;
void fexpa_init()
{
    if (g_fexpa_ready) return;
    for (int i = 0; i < 64; ++i) {
        float v = (float)std::exp2((double)i / 64.0);  // correctly rounded to fp32, in [1,2)
        uint32_t u;
        std::memcpy(&u, &v, 4);
        g_fexpa_frac[i] = u & 0x007fffffu;
    }
    g_fexpa_ready = true;
}
inline float fexpa_exp(float x)
{
    const float k = 92.33248f;
    const float lnmax = 88.72284f;
    float t = std::fmaf(std::min(x, lnmax), k, 8128.0f);  // svmad: fused
    t = std::round(t);                                     // svrinta: half away from zero
    uint32_t n;
    if (!(t > 0.0f)) {
        n = 0;  // svcvt_u32 saturates negatives (and NaN) to 0
    } else if (t >= 4294967296.0f) {
        n = 0xffffffffu;
    } else {
        n = (uint32_t)t;
    }
    uint32_t bits = (((n >> 6) & 0xffu) << 23) | g_fexpa_frac[n & 63u];
    float r;
    std::memcpy(&r, &bits, 4);
    return r;
}
// src/activation/sigmoid.h:31-35 (vector overload): 1 / (1 + fast_exp(-x)), true division.
inline float fexpa_sigmoid(float x) { return 1.0f / (fexpa_exp(-x) + 1.0f); }

// ---- GEMM stand-in ---------------------------------------------------------------------------
// c[m,n] = bf16( sum_k a[m,k]*w[n,k] + bias[n] ), a and w given as fp32 copies of bf16 data.
// Stands in for addmm -> kutacc_core_bgemm_ex (src/linear/mm.cpp:46-86).
void gemm_nt_bf16out(const float *a, int64_t lda, const float *w, int64_t ldw, const float *bias, int64_t M,
                     int64_t N, int64_t K, float *c, int64_t ldc, bool round_out)
{
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        const float *ar = a + m * lda;
        for (int64_t n = 0; n < N; ++n) {
            const float *wr = w + n * ldw;
            float acc = 0.f;
#pragma omp simd reduction(+ : acc)
            for (int64_t k = 0; k < K; ++k) acc += ar[k] * wr[k];
            if (bias) acc += bias[n];
            c[m * ldc + n] = round_out ? rbf(acc) : acc;
        }
    }
}

void widen(const uint16_t *src, int64_t n, std::vector<float> &dst)
{
    dst.resize((size_t)n);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) dst[(size_t)i] = bf2f(src[i]);
}

}  // namespace

extern "C" {

// number of OpenMP threads later parallel regions use (a launcher may have exported OMP_NUM_THREADS=1)
void orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads()
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_f32_to_bf16(const float *src, uint16_t *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) dst[i] = f2bf(src[i]);
}
void orc_bf16_to_f32(const uint16_t *src, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) dst[i] = bf2f(src[i]);
}
float orc_fexpa_exp(float x)
{
    fexpa_init();
    return fexpa_exp(x);
}

// ------------------------------------------------------------------------------------------------
// Gating attention, faithful mode. Follows src/attention/gating_attention.cpp:33-158.
//   x      [B*S, C] bf16          wq,wk,wv,wg,wo [C_out, C_in] bf16 (memory order W[out][in])
//   bg,bo  [C] fp32               bias [B, S] bf16 (row stride bias_stride0)
//   nb     [H, S, S] bf16 or NULL (strides nb_stride_h, nb_stride_q, unit key stride)
//   out    [B*S, C] bf16
// Optional dumps (may be NULL): q,k,g,avg as [B,S,H,D] bf16; v as [H,D,B,S] bf16 (the layout the
// reference writes, gating_attention.cpp:57-61).
// Rounding points: projections (:47-66), raw logits before scaling (:97-101), probabilities
// (softmax.h:40-41), weighted average (:128-133), gated average (:145), output (:152-157).
// ------------------------------------------------------------------------------------------------
void orc_gating_attention_bf16(const uint16_t *x, const uint16_t *wq, const uint16_t *wk, const uint16_t *wv,
                               const uint16_t *wg, const float *bg, const uint16_t *wo, const float *bo,
                               const uint16_t *bias, int64_t bias_stride0, const uint16_t *nb, int64_t nb_stride_h,
                               int64_t nb_stride_q, int64_t B, int64_t S, int64_t H, int64_t D, int64_t block_size,
                               uint16_t *out, uint16_t *q_dump, uint16_t *k_dump, uint16_t *v_dump, uint16_t *g_dump,
                               uint16_t *avg_dump)
{
    fexpa_init();
    const int64_t C = H * D;
    const int64_t M = B * S;
    std::vector<float> xf, wqf, wkf, wvf, wgf, wof;
    widen(x, M * C, xf);
    widen(wq, C * C, wqf);
    widen(wk, C * C, wkf);
    widen(wv, C * C, wvf);
    widen(wg, C * C, wgf);
    widen(wo, C * C, wof);
    std::vector<float> q((size_t)(M * C)), k((size_t)(M * C)), v((size_t)(M * C)), g((size_t)(M * C)),
        avg((size_t)(M * C));
    gemm_nt_bf16out(xf.data(), C, wqf.data(), C, nullptr, M, C, C, q.data(), C, true);
    gemm_nt_bf16out(xf.data(), C, wkf.data(), C, nullptr, M, C, C, k.data(), C, true);
    gemm_nt_bf16out(xf.data(), C, wvf.data(), C, nullptr, M, C, C, v.data(), C, true);
    gemm_nt_bf16out(xf.data(), C, wgf.data(), C, bg, M, C, C, g.data(), C, true);

    const float scale = (float)(1.0 / std::sqrt((double)D));  // gating_attention.cpp:68
    const int64_t nblocks = (S + block_size - 1) / block_size;

#pragma omp parallel
    {
        std::vector<float> logits((size_t)S), xs((size_t)S), p((size_t)S), kh((size_t)(S * D)), vh((size_t)(S * D)),
            acc_d((size_t)D);
        // (b, h, q-block) flattened with the block index fastest (src/utils/collapse.h:31-58)
#pragma omp for schedule(static)
        for (int64_t bh = 0; bh < B * H; ++bh) {
            const int64_t b = bh / H, h = bh % H;
            const uint16_t *brow = bias + b * bias_stride0;
            // per-(b,h) K and V panels, the analogue of the gemm_pack calls (:92-96, :123-127)
            for (int64_t j = 0; j < S; ++j)
                for (int64_t d = 0; d < D; ++d) {
                    kh[(size_t)(j * D + d)] = k[(size_t)((b * S + j) * C + h * D + d)];
                    vh[(size_t)(j * D + d)] = v[(size_t)((b * S + j) * C + h * D + d)];
                }
            for (int64_t blk = 0; blk < nblocks; ++blk) {
                const int64_t q0 = blk * block_size, q1 = std::min(q0 + block_size, S);
                for (int64_t i = q0; i < q1; ++i) {
                    const float *qi = &q[(size_t)((b * S + i) * C + h * D)];
                    for (int64_t j = 0; j < S; ++j) {
                        const float *kj = &kh[(size_t)(j * D)];
                        float acc = 0.f;
#pragma omp simd reduction(+ : acc)
                        for (int64_t d = 0; d < D; ++d) acc += qi[d] * kj[d];
                        logits[(size_t)j] = rbf(acc);  // logits scratch is bf16 (:77,91)
                    }
                    const uint16_t *nbrow = nb ? nb + h * nb_stride_h + i * nb_stride_q : nullptr;
                    float mx = -INFINITY;
                    for (int64_t j = 0; j < S; ++j) {
                        float val = logits[(size_t)j] * scale;  // :113
                        val = val + bf2f(brow[j]);              // :114
                        if (nbrow) val = val + bf2f(nbrow[j]);  // :115-117
                        mx = std::max(mx, val);
                        xs[(size_t)j] = val;
                    }
                    // softmax_with_max (src/softmax/softmax.h:22-43)
                    float sum = 0.f;
                    for (int64_t j = 0; j < S; ++j) {
                        float e = fexpa_exp(xs[(size_t)j] - mx);
                        xs[(size_t)j] = e;
                        sum += e;
                    }
                    const float inv = 1.0f / sum;
                    for (int64_t j = 0; j < S; ++j) p[(size_t)j] = rbf(xs[(size_t)j] * inv);
                    for (int64_t d = 0; d < D; ++d) acc_d[(size_t)d] = 0.f;
                    for (int64_t j = 0; j < S; ++j) {
                        const float pj = p[(size_t)j];
                        const float *vj = &vh[(size_t)(j * D)];
#pragma omp simd
                        for (int64_t d = 0; d < D; ++d) acc_d[(size_t)d] += pj * vj[d];
                    }
                    float *ai = &avg[(size_t)((b * S + i) * C + h * D)];
                    const float *gi = &g[(size_t)((b * S + i) * C + h * D)];
                    for (int64_t d = 0; d < D; ++d) {
                        float wa = rbf(acc_d[(size_t)d]);         // :128-133
                        ai[d] = rbf(wa * fexpa_sigmoid(gi[d]));  // :134-147
                    }
                }
            }
        }
    }

    std::vector<float> of((size_t)(M * C));
    gemm_nt_bf16out(avg.data(), C, wof.data(), C, bo, M, C, C, of.data(), C, true);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M * C; ++i) out[i] = f2bf(of[(size_t)i]);

    auto dump = [&](uint16_t *dst, const std::vector<float> &src) {
        if (!dst) return;
        for (int64_t i = 0; i < M * C; ++i) dst[i] = f2bf(src[(size_t)i]);
    };
    dump(q_dump, q);
    dump(k_dump, k);
    dump(g_dump, g);
    dump(avg_dump, avg);
    if (v_dump) {
        for (int64_t m = 0; m < M; ++m)
            for (int64_t c = 0; c < C; ++c) v_dump[c * M + m] = f2bf(v[(size_t)(m * C + c)]);
    }
}

// ------------------------------------------------------------------------------------------------
// Gating attention, exact mode: same formula, fp32 inputs, double accumulation, std::exp, no
// intermediate rounding. bias/nb are fp32. Used for the fp32 configuration and as the
// "how far is faithful from the textbook formula" yardstick.
// ------------------------------------------------------------------------------------------------
void orc_gating_attention_exact(const float *x, const float *wq, const float *wk, const float *wv, const float *wg,
                                const float *bg, const float *wo, const float *bo, const float *bias,
                                int64_t bias_stride0, const float *nb, int64_t nb_stride_h, int64_t nb_stride_q,
                                int64_t B, int64_t S, int64_t H, int64_t D, float *out)
{
    const int64_t C = H * D;
    const int64_t M = B * S;
    std::vector<double> q((size_t)(M * C)), k((size_t)(M * C)), v((size_t)(M * C)), g((size_t)(M * C)),
        avg((size_t)(M * C));
    auto proj = [&](const float *w, const float *bvec, std::vector<double> &dst) {
#pragma omp parallel for schedule(static)
        for (int64_t m = 0; m < M; ++m)
            for (int64_t n = 0; n < C; ++n) {
                double acc = 0;
                for (int64_t c = 0; c < C; ++c) acc += (double)x[m * C + c] * (double)w[n * C + c];
                dst[(size_t)(m * C + n)] = acc + (bvec ? (double)bvec[n] : 0.0);
            }
    };
    proj(wq, nullptr, q);
    proj(wk, nullptr, k);
    proj(wv, nullptr, v);
    proj(wg, bg, g);
    const double scale = 1.0 / std::sqrt((double)D);
#pragma omp parallel
    {
        std::vector<double> xs((size_t)S);
#pragma omp for schedule(static)
        for (int64_t bhi = 0; bhi < B * H * S; ++bhi) {
            const int64_t i = bhi % S, h = (bhi / S) % H, b = bhi / (S * H);
            const double *qi = &q[(size_t)((b * S + i) * C + h * D)];
            double mx = -INFINITY;
            for (int64_t j = 0; j < S; ++j) {
                const double *kj = &k[(size_t)((b * S + j) * C + h * D)];
                double acc = 0;
                for (int64_t d = 0; d < D; ++d) acc += qi[d] * kj[d];
                // the reference forms (logit*scale + bias) + nb in fp32; keep the fp32 absorption of
                // small logits by a -1e9 mask bias so fully masked rows stay uniform.
                float val = (float)(acc * scale);
                val = val + bias[b * bias_stride0 + j];
                if (nb) val = val + nb[h * nb_stride_h + i * nb_stride_q + j];
                xs[(size_t)j] = (double)val;
                mx = std::max(mx, (double)val);
            }
            double sum = 0;
            for (int64_t j = 0; j < S; ++j) {
                xs[(size_t)j] = std::exp(xs[(size_t)j] - mx);
                sum += xs[(size_t)j];
            }
            for (int64_t d = 0; d < D; ++d) {
                double acc = 0;
                for (int64_t j = 0; j < S; ++j) acc += xs[(size_t)j] * v[(size_t)((b * S + j) * C + h * D + d)];
                const double gate = 1.0 / (1.0 + std::exp(-g[(size_t)((b * S + i) * C + h * D + d)]));
                avg[(size_t)((b * S + i) * C + h * D + d)] = acc / sum * gate;
            }
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < C; ++n) {
            double acc = 0;
            for (int64_t c = 0; c < C; ++c) acc += avg[(size_t)(m * C + c)] * (double)wo[n * C + c];
            out[m * C + n] = (float)(acc + (double)bo[n]);
        }
}

// ------------------------------------------------------------------------------------------------
// Global attention, faithful mode. Follows src/attention/global_attention.cpp:30-164.
//   x [B,S,C] bf16 contiguous (:53), mask [B,S] bf16 (:55), wq [C,C], wk [D,C], wv [D,C], wg [C,C],
//   wo [C,C] (all W[out][in]), bg, bo fp32; out [B,S,C] bf16.
// ------------------------------------------------------------------------------------------------
void orc_global_attention_bf16(const uint16_t *x, const uint16_t *mask, const uint16_t *wq, const uint16_t *wk,
                               const uint16_t *wv, const uint16_t *wg, const float *bg, const uint16_t *wo,
                               const float *bo, int64_t B, int64_t S, int64_t H, int64_t D, uint16_t *out)
{
    fexpa_init();
    const int64_t C = H * D;
    const int64_t M = B * S;
    std::vector<float> xf, wqf, wkf, wvf, wgf, wof;
    widen(x, M * C, xf);
    widen(wq, C * C, wqf);
    widen(wk, D * C, wkf);
    widen(wv, D * C, wvf);
    widen(wg, C * C, wgf);
    widen(wo, C * C, wof);
    std::vector<float> qavg((size_t)(B * C)), q((size_t)(B * C)), k((size_t)(M * D)), v((size_t)(M * D)),
        g((size_t)(M * C));
    // masked mean (:44-75): fp32 fused multiply-add per row, 1/(sum+1e-10), bf16 store
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        std::vector<float> acc((size_t)C, 0.f);
        float msum = 0.f;
        for (int64_t s = 0; s < S; ++s) {
            const float mv = bf2f(mask[b * S + s]);
            msum += mv;
            const float *xr = &xf[(size_t)((b * S + s) * C)];
            for (int64_t c = 0; c < C; ++c) acc[(size_t)c] = std::fmaf(xr[c], mv, acc[(size_t)c]);
        }
        const float inv = 1.0f / (msum + 1e-10f);
        for (int64_t c = 0; c < C; ++c) qavg[(size_t)(b * C + c)] = rbf(acc[(size_t)c] * inv);
    }
    gemm_nt_bf16out(qavg.data(), C, wqf.data(), C, nullptr, B, C, C, q.data(), C, true);  // :76-79
    gemm_nt_bf16out(xf.data(), C, wkf.data(), C, nullptr, M, D, C, k.data(), D, true);    // :80-84
    gemm_nt_bf16out(xf.data(), C, wvf.data(), C, nullptr, M, D, C, v.data(), D, true);    // :85-89
    gemm_nt_bf16out(xf.data(), C, wgf.data(), C, bg, M, C, C, g.data(), C, true);         // :90-94
    const float scale = (float)(1.0 / std::sqrt((double)D));
#pragma omp parallel
    {
        std::vector<float> xs((size_t)S), p((size_t)(H * S)), wa((size_t)C);
#pragma omp for schedule(static)
        for (int64_t b = 0; b < B; ++b) {
            for (int64_t h = 0; h < H; ++h) {
                float mx = -INFINITY;
                for (int64_t s = 0; s < S; ++s) {
                    float acc = 0.f;
                    for (int64_t d = 0; d < D; ++d) acc += q[(size_t)(b * C + h * D + d)] * k[(size_t)((b * S + s) * D + d)];
                    const float l = rbf(acc);  // logits bf16 (:97-98,109-112)
                    const float mb = std::fmaf(bf2f(mask[b * S + s]), 1e9f, -1e9f);  // :120-121
                    const float val = l * scale + mb;                                 // :122-123
                    xs[(size_t)s] = val;
                    mx = std::max(mx, val);
                }
                float sum = 0.f;
                for (int64_t s = 0; s < S; ++s) {
                    xs[(size_t)s] = fexpa_exp(xs[(size_t)s] - mx);
                    sum += xs[(size_t)s];
                }
                const float inv = 1.0f / sum;
                for (int64_t s = 0; s < S; ++s) p[(size_t)(h * S + s)] = rbf(xs[(size_t)s] * inv);
                for (int64_t d = 0; d < D; ++d) {
                    float acc = 0.f;
                    for (int64_t s = 0; s < S; ++s) acc += p[(size_t)(h * S + s)] * v[(size_t)((b * S + s) * D + d)];
                    wa[(size_t)(h * D + d)] = rbf(acc);  // :129-133
                }
            }
            for (int64_t s = 0; s < S; ++s) {
                float *gr = &g[(size_t)((b * S + s) * C)];
                for (int64_t c = 0; c < C; ++c) gr[c] = rbf(fexpa_sigmoid(gr[c]) * wa[(size_t)c]);  // :134-156
            }
        }
    }
    std::vector<float> of((size_t)(M * C));
    gemm_nt_bf16out(g.data(), C, wof.data(), C, bo, M, C, C, of.data(), C, true);  // :159-163
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M * C; ++i) out[i] = f2bf(of[(size_t)i]);
}

// Global attention, exact mode (fp32 in, double accumulate, std::exp).
void orc_global_attention_exact(const float *x, const float *mask, const float *wq, const float *wk, const float *wv,
                                const float *wg, const float *bg, const float *wo, const float *bo, int64_t B,
                                int64_t S, int64_t H, int64_t D, float *out)
{
    const int64_t C = H * D;
    const double scale = 1.0 / std::sqrt((double)D);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        std::vector<double> qa((size_t)C, 0.0), q((size_t)C), k((size_t)(S * D)), v((size_t)(S * D)), wa((size_t)C),
            xs((size_t)S), gated((size_t)C);
        double msum = 0;
        for (int64_t s = 0; s < S; ++s) {
            const double mv = mask[b * S + s];
            msum += mv;
            for (int64_t c = 0; c < C; ++c) qa[(size_t)c] += mv * (double)x[(b * S + s) * C + c];
        }
        for (int64_t c = 0; c < C; ++c) qa[(size_t)c] /= (msum + 1e-10);
        for (int64_t n = 0; n < C; ++n) {
            double acc = 0;
            for (int64_t c = 0; c < C; ++c) acc += qa[(size_t)c] * (double)wq[n * C + c];
            q[(size_t)n] = acc;
        }
        for (int64_t s = 0; s < S; ++s)
            for (int64_t d = 0; d < D; ++d) {
                double ak = 0, av = 0;
                for (int64_t c = 0; c < C; ++c) {
                    const double xv = x[(b * S + s) * C + c];
                    ak += xv * (double)wk[d * C + c];
                    av += xv * (double)wv[d * C + c];
                }
                k[(size_t)(s * D + d)] = ak;
                v[(size_t)(s * D + d)] = av;
            }
        for (int64_t h = 0; h < H; ++h) {
            double mx = -INFINITY;
            for (int64_t s = 0; s < S; ++s) {
                double acc = 0;
                for (int64_t d = 0; d < D; ++d) acc += q[(size_t)(h * D + d)] * k[(size_t)(s * D + d)];
                const float mb = std::fmaf(mask[b * S + s], 1e9f, -1e9f);
                const float val = (float)(acc * scale) + mb;
                xs[(size_t)s] = val;
                mx = std::max(mx, (double)val);
            }
            double sum = 0;
            for (int64_t s = 0; s < S; ++s) {
                xs[(size_t)s] = std::exp(xs[(size_t)s] - mx);
                sum += xs[(size_t)s];
            }
            for (int64_t d = 0; d < D; ++d) {
                double acc = 0;
                for (int64_t s = 0; s < S; ++s) acc += xs[(size_t)s] * v[(size_t)(s * D + d)];
                wa[(size_t)(h * D + d)] = acc / sum;
            }
        }
        for (int64_t s = 0; s < S; ++s) {
            for (int64_t n = 0; n < C; ++n) {
                double acc = bg[n];
                for (int64_t c = 0; c < C; ++c) acc += (double)x[(b * S + s) * C + c] * (double)wg[n * C + c];
                gated[(size_t)n] = wa[(size_t)n] / (1.0 + std::exp(-acc));
            }
            for (int64_t n = 0; n < C; ++n) {
                double acc = bo[n];
                for (int64_t c = 0; c < C; ++c) acc += gated[(size_t)c] * (double)wo[n * C + c];
                out[(b * S + s) * C + n] = (float)acc;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Linear: result[m,n] = bf16( act[m,k] . weight[n,k] + beta*result + bias[n] ).
// Follows src/linear/linear.cpp:21-42 (beta is an integer cast to bf16, :32).
// ------------------------------------------------------------------------------------------------
void orc_linear_bf16(const uint16_t *act, int64_t lda, const uint16_t *w, int64_t ldw, const float *bias, int64_t M,
                     int64_t N, int64_t K, int64_t beta, uint16_t *result)
{
    const float betaf = rbf((float)beta);
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float acc = 0.f;
            for (int64_t k = 0; k < K; ++k) acc += bf2f(act[m * lda + k]) * bf2f(w[n * ldw + k]);
            if (betaf != 0.f) acc += betaf * bf2f(result[m * N + n]);
            if (bias) acc += bias[n];
            result[m * N + n] = f2bf(acc);
        }
}
void orc_linear_exact(const float *act, int64_t lda, const float *w, int64_t ldw, const float *bias, int64_t M,
                      int64_t N, int64_t K, int64_t beta, float *result)
{
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            double acc = 0;
            for (int64_t k = 0; k < K; ++k) acc += (double)act[m * lda + k] * (double)w[n * ldw + k];
            if (beta != 0) acc += (double)beta * (double)result[m * N + n];
            if (bias) acc += (double)bias[n];
            result[m * N + n] = (float)acc;
        }
}

// ------------------------------------------------------------------------------------------------
// All-gather over simulated ranks. Follows src/comm/all_gather.cpp:21-83: byte-typed tensors
// [m,n,len] sharded on dim 0 (data.sizes[0] != out.sizes[0]) or on dim 1 (data.sizes[0] ==
// out.sizes[0]); block = ceil(x/world); rank r owns rows [r*block, min((r+1)*block, x)).
//   shards[r] : rank r's local tensor with byte strides (ds0[r], ds1)
//   out       : [m, n, len] bytes with byte strides (os0, os1)
// ------------------------------------------------------------------------------------------------
void orc_all_gather_bytes(const uint8_t *const *shards, int64_t world, int64_t data_size0, const int64_t *ds0, int64_t ds1,
                          uint8_t *out, int64_t m, int64_t n, int64_t len, int64_t os0, int64_t os1)
{
    const bool dim1 = (data_size0 == m);
    const int64_t full = dim1 ? n : m;    // extent of the sharded axis
    const int64_t other = dim1 ? m : n;   // extent of the whole axis
    const int64_t block = (full + world - 1) / world;
    for (int64_t r = 0; r < world; ++r) {
        const int64_t have = std::min(block, full - r * block);
        for (int64_t a = 0; a < have; ++a)
            for (int64_t o = 0; o < other; ++o) {
                const int64_t src = dim1 ? (o * ds0[r] + a * ds1) : (a * ds0[r] + o * ds1);
                const int64_t g = a + r * block;
                const int64_t dst = dim1 ? (o * os0 + g * os1) : (g * os0 + o * os1);
                std::memcpy(out + dst, shards[r] + src, (size_t)len);
            }
    }
}

// ------------------------------------------------------------------------------------------------
// Transpose (re-shard) over simulated ranks. Follows src/comm/transpose.cpp:21-86 in its normalised form
// (after the swap of :27-33): rank r holds data [chunk_r(m), n, len] and receives out [m, chunk_r(n), len];
// the element at local row bmi of rank s, column bni + d*block_n goes to rank d, row bmi + s*block_m, column
// bni (:52-57 for the part that stays, :46-51 and :70-77 for the part that travels through the window).
//   data[r] : dense [chunk_r(m)][n][len] bytes        out[r] : dense [m][chunk_r(n)][len] bytes
// ------------------------------------------------------------------------------------------------
void orc_transpose_bytes(const uint8_t *const *data, uint8_t *const *out, int64_t world, int64_t m, int64_t n, int64_t len)
{
    const int64_t bm = (m + world - 1) / world, bn = (n + world - 1) / world;
    for (int64_t s = 0; s < world; ++s) {
        const int64_t cm = std::max<int64_t>(0, std::min(bm, m - s * bm));
        for (int64_t d = 0; d < world; ++d) {
            const int64_t cn = std::max<int64_t>(0, std::min(bn, n - d * bn));
            for (int64_t bmi = 0; bmi < cm; ++bmi)
                for (int64_t bni = 0; bni < cn; ++bni)
                    std::memcpy(out[d] + ((bmi + s * bm) * cn + bni) * len, data[s] + (bmi * n + bni + d * bn) * len,
                                (size_t)len);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// LayerNorm of each row. Follows src/normalization/layernorm_kernel.h:22-53 (one row per call there):
// sums of (x - x[0]) accumulated per vector lane (16 fp32 lanes) and then across the lanes, mean = sum/n +
// x[0], var = max((sum2 - sum*sum/n)/n, 0), rstd = 1/sqrt(var + eps), y = fma(fma(x, rstd, -rstd*mean),
// gamma, beta), bf16 RNE on store. The exact variant uses the textbook two-pass formula in double.
// ------------------------------------------------------------------------------------------------
void orc_layernorm_bf16(const uint16_t *x, const float *gamma, const float *beta, int64_t rows, int64_t size, float eps,
                        uint16_t *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t *xr = x + r * size;
        const float delta = bf2f(xr[0]);
        float lane_sum[16] = {0}, lane_sum2[16] = {0};
        for (int64_t i = 0; i < size; ++i) {
            const float v = bf2f(xr[i]) - delta;
            lane_sum[i & 15] += v;
            lane_sum2[i & 15] = std::fma(v, v, lane_sum2[i & 15]);
        }
        float sum = 0.f, sum2 = 0.f;
        for (int l = 0; l < 16; ++l) {
            sum += lane_sum[l];
            sum2 += lane_sum2[l];
        }
        const float mean = sum / (float)size + delta;
        const float var = std::max((sum2 - sum * sum / (float)size) / (float)size, 0.f);
        const float rstd = 1 / std::sqrt(var + eps);
        const float bias = -rstd * mean;
        for (int64_t i = 0; i < size; ++i)
            out[r * size + i] = f2bf(std::fma(std::fma(bf2f(xr[i]), rstd, bias), gamma[i], beta[i]));
    }
}

void orc_layernorm_exact(const float *x, const float *gamma, const float *beta, int64_t rows, int64_t size, float eps,
                         float *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float *xr = x + r * size;
        double mean = 0, var = 0;
        for (int64_t i = 0; i < size; ++i) mean += xr[i];
        mean /= (double)size;
        for (int64_t i = 0; i < size; ++i) var += (xr[i] - mean) * (xr[i] - mean);
        var /= (double)size;
        const double rstd = 1.0 / std::sqrt(var + (double)eps);
        for (int64_t i = 0; i < size; ++i) out[r * size + i] = (float)((xr[i] - mean) * rstd * gamma[i] + beta[i]);
    }
}

// ------------------------------------------------------------------------------------------------
// Triangle multiplication (src/attention/triangle_multiplication.cpp:25-150), in the four steps the
// reference exports. Layouts: the input activations x are [n_res, n_gather, c_o]; the projections and
// the per-channel products are channel-major, [c_i, n_res, n_gather]; gate and out of the last two steps
// are [n_res, n_gather, c_o]. Biases are fp32.
//
//   calc_proj (:25-70)  p = bf16(x.pw^T + pb), g = bf16(x.gw^T + gb) (both stored), then in place
//                       p = bf16((f32(p) * f32(mask)) * sigmoid(f32(g)))        (:56-65, this order)
//   equation (:75-104)  outgoing: c[ch, a, b] = bf16(sum_k left[ch, a, k] * right[ch, b, k])
//                       incoming: c[ch, a, b] = bf16(sum_k right[ch, k, a] * left[ch, k, b])
//   gate_and_out_linear (:109-133)  two row-bias linears (orc_linear_bf16)
//   last (:138-158)     out = bf16(f32(out) * sigmoid(f32(gate)))
// ------------------------------------------------------------------------------------------------
void orc_tm_calc_proj_bf16(const uint16_t *x, const uint16_t *mask, const uint16_t *pw, const float *pb,
                           const uint16_t *gw, const float *gb, int64_t n_res, int64_t n_gather, int64_t c_o,
                           int64_t c_i, uint16_t *proj, uint16_t *gate)
{
    fexpa_init();
    const int64_t P = n_res * n_gather;
#pragma omp parallel for schedule(static)
    for (int64_t pos = 0; pos < P; ++pos) {
        const uint16_t *xr = x + pos * c_o;
        const float mk = bf2f(mask[pos]);
        for (int64_t ci = 0; ci < c_i; ++ci) {
            float ap = 0.f, ag = 0.f;
            for (int64_t k = 0; k < c_o; ++k) {
                const float xv = bf2f(xr[k]);
                ap += xv * bf2f(pw[ci * c_o + k]);
                ag += xv * bf2f(gw[ci * c_o + k]);
            }
            const uint16_t pbf = f2bf(ap + pb[ci]), gbf = f2bf(ag + gb[ci]);
            gate[ci * P + pos] = gbf;
            float v = bf2f(pbf) * mk;
            v = v * fexpa_sigmoid(bf2f(gbf));
            proj[ci * P + pos] = f2bf(v);
        }
    }
}
void orc_tm_calc_proj_exact(const float *x, const float *mask, const float *pw, const float *pb, const float *gw,
                            const float *gb, int64_t n_res, int64_t n_gather, int64_t c_o, int64_t c_i, float *proj)
{
    const int64_t P = n_res * n_gather;
#pragma omp parallel for schedule(static)
    for (int64_t pos = 0; pos < P; ++pos)
        for (int64_t ci = 0; ci < c_i; ++ci) {
            double ap = pb[ci], ag = gb[ci];
            for (int64_t k = 0; k < c_o; ++k) {
                ap += (double)x[pos * c_o + k] * pw[ci * c_o + k];
                ag += (double)x[pos * c_o + k] * gw[ci * c_o + k];
            }
            proj[ci * P + pos] = (float)(ap * mask[pos] / (1.0 + std::exp(-ag)));
        }
}
void orc_tm_equation_bf16(const uint16_t *left, const uint16_t *right, int64_t c_i, int64_t n, int incoming,
                          uint16_t *center)
{
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t ch = 0; ch < c_i; ++ch)
        for (int64_t a = 0; a < n; ++a) {
            const uint16_t *L = left + ch * n * n, *R = right + ch * n * n;
            for (int64_t b = 0; b < n; ++b) {
                float acc = 0.f;
                if (!incoming)
                    for (int64_t k = 0; k < n; ++k) acc += bf2f(L[a * n + k]) * bf2f(R[b * n + k]);
                else
                    for (int64_t k = 0; k < n; ++k) acc += bf2f(R[k * n + a]) * bf2f(L[k * n + b]);
                center[(ch * n + a) * n + b] = f2bf(acc);
            }
        }
}
void orc_tm_equation_exact(const float *left, const float *right, int64_t c_i, int64_t n, int incoming, float *center)
{
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t ch = 0; ch < c_i; ++ch)
        for (int64_t a = 0; a < n; ++a) {
            const float *L = left + ch * n * n, *R = right + ch * n * n;
            for (int64_t b = 0; b < n; ++b) {
                double acc = 0;
                if (!incoming)
                    for (int64_t k = 0; k < n; ++k) acc += (double)L[a * n + k] * R[b * n + k];
                else
                    for (int64_t k = 0; k < n; ++k) acc += (double)R[k * n + a] * L[k * n + b];
                center[(ch * n + a) * n + b] = (float)acc;
            }
        }
}
void orc_tm_last_bf16(uint16_t *out, const uint16_t *gate, int64_t n)
{
    fexpa_init();
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = f2bf(bf2f(out[i]) * fexpa_sigmoid(bf2f(gate[i])));
}

}  // extern "C"
