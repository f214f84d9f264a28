// Launchers of the device kernels. Plain pointers and integers only: the operator entry points
// translate tensor descriptors into these calls. Every launcher enqueues on `stream` and returns
// false (after reporting through KUTACC_CHECK) when the shape is outside what it supports.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace kutacc {
namespace dev {

enum ElemType { kElemBF16 = 0, kElemF32 = 1 };

// ---- projections ---------------------------------------------------------------------------------
// Fused Q/K/V/gate projection of x [M = B*S, C] with four [C, C] weights (W[out][in]).
//   q, k, v : [B, H, S, D] (q pre-multiplied by q_scale), gate : [B, S, C] with bg added.
// bf16 in / bf16 out, fp32 accumulate. Needs C % 64 == 0.
bool launch_proj_qkvg_bf16(cudaStream_t stream, const void *x, const void *wq, const void *wk, const void *wv,
                           const void *wg, const float *bg, void *q, void *k, void *v, void *gate, int B, int S,
                           int H, int D, float q_scale);

// out[m, :] = a[m, :] . w^T + bias, a [M, K] (row stride lda), w [N, K], out row stride ldo.
// bf16 in / bf16 out, fp32 accumulate. Needs K % 64 == 0 and N % 64 == 0.
bool launch_linear_bias_bf16(cudaStream_t stream, const void *a, int64_t lda, const void *w, const float *bias,
                             void *out, int64_t ldo, int64_t M, int N, int K);

// tcgen05/TMEM/TMA versions of the two GEMMs above (C % 128 == 0, D in {32, 64}; N % 128 == 0,
// K % 64 == 0, out row stride % 8 == 0). q is written unscaled. With v_transposed, v is written as
// [B, H, D, S] with row pitch v_pitch (what the tcgen05 attention core consumes) instead of [B, H, S, D].
// Return false when the shape is not covered.
// With gate_sigmoid the gate segment stores bf16(sigmoid(bf16(x.Wg + bg))) instead of bf16(x.Wg + bg).
// With ln_stats (float2 mean/rstd per row of x) the four weights are LayerNorm-folded ones (launch_ln_fold) and the
// epilogue applies y = rstd * (acc - mean * ln_s[seg][n]) + ln_t[seg][n] (ln_t carries the gate bias; bg is ignored).
bool tcgen05_proj_qkvg_bf16(cudaStream_t stream, const void *x, const void *wq, const void *wk, const void *wv,
                            const void *wg, const float *bg, void *q, void *k, void *v, void *gate, int B, int S,
                            int H, int D, bool v_transposed, int64_t v_pitch, bool gate_sigmoid = false,
                            const void *ln_stats = nullptr, const float *const *ln_s = nullptr,
                            const float *const *ln_t = nullptr);
// a_row_stride (elements, 0 = K): row stride of a, whose batch rows are S rows apart.
bool tcgen05_linear_bias_bf16(cudaStream_t stream, const void *a, const void *w, const float *bias, void *out,
                              int64_t out_row_stride, int B, int S, int N, int K, bool relu = false,
                              int64_t a_row_stride = 0);
// out_i[n, b, s] = x[b, s, :] . w_i[n, :] + bias_i[n], i = 0, 1: two projections stored channel-major
// (N % 128 == 0, K % 64 == 0, strides multiples of 8 elements). False when the shape is not covered.
bool tcgen05_proj2_chanmajor_bf16(cudaStream_t stream, const void *x, const void *w0, const float *bias0, const void *w1,
                                  const float *bias1, void *out0, void *out1, int64_t out_c_stride, int64_t out_b_stride,
                                  int B, int S, int N, int K);
// out[b, m, n] = sum_k a[b, m, k] * w[b, n, k]: one right-hand matrix per batch (strides multiples of 8 elements).
bool tcgen05_batched_nt_bf16(cudaStream_t stream, const void *a, int64_t a_row_stride, int64_t a_batch_stride,
                             const void *w, int64_t w_row_stride, int64_t w_batch_stride, void *out,
                             int64_t out_row_stride, int64_t out_batch_stride, int B, int M, int N, int K);

// fp32 GEMM on tcgen05 (gemm_tf32_tcgen05.cu): operands pre-split into tf32 head and tail, stored as rows
// [hi(0..K) | lo(0..K)] by launch_split_tf32 (src [rows, K] fp32 with row stride src_ld; dst [rows, 2K] dense).
// out_i[m, :] = a[m, :] . w_i^T (+ bias_i) for up to four weight matrices [N, K] in one pass over a; out row stride
// ldo. Needs N % 128 == 0, K % 32 == 0, 16-byte aligned pointers. False when the shape is not covered.
bool launch_split_tf32(cudaStream_t stream, const void *src, int64_t src_ld, void *dst, int64_t rows, int K);
// the same for up to eight matrices of one shape in a single launch
bool launch_split_tf32_many(cudaStream_t stream, int count, const void *const *src, int64_t src_ld, void *const *dst,
                            int64_t rows, int K);
bool tcgen05_gemm_tf32x3(cudaStream_t stream, const void *a_split, const void *const *w_split, const float *const *bias,
                         void *const *out, int64_t ldo, int64_t M, int N, int K, int nseg);

// ---- triangle multiplication: element-wise steps and fallbacks (tm_kernels.cu) ------------------------
// proj[c, b, i] = bf16((f32(proj) * f32(mask[b, i])) * sigmoid(f32(gate[c, b, i]))) in place; strides in elements.
bool launch_tm_mask_gate(cudaStream_t stream, void *proj, const void *gate, const void *mask, int64_t c_i, int64_t n_res,
                         int64_t n_gather, int64_t p_s0, int64_t p_s1, int64_t g_s0, int64_t g_s1, int64_t m_s0);
// proj and gate of the projection step on CUDA cores (any shape): see tcgen05_proj2_chanmajor_bf16.
bool launch_tm_proj_generic(cudaStream_t stream, const void *x, const void *w0, const float *b0, const void *w1,
                            const float *b1, void *out0, void *out1, int64_t p_s0, int64_t p_s1, int64_t g_s0,
                            int64_t g_s1, int64_t n_res, int64_t n_gather, int64_t c_o, int64_t c_i);
// center[c, a, b] = sum_k left[c, a, k] * right[c, b, k] (incoming = 0) or sum_k right[c, k, a] * left[c, k, b]
// on CUDA cores (any shape).
bool launch_tm_equation_generic(cudaStream_t stream, const void *left, int64_t l_s0, int64_t l_s1, const void *right,
                                int64_t r_s0, int64_t r_s1, void *center, int64_t c_s0, int64_t c_s1, int64_t c_i,
                                int64_t n, bool incoming);
// dst[c, a, k] = src[c, k, a] for every channel c (n x n matrices; dst dense with row pitch d_pitch)
bool launch_tm_transpose(cudaStream_t stream, const void *src, int64_t s_s0, int64_t s_s1, void *dst, int64_t d_pitch,
                         int64_t c_i, int64_t n);
// out[r, :] = bf16(f32(out[r, :]) * sigmoid(f32(gate[r, :]))) for rows of c_o elements
bool launch_tm_last(cudaStream_t stream, void *out, int64_t o_rs, const void *gate, int64_t g_rs, int64_t rows, int64_t c_o);

// ---- fused attention core ------------------------------------------------------------------------
// avg[b, s, h*D + d] = sigmoid(gate[b, s, h*D + d]) * softmax_k(bf16(q.k)*scale + bias[b,k] + nb[h,s,k]) . v
// q, k, v are [B, H, S, D]. bf16; D in {16, 32, 64}. nb may be null; its strides must be multiples
// of 8 elements and its base 16-byte aligned (TMA).
bool launch_attn_core_bf16(cudaStream_t stream, const void *q, const void *k, const void *v, const void *gate,
                           const void *bias, int64_t bias_stride0, const void *nb, int64_t nb_stride_h,
                           int64_t nb_stride_q, void *avg, int B, int S, int H, int D, float scale);

// The same operator with both products on tcgen05 and the accumulators in tensor memory (head size 32).
// vt is v transposed, [B, H, D, S] with row pitch vt_pitch, as tcgen05_proj_qkvg_bf16 writes it. With
// gate_is_sigmoid, `gate` already holds bf16(sigmoid(bf16(x.Wg + bg))) (the projection kernel's gate_sigmoid
// option) and the kernel only multiplies.
bool tcgen05_attn_core_bf16(cudaStream_t stream, const void *q, const void *k, const void *vt, int64_t vt_pitch,
                            const void *gate, const void *bias, int64_t bias_stride0, const void *nb,
                            int64_t nb_stride_h, int64_t nb_stride_q, void *avg, int B, int S, int H, int D,
                            float scale, bool gate_is_sigmoid);

// ---- generic (any shape, bf16 or fp32 storage, fp32 math) ------------------------------------------
// c[m, n] = sum_k a[m, k] * w[n, k] (+ bias[n]) (+ beta * c[m, n]); a row stride lda, w row stride
// ldw, c row stride ldc.
bool launch_gemm_generic(cudaStream_t stream, ElemType t, const void *a, int64_t lda, const void *w, int64_t ldw,
                         const float *bias, float beta, void *c, int64_t ldc, int64_t M, int64_t N, int64_t K);
bool launch_relu_bf16(cudaStream_t stream, void *x, int64_t n);
// Attention core on [B, S, C]-shaped q/k/v/gate (head h at channel offset h*D); scale applied here.
bool launch_attn_generic(cudaStream_t stream, ElemType t, const void *q, const void *k, const void *v,
                         const void *gate, const void *bias, int64_t bias_stride0, const void *nb,
                         int64_t nb_stride_h, int64_t nb_stride_q, void *avg, int B, int S, int H, int D,
                         float scale);

// ---- pair-bias projection --------------------------------------------------------------------------
// y[h * head_stride + (r * Nk + k) * pos_stride] = z[r, k, :] . wb[h, :], z [R, Nk, Cz] contiguous.
// (head_stride = R*Nk, pos_stride = 1) writes [H, R, Nk]; (1, H) writes [R*Nk, H]. H <= 16.
// nb_row_stride (elements, 0 = Nk): distance between the output rows of one head when they are not dense, e.g.
// H * Nk for a [R, H, Nk] layout with head stride Nk (bf16, c_z 64 or 128, pos_stride 1 only).
bool launch_pair_bias(cudaStream_t stream, ElemType t, const void *z, const void *wb, void *nb,
                      int64_t nb_head_stride, int64_t pos_stride, int64_t R, int64_t Nk, int Cz, int H,
                      int64_t nb_row_stride = 0);
// The same projection of LayerNorm(z) with folded weights (launch_ln_fold) and per-position statistics: only the
// tensor-core kernel (bf16, c_z 64 or 128, up to 8 heads, [H, R, Nk] output); false otherwise.
bool launch_pair_bias_ln(cudaStream_t stream, const void *z, const void *wb_folded, const void *stats, const float *ln_s,
                         const float *ln_t, void *nb, int64_t nb_head_stride, int64_t R, int64_t Nk, int Cz, int H);

// ---- global attention (bf16, C = 64) ---------------------------------------------------------------
// scratch: qk [B, H, 64] fp32-sized slots and wa [B, 64]; see global_attention.cu
// fp32 attention core on tensor cores (error-compensated tf32), head size 32; false for other shapes.
// With avg_split the result is written as rows [tf32 head | tail] of 2 * H * D floats (the operand layout of
// tcgen05_gemm_tf32x3) instead of into avg.
bool launch_attn_f32(cudaStream_t stream, const void *q, const void *k, const void *v, const void *gate, const void *bias,
                     int64_t bias_stride0, const void *nb, int64_t nb_stride_h, int64_t nb_stride_q, void *avg, int B,
                     int S, int H, int D, float scale, void *avg_split = nullptr);

// LayerNorm folded into the projection that follows (ln_fold.cu): per-row (mean, rstd) pairs as float2, and
// for up to four [N, K] weight matrices the folded, centred bf16 weights with the epilogue terms s and t
// (y = rstd * (acc - mean * s[n]) + t[n]).
bool launch_ln_stats(cudaStream_t stream, const void *x, int64_t rows, int64_t size, int64_t x_stride, float eps, void *stats);
bool launch_ln_fold(cudaStream_t stream, int nmat, const void *const *w, const float *const *bias, const float *gamma,
                    const float *beta, void *const *w2, float *const *s, float *const *t, int N, int K);

// LayerNorm of every row of a [rows, size] bf16 matrix (strides in elements); fp32 gamma and beta.
bool launch_layernorm_rows(cudaStream_t stream, const void *x, const float *gamma, const float *beta, void *out,
                           int64_t rows, int64_t size, int64_t x_stride, int64_t out_stride, float eps);

// Global attention in one pass over HBM (thread-block clusters hold a column in shared memory); 8 heads x 8
// only. Returns false when the shape is not covered.
bool launch_global_fused_bf16(cudaStream_t stream, const void *x, const void *mask, const void *wq, const void *wk,
                              const void *wv, const void *wg, const float *bg, const void *wo, const float *bo,
                              void *out, int64_t out_row_stride, int B, int S, int H, int D);
size_t global_attention_scratch_bytes(int B, int S, int H, int D);
bool launch_global_attention_bf16(cudaStream_t stream, const void *x, const void *mask, const void *wq,
                                  const void *wk, const void *wv, const void *wg, const float *bg, const void *wo,
                                  const float *bo, void *out, int64_t out_row_stride, void *scratch, int B, int S,
                                  int H, int D);

}  // namespace dev
}  // namespace kutacc
