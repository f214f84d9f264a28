// The four exported steps of the triangle multiplication (outgoing and incoming edges).
// Replaces src/attention/triangle_multiplication.cpp:25-262 of the reference. The matrix products run on the
// tcgen05 projection kernel (channel-major stores for the projections, one right-hand matrix per channel for the
// per-channel products) where the shape allows it, and on plain CUDA-core kernels otherwise; the mask, gate and
// sigmoid steps are element-wise kernels. Host or device tensors (host tensors are staged like everywhere else).
#include <cuda_runtime.h>

#include <climits>

#include "common.h"
#include "kernels.h"

namespace kutacc {
namespace {

// bytes spanned by a [d0, d1, d2] bf16 view with unit last stride
size_t span3(const Tensor &t, int64_t d0, int64_t d1, int64_t d2)
{
    return (size_t)((d0 - 1) * t.strides()[0] + (d1 - 1) * t.strides()[1] + d2) * 2;
}
bool dense3(const Tensor &t, int64_t d1, int64_t d2) { return t.strides()[1] == d2 && t.strides()[0] == d1 * d2; }

// an output whose strides leave gaps is brought in first, so that the bytes between its elements survive the
// copy back of a staged host tensor
DeviceArg resolve_out_keeping_gaps(void *p, size_t bytes, bool dense)
{
    return dense ? resolve_out(p, bytes) : resolve_in(p, bytes);
}

}  // namespace
}  // namespace kutacc

extern "C" void kutacc_af2_triangle_multiplication_calc_proj(kutacc_af2_tm_act_inputs_t *tm_acts_ptr, kutacc_tensor_h mask_h,
                                                             kutacc_af2_tm_proj_weights_t *tm_weights_ptr, bool input_prepack)
{
    using namespace kutacc;
    (void)input_prepack;
    KUTACC_CHECK(tm_acts_ptr != nullptr && mask_h != nullptr && tm_weights_ptr != nullptr,
                 "kutacc_af2_triangle_multiplication_calc_proj: input args nullptr error");
    if (kutacc_check_err_set) return;
    const int64_t n_res = tm_acts_ptr->n_res, n_gather = tm_acts_ptr->n_res_gather;
    const int64_t c_o = tm_weights_ptr->c_o, c_i = tm_weights_ptr->c_i;
    // triangle_multiplication.cpp:29-34
    KUTACC_CHECK(n_res > 0 && n_gather > 0 && c_o > 0 && c_i > 0 && n_res <= INT64_MAX / n_gather && n_res <= INT64_MAX / c_i &&
                     c_o <= INT32_MAX && c_i <= INT32_MAX && n_res <= INT32_MAX && n_gather <= INT32_MAX,
                 "input param <= 0 or overflow");
    if (kutacc_check_err_set) return;
    KUTACC_CHECK(tm_acts_ptr->proj_act && tm_acts_ptr->input_act && tm_acts_ptr->proj_act_gate && tm_weights_ptr->proj_w &&
                     tm_weights_ptr->proj_b && tm_weights_ptr->gate_w && tm_weights_ptr->gate_b,
                 "kutacc_af2_triangle_multiplication_calc_proj: tensor handle nullptr error");
    if (kutacc_check_err_set) return;
    Tensor &proj = *as_tensor(tm_acts_ptr->proj_act), &x = *as_tensor(tm_acts_ptr->input_act),
           &gate = *as_tensor(tm_acts_ptr->proj_act_gate), &mask = *as_tensor(mask_h);
    const Tensor &pw = *as_tensor(tm_weights_ptr->proj_w), &pb = *as_tensor(tm_weights_ptr->proj_b),
                 &gw = *as_tensor(tm_weights_ptr->gate_w), &gb = *as_tensor(tm_weights_ptr->gate_b);
    KUTACC_CHECK(proj.data_ptr() && x.data_ptr() && gate.data_ptr() && mask.data_ptr() && pw.data_ptr() && pb.data_ptr() &&
                     gw.data_ptr() && gb.data_ptr(),
                 "kutacc_af2_triangle_multiplication_calc_proj: null data pointer");
    KUTACC_CHECK(x.dtype() == kBF16, "addmm dtype invalid, a: [", (int)x.dtype(), "]");
    KUTACC_CHECK(proj.dim() >= 2 && gate.dim() >= 2 && mask.dim() >= 1, "triangle_multiplication_calc_proj: tensor rank invalid");
    if (kutacc_check_err_set) return;
    const int64_t P = n_res * n_gather;
    // channel-major outputs: strides()[0] between channels, strides()[1] between rows of n_res_gather positions
    const int64_t p_s0 = proj.strides()[0], p_s1 = proj.dim() >= 3 ? proj.strides()[1] : n_gather;
    const int64_t g_s0 = gate.strides()[0], g_s1 = gate.dim() >= 3 ? gate.strides()[1] : n_gather;
    const int64_t m_s0 = mask.dim() >= 2 ? mask.strides()[0] : n_gather;
    const size_t x_bytes = (size_t)P * c_o * 2, w_bytes = (size_t)c_i * c_o * 2, b_bytes = (size_t)c_i * 4;
    const size_t p_bytes = (size_t)((c_i - 1) * p_s0 + (n_res - 1) * p_s1 + n_gather) * 2;
    const size_t g_bytes = (size_t)((c_i - 1) * g_s0 + (n_res - 1) * g_s1 + n_gather) * 2;
    const size_t m_bytes = (size_t)((n_res - 1) * m_s0 + n_gather) * 2;
    const bool p_dense = p_s1 == n_gather && p_s0 == P, g_dense = g_s1 == n_gather && g_s0 == P;

    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    const size_t stage = staged_bytes_needed(x.data_ptr(), x_bytes) + staged_bytes_needed(mask.data_ptr(), m_bytes) +
                         staged_bytes_needed(proj.data_ptr(), p_bytes) + staged_bytes_needed(gate.data_ptr(), g_bytes) +
                         2 * staged_bytes_needed(pw.data_ptr(), w_bytes) + 2 * staged_bytes_needed(pb.data_ptr(), b_bytes) + 1024;
    if (!rt.reserve_stage(stage)) return;
    DeviceArg d_x = resolve_in(x.data_ptr(), x_bytes), d_m = resolve_in(mask.data_ptr(), m_bytes),
              d_pw = resolve_in(pw.data_ptr(), w_bytes), d_gw = resolve_in(gw.data_ptr(), w_bytes),
              d_pb = resolve_in(pb.data_ptr(), b_bytes), d_gb = resolve_in(gb.data_ptr(), b_bytes);
    DeviceArg d_p = resolve_out_keeping_gaps(proj.data_ptr(), p_bytes, p_dense),
              d_g = resolve_out_keeping_gaps(gate.data_ptr(), g_bytes, g_dense);
    if (kutacc_check_err_set) return;

    bool ok = p_s0 == g_s0 && p_s1 == g_s1 &&
              dev::tcgen05_proj2_chanmajor_bf16(stream, d_x.dev, d_pw.dev, (const float *)d_pb.dev, d_gw.dev,
                                                (const float *)d_gb.dev, d_p.dev, d_g.dev, p_s0, p_s1, (int)n_res,
                                                (int)n_gather, (int)c_i, (int)c_o);
    if (kutacc_check_err_set) return;
    if (!ok)
        ok = dev::launch_tm_proj_generic(stream, d_x.dev, d_pw.dev, (const float *)d_pb.dev, d_gw.dev, (const float *)d_gb.dev,
                                         d_p.dev, d_g.dev, p_s0, p_s1, g_s0, g_s1, n_res, n_gather, c_o, c_i);
    ok = ok && dev::launch_tm_mask_gate(stream, d_p.dev, d_g.dev, d_m.dev, c_i, n_res, n_gather, p_s0, p_s1, g_s0, g_s1, m_s0);
    KUTACC_CHECK(ok, "triangle_multiplication_calc_proj: no device kernel for c_o=", c_o, " c_i=", c_i);
    finish_out(d_p);
    finish_out(d_g);
    end_of_call();
}

extern "C" void kutacc_af2_triangle_multiplication_equation(kutacc_tensor_h center_h, kutacc_tensor_h left_h,
                                                            kutacc_tensor_h right_h, int64_t n_res_gather, bool is_incoming)
{
    using namespace kutacc;
    KUTACC_CHECK(center_h != nullptr && left_h != nullptr && right_h != nullptr,
                 "kutacc_af2_triangle_multiplication_equation: input args nullptr error");
    KUTACC_CHECK(n_res_gather > 0, "kutacc_af2_triangle_multiplication_equation: input args int values error, values "
                                   "are less than or equal to zero");
    if (kutacc_check_err_set) return;
    Tensor &center = *as_tensor(center_h), &left = *as_tensor(left_h), &right = *as_tensor(right_h);
    KUTACC_CHECK(center.dim() >= 2 && left.dim() >= 2 && right.dim() >= 2 && center.data_ptr() && left.data_ptr() &&
                     right.data_ptr() && n_res_gather <= INT32_MAX,
                 "triangle_multiplication_equation: [c_i, n, n] tensors expected");
    KUTACC_CHECK(left.dtype() == kBF16, "addmm dtype invalid, a: [", (int)left.dtype(), "]");
    if (kutacc_check_err_set) return;
    const int64_t c_i = left.sizes()[0], n = n_res_gather;          // :77, the loop runs over left's channels
    KUTACC_CHECK(c_i > 0 && c_i <= INT32_MAX, "triangle_multiplication_equation: channel count invalid");
    if (kutacc_check_err_set) return;
    const int64_t l_s0 = left.strides()[0], l_s1 = left.strides()[1], r_s0 = right.strides()[0], r_s1 = right.strides()[1],
                  c_s0 = center.strides()[0], c_s1 = center.strides()[1];
    const size_t l_bytes = span3(left, c_i, n, n), r_bytes = span3(right, c_i, n, n), c_bytes = span3(center, c_i, n, n);
    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    if (!rt.reserve_stage(staged_bytes_needed(left.data_ptr(), l_bytes) + staged_bytes_needed(right.data_ptr(), r_bytes) +
                          staged_bytes_needed(center.data_ptr(), c_bytes)))
        return;
    const int64_t pitch = (n + 7) / 8 * 8;                           // transposed copies for the incoming product
    if (is_incoming && !rt.reserve_workspace(2 * ((size_t)c_i * n * pitch * 2 + 256))) return;
    DeviceArg d_l = resolve_in(left.data_ptr(), l_bytes), d_r = resolve_in(right.data_ptr(), r_bytes);
    DeviceArg d_c = resolve_out_keeping_gaps(center.data_ptr(), c_bytes, dense3(center, n, n));
    if (kutacc_check_err_set) return;
    bool ok = false;
    if (!is_incoming) {
        // center[a, b] = sum_k left[a, k] * right[b, k]
        ok = dev::tcgen05_batched_nt_bf16(stream, d_l.dev, l_s1, l_s0, d_r.dev, r_s1, r_s0, d_c.dev, c_s1, c_s0, (int)c_i, (int)n,
                                          (int)n, (int)n);
    } else {
        // center[a, b] = sum_k right[k, a] * left[k, b] = sum_k right^T[a, k] * left^T[b, k]: both operands are
        // transposed once (a pass over HBM each), then the same product runs
        void *lt = rt.take_workspace((size_t)c_i * n * pitch * 2), *rtp = rt.take_workspace((size_t)c_i * n * pitch * 2);
        if (kutacc_check_err_set) return;
        ok = dev::launch_tm_transpose(stream, d_l.dev, l_s0, l_s1, lt, pitch, c_i, n) &&
             dev::launch_tm_transpose(stream, d_r.dev, r_s0, r_s1, rtp, pitch, c_i, n) &&
             dev::tcgen05_batched_nt_bf16(stream, rtp, pitch, n * pitch, lt, pitch, n * pitch, d_c.dev, c_s1, c_s0, (int)c_i,
                                          (int)n, (int)n, (int)n);
    }
    if (kutacc_check_err_set) return;
    if (!ok)
        ok = dev::launch_tm_equation_generic(stream, d_l.dev, l_s0, l_s1, d_r.dev, r_s0, r_s1, d_c.dev, c_s0, c_s1, c_i, n,
                                             is_incoming);
    KUTACC_CHECK(ok, "triangle_multiplication_equation: no device kernel for n=", n);
    finish_out(d_c);
    end_of_call();
}

extern "C" void kutacc_af2_triangle_multiplication_gate_and_out_linear(kutacc_tensor_h gate_h, kutacc_tensor_h out_h,
                                                                       kutacc_af2_tm_act_inputs_t *tm_acts_ptr,
                                                                       kutacc_tensor_h center_h,
                                                                       kutacc_af2_tm_linear_weights_t *tm_weights_ptr,
                                                                       bool input_prepack)
{
    using namespace kutacc;
    (void)input_prepack;
    KUTACC_CHECK(gate_h != nullptr && out_h != nullptr && tm_acts_ptr != nullptr && center_h != nullptr &&
                     tm_weights_ptr != nullptr,
                 "kutacc_af2_triangle_multiplication_gate_and_out_linear: input args nullptr error");
    if (kutacc_check_err_set) return;
    const int64_t n_res = tm_acts_ptr->n_res, n_gather = tm_acts_ptr->n_res_gather;
    const int64_t c_o = tm_weights_ptr->c_o, c_i = tm_weights_ptr->c_i;
    // triangle_multiplication.cpp:113-118
    KUTACC_CHECK(n_res > 0 && n_gather > 0 && c_o > 0 && c_i > 0 && n_res <= INT64_MAX / n_gather && c_o <= INT32_MAX &&
                     c_i <= INT32_MAX && n_res <= INT32_MAX && n_gather <= INT32_MAX,
                 "input param <= 0 or overflow");
    if (kutacc_check_err_set) return;
    KUTACC_CHECK(tm_acts_ptr->input_act && tm_weights_ptr->gating_w && tm_weights_ptr->gating_b &&
                     tm_weights_ptr->output_proj_w && tm_weights_ptr->output_proj_b,
                 "kutacc_af2_triangle_multiplication_gate_and_out_linear: tensor handle nullptr error");
    if (kutacc_check_err_set) return;
    Tensor &gate = *as_tensor(gate_h), &out = *as_tensor(out_h), &x = *as_tensor(tm_acts_ptr->input_act),
           &center = *as_tensor(center_h);
    const Tensor &gw = *as_tensor(tm_weights_ptr->gating_w), &gb = *as_tensor(tm_weights_ptr->gating_b),
                 &ow = *as_tensor(tm_weights_ptr->output_proj_w), &ob = *as_tensor(tm_weights_ptr->output_proj_b);
    KUTACC_CHECK(gate.data_ptr() && out.data_ptr() && x.data_ptr() && center.data_ptr() && gw.data_ptr() && gb.data_ptr() &&
                     ow.data_ptr() && ob.data_ptr(),
                 "kutacc_af2_triangle_multiplication_gate_and_out_linear: null data pointer");
    KUTACC_CHECK(x.dtype() == kBF16, "addmm dtype invalid, a: [", (int)x.dtype(), "]");
    KUTACC_CHECK(gate.dim() >= 2 && out.dim() >= 2 && center.dim() >= 2, "triangle_multiplication_gate_and_out_linear: tensor rank invalid");
    if (kutacc_check_err_set) return;
    const int64_t P = n_res * n_gather;
    // row strides as the reference reads them: strides()[1] of [n_res, n_res_gather, channels] tensors (:121,128,130)
    const int64_t g_rs = gate.strides()[1], o_rs = out.strides()[1], c_rs = center.strides()[1];
    KUTACC_CHECK(g_rs >= c_o && o_rs >= c_o && c_rs >= c_i, "triangle_multiplication_gate_and_out_linear: row stride below the channel count");
    if (kutacc_check_err_set) return;
    const size_t x_bytes = (size_t)P * c_o * 2, g_bytes = (size_t)((P - 1) * g_rs + c_o) * 2,
                 o_bytes = (size_t)((P - 1) * o_rs + c_o) * 2, c_bytes = (size_t)((P - 1) * c_rs + c_i) * 2;
    const size_t gw_bytes = (size_t)c_o * c_o * 2, ow_bytes = (size_t)c_o * c_i * 2, b_bytes = (size_t)c_o * 4;
    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    if (!rt.reserve_stage(staged_bytes_needed(x.data_ptr(), x_bytes) + staged_bytes_needed(gate.data_ptr(), g_bytes) +
                          staged_bytes_needed(out.data_ptr(), o_bytes) + staged_bytes_needed(center.data_ptr(), c_bytes) +
                          staged_bytes_needed(gw.data_ptr(), gw_bytes) + staged_bytes_needed(ow.data_ptr(), ow_bytes) +
                          2 * staged_bytes_needed(gb.data_ptr(), b_bytes)))
        return;
    DeviceArg d_x = resolve_in(x.data_ptr(), x_bytes), d_c = resolve_in(center.data_ptr(), c_bytes),
              d_gw = resolve_in(gw.data_ptr(), gw_bytes), d_ow = resolve_in(ow.data_ptr(), ow_bytes),
              d_gb = resolve_in(gb.data_ptr(), b_bytes), d_ob = resolve_in(ob.data_ptr(), b_bytes);
    DeviceArg d_g = resolve_out_keeping_gaps(gate.data_ptr(), g_bytes, g_rs == c_o),
              d_o = resolve_out_keeping_gaps(out.data_ptr(), o_bytes, o_rs == c_o);
    if (kutacc_check_err_set) return;
    bool ok = dev::tcgen05_linear_bias_bf16(stream, d_x.dev, d_gw.dev, (const float *)d_gb.dev, d_g.dev, g_rs, (int)n_res,
                                            (int)n_gather, (int)c_o, (int)c_o, false, c_o);
    if (kutacc_check_err_set) return;
    if (!ok)
        ok = dev::launch_gemm_generic(stream, dev::kElemBF16, d_x.dev, c_o, d_gw.dev, c_o, (const float *)d_gb.dev, 0.f, d_g.dev,
                                      g_rs, P, c_o, c_o);
    bool ok2 = ok && dev::tcgen05_linear_bias_bf16(stream, d_c.dev, d_ow.dev, (const float *)d_ob.dev, d_o.dev, o_rs, (int)n_res,
                                                   (int)n_gather, (int)c_o, (int)c_i, false, c_rs);
    if (kutacc_check_err_set) return;
    if (ok && !ok2)
        ok2 = dev::launch_gemm_generic(stream, dev::kElemBF16, d_c.dev, c_rs, d_ow.dev, c_i, (const float *)d_ob.dev, 0.f, d_o.dev,
                                       o_rs, P, c_o, c_i);
    KUTACC_CHECK(ok && ok2, "triangle_multiplication_gate_and_out_linear: no device kernel for c_o=", c_o, " c_i=", c_i);
    finish_out(d_g);
    finish_out(d_o);
    end_of_call();
}

extern "C" void kutacc_af2_triangle_multiplication_last(kutacc_tensor_h out_h, kutacc_tensor_h gate_h, int64_t n_res,
                                                        int64_t n_res_gather, int64_t c_o)
{
    using namespace kutacc;
    KUTACC_CHECK(out_h != nullptr && gate_h != nullptr, "kutacc_af2_triangle_multiplication_last: input args nullptr error");
    KUTACC_CHECK(n_res > 0 && n_res_gather > 0 && c_o > 0 && n_res <= INT64_MAX / n_res_gather,
                 "kutacc_af2_triangle_multiplication_last: input args int values error, values are less than or equal "
                 "to zero, or overflow");
    if (kutacc_check_err_set) return;
    Tensor &out = *as_tensor(out_h), &gate = *as_tensor(gate_h);
    KUTACC_CHECK(out.dim() >= 2 && gate.dim() >= 2 && out.data_ptr() && gate.data_ptr(),
                 "triangle_multiplication_last: [n_res, n_res_gather, c_o] tensors expected");
    if (kutacc_check_err_set) return;
    // rows are addressed as bi * strides()[0] + si * strides()[1] (:144-145); the kernel takes one row stride, so the
    // batch stride must be n_res_gather rows
    const int64_t o_rs = out.strides()[1], g_rs = gate.strides()[1];
    KUTACC_CHECK(out.strides()[0] == n_res_gather * o_rs && gate.strides()[0] == n_res_gather * g_rs && o_rs >= c_o && g_rs >= c_o,
                 "triangle_multiplication_last: rows of out and gate must be evenly spaced");
    if (kutacc_check_err_set) return;
    const int64_t P = n_res * n_res_gather;
    const size_t o_bytes = (size_t)((P - 1) * o_rs + c_o) * 2, g_bytes = (size_t)((P - 1) * g_rs + c_o) * 2;
    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    if (!rt.reserve_stage(staged_bytes_needed(out.data_ptr(), o_bytes) + staged_bytes_needed(gate.data_ptr(), g_bytes))) return;
    DeviceArg d_o = resolve_in(out.data_ptr(), o_bytes), d_g = resolve_in(gate.data_ptr(), g_bytes);
    if (kutacc_check_err_set) return;
    const bool ok = dev::launch_tm_last(stream, d_o.dev, o_rs, d_g.dev, g_rs, P, c_o);
    KUTACC_CHECK(ok, "triangle_multiplication_last: launch failed");
    finish_out(d_o);
    end_of_call();
}
