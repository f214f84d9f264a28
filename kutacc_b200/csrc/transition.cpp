// kutacc_af2_transition: out = relu(x . W1^T + b1) . W2^T + b2, the transition MLP of the Evoformer.
// Replaces src/attention/transition.cpp:21-61 (two addmm calls with a row bias, the first with ReLU; the
// intermediate is a bf16 tensor). Both products run on the tcgen05 projection kernel (ReLU in its epilogue);
// shapes it does not cover take the generic GEMM. The intermediate lives in the library's workspace: the
// caller's intermediate_act tensor is not written, like the scratch tensors of the attention operators.
#include <cuda_runtime.h>

#include <climits>

#include "common.h"
#include "kernels.h"

extern "C" void kutacc_af2_transition(kutacc_af2_trans_act_inputs_t *trans_inputs_ptr,
                                      kutacc_af2_trans_weights_t *trans_weights_ptr, kutacc_tensor_h out_h)
{
    using namespace kutacc;
    // handle / struct nulls first (transition.cpp:44-51), then the scalars (:25-30), then the tensors
    KUTACC_CHECK(trans_inputs_ptr != nullptr && trans_weights_ptr != nullptr && out_h != nullptr,
                 "kutacc_af2_transition: input args nullptr error");
    if (kutacc_check_err_set) return;
    const int64_t batch = trans_inputs_ptr->batch, n_res = trans_inputs_ptr->n_res;
    const int64_t c_o = trans_weights_ptr->c_o, c_i = trans_weights_ptr->c_i;
    KUTACC_CHECK(batch > 0 && n_res > 0 && c_o > 0 && c_i > 0 && batch <= INT64_MAX / n_res && c_o <= INT32_MAX &&
                     c_i <= INT32_MAX && n_res <= INT32_MAX && batch <= INT32_MAX,
                 "input param <= 0 or overflow");
    if (kutacc_check_err_set) return;
    KUTACC_CHECK(trans_inputs_ptr->input_act && trans_weights_ptr->linear1_w && trans_weights_ptr->linear1_b &&
                     trans_weights_ptr->linear2_w && trans_weights_ptr->linear2_b,
                 "kutacc_af2_transition: tensor handle nullptr error");
    if (kutacc_check_err_set) return;
    Tensor &x = *as_tensor(trans_inputs_ptr->input_act), &o = *as_tensor(out_h);
    const Tensor &w1 = *as_tensor(trans_weights_ptr->linear1_w), &b1 = *as_tensor(trans_weights_ptr->linear1_b),
                 &w2 = *as_tensor(trans_weights_ptr->linear2_w), &b2 = *as_tensor(trans_weights_ptr->linear2_b);
    KUTACC_CHECK(x.data_ptr() && o.data_ptr() && w1.data_ptr() && b1.data_ptr() && w2.data_ptr() && b2.data_ptr(),
                 "kutacc_af2_transition: null data pointer");
    KUTACC_CHECK(x.dtype() == kBF16, "addmm dtype invalid, a: [", (int)x.dtype(), "]");
    if (kutacc_check_err_set) return;
    const int64_t M = batch * n_res;
    const size_t x_bytes = (size_t)M * c_o * 2, h_bytes = (size_t)M * c_i * 2, w_bytes = (size_t)c_o * c_i * 2;
    const size_t b1_bytes = (size_t)c_i * 4, b2_bytes = (size_t)c_o * 4;

    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    const size_t stage = staged_bytes_needed(x.data_ptr(), x_bytes) + staged_bytes_needed(o.data_ptr(), x_bytes) +
                         staged_bytes_needed(w1.data_ptr(), w_bytes) + staged_bytes_needed(w2.data_ptr(), w_bytes) +
                         staged_bytes_needed(b1.data_ptr(), b1_bytes) + staged_bytes_needed(b2.data_ptr(), b2_bytes);
    if (!rt.reserve_stage(stage)) return;
    if (!rt.reserve_workspace(h_bytes + 256)) return;
    DeviceArg d_x = resolve_in(x.data_ptr(), x_bytes), d_w1 = resolve_in(w1.data_ptr(), w_bytes),
              d_w2 = resolve_in(w2.data_ptr(), w_bytes), d_b1 = resolve_in(b1.data_ptr(), b1_bytes),
              d_b2 = resolve_in(b2.data_ptr(), b2_bytes);
    DeviceArg d_o = resolve_out(o.data_ptr(), x_bytes);
    void *hid = rt.take_workspace(h_bytes);
    if (kutacc_check_err_set) return;

    // hidden = relu(x . W1^T + b1): W1 is stored [c_i][c_o] (transition.cpp:32, the {c_o, c_i} view with strides {1, c_o})
    bool ok = dev::tcgen05_linear_bias_bf16(stream, d_x.dev, d_w1.dev, (const float *)d_b1.dev, hid, c_i, (int)batch,
                                            (int)n_res, (int)c_i, (int)c_o, true);
    if (kutacc_check_err_set) return;
    if (!ok) {
        ok = dev::launch_gemm_generic(stream, dev::kElemBF16, d_x.dev, c_o, d_w1.dev, c_o, (const float *)d_b1.dev, 0.f, hid,
                                      c_i, M, c_i, c_o) &&
             dev::launch_relu_bf16(stream, hid, M * c_i);
    }
    // out = hidden . W2^T + b2: W2 is stored [c_o][c_i] (transition.cpp:36)
    if (ok) {
        bool ok2 = dev::tcgen05_linear_bias_bf16(stream, hid, d_w2.dev, (const float *)d_b2.dev, d_o.dev, c_o, (int)batch,
                                                 (int)n_res, (int)c_o, (int)c_i, false);
        if (kutacc_check_err_set) return;
        if (!ok2)
            ok2 = dev::launch_gemm_generic(stream, dev::kElemBF16, hid, c_i, d_w2.dev, c_i, (const float *)d_b2.dev, 0.f,
                                           d_o.dev, c_o, M, c_o, c_i);
        ok = ok2;
    }
    KUTACC_CHECK(ok, "kutacc_af2_transition: no device kernel for c_o=", c_o, " c_i=", c_i);
    finish_out(d_o);
    end_of_call();
}
