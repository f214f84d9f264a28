// kutacc_af2_linear, weight prepack, pack size query, and the fused pair-bias projection.
// Replaces src/linear/linear.cpp:21-50, src/linear/mm.cpp:94-110, src/utils/blas.cpp:93-98.
#include <cuda_runtime.h>

#include <climits>
#include <cstring>

#include "common.h"
#include "kernels.h"

extern "C" void kutacc_af2_linear(kutacc_tensor_h act_h, kutacc_tensor_h weight_h, float *bias_data,
                                  kutacc_tensor_h result_h, int64_t beta)
{
    using namespace kutacc;
    KUTACC_CHECK(act_h != nullptr && weight_h != nullptr && result_h != nullptr, "kutacc_af2_linear: nullptr error");
    if (kutacc_check_err_set) return;
    Tensor &act = *as_tensor(act_h), &weight = *as_tensor(weight_h), &result = *as_tensor(result_h);
    KUTACC_CHECK(act.dim() >= 1 && weight.dim() >= 1 && act.data_ptr() && weight.data_ptr() && result.data_ptr(),
                 "kutacc_af2_linear: empty tensor");
    if (kutacc_check_err_set) return;
    // shapes as linear.cpp:23-25: m = numel / last, n = rows of weight, k = last dim of act
    const int64_t k = act.sizes().back();
    KUTACC_CHECK(k > 0 && weight.sizes().back() == k, "shape invalid, act k: [", k, "], weight k: [",
                 weight.sizes().back(), "]");
    if (kutacc_check_err_set) return;
    const int64_t m = act.numel() / k, n = weight.numel() / k;
    const int64_t lda = act.dim() >= 2 ? act.strides()[(size_t)act.dim() - 2] : k;
    const int64_t ldw = weight.dim() >= 2 ? weight.strides()[(size_t)weight.dim() - 2] : k;
    const DType dt = act.dtype();
    KUTACC_CHECK(dt == kBF16 || dt == kFP32, "addmm dtype invalid, a: [", (int)dt, "]");
    KUTACC_CHECK(m > 0 && n > 0 && lda >= k && ldw >= k, "kutacc_af2_linear: shape/stride invalid m=", m, " n=", n,
                 " lda=", lda, " ldw=", ldw);
    if (kutacc_check_err_set) return;
    const size_t es = dtype_size(dt);
    const size_t a_bytes = (size_t)((m - 1) * lda + k) * es, w_bytes = (size_t)((n - 1) * ldw + k) * es,
                 r_bytes = (size_t)m * n * es, b_bytes = bias_data ? (size_t)n * 4 : 0;

    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    const size_t stage = staged_bytes_needed(act.data_ptr(), a_bytes) + staged_bytes_needed(weight.data_ptr(), w_bytes) +
                         staged_bytes_needed(result.data_ptr(), r_bytes) + staged_bytes_needed(bias_data, b_bytes);
    if (!rt.reserve_stage(stage)) return;
    DeviceArg d_a = resolve_in(act.data_ptr(), a_bytes), d_w = resolve_in(weight.data_ptr(), w_bytes);
    DeviceArg d_b = bias_data ? resolve_in(bias_data, b_bytes) : DeviceArg{};
    // beta != 0 reads the old result (linear.cpp:32)
    DeviceArg d_r = beta != 0 ? resolve_in(result.data_ptr(), r_bytes) : resolve_out(result.data_ptr(), r_bytes);
    if (d_r.staged && beta != 0) d_r.host = result.data_ptr();
    if (kutacc_check_err_set) return;

    const dev::ElemType et = dt == kFP32 ? dev::kElemF32 : dev::kElemBF16;
    bool ok = false;
    const bool a16 = (((uintptr_t)d_a.dev | (uintptr_t)d_w.dev) & 15u) == 0;
    if (dt == kBF16 && beta == 0 && a16 && k % 64 == 0 && n % 128 == 0 && lda == k && ldw == k && m <= INT32_MAX) {
        // the tcgen05 projection kernel on the [1, m, k] view of the activations
        ok = dev::tcgen05_linear_bias_bf16(stream, d_a.dev, d_w.dev, (const float *)d_b.dev, d_r.dev, n, 1, (int)m, (int)n,
                                           (int)k);
        if (kutacc_check_err_set) return;
    }
    if (dt == kFP32 && beta == 0 && a16 && k % 32 == 0 && n % 128 == 0 && lda % 4 == 0 && ldw % 4 == 0 && k <= INT32_MAX / 2 &&
        n <= INT32_MAX && (((uintptr_t)d_r.dev | (uintptr_t)d_b.dev) & 15u) == 0) {
        // fp32 on the tensor-memory GEMM: both operands split into tf32 head and tail in the workspace
        const size_t as_bytes = (size_t)m * 2 * k * 4, ws_bytes = (size_t)n * 2 * k * 4;
        if (rt.reserve_workspace(as_bytes + ws_bytes + 512)) {
            void *a_split = rt.take_workspace(as_bytes), *w_split = rt.take_workspace(ws_bytes);
            const void *wp[1] = {w_split};
            const float *bp[1] = {(const float *)d_b.dev};
            void *op[1] = {d_r.dev};
            ok = a_split && w_split && dev::launch_split_tf32(stream, d_a.dev, lda, a_split, m, (int)k) &&
                 dev::launch_split_tf32(stream, d_w.dev, ldw, w_split, n, (int)k) &&
                 dev::tcgen05_gemm_tf32x3(stream, a_split, wp, bp, op, n, m, (int)n, (int)k, 1);
        }
        if (kutacc_check_err_set) return;
    }
    if (!ok && dt == kBF16 && beta == 0 && a16 && k % 64 == 0 && n % 64 == 0 && lda % 8 == 0 && ldw == k) {
        ok = dev::launch_linear_bias_bf16(stream, d_a.dev, lda, d_w.dev, (const float *)d_b.dev, d_r.dev, n, m, (int)n,
                                          (int)k);
    } else if (beta == 0 && bias_data == nullptr && n <= 16 && lda == k && ldw == k && k <= INT32_MAX) {
        // skinny projection (the pair-bias shape): bandwidth-bound kernel, result [m, n]
        ok = dev::launch_pair_bias(stream, et, d_a.dev, d_w.dev, d_r.dev, 1, n, m, 1, (int)k, (int)n);
    }
    if (!ok) {
        float betaf = (float)beta;
        if (dt == kBF16) {  // beta passes through bf16 in the reference (linear.cpp:32)
            uint32_t u;
            std::memcpy(&u, &betaf, 4);
            u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
            std::memcpy(&betaf, &u, 4);
        }
        ok = dev::launch_gemm_generic(stream, et, d_a.dev, lda, d_w.dev, ldw, (const float *)d_b.dev, betaf, d_r.dev, n,
                                      m, n, k);
    }
    KUTACC_CHECK(ok, "kutacc_af2_linear: no device kernel for m=", m, " n=", n, " k=", k);
    finish_out(d_r);
    end_of_call();
}

// The packed image is the dense row-major [n, k] matrix; rows are copied block by block as the
// reference does (mm.cpp:97-106). Host or device pointers; num_threads is ignored.
extern "C" void kutacc_af2_linear_weight_prepack(const uint16_t *weight, uint16_t *result, int64_t n, int64_t k,
                                                 int64_t ldb, int64_t num_threads)
{
    using namespace kutacc;
    (void)num_threads;
    KUTACC_CHECK(weight != nullptr && result != nullptr && n > 0 && k > 0 && ldb >= k,
                 "kutacc_af2_linear_weight_prepack: invalid argument");
    if (kutacc_check_err_set) return;
    const bool dsrc = is_device_pointer(weight), ddst = is_device_pointer(result);
    if (!dsrc && !ddst) {
        for (int64_t r = 0; r < n; ++r) std::memcpy(result + r * k, weight + r * ldb, (size_t)k * 2);
        return;
    }
    KUTACC_CUDA(cudaMemcpy2DAsync(result, (size_t)k * 2, weight, (size_t)ldb * 2, (size_t)k * 2, (size_t)n,
                                  cudaMemcpyDefault, (cudaStream_t)runtime().stream));
    end_of_call();
}

extern "C" size_t kutacc_af2_gemm_pack_get_size(char identifier, char transa, char transb, int m, int n, int k)
{
    (void)transa;
    (void)transb;
    if (m < 0 || n < 0 || k < 0) return 0;
    if (identifier == 'A' || identifier == 'a') return (size_t)m * (size_t)k;
    return (size_t)k * (size_t)n;
}

// nb[h, r, c] = z[r, c, :] . wb[h, :]
extern "C" void kutacc_b200_pair_bias(kutacc_tensor_h z_h, kutacc_tensor_h wb_h, kutacc_tensor_h nb_h)
{
    using namespace kutacc;
    KUTACC_CHECK(z_h != nullptr && wb_h != nullptr && nb_h != nullptr, "kutacc_b200_pair_bias: nullptr error");
    if (kutacc_check_err_set) return;
    Tensor &z = *as_tensor(z_h), &wb = *as_tensor(wb_h), &nb = *as_tensor(nb_h);
    KUTACC_CHECK(z.dim() == 3 && wb.dim() == 2 && nb.dim() == 3 && z.data_ptr() && wb.data_ptr() && nb.data_ptr(),
                 "kutacc_b200_pair_bias: z [rows, keys, c_z], wb [nheads, c_z], nb [nheads, rows, keys] expected");
    if (kutacc_check_err_set) return;
    const int64_t R = z.sizes()[0], Nk = z.sizes()[1], Cz = z.sizes()[2], H = wb.sizes()[0];
    const DType dt = z.dtype();
    KUTACC_CHECK((dt == kBF16 || dt == kFP32) && wb.sizes()[1] == Cz && nb.sizes()[0] == H && nb.sizes()[1] == R &&
                     nb.sizes()[2] == Nk && z.strides()[2] == 1 && z.strides()[1] == Cz && z.strides()[0] == Nk * Cz &&
                     nb.strides()[2] == 1 && nb.strides()[1] >= Nk && wb.strides()[1] == 1 && wb.strides()[0] == Cz &&
                     R > 0 && Nk > 0 && Cz > 0 && H > 0 && H <= 16 && Cz <= 4096,
                 "kutacc_b200_pair_bias: shape/stride invalid");
    if (kutacc_check_err_set) return;
    const size_t es = dtype_size(dt);
    const int64_t hs = nb.strides()[0], rs = nb.strides()[1];   // rs > Nk: rows apart, e.g. [rows, nheads, keys] storage
    const size_t z_bytes = (size_t)R * Nk * Cz * es, w_bytes = (size_t)H * Cz * es,
                 nb_bytes = (size_t)((H - 1) * hs + (R - 1) * rs + Nk) * es;
    Runtime &rt = runtime();
    const size_t stage = staged_bytes_needed(z.data_ptr(), z_bytes) + staged_bytes_needed(wb.data_ptr(), w_bytes) +
                         staged_bytes_needed(nb.data_ptr(), nb_bytes);
    if (!rt.reserve_stage(stage)) return;
    DeviceArg d_z = resolve_in(z.data_ptr(), z_bytes), d_w = resolve_in(wb.data_ptr(), w_bytes),
              d_n = resolve_out(nb.data_ptr(), nb_bytes);
    if (kutacc_check_err_set) return;
    const bool ok = dev::launch_pair_bias((cudaStream_t)rt.stream, dt == kFP32 ? dev::kElemF32 : dev::kElemBF16,
                                          d_z.dev, d_w.dev, d_n.dev, hs, 1, R, Nk, (int)Cz, (int)H, rs);
    KUTACC_CHECK(ok, "kutacc_b200_pair_bias: no device kernel for nheads=", H, " c_z=", Cz, " row stride ", rs);
    finish_out(d_n);
    end_of_call();
}

// Pair bias of LayerNorm(z): nb[h, r, k] = LayerNorm(z[r, k, :]) . wb[h, :]. The normalisation is folded into the
// projection (one read of z for the row statistics, one for the product; the normalised tensor is never written).
// Shapes the folded tensor-core kernel does not cover normalise into the workspace first.
extern "C" void kutacc_b200_pair_bias_ln(kutacc_tensor_h z_h, const float *ln_gamma, const float *ln_beta, float eps,
                                         kutacc_tensor_h wb_h, kutacc_tensor_h nb_h)
{
    using namespace kutacc;
    KUTACC_CHECK(z_h != nullptr && wb_h != nullptr && nb_h != nullptr && ln_gamma != nullptr && ln_beta != nullptr,
                 "kutacc_b200_pair_bias_ln: nullptr error");
    if (kutacc_check_err_set) return;
    Tensor &z = *as_tensor(z_h), &wb = *as_tensor(wb_h), &nb = *as_tensor(nb_h);
    KUTACC_CHECK(z.dim() == 3 && wb.dim() == 2 && nb.dim() == 3 && z.data_ptr() && wb.data_ptr() && nb.data_ptr(),
                 "kutacc_b200_pair_bias_ln: z [rows, keys, c_z], wb [nheads, c_z], nb [nheads, rows, keys] expected");
    if (kutacc_check_err_set) return;
    const int64_t R = z.sizes()[0], Nk = z.sizes()[1], Cz = z.sizes()[2], H = wb.sizes()[0];
    KUTACC_CHECK(z.dtype() == kBF16 && wb.sizes()[1] == Cz && nb.sizes()[0] == H && nb.sizes()[1] == R && nb.sizes()[2] == Nk &&
                     z.strides()[2] == 1 && z.strides()[1] == Cz && z.strides()[0] == Nk * Cz && nb.strides()[2] == 1 &&
                     nb.strides()[1] == Nk && wb.strides()[1] == 1 && wb.strides()[0] == Cz && R > 0 && Nk > 0 && Cz > 0 &&
                     H > 0 && H <= 16 && Cz <= 4096 && eps >= 0.f,
                 "kutacc_b200_pair_bias_ln: shape/stride invalid (bf16 only)");
    if (kutacc_check_err_set) return;
    const int64_t hs = nb.strides()[0], P = R * Nk;
    const size_t z_bytes = (size_t)P * Cz * 2, w_bytes = (size_t)H * Cz * 2, nb_bytes = (size_t)((H - 1) * hs + P) * 2,
                 g_bytes = (size_t)Cz * 4;
    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    if (!rt.reserve_stage(staged_bytes_needed(z.data_ptr(), z_bytes) + staged_bytes_needed(wb.data_ptr(), w_bytes) +
                          staged_bytes_needed(nb.data_ptr(), nb_bytes) + 2 * staged_bytes_needed(ln_gamma, g_bytes)))
        return;
    // workspace: statistics, folded weights with s and t, and room for the normalised copy of the fallback
    if (!rt.reserve_workspace((size_t)P * 8 + w_bytes + 2 * (size_t)H * 4 + z_bytes + 4 * 256)) return;
    DeviceArg d_z = resolve_in(z.data_ptr(), z_bytes), d_w = resolve_in(wb.data_ptr(), w_bytes),
              d_g = resolve_in(ln_gamma, g_bytes), d_b = resolve_in(ln_beta, g_bytes), d_n = resolve_out(nb.data_ptr(), nb_bytes);
    void *stats = rt.take_workspace((size_t)P * 8), *w2 = rt.take_workspace(w_bytes);
    float *s = (float *)rt.take_workspace((size_t)H * 4), *t = (float *)rt.take_workspace((size_t)H * 4);
    if (kutacc_check_err_set) return;
    const void *w_in[1] = {d_w.dev};
    const float *no_bias[1] = {nullptr};
    void *w_out[1] = {w2};
    float *s_out[1] = {s}, *t_out[1] = {t};
    bool ok = H <= 8 && (Cz == 128 || Cz == 64) && ((uintptr_t)d_z.dev % 16) == 0 &&
              dev::launch_ln_stats(stream, d_z.dev, P, Cz, Cz, eps, stats) &&
              dev::launch_ln_fold(stream, 1, w_in, no_bias, (const float *)d_g.dev, (const float *)d_b.dev, w_out, s_out, t_out,
                                  (int)H, (int)Cz) &&
              dev::launch_pair_bias_ln(stream, d_z.dev, w2, stats, s, t, d_n.dev, hs, R, Nk, (int)Cz, (int)H);
    if (!ok && !kutacc_check_err_set) {
        void *zn = rt.take_workspace(z_bytes);
        ok = zn != nullptr &&
             dev::launch_layernorm_rows(stream, d_z.dev, (const float *)d_g.dev, (const float *)d_b.dev, zn, P, Cz, Cz, Cz, eps) &&
             dev::launch_pair_bias(stream, dev::kElemBF16, zn, d_w.dev, d_n.dev, hs, 1, R, Nk, (int)Cz, (int)H);
    }
    KUTACC_CHECK(ok, "kutacc_b200_pair_bias_ln: no device kernel for nheads=", H, " c_z=", Cz);
    finish_out(d_n);
    end_of_call();
}
