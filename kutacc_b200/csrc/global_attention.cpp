// kutacc_af2_global_attention: validation, device resolution, kernel sequence.
// Replaces src/attention/global_attention.cpp:30-205 of the reference.
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>

#include "common.h"
#include "kernels.h"

extern "C" void kutacc_af2_global_attention(kutacc_af2_attention_inputs_t *q_based_ptr, kutacc_tensor_h q_data,
                                            kutacc_tensor_h q_mask, kutacc_af2_attention_weights_t *weight_ptr,
                                            kutacc_tensor_h out)
{
    using namespace kutacc;
    // nulls and the 64-channel restriction are rejected up front (global_attention.cpp:171-173)
    KUTACC_CHECK(q_based_ptr != nullptr && q_data != nullptr && q_mask != nullptr && weight_ptr != nullptr &&
                     out != nullptr && weight_ptr->nchannels == 64,
                 "kutacc_af2_global_attention: input args nullptr error or invalid int value error");
    if (kutacc_check_err_set) return;
    const int64_t B = q_based_ptr->batch, S = q_based_ptr->seq_len;
    const int64_t C = weight_ptr->nchannels, H = weight_ptr->nheads, D = weight_ptr->head_size;
    // scalar ranges (global_attention.cpp:36-39)
    KUTACC_CHECK(B > 0 && S > 0 && C > 0 && H > 0 && D > 0 && B <= INT32_MAX / S && S <= INT32_MAX && C <= INT32_MAX &&
                     D <= INT32_MAX && H <= INT64_MAX / S && H <= INT64_MAX / D,
                 "input param <= 0 or overflow");
    KUTACC_CHECK(weight_ptr->query_w && weight_ptr->key_w && weight_ptr->value_w && weight_ptr->gating_w &&
                     weight_ptr->gating_b && weight_ptr->output_w && weight_ptr->output_b,
                 "kutacc_af2_global_attention: weight handle nullptr error");
    if (kutacc_check_err_set) return;
    KUTACC_CHECK(H * D == C, "nchannels != nheads * head_size: ", C, " ", H, " ", D);
    if (kutacc_check_err_set) return;

    Tensor &x = *as_tensor(q_data), &mask = *as_tensor(q_mask), &o = *as_tensor(out);
    const Tensor &wq = *as_tensor(weight_ptr->query_w), &wk = *as_tensor(weight_ptr->key_w),
                 &wv = *as_tensor(weight_ptr->value_w), &wg = *as_tensor(weight_ptr->gating_w),
                 &bg = *as_tensor(weight_ptr->gating_b), &wo = *as_tensor(weight_ptr->output_w),
                 &bo = *as_tensor(weight_ptr->output_b);
    KUTACC_CHECK(x.dtype() == kBF16, "global_attention dtype invalid: [", (int)x.dtype(), "]");
    KUTACC_CHECK(x.data_ptr() && mask.data_ptr() && o.data_ptr() && wq.data_ptr() && wk.data_ptr() && wv.data_ptr() &&
                     wg.data_ptr() && bg.data_ptr() && wo.data_ptr() && bo.data_ptr(),
                 "global_attention: null data pointer");
    KUTACC_CHECK(o.dim() >= 2, "global_attention: out rank invalid");
    if (kutacc_check_err_set) return;
    const int64_t out_rs = o.dim() >= 3 ? o.strides()[1] : o.strides()[0];
    const int64_t M = B * S;
    const size_t x_bytes = (size_t)M * C * 2, m_bytes = (size_t)M * 2, out_bytes = (size_t)((M - 1) * out_rs + C) * 2;
    const size_t wcc = (size_t)C * C * 2, wdc = (size_t)D * C * 2, bb = (size_t)C * 4;

    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    size_t stage = staged_bytes_needed(x.data_ptr(), x_bytes) + staged_bytes_needed(mask.data_ptr(), m_bytes) +
                   staged_bytes_needed(o.data_ptr(), out_bytes) + staged_bytes_needed(wq.data_ptr(), wcc) +
                   staged_bytes_needed(wk.data_ptr(), wdc) + staged_bytes_needed(wv.data_ptr(), wdc) +
                   staged_bytes_needed(wg.data_ptr(), wcc) + staged_bytes_needed(wo.data_ptr(), wcc) +
                   staged_bytes_needed(bg.data_ptr(), bb) + staged_bytes_needed(bo.data_ptr(), bb);
    if (!rt.reserve_stage(stage)) return;
    const size_t scratch_bytes = dev::global_attention_scratch_bytes((int)B, (int)S, (int)H, (int)D);
    if (!rt.reserve_workspace(scratch_bytes + 256)) return;
    // Host-resident activations and result: the batch columns are independent, so they go through in
    // chunks with upload, kernels and download overlapped on three streams (as in the gated attention).
    const bool pipelined = staged_bytes_needed(x.data_ptr(), x_bytes) != 0 && staged_bytes_needed(o.data_ptr(), out_bytes) != 0 &&
                           B >= 8 && x_bytes >= ((size_t)4 << 20) && out_rs == C;
    DeviceArg d_x = pipelined ? resolve_out(x.data_ptr(), x_bytes) : resolve_in(x.data_ptr(), x_bytes);
    DeviceArg d_m = resolve_in(mask.data_ptr(), m_bytes);
    DeviceArg d_wq = resolve_in(wq.data_ptr(), wcc), d_wk = resolve_in(wk.data_ptr(), wdc),
              d_wv = resolve_in(wv.data_ptr(), wdc), d_wg = resolve_in(wg.data_ptr(), wcc),
              d_wo = resolve_in(wo.data_ptr(), wcc), d_bg = resolve_in(bg.data_ptr(), bb),
              d_bo = resolve_in(bo.data_ptr(), bb);
    DeviceArg d_out = resolve_out(o.data_ptr(), out_bytes);
    if (pipelined) {
        // the copy streams start once the previous work on the runtime stream and the small uploads above are done
        CopyPipeline &cp0 = copy_pipeline(1);
        if (kutacc_check_err_set) return;
        KUTACC_CUDA(cudaEventRecord((cudaEvent_t)cp0.start, stream));
        KUTACC_CUDA(cudaStreamWaitEvent((cudaStream_t)cp0.in, (cudaEvent_t)cp0.start, 0));
        KUTACC_CUDA(cudaStreamWaitEvent((cudaStream_t)cp0.out, (cudaEvent_t)cp0.start, 0));
    }
    void *scratch = rt.take_workspace(scratch_bytes);
    if (kutacc_check_err_set) return;
    // the kernels read activations and weights with 4- to 16-byte vector loads
    KUTACC_CHECK((((uintptr_t)d_x.dev | (uintptr_t)d_out.dev | (uintptr_t)d_wg.dev | (uintptr_t)d_wo.dev |
                   (uintptr_t)d_wq.dev | (uintptr_t)d_wk.dev | (uintptr_t)d_wv.dev) & 15u) == 0,
                 "global_attention: q_data, out and the five weights must be 16-byte aligned");
    if (kutacc_check_err_set) return;
    // one pass over HBM where the shape allows it (a cluster of CTAs holds each column in shared memory),
    // otherwise three kernels per L2-sized group of columns with the split-softmax state in `scratch`
    auto run_cols = [&](int64_t b0, int64_t nb) -> bool {
        const char *xc = (const char *)d_x.dev + (size_t)b0 * S * C * 2;
        const char *mc = (const char *)d_m.dev + (size_t)b0 * S * 2;
        char *oc = (char *)d_out.dev + (size_t)b0 * S * out_rs * 2;
        bool done = dev::launch_global_fused_bf16(stream, xc, mc, d_wq.dev, d_wk.dev, d_wv.dev, d_wg.dev,
                                                  (const float *)d_bg.dev, d_wo.dev, (const float *)d_bo.dev, oc, out_rs,
                                                  (int)nb, (int)S, (int)H, (int)D);
        if (kutacc_check_err_set) return false;
        if (!done)
            done = dev::launch_global_attention_bf16(stream, xc, mc, d_wq.dev, d_wk.dev, d_wv.dev, d_wg.dev,
                                                     (const float *)d_bg.dev, d_wo.dev, (const float *)d_bo.dev, oc,
                                                     out_rs, scratch, (int)nb, (int)S, (int)H, (int)D);
        return done;
    };
    bool ok = true;
    if (!pipelined) {
        ok = run_cols(0, B);
    } else {
        int nchunks = (int)std::max<int64_t>(2, std::min<int64_t>(12, (int64_t)((x_bytes + ((size_t)4 << 20)) >> 23)));
        nchunks = (int)std::max<int64_t>(1, std::min<int64_t>(nchunks, B / 4));
        // chunk sizes shrink towards the end: the kernels and the download of the last chunk overlap nothing
        int64_t chunk_begin[17];
        const int64_t wsum = (int64_t)nchunks * (nchunks + 5) / 2;
        int64_t acc = 0;
        for (int i = 0; i < nchunks; ++i) {
            chunk_begin[i] = std::min<int64_t>(B, (acc * B + wsum / 2) / wsum);
            acc += nchunks + 2 - i;
        }
        chunk_begin[nchunks] = B;
        CopyPipeline &cp = copy_pipeline(nchunks);
        if (kutacc_check_err_set) return;
        cudaStream_t s_in = (cudaStream_t)cp.in, s_out = (cudaStream_t)cp.out;
        const size_t col_bytes = (size_t)S * C * 2;
        for (int i = 0; i < nchunks; ++i) {                 // every upload is queued before the first kernel
            const int64_t b0 = chunk_begin[i], nb = chunk_begin[i + 1] - b0;
            if (nb <= 0) continue;
            KUTACC_CUDA(cudaMemcpyAsync((char *)d_x.dev + b0 * col_bytes, (const char *)x.data_ptr() + b0 * col_bytes,
                                        (size_t)nb * col_bytes, cudaMemcpyHostToDevice, s_in));
            KUTACC_CUDA(cudaEventRecord((cudaEvent_t)cp.uploaded[i], s_in));
        }
        for (int i = 0; i < nchunks && ok; ++i) {
            const int64_t b0 = chunk_begin[i], nb = chunk_begin[i + 1] - b0;
            if (nb <= 0) continue;
            KUTACC_CUDA(cudaStreamWaitEvent(stream, (cudaEvent_t)cp.uploaded[i], 0));
            ok = run_cols(b0, nb);
            KUTACC_CUDA(cudaEventRecord((cudaEvent_t)cp.computed[i], stream));
            KUTACC_CUDA(cudaStreamWaitEvent(s_out, (cudaEvent_t)cp.computed[i], 0));
            KUTACC_CUDA(cudaMemcpyAsync((char *)o.data_ptr() + b0 * col_bytes, (const char *)d_out.dev + b0 * col_bytes,
                                        (size_t)nb * col_bytes, cudaMemcpyDeviceToHost, s_out));
        }
        KUTACC_CUDA(cudaStreamSynchronize(s_out));
    }
    if (kutacc_check_err_set) return;
    KUTACC_CHECK(ok, "global_attention: no device kernel for nheads=", H, " head_size=", D, " out row stride ", out_rs);
    if (!pipelined && d_out.staged)   // only the C elements of each row: gaps of a strided host `out` stay untouched
        copy_rows_d2h(d_out.host, d_out.dev, (size_t)M, (size_t)C * 2, (size_t)out_rs * 2, stream);
    end_of_call();
}
