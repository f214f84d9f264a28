// kutacc_af2_gating_attention: validation, device resolution of the arguments, kernel sequence.
// Replaces src/attention/gating_attention.cpp:33-200 of the reference.
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cmath>

#include "common.h"
#include "kernels.h"

namespace kutacc {

namespace {
bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

// LayerNorm applied to `input` before the projections (kutacc_b200_gating_attention_ln): fp32 gamma and beta of
// nchannels elements, host or device.
struct LayerNormArgs {
    const float *gamma, *beta;
    float eps;
};
}  // namespace

static void gating_attention_impl(Tensor &input, int64_t batch, int64_t seq_len, Tensor &bias, Tensor &nonbatched_bias,
                                  const Tensor &query_w, const Tensor &key_w, const Tensor &value_w,
                                  const Tensor &gating_w, const Tensor &gating_b, const Tensor &output_w,
                                  const Tensor &output_b, Tensor &out, int64_t block_size, int64_t head_size,
                                  int64_t nheads, int64_t nchannels, const LayerNormArgs *ln = nullptr)
{
    // same scalar validation, in the same place, as gating_attention.cpp:39-45 and :69
    KUTACC_CHECK(batch > 0 && seq_len > 0 && block_size > 0 && head_size > 0 && nheads > 0 && nchannels > 0 &&
                     batch <= INT32_MAX / seq_len && seq_len <= INT32_MAX && nchannels <= INT32_MAX &&
                     head_size <= INT32_MAX && block_size <= INT64_MAX / seq_len,
                 "input param <= 0 or overflow");
    if (kutacc_check_err_set) return;
    const int64_t nblocks = (seq_len + block_size - 1) / block_size;
    KUTACC_CHECK(batch <= INT64_MAX / nheads / nblocks, "parallel end overflow");
    KUTACC_CHECK(nheads * head_size == nchannels, "nchannels != nheads * head_size: ", nchannels, " ", nheads, " ",
                 head_size);
    if (kutacc_check_err_set) return;

    const DType dt = input.dtype();
    KUTACC_CHECK(dt == kBF16 || dt == kFP32, "gating_attention dtype invalid: [", (int)dt, "]");
    KUTACC_CHECK(ln == nullptr || dt == kBF16, "gating_attention with LayerNorm: bf16 only");
    KUTACC_CHECK(input.data_ptr() && bias.data_ptr() && out.data_ptr() && query_w.data_ptr() && key_w.data_ptr() &&
                     value_w.data_ptr() && gating_w.data_ptr() && gating_b.data_ptr() && output_w.data_ptr() &&
                     output_b.data_ptr(),
                 "gating_attention: null data pointer");
    KUTACC_CHECK(bias.dim() >= 1 && out.dim() >= 2, "gating_attention: bias/out rank invalid");
    if (kutacc_check_err_set) return;

    const bool has_nb = nonbatched_bias.dim() > 0 && nonbatched_bias.sizes()[0] != 0;  // :103
    if (has_nb) {
        KUTACC_CHECK(nonbatched_bias.dim() >= 3 && nonbatched_bias.data_ptr() != nullptr,
                     "gating_attention: nonbatched_bias must be [nheads, seq_len, seq_len]");
        if (kutacc_check_err_set) return;
    }

    const int64_t B = batch, S = seq_len, H = nheads, D = head_size, C = nchannels, M = B * S;
    const size_t es = dtype_size(dt);
    const int64_t bias_s0 = bias.dim() >= 2 ? bias.strides()[0] : 0;
    const int64_t nb_s0 = has_nb ? nonbatched_bias.strides()[0] : 0, nb_s1 = has_nb ? nonbatched_bias.strides()[1] : 0;
    const int64_t out_rs = out.dim() >= 3 ? out.strides()[1] : out.strides()[0];
    KUTACC_CHECK(out_rs >= C, "gating_attention: out row stride ", out_rs, " < nchannels ", C);
    if (kutacc_check_err_set) return;

    const size_t x_bytes = (size_t)M * C * es, w_bytes = (size_t)C * C * es, b_bytes = (size_t)C * sizeof(float);
    const size_t bias_bytes = (size_t)((B - 1) * bias_s0 + S) * es;
    const size_t nb_bytes = has_nb ? (size_t)((H - 1) * nb_s0 + (S - 1) * nb_s1 + S) * es : 0;
    const size_t out_bytes = (size_t)((M - 1) * out_rs + C) * es;

    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;

    // When the result lives in host memory, the batch rows (independent problems) are processed in chunks so
    // that the upload of chunk i+1 (when the activations are in host memory too), the kernels of chunk i and
    // the download of chunk i-1 overlap on three streams. Otherwise the call is a single chunk on the runtime
    // stream.
    const bool x_host = staged_bytes_needed(input.data_ptr(), x_bytes) != 0;
    const bool out_host = staged_bytes_needed(out.data_ptr(), out_bytes) != 0;
    const bool pipelined = out_host && B >= 8 && x_bytes >= ((size_t)4 << 20);

    size_t stage = staged_bytes_needed(input.data_ptr(), x_bytes) + staged_bytes_needed(bias.data_ptr(), bias_bytes) +
                   staged_bytes_needed(out.data_ptr(), out_bytes) + staged_bytes_needed(gating_b.data_ptr(), b_bytes) +
                   staged_bytes_needed(output_b.data_ptr(), b_bytes);
    if (has_nb) stage += staged_bytes_needed(nonbatched_bias.data_ptr(), nb_bytes);
    for (const Tensor *w : {&query_w, &key_w, &value_w, &gating_w, &output_w})
        stage += staged_bytes_needed(w->data_ptr(), w_bytes);
    if (ln) stage += 2 * staged_bytes_needed(ln->gamma, b_bytes);
    const bool downloads_in_flight = rt.out_hazard;          // of an earlier enqueue-only call with a HOST result
    if (!rt.reserve_stage(stage, pipelined)) return;
    const int64_t s_pad8 = (S + 7) / 8 * 8;
    const size_t nb_pad_bytes = has_nb ? (size_t)H * S * s_pad8 * 2 : 0;
    const size_t v_bytes = std::max(x_bytes, (size_t)B * C * s_pad8 * es);   // v may be stored key-major with padded rows
    // with LayerNorm: row statistics, four folded weights with their s and t, and (for shapes the folded projection does
    // not cover) a normalised copy of the activations
    const size_t ln_bytes = ln ? (size_t)M * 8 + 4 * (w_bytes + 256) + 8 * (b_bytes + 256) + x_bytes + 1024 : 0;
    // fp32 on the tensor-memory GEMM: operands split into tf32 head and tail (activations: one [M, 2C] buffer that the
    // projection and, later, the output projection use in turn; five weights [C, 2C])
    const bool f32_tc = dt == kFP32 && C % 128 == 0 && out_rs % 4 == 0;
    const size_t f32_bytes = f32_tc ? 2 * x_bytes + 256 + 5 * (2 * w_bytes + 256) : 0;
    if (!rt.reserve_workspace(4 * (x_bytes + 256) + v_bytes + 256 + nb_pad_bytes + 256 + ln_bytes + f32_bytes)) return;

    // The staged output is placed first: its address tells whether downloads of an earlier enqueue-only call, still
    // in flight, read the very block this call will fill. A call of the same shape (same block, same chunks) lets its
    // chunk i wait for the earlier download of chunk i only, so its first chunks run beside the tail of those
    // downloads; any other call waits for all of them before it writes anything into the staging area.
    DeviceArg d_out = resolve_out(out.data_ptr(), out_bytes);
    // about 8 MiB of activations per chunk on average, between 2 and 12 chunks of at least 4 rows
    int nchunks = (int)std::max<int64_t>(2, std::min<int64_t>(12, (int64_t)((x_bytes + ((size_t)4 << 20)) >> 23)));
    nchunks = (int)std::max<int64_t>(1, std::min<int64_t>(nchunks, B / 4));
    const bool same_chunks = pipelined && downloads_in_flight && rt.pend_dev == d_out.dev && rt.pend_bytes == out_bytes &&
                             rt.pend_nchunks == nchunks && rt.pend_rows == B;
    if (pipelined && downloads_in_flight && !same_chunks) {
        KUTACC_CUDA(cudaStreamWaitEvent(stream, (cudaEvent_t)rt.out_done, 0));
        rt.out_hazard = false;
    }

    DeviceArg d_x = pipelined ? resolve_out(input.data_ptr(), x_bytes) : resolve_in(input.data_ptr(), x_bytes);
    DeviceArg d_bias = resolve_in(bias.data_ptr(), bias_bytes);
    DeviceArg d_nb = has_nb ? resolve_in(nonbatched_bias.data_ptr(), nb_bytes) : DeviceArg{};
    DeviceArg d_wq = resolve_in(query_w.data_ptr(), w_bytes), d_wk = resolve_in(key_w.data_ptr(), w_bytes),
              d_wv = resolve_in(value_w.data_ptr(), w_bytes), d_wg = resolve_in(gating_w.data_ptr(), w_bytes),
              d_wo = resolve_in(output_w.data_ptr(), w_bytes);
    DeviceArg d_bg = resolve_in(gating_b.data_ptr(), b_bytes), d_bo = resolve_in(output_b.data_ptr(), b_bytes);
    if (pipelined) {
        // The copy streams start once the previous work on the runtime stream AND the small uploads queued above are
        // done. (Letting the first chunk travel beside the small uploads was tried: the copy engine then served
        // some of the small uploads only after every chunk, and the first kernel waited for all of them.)
        CopyPipeline &cp0 = copy_pipeline(1);
        if (kutacc_check_err_set) return;
        KUTACC_CUDA(cudaEventRecord((cudaEvent_t)cp0.start, stream));
        KUTACC_CUDA(cudaStreamWaitEvent((cudaStream_t)cp0.in, (cudaEvent_t)cp0.start, 0));
        KUTACC_CUDA(cudaStreamWaitEvent((cudaStream_t)cp0.out, (cudaEvent_t)cp0.start, 0));
    }
    char *wq_ = (char *)rt.take_workspace(x_bytes), *wk_ = (char *)rt.take_workspace(x_bytes),
         *wv_ = (char *)rt.take_workspace(v_bytes), *wg_ = (char *)rt.take_workspace(x_bytes),
         *wavg = (char *)rt.take_workspace(x_bytes);
    void *nb_pad = nb_pad_bytes ? rt.take_workspace(nb_pad_bytes) : nullptr;
    DeviceArg d_lg = ln ? resolve_in(ln->gamma, b_bytes) : DeviceArg{}, d_lb = ln ? resolve_in(ln->beta, b_bytes) : DeviceArg{};
    char *ln_stats = ln ? (char *)rt.take_workspace((size_t)M * 8) : nullptr;
    void *ln_w[4] = {nullptr, nullptr, nullptr, nullptr};
    float *ln_s[4] = {nullptr, nullptr, nullptr, nullptr}, *ln_t[4] = {nullptr, nullptr, nullptr, nullptr};
    char *x_norm = nullptr;
    if (ln) {
        for (int i = 0; i < 4; ++i) {
            ln_w[i] = rt.take_workspace(w_bytes);
            ln_s[i] = (float *)rt.take_workspace(b_bytes);
            ln_t[i] = (float *)rt.take_workspace(b_bytes);
        }
        x_norm = (char *)rt.take_workspace(x_bytes);
    }
    char *a_split = f32_tc ? (char *)rt.take_workspace(2 * x_bytes) : nullptr;
    void *w_split[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    for (int i = 0; i < 5 && f32_tc; ++i) w_split[i] = rt.take_workspace(2 * w_bytes);
    if (kutacc_check_err_set) return;

    const float scale = (float)(1 / std::sqrt((double)head_size));  // gating_attention.cpp:68

    const bool fast = dt == kBF16 && (C % 64 == 0) && (D == 16 || D == 32 || D == 64) && B <= 65535 && H <= 65535 &&
                      aligned16(d_x.dev) && aligned16(d_wq.dev) && aligned16(d_wk.dev) && aligned16(d_wv.dev) &&
                      aligned16(d_wg.dev) && aligned16(d_wo.dev) && (out_rs % 2 == 0) &&
                      (((uintptr_t)d_out.dev & 3u) == 0);

    // The pair bias may still be on its way (kutacc_b200_set_pair_bias_event): everything that reads it waits for the
    // event, once. The projections do not read it, so they are queued first where the pair bias is used as it lies.
    void *nb_event = rt.pair_bias_event;
    rt.pair_bias_event = nullptr;
    auto wait_for_pair_bias = [&]() {
        if (nb_event) KUTACC_CUDA(cudaStreamWaitEvent(stream, (cudaEvent_t)nb_event, 0));
        nb_event = nullptr;
    };
    if (!has_nb || staged_bytes_needed(nonbatched_bias.data_ptr(), nb_bytes) != 0) nb_event = nullptr;   // nothing to wait for / host data

    // The TMA loads of the pair bias need 16-byte aligned rows. A pair bias whose strides are not
    // multiples of 8 elements is first copied into the workspace with padded rows.
    const void *nb_dev = has_nb ? d_nb.dev : nullptr;
    int64_t nb_sh = nb_s0, nb_sq = nb_s1;
    if (fast && has_nb && ((nb_s0 % 8) || (nb_s1 % 8) || !aligned16(d_nb.dev))) {
        wait_for_pair_bias();                         // the re-pitching copy reads it
        KUTACC_CUDA(cudaMemcpy2DAsync(nb_pad, (size_t)s_pad8 * 2, d_nb.dev, (size_t)nb_s1 * 2, (size_t)S * 2,
                                      (size_t)(nb_s0 == S * nb_s1 ? H * S : S), cudaMemcpyDeviceToDevice, stream));
        for (int64_t hh = 1; nb_s0 != S * nb_s1 && hh < H; ++hh)
            KUTACC_CUDA(cudaMemcpy2DAsync((char *)nb_pad + (size_t)hh * S * s_pad8 * 2, (size_t)s_pad8 * 2,
                                          (const char *)d_nb.dev + (size_t)hh * nb_s0 * 2, (size_t)nb_s1 * 2,
                                          (size_t)S * 2, (size_t)S, cudaMemcpyDeviceToDevice, stream));
        nb_dev = nb_pad;
        nb_sq = s_pad8;
        nb_sh = S * s_pad8;
    }

    // LayerNorm in front: folded into the tcgen05 projection where that kernel runs (head size 32), otherwise the
    // rows are normalised into the workspace chunk by chunk and the usual sequence runs on the copy
    const bool ln_folded = ln && fast && D == 32 && C % 128 == 0;
    if (ln_folded) {
        const void *w_in[4] = {d_wq.dev, d_wk.dev, d_wv.dev, d_wg.dev};
        const float *b_in[4] = {nullptr, nullptr, nullptr, (const float *)d_bg.dev};
        const bool folded = dev::launch_ln_fold(stream, 4, w_in, b_in, (const float *)d_lg.dev, (const float *)d_lb.dev, ln_w,
                                                ln_s, ln_t, (int)C, (int)C);
        KUTACC_CHECK(folded, "gating_attention with LayerNorm: weight folding failed");
        if (kutacc_check_err_set) return;
    }

    bool f32_tc_ok = f32_tc && aligned16(d_x.dev) && aligned16(d_out.dev);
    if (f32_tc_ok) {
        const void *w_in[5] = {d_wq.dev, d_wk.dev, d_wv.dev, d_wg.dev, d_wo.dev};
        f32_tc_ok = dev::launch_split_tf32_many(stream, 5, w_in, C, w_split, C, (int)C);
    }

    // kernel sequence for batch rows [b0, b0 + nb): every buffer is batch-major, so a chunk is an offset
    auto run_rows = [&](int64_t b0, int64_t nbr) -> bool {
        const size_t row_bytes = (size_t)S * C * es;                       // one batch row of a [B, S, C]-sized buffer
        const char *x_c = (const char *)d_x.dev + b0 * row_bytes;
        char *st_c = ln ? ln_stats + (size_t)b0 * S * 8 : nullptr;
        if (ln && !ln_folded) {
            if (!dev::launch_layernorm_rows(stream, x_c, (const float *)d_lg.dev, (const float *)d_lb.dev, x_norm + b0 * row_bytes,
                                            nbr * S, C, C, C, ln->eps))
                return false;
            x_c = x_norm + b0 * row_bytes;
        }
        char *q_c = wq_ + b0 * row_bytes, *k_c = wk_ + b0 * row_bytes, *g_c = wg_ + b0 * row_bytes,
             *a_c = wavg + b0 * row_bytes;
        const char *bias_c = (const char *)d_bias.dev + (size_t)b0 * bias_s0 * es;
        char *out_c = (char *)d_out.dev + (size_t)b0 * S * out_rs * es;
        const int64_t Mc = nbr * S;
        bool ok;
        if (fast) {
            // Tensor-memory kernels where the shape allows it (head size 32: projection with v stored
            // key-major plus the tcgen05 attention core), warp-level MMA kernels otherwise.
            char *v_km = wv_ + (size_t)b0 * C * s_pad8 * es;                   // key-major v: [B, H, D, s_pad8]
            char *v_c = wv_ + b0 * row_bytes;                                  // [B, H, S, D]
            bool v_key_major = false;
            ok = false;
            if (ln_folded) {
                ok = dev::launch_ln_stats(stream, x_c, nbr * S, C, C, ln->eps, st_c) &&
                     dev::tcgen05_proj_qkvg_bf16(stream, x_c, ln_w[0], ln_w[1], ln_w[2], ln_w[3], nullptr, q_c, k_c, v_km, g_c,
                                                 (int)nbr, (int)S, (int)H, (int)D, true, s_pad8, /*gate_sigmoid=*/true, st_c,
                                                 ln_s, ln_t);
                if (!ok) return false;
                v_key_major = true;
            } else if (D == 32) {
                ok = dev::tcgen05_proj_qkvg_bf16(stream, x_c, d_wq.dev, d_wk.dev, d_wv.dev, d_wg.dev,
                                                 (const float *)d_bg.dev, q_c, k_c, v_km, g_c, (int)nbr, (int)S, (int)H,
                                                 (int)D, true, s_pad8, /*gate_sigmoid=*/true);
                v_key_major = ok;
            }
            if (!ok)
                ok = dev::tcgen05_proj_qkvg_bf16(stream, x_c, d_wq.dev, d_wk.dev, d_wv.dev, d_wg.dev,
                                                 (const float *)d_bg.dev, q_c, k_c, v_c, g_c, (int)nbr, (int)S, (int)H,
                                                 (int)D, false, 0) ||
                     dev::launch_proj_qkvg_bf16(stream, x_c, d_wq.dev, d_wk.dev, d_wv.dev, d_wg.dev,
                                                (const float *)d_bg.dev, q_c, k_c, v_c, g_c, (int)nbr, (int)S, (int)H,
                                                (int)D, 1.0f);
            wait_for_pair_bias();
            if (ok && v_key_major)
                ok = dev::tcgen05_attn_core_bf16(stream, q_c, k_c, v_km, s_pad8, g_c, bias_c, bias_s0, nb_dev, nb_sh,
                                                 nb_sq, a_c, (int)nbr, (int)S, (int)H, (int)D, scale, /*gate_is_sigmoid=*/true);
            else
                ok = ok && dev::launch_attn_core_bf16(stream, q_c, k_c, v_c, g_c, bias_c, bias_s0, nb_dev, nb_sh, nb_sq,
                                                      a_c, (int)nbr, (int)S, (int)H, (int)D, scale);
            ok = ok && (dev::tcgen05_linear_bias_bf16(stream, a_c, d_wo.dev, (const float *)d_bo.dev, out_c, out_rs,
                                                      (int)nbr, (int)S, (int)C, (int)C) ||
                        dev::launch_linear_bias_bf16(stream, a_c, C, d_wo.dev, (const float *)d_bo.dev, out_c, out_rs,
                                                     Mc, (int)C, (int)C));
        } else {
            const dev::ElemType et = dt == kFP32 ? dev::kElemF32 : dev::kElemBF16;
            char *v_c = wv_ + b0 * row_bytes;
            char *as_c = f32_tc_ok ? a_split + 2 * b0 * row_bytes : nullptr;
            bool projected = false;
            if (f32_tc_ok) {
                // fp32: all four projections in one pass of the tensor-memory GEMM over the split activations
                const float *pb[4] = {nullptr, nullptr, nullptr, (const float *)d_bg.dev};
                void *po[4] = {q_c, k_c, v_c, g_c};
                projected = dev::launch_split_tf32(stream, x_c, C, as_c, Mc, (int)C) &&
                            dev::tcgen05_gemm_tf32x3(stream, as_c, w_split, pb, po, C, Mc, (int)C, (int)C, 4);
            }
            ok = projected || dev::launch_gemm_generic(stream, et, x_c, C, d_wq.dev, C, nullptr, 0.f, q_c, C, Mc, C, C);
            ok = ok && (projected || dev::launch_gemm_generic(stream, et, x_c, C, d_wk.dev, C, nullptr, 0.f, k_c, C, Mc, C, C));
            ok = ok && (projected || dev::launch_gemm_generic(stream, et, x_c, C, d_wv.dev, C, nullptr, 0.f, v_c, C, Mc, C, C));
            ok = ok && (projected || dev::launch_gemm_generic(stream, et, x_c, C, d_wg.dev, C, (const float *)d_bg.dev, 0.f,
                                                              g_c, C, Mc, C, C));
            wait_for_pair_bias();
            // fp32 with the tensor-memory GEMM after it: the attention core writes its result already split into
            // tf32 head and tail, in the rows of the output projection's operand
            bool avg_is_split = false;
            if (ok && dt == kFP32 && f32_tc_ok)
                avg_is_split = dev::launch_attn_f32(stream, q_c, k_c, v_c, g_c, bias_c, bias_s0, has_nb ? d_nb.dev : nullptr,
                                                    nb_s0, nb_s1, a_c, (int)nbr, (int)S, (int)H, (int)D, scale, as_c);
            ok = ok && (avg_is_split ||
                        (dt == kFP32 && dev::launch_attn_f32(stream, q_c, k_c, v_c, g_c, bias_c, bias_s0,
                                                              has_nb ? d_nb.dev : nullptr, nb_s0, nb_s1, a_c, (int)nbr,
                                                              (int)S, (int)H, (int)D, scale)) ||
                        dev::launch_attn_generic(stream, et, q_c, k_c, v_c, g_c, bias_c, bias_s0,
                                                 has_nb ? d_nb.dev : nullptr, nb_s0, nb_s1, a_c, (int)nbr, (int)S, (int)H,
                                                 (int)D, scale));
            bool out_done = false;
            if (ok && f32_tc_ok) {
                const float *pb[1] = {(const float *)d_bo.dev};
                void *po[1] = {out_c};
                out_done = (avg_is_split || dev::launch_split_tf32(stream, a_c, C, as_c, Mc, (int)C)) &&
                           dev::tcgen05_gemm_tf32x3(stream, as_c, &w_split[4], pb, po, out_rs, Mc, (int)C, (int)C, 1);
            }
            // (when the average exists only in split form, the tensor-memory GEMM is the only kernel that can read it)
            ok = ok && (out_done || (!avg_is_split && dev::launch_gemm_generic(stream, et, a_c, C, d_wo.dev, C,
                                                                               (const float *)d_bo.dev, 0.f, out_c, out_rs,
                                                                               Mc, C, C)));
        }
        return ok;
    };

    bool ok = true;
    if (!pipelined) {
        ok = run_rows(0, B);
        if (d_out.staged)
            copy_rows_d2h((char *)d_out.host, (const char *)d_out.dev, (size_t)M, (size_t)C * es, (size_t)out_rs * es, stream);
    } else {
        // Chunk i gets a share of the rows proportional to nchunks + 2 - i: the chunks shrink towards the end,
        // because the kernels and the download of the last chunk are the part of the call nothing overlaps.
        int64_t chunk_begin[17];
        {
            const int64_t wsum = (int64_t)nchunks * (nchunks + 5) / 2;      // sum of (nchunks + 2 - i), i = 0..nchunks-1
            int64_t acc = 0;
            for (int i = 0; i < nchunks; ++i) {
                chunk_begin[i] = std::min<int64_t>(B, (acc * B + wsum / 2) / wsum);
                acc += nchunks + 2 - i;
            }
            chunk_begin[nchunks] = B;
        }
        CopyPipeline &cp = copy_pipeline(nchunks);
        if (kutacc_check_err_set) return;
        cudaStream_t s_in = (cudaStream_t)cp.in, s_out = (cudaStream_t)cp.out;
        const size_t row_bytes = (size_t)S * C * es;
        // every upload is queued before the first kernel: the copy-in stream then never waits for the host, which
        // needs a while per chunk to encode tensor maps and launch
        for (int i = 0; i < nchunks && x_host; ++i) {
            const int64_t b0 = chunk_begin[i], nbr = chunk_begin[i + 1] - b0;
            if (nbr <= 0) continue;
            KUTACC_CUDA(cudaMemcpyAsync((char *)d_x.dev + b0 * row_bytes, (const char *)input.data_ptr() + b0 * row_bytes,
                                        (size_t)nbr * row_bytes, cudaMemcpyHostToDevice, s_in));
            KUTACC_CUDA(cudaEventRecord((cudaEvent_t)cp.uploaded[i], s_in));
        }
        for (int i = 0; i < nchunks && ok; ++i) {
            const int64_t b0 = chunk_begin[i], nbr = chunk_begin[i + 1] - b0;
            if (nbr <= 0) continue;
            if (same_chunks) KUTACC_CUDA(cudaStreamWaitEvent(stream, (cudaEvent_t)cp.downloaded[i], 0));
            if (x_host) KUTACC_CUDA(cudaStreamWaitEvent(stream, (cudaEvent_t)cp.uploaded[i], 0));
            ok = run_rows(b0, nbr);
            KUTACC_CUDA(cudaEventRecord((cudaEvent_t)cp.computed[i], stream));
            KUTACC_CUDA(cudaStreamWaitEvent(s_out, (cudaEvent_t)cp.computed[i], 0));
            // only the C elements of each row travel back: a host `out` whose row stride leaves gaps keeps
            // the bytes between its rows (the reference writes through strides()[1] and touches nothing else)
            const size_t o_off = (size_t)b0 * S * out_rs * es;
            copy_rows_d2h((char *)out.data_ptr() + o_off, (const char *)d_out.dev + o_off, (size_t)nbr * S, (size_t)C * es,
                          (size_t)out_rs * es, s_out);
            KUTACC_CUDA(cudaEventRecord((cudaEvent_t)cp.downloaded[i], s_out));
        }
        if (rt.async) {
            // enqueue-only: the call returns with its downloads in flight; kutacc_b200_synchronize waits for them
            if (rt.out_done == nullptr) {
                cudaEvent_t e = nullptr;
                KUTACC_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
                rt.out_done = e;
            }
            if (rt.out_done) {
                KUTACC_CUDA(cudaEventRecord((cudaEvent_t)rt.out_done, s_out));
                rt.out_unsynced = rt.out_hazard = true;
                rt.pend_dev = d_out.dev;
                rt.pend_bytes = out_bytes;
                rt.pend_nchunks = nchunks;
                rt.pend_rows = B;
            } else {
                KUTACC_CUDA(cudaStreamSynchronize(s_out));
            }
        } else {
            KUTACC_CUDA(cudaStreamSynchronize(s_out));
            rt.out_unsynced = rt.out_hazard = false;
        }
    }
    KUTACC_CHECK(ok, "gating_attention: no device kernel for this shape (B=", B, " S=", S, " H=", H, " D=", D, ")");
    end_of_call();
}

}  // namespace kutacc

// The argument checks of the two entry points, expanded inside each of them so that a failed check names the
// entry point the caller used (the reference prints __func__: src/utils/check.h:38-45).
#define KUTACC_GATING_ENTRY(ln_ptr) \
 /* handle / struct nulls first (gating_attention.cpp:165-170) ... */ \
    KUTACC_CHECK(input != nullptr && q_based_ptr != nullptr && bias != nullptr && nonbatched_bias != nullptr && \
                     weight_ptr != nullptr && out != nullptr, \
                 "kutacc_af2_gating_attention: input args nullptr error"); \
    if (kutacc_check_err_set) return; \
 /* ... then the scalars, before any handle is dereferenced: the reference's robustness tests */ \
 /* pass pointers to stack floats as handles together with one bad integer. */ \
    const int64_t batch = q_based_ptr->batch, seq_len = q_based_ptr->seq_len; \
    const int64_t head_size = weight_ptr->head_size, nheads = weight_ptr->nheads, nchannels = weight_ptr->nchannels; \
    KUTACC_CHECK(batch > 0 && seq_len > 0 && block_size > 0 && head_size > 0 && nheads > 0 && nchannels > 0, \
                 "input param <= 0 or overflow"); \
    KUTACC_CHECK(weight_ptr->query_w && weight_ptr->key_w && weight_ptr->value_w && weight_ptr->gating_w && \
                     weight_ptr->gating_b && weight_ptr->output_w && weight_ptr->output_b, \
                 "kutacc_af2_gating_attention: weight handle nullptr error"); \
    if (kutacc_check_err_set) return; \
    gating_attention_impl(*as_tensor(input), batch, seq_len, *as_tensor(bias), *as_tensor(nonbatched_bias), \
                          *as_tensor(weight_ptr->query_w), *as_tensor(weight_ptr->key_w), \
                          *as_tensor(weight_ptr->value_w), *as_tensor(weight_ptr->gating_w), \
                          *as_tensor(weight_ptr->gating_b), *as_tensor(weight_ptr->output_w), \
                          *as_tensor(weight_ptr->output_b), *as_tensor(out), block_size, head_size, nheads, nchannels, ln_ptr);

extern "C" void kutacc_af2_gating_attention(kutacc_tensor_h input, kutacc_af2_attention_inputs_t *q_based_ptr,
                                            kutacc_tensor_h bias, kutacc_tensor_h nonbatched_bias,
                                            kutacc_af2_attention_weights_t *weight_ptr, kutacc_tensor_h out,
                                            int64_t block_size)
{
    using namespace kutacc;
    KUTACC_GATING_ENTRY(nullptr)
}

// kutacc_af2_gating_attention applied to LayerNorm(input): same arguments plus the LayerNorm's fp32 gamma and beta
// (nchannels elements each, host or device) and eps. For head size 32 the normalisation is folded into the
// projection kernel: the normalised activations are never written to memory.
extern "C" void kutacc_b200_gating_attention_ln(kutacc_tensor_h input, kutacc_af2_attention_inputs_t *q_based_ptr,
                                                kutacc_tensor_h bias, kutacc_tensor_h nonbatched_bias,
                                                kutacc_af2_attention_weights_t *weight_ptr, const float *ln_gamma,
                                                const float *ln_beta, float eps, kutacc_tensor_h out, int64_t block_size)
{
    using namespace kutacc;
    KUTACC_CHECK(ln_gamma != nullptr && ln_beta != nullptr && eps >= 0.f, "kutacc_b200_gating_attention_ln: LayerNorm arguments invalid");
    if (kutacc_check_err_set) return;
    const LayerNormArgs ln{ln_gamma, ln_beta, eps};
    KUTACC_GATING_ENTRY(&ln)
}
