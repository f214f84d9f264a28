// kutacc_af2_layernorm (one row, the reference's signature) and kutacc_b200_layernorm_rows (every row of a
// matrix in one launch). Replaces src/normalization/layernorm.cpp:17-20 and the caller's loop over rows.
#include <cuda_runtime.h>

#include "common.h"
#include "kernels.h"

namespace kutacc {
namespace {

void layernorm_impl(const char *who, const void *data, const float *gamma, const float *beta, int64_t rows, int64_t size,
                    int64_t row_stride, int64_t out_row_stride, float eps, void *out)
{
    KUTACC_CHECK(data != nullptr && gamma != nullptr && beta != nullptr && out != nullptr, who, ": nullptr error");
    if (kutacc_check_err_set) return;
    KUTACC_CHECK(rows > 0 && size > 0 && row_stride >= size && out_row_stride >= size, who,
                 ": input param <= 0 or row stride shorter than a row");
    if (kutacc_check_err_set) return;
    const size_t x_bytes = (size_t)((rows - 1) * row_stride + size) * 2, o_bytes = (size_t)((rows - 1) * out_row_stride + size) * 2;
    const size_t p_bytes = (size_t)size * 4;
    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    const size_t stage = staged_bytes_needed(data, x_bytes) + staged_bytes_needed(out, o_bytes) +
                         staged_bytes_needed(gamma, p_bytes) + staged_bytes_needed(beta, p_bytes);
    if (!rt.reserve_stage(stage)) return;
    DeviceArg d_x = resolve_in(data, x_bytes), d_g = resolve_in(gamma, p_bytes), d_b = resolve_in(beta, p_bytes);
    // a strided host output keeps the bytes between its rows: bring them in before they are copied back
    DeviceArg d_o = out_row_stride == size ? resolve_out(out, o_bytes) : resolve_in(out, o_bytes);
    if (kutacc_check_err_set) return;
    const bool ok = dev::launch_layernorm_rows(stream, d_x.dev, (const float *)d_g.dev, (const float *)d_b.dev, d_o.dev, rows,
                                               size, row_stride, out_row_stride, eps);
    KUTACC_CHECK(ok, who, ": no device kernel for rows=", rows, " size=", size);
    finish_out(d_o);
    end_of_call();
}

}  // namespace
}  // namespace kutacc

extern "C" void kutacc_af2_layernorm(uint16_t *data, float *gamma, float *beta, int64_t size, float eps, uint16_t *out)
{
    kutacc::layernorm_impl("kutacc_af2_layernorm", data, gamma, beta, 1, size, size, size, eps, out);
}

extern "C" void kutacc_b200_layernorm_rows(const void *data, const float *gamma, const float *beta, int64_t rows,
                                           int64_t size, int64_t row_stride, int64_t out_row_stride, float eps, void *out)
{
    kutacc::layernorm_impl("kutacc_b200_layernorm_rows", data, gamma, beta, rows, size, row_stride, out_row_stride, eps,
                           out);
}
