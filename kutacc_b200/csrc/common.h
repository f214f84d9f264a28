// Host-side plumbing shared by the operator entry points: tensor descriptor, error convention,
// device runtime (stream, workspace pool, host-pointer staging).
#pragma once
#include <cstddef>
#include <cstdint>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/kutacc_b200.h"

namespace kutacc {

// ---- tensor descriptor (reference: src/tensor/tensor.h:21-51) ---------------------------------
// Field order {dim, data_ptr, sizes, strides, dtype} is kept so that a handle made by a caller
// compiled against the reference's TensorWrapper has the same object layout.
struct Tensor {
    int64_t dim_;
    void *data_;
    std::vector<int64_t> sizes_;
    std::vector<int64_t> strides_;
    DType dtype_;

    Tensor(void *data, std::vector<int64_t> &&sizes, std::vector<int64_t> &&strides, int64_t dim, DType dtype);
    void *data_ptr() const { return data_; }
    const std::vector<int64_t> &sizes() const { return sizes_; }
    const std::vector<int64_t> &strides() const { return strides_; }
    DType dtype() const { return dtype_; }
    int64_t dim() const { return dim_; }
    int64_t numel() const;  // 0 for dim 0 (reference: src/tensor/tensor.cpp:67-77)
};
inline Tensor *as_tensor(kutacc_tensor_h h) { return static_cast<Tensor *>(h); }
inline size_t dtype_size(DType t) { return t == kBF16 ? 2 : (t == kFP32 ? 4 : 8); }

// ---- error convention (reference: src/utils/check.h:38-56, src/utils/check.cpp:16) ------------
extern bool kutacc_check_err_set;
void check_fail(const char *func, const char *file, int line, const std::string &msg);

namespace detail {
inline void cat(std::ostringstream &) {}
template <typename A, typename... R>
inline void cat(std::ostringstream &os, A &&a, R &&...r)
{
    os << a;
    cat(os, r...);
}
}  // namespace detail
}  // namespace kutacc

#define KUTACC_CHECK(cond, ...)                                              \
    do {                                                                     \
        if (__builtin_expect(!(cond), 0)) {                                  \
            std::ostringstream os__;                                         \
            ::kutacc::detail::cat(os__, __VA_ARGS__);                        \
            ::kutacc::check_fail(__func__, __FILE_NAME__, __LINE__, os__.str()); \
        }                                                                    \
    } while (0)

// A CUDA runtime status other than success is reported through the same sticky flag.
#define KUTACC_CUDA(call)                                                                      \
    do {                                                                                       \
        cudaError_t e__ = (call);                                                              \
        KUTACC_CHECK(e__ == cudaSuccess, "CUDA error: ", cudaGetErrorString(e__), " (", #call, ")"); \
    } while (0)

namespace kutacc {

// ---- device runtime ------------------------------------------------------------------------------
// One per process. Holds the stream operators launch on, a grow-only device workspace carved by a
// bump pointer per call, and a second grow-only pool that stages host-resident tensors.
struct Runtime {
    void *stream = nullptr;   // cudaStream_t
    bool async = false;
    int sm_margin = 0;        // SMs the persistent kernels leave free (for a collective running beside them)
    void *pair_bias_event = nullptr;   // cudaEvent_t the next gated-attention call waits for before its attention kernel

    char *ws_base = nullptr;
    size_t ws_cap = 0, ws_off = 0;
    char *stage_base = nullptr;
    size_t stage_cap = 0, stage_off = 0;

    // An enqueue-only call (async) whose result goes to HOST memory in chunks returns while its downloads are still
    // running on the copy-out stream. `out_done` (cudaEvent_t) follows the last of them. out_unsynced: the host has
    // not waited for it yet (kutacc_b200_synchronize does); out_hazard: later work on the runtime stream has not been
    // ordered after it yet, so the staging block the downloads read must not be rewritten. pend_*: which staged
    // output and which chunking the downloads belong to, for a following call of the same shape that orders itself
    // chunk by chunk instead.
    void *out_done = nullptr;
    bool out_unsynced = false, out_hazard = false;
    const void *pend_dev = nullptr;
    size_t pend_bytes = 0;
    int pend_nchunks = 0;
    int64_t pend_rows = 0;

    // reserve() must be called once per operator call with the total need, before any take()
    bool reserve_workspace(size_t bytes);
    void *take_workspace(size_t bytes);   // 256-byte aligned slices of the reserved block
    // caller_orders_downloads: the caller itself orders its writes after downloads still in flight (see out_hazard)
    bool reserve_stage(size_t bytes, bool caller_orders_downloads = false);
    void *take_stage(size_t bytes);
    void release();
};
Runtime &runtime();
bool is_device_pointer(const void *p);
void count_launch(int n = 1);

// Optional per-kernel timing (kutacc_b200_set_profile): a launcher wraps each launch in a
// KernelTimer, which brackets it with CUDA events on the stream of the launch.
struct KernelTimer {
    // `cuda_stream` is the stream the kernel is launched on
    KernelTimer(const char *name, void *cuda_stream);
    ~KernelTimer();
    int slot;
    void *stream;
};

// A tensor argument resolved to device memory: either the caller's own device pointer or a staged
// copy of a host buffer (copied in on demand, copied back by finish()).
struct DeviceArg {
    void *dev = nullptr;
    void *host = nullptr;
    size_t bytes = 0;
    bool staged = false;
};
size_t staged_bytes_needed(const void *p, size_t bytes);               // 0 when p is a device pointer
DeviceArg resolve_in(const void *p, size_t bytes);                     // copies host -> device when staged
DeviceArg resolve_out(void *p, size_t bytes);                          // no copy in
void finish_out(const DeviceArg &a);                                    // device -> host when staged
// Device -> host copy of `rows` rows of `width` bytes that are `pitch` bytes apart in both buffers. Only the
// `width` bytes of a row are written, so a host tensor whose row stride leaves gaps keeps what lies between
// its rows (the reference writes through the row stride and touches nothing else).
void copy_rows_d2h(void *host, const void *dev, size_t rows, size_t width, size_t pitch, void *cuda_stream);
void end_of_call();                                                    // stream sync unless async
void sync_and_check();                                                 // stream sync + device-side timeout report

// Two extra non-blocking streams and a pool of events for calls that overlap host<->device copies with
// compute on the runtime stream (created on first use, reused afterwards).
struct CopyPipeline {
    void *in = nullptr, *out = nullptr;       // cudaStream_t
    void *start = nullptr;                    // cudaEvent_t
    std::vector<void *> uploaded, computed, downloaded;   // cudaEvent_t per chunk
};
CopyPipeline &copy_pipeline(int nchunks);

}  // namespace kutacc
