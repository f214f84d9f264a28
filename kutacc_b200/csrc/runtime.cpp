// Device runtime: stream, grow-only workspace, staging of host-resident tensors.
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <vector>

#include "common.h"
#include "tma_utils.cuh"

namespace kutacc {

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

namespace {
struct ProfRecord {
    const char *name;
    cudaEvent_t start, stop;
};
bool g_profile = false;
std::vector<ProfRecord> g_prof;
}  // namespace

KernelTimer::KernelTimer(const char *name, void *cuda_stream) : slot(-1), stream(cuda_stream)
{
    if (!g_profile) return;
    ProfRecord r;
    r.name = name;
    if (cudaEventCreate(&r.start) != cudaSuccess || cudaEventCreate(&r.stop) != cudaSuccess) return;
    cudaEventRecord(r.start, (cudaStream_t)stream);
    g_prof.push_back(r);
    slot = (int)g_prof.size() - 1;
}
KernelTimer::~KernelTimer()
{
    if (slot >= 0) cudaEventRecord(g_prof[(size_t)slot].stop, (cudaStream_t)stream);
}

Runtime &runtime()
{
    static Runtime rt;
    return rt;
}

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static bool grow(char *&base, size_t &cap, size_t need)
{
    if (need <= cap) return true;
    // Blocks are handed to kernels enqueued on the stream (and to downloads on the copy-out stream); let them
    // drain before the old block goes.
    KUTACC_CUDA(cudaStreamSynchronize((cudaStream_t)runtime().stream));
    if (runtime().out_unsynced && runtime().out_done) {
        KUTACC_CUDA(cudaEventSynchronize((cudaEvent_t)runtime().out_done));
        runtime().out_unsynced = runtime().out_hazard = false;
    }
    if (base) KUTACC_CUDA(cudaFree(base));
    base = nullptr;
    cap = 0;
    const size_t want = round_up(need + need / 8, (size_t)2 << 20);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    KUTACC_CHECK(e == cudaSuccess, "device allocation of ", want, " bytes failed: ", cudaGetErrorString(e));
    if (e != cudaSuccess) return false;
    base = (char *)p;
    cap = want;
    return true;
}

bool Runtime::reserve_workspace(size_t bytes)
{
    ws_off = 0;
    return grow(ws_base, ws_cap, bytes);
}
void *Runtime::take_workspace(size_t bytes)
{
    const size_t off = ws_off;
    ws_off = round_up(ws_off + bytes, 256);
    KUTACC_CHECK(ws_off <= ws_cap, "workspace slice beyond reservation: ", ws_off, " > ", ws_cap);
    return ws_off <= ws_cap ? ws_base + off : nullptr;
}
bool Runtime::reserve_stage(size_t bytes, bool caller_orders_downloads)
{
    stage_off = 0;
    if (bytes == 0) return true;
    if (out_hazard && !caller_orders_downloads) {
        // downloads of an earlier enqueue-only call still read the staging block this call is about to fill
        KUTACC_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)out_done, 0));
        out_hazard = false;
    }
    return grow(stage_base, stage_cap, bytes);
}
void *Runtime::take_stage(size_t bytes)
{
    const size_t off = stage_off;
    stage_off = round_up(stage_off + bytes, 256);
    KUTACC_CHECK(stage_off <= stage_cap, "staging slice beyond reservation: ", stage_off, " > ", stage_cap);
    return stage_off <= stage_cap ? stage_base + off : nullptr;
}
void Runtime::release()
{
    cudaStreamSynchronize((cudaStream_t)stream);
    if (ws_base) cudaFree(ws_base);
    if (stage_base) cudaFree(stage_base);
    ws_base = stage_base = nullptr;
    ws_cap = ws_off = stage_cap = stage_off = 0;
}

bool is_device_pointer(const void *p)
{
    if (p == nullptr) return false;
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, p);
    if (e != cudaSuccess) {
        cudaGetLastError();  // unregistered host memory on old drivers reports an error: not sticky
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

size_t staged_bytes_needed(const void *p, size_t bytes)
{
    if (p == nullptr || bytes == 0 || is_device_pointer(p)) return 0;
    return round_up(bytes, 256);
}

DeviceArg resolve_in(const void *p, size_t bytes)
{
    DeviceArg a;
    a.bytes = bytes;
    if (p == nullptr || bytes == 0) return a;
    if (is_device_pointer(p)) {
        a.dev = const_cast<void *>(p);
        return a;
    }
    a.staged = true;
    a.host = const_cast<void *>(p);
    a.dev = runtime().take_stage(bytes);
    if (a.dev) KUTACC_CUDA(cudaMemcpyAsync(a.dev, p, bytes, cudaMemcpyHostToDevice, (cudaStream_t)runtime().stream));
    return a;
}

DeviceArg resolve_out(void *p, size_t bytes)
{
    DeviceArg a;
    a.bytes = bytes;
    if (p == nullptr || bytes == 0) return a;
    if (is_device_pointer(p)) {
        a.dev = p;
        return a;
    }
    a.staged = true;
    a.host = p;
    a.dev = runtime().take_stage(bytes);
    return a;
}

void finish_out(const DeviceArg &a)
{
    if (a.staged && a.dev && a.host)
        KUTACC_CUDA(cudaMemcpyAsync(a.host, a.dev, a.bytes, cudaMemcpyDeviceToHost, (cudaStream_t)runtime().stream));
}

void copy_rows_d2h(void *host, const void *dev, size_t rows, size_t width, size_t pitch, void *cuda_stream)
{
    if (rows == 0 || width == 0) return;
    if (width == pitch) {
        KUTACC_CUDA(cudaMemcpyAsync(host, dev, rows * width, cudaMemcpyDeviceToHost, (cudaStream_t)cuda_stream));
        return;
    }
    KUTACC_CUDA(cudaMemcpy2DAsync(host, pitch, dev, pitch, width, rows, cudaMemcpyDeviceToHost, (cudaStream_t)cuda_stream));
}

CopyPipeline &copy_pipeline(int nchunks)
{
    static CopyPipeline cp;
    if (cp.in == nullptr) {
        cudaStream_t a = nullptr, b = nullptr;
        KUTACC_CUDA(cudaStreamCreateWithFlags(&a, cudaStreamNonBlocking));
        KUTACC_CUDA(cudaStreamCreateWithFlags(&b, cudaStreamNonBlocking));
        cudaEvent_t e = nullptr;
        KUTACC_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        cp.in = a;
        cp.out = b;
        cp.start = e;
    }
    while ((int)cp.uploaded.size() < nchunks) {
        cudaEvent_t e1 = nullptr, e2 = nullptr, e3 = nullptr;
        KUTACC_CUDA(cudaEventCreateWithFlags(&e1, cudaEventDisableTiming));
        KUTACC_CUDA(cudaEventCreateWithFlags(&e2, cudaEventDisableTiming));
        KUTACC_CUDA(cudaEventCreateWithFlags(&e3, cudaEventDisableTiming));
        cp.uploaded.push_back(e1);
        cp.computed.push_back(e2);
        cp.downloaded.push_back(e3);
    }
    return cp;
}

void end_of_call()
{
    cudaError_t e = cudaGetLastError();
    KUTACC_CHECK(e == cudaSuccess, "kernel launch failed: ", cudaGetErrorString(e));
    if (!runtime().async) sync_and_check();
}

// Wait for the runtime stream and report a device-side wait that ran out of time (the kernels write the
// site into a host-visible word instead of hanging).
void sync_and_check()
{
    KUTACC_CUDA(cudaStreamSynchronize((cudaStream_t)runtime().stream));
    if (runtime().out_unsynced && runtime().out_done) {
        // chunked downloads of an enqueue-only call: the host result is complete only now
        KUTACC_CUDA(cudaEventSynchronize((cudaEvent_t)runtime().out_done));
        runtime().out_unsynced = runtime().out_hazard = false;
    }
    dev::KernelErrorWord &ew = dev::kernel_error_word();
    if (ew.host && *ew.host != 0) {
        const int code = *ew.host;
        *ew.host = 0;
        KUTACC_CHECK(false, "a device-side wait ran out of time (site ", code, "); the result is invalid");
    }
}

}  // namespace kutacc

extern "C" {

void kutacc_b200_set_stream(void *cuda_stream) { kutacc::runtime().stream = cuda_stream; }
void kutacc_b200_set_async(int enabled) { kutacc::runtime().async = enabled != 0; }
void kutacc_b200_set_sm_margin(int sms) { kutacc::runtime().sm_margin = sms < 0 ? 0 : (sms > 64 ? 64 : sms); }
void kutacc_b200_set_pair_bias_event(void *cuda_event) { kutacc::runtime().pair_bias_event = cuda_event; }
void kutacc_b200_synchronize(void) { kutacc::sync_and_check(); }

void *kutacc_b200_device_malloc(size_t bytes)
{
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    KUTACC_CHECK(e == cudaSuccess, "kutacc_b200_device_malloc(", bytes, "): ", cudaGetErrorString(e));
    return e == cudaSuccess ? p : nullptr;
}
void kutacc_b200_device_free(void *p)
{
    if (p) KUTACC_CUDA(cudaFree(p));
}
void kutacc_b200_memcpy_h2d(void *dst, const void *src, size_t bytes)
{
    KUTACC_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
}
void kutacc_b200_memcpy_d2h(void *dst, const void *src, size_t bytes)
{
    KUTACC_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
}
size_t kutacc_b200_workspace_bytes(void) { return kutacc::runtime().ws_cap + kutacc::runtime().stage_cap; }
void kutacc_b200_release_workspace(void) { kutacc::runtime().release(); }
uint64_t kutacc_b200_launch_count(void) { return kutacc::g_launches.load(); }

void kutacc_b200_set_profile(int enabled)
{
    kutacc::g_profile = enabled != 0;
}

int kutacc_b200_profile_read(char *names, size_t names_cap, float *ms, int cap)
{
    using namespace kutacc;
    cudaStreamSynchronize((cudaStream_t)runtime().stream);
    int n = 0;
    size_t off = 0;
    if (names && names_cap) names[0] = 0;
    for (auto &r : g_prof) {
        float t = 0.f;
        cudaEventElapsedTime(&t, r.start, r.stop);
        if (n < cap) {
            if (ms) ms[n] = t;
            if (names) {
                const size_t len = std::strlen(r.name);
                if (off + len + 2 <= names_cap) {
                    std::memcpy(names + off, r.name, len);
                    names[off + len] = ';';
                    names[off + len + 1] = 0;
                    off += len + 1;
                }
            }
            ++n;
        }
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    g_prof.clear();
    return n;
}

}  // extern "C"
