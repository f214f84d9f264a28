// Rank bookkeeping and the byte-typed all-gather on NCCL.
// Replaces src/comm/kupl.cpp:25-68 and src/comm/all_gather.cpp:21-100 of the reference, where the
// transport is a shared-memory window plus MPI barriers; here it is ncclAllGather over NVLink into
// this GPU's own memory. NCCL is resolved with dlopen at kutacc_comm_init, so single-GPU users do
// not need the library at all.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <nccl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>

#include "common.h"

extern "C" {
KUTACC_B200_API int64_t world_size = 1;
KUTACC_B200_API int64_t rank = 0;
}
int64_t buffer_size = 0;  // declared by the reference header, not exported (include/kutacc.h:53)

namespace kutacc {

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommFinalize)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
NcclApi g_nccl;
ncclComm_t g_comm = nullptr;
std::string g_id_file;

bool load_nccl()
{
    if (g_nccl.handle) return true;
    // KUTACC_NCCL_LIB names another library with the NCCL interface (the tests use it to put a stand-in there)
    const char *override_name = std::getenv("KUTACC_NCCL_LIB");
    const char *names[] = {override_name && *override_name ? override_name : "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle || (override_name && *override_name)) break;
    }
    KUTACC_CHECK(g_nccl.handle != nullptr, "cannot load libnccl.so.2: ", dlerror());
    if (!g_nccl.handle) return false;
#define KUTACC_SYM(field, name) \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(g_nccl.handle, name))
    KUTACC_SYM(GetUniqueId, "ncclGetUniqueId");
    KUTACC_SYM(CommInitRankConfig, "ncclCommInitRankConfig");
    KUTACC_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    KUTACC_SYM(CommAbort, "ncclCommAbort");
    KUTACC_SYM(CommFinalize, "ncclCommFinalize");
    KUTACC_SYM(CommDestroy, "ncclCommDestroy");
    KUTACC_SYM(AllGather, "ncclAllGather");
    KUTACC_SYM(Send, "ncclSend");
    KUTACC_SYM(Recv, "ncclRecv");
    KUTACC_SYM(GroupStart, "ncclGroupStart");
    KUTACC_SYM(GroupEnd, "ncclGroupEnd");
    KUTACC_SYM(GetErrorString, "ncclGetErrorString");
#undef KUTACC_SYM
    const bool ok = g_nccl.GetUniqueId && g_nccl.CommInitRankConfig && g_nccl.CommGetAsyncError && g_nccl.CommAbort &&
                    g_nccl.CommDestroy && g_nccl.AllGather &&
                    g_nccl.Send && g_nccl.Recv && g_nccl.GroupStart && g_nccl.GroupEnd && g_nccl.GetErrorString;
    KUTACC_CHECK(ok, "libnccl lacks a required symbol");
    return ok;
}

double env_seconds(const char *name, double dflt)
{
    const char *v = std::getenv(name);
    return v && *v ? std::atof(v) : dflt;
}

// The communicator is non-blocking (ncclCommInitRankConfig with blocking = 0), so that a rank that never
// arrives cannot park this process inside NCCL: a call may answer ncclInProgress, and the host then polls
// ncclCommGetAsyncError under a time limit (KUTACC_COMM_TIMEOUT_S, 120 s by default). When the limit runs out the
// communicator is aborted and the failure goes through the usual error flag.
ncclResult_t settle(ncclResult_t r)
{
    if (r != ncclInProgress || g_comm == nullptr) return r;
    const double limit = env_seconds("KUTACC_COMM_TIMEOUT_S", 120.0);
    const auto t0 = std::chrono::steady_clock::now();
    for (long polls = 0;; ++polls) {
        ncclResult_t state = ncclSuccess;
        const ncclResult_t q = g_nccl.CommGetAsyncError(g_comm, &state);
        if (q != ncclSuccess) return q;
        if (state != ncclInProgress) return state;
        // an enqueue settles within microseconds: poll without yielding first, sleep only when it takes long
        if ((polls & 63) == 63) {
            const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (waited > limit) {
                g_nccl.CommAbort(g_comm);
                g_comm = nullptr;
                return ncclSystemError;
            }
            if (waited > 2e-3) std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
    }
}

#define KUTACC_NCCL(call)                                                                                   \
    do {                                                                                                    \
        ncclResult_t r__ = settle(call);                                                                    \
        KUTACC_CHECK(r__ == ncclSuccess, "NCCL error: ", g_nccl.GetErrorString(r__), " (", #call, ")");    \
    } while (0)

// Name of the file through which rank 0 hands the NCCL id to the other ranks when the caller gives none.
// The default name carries the user id and what identifies the job (MASTER_ADDR, MASTER_PORT and the launcher's
// run id), so that two jobs or two users on one machine do not meet in the same file.
std::string rendezvous_path()
{
    const char *name = std::getenv("KUTACC_RENDEZVOUS");
    if (!name || !*name) name = std::getenv("SHMID");
    std::string base;
    if (name && *name) {
        base = name;
    } else {
        const char *addr = std::getenv("MASTER_ADDR"), *port = std::getenv("MASTER_PORT"),
                   *run = std::getenv("TORCHELASTIC_RUN_ID");
        base = "kutacc_nccl_u" + std::to_string((long long)getuid()) + "_" + (addr ? addr : "local") + "_" +
               (port ? port : "default") + "_" + (run ? run : "norun");
        for (char &c : base)
            if (c == '/' || c == ' ') c = '_';
    }
    if (base.find('/') != std::string::npos) return base;
    return "/dev/shm/" + base + ".ncclid";
}

struct IdRecord {
    ncclUniqueId id;
    int64_t stamp;  // seconds since the epoch when rank 0 wrote the file
    int64_t world;
};

// Rank 0 publishes the id through a file that it creates itself (O_EXCL, no symlink followed, mode 0600) and
// renames into place; the others poll for a record that is owned by this user, has the right world size and was
// written no earlier than KUTACC_RENDEZVOUS_SLACK_S (60 s) before this rank began to wait: an id left by a job
// that crashed, or by the previous job of a back-to-back pair, is refused. The poll gives up after
// KUTACC_RENDEZVOUS_TIMEOUT_S (120 s).
bool exchange_id(int64_t nranks, int64_t me, ncclUniqueId &id)
{
    using clock = std::chrono::system_clock;
    const int64_t now = std::chrono::duration_cast<std::chrono::seconds>(clock::now().time_since_epoch()).count();
    g_id_file = rendezvous_path();
    if (me == 0) {
        KUTACC_NCCL(g_nccl.GetUniqueId(&id));
        if (kutacc_check_err_set) return false;
        IdRecord rec;
        std::memset(&rec, 0, sizeof(rec));
        rec.id = id;
        rec.stamp = now;
        rec.world = nranks;
        const std::string tmp = g_id_file + ".tmp" + std::to_string((long long)getpid());
        ::unlink(g_id_file.c_str());
        ::unlink(tmp.c_str());
        const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_EXCL | O_NOFOLLOW | O_CLOEXEC, 0600);
        KUTACC_CHECK(fd >= 0, "cannot create rendezvous file ", tmp, ": ", std::strerror(errno));
        if (fd < 0) return false;
        const ssize_t w = ::write(fd, &rec, sizeof(rec));
        ::close(fd);
        KUTACC_CHECK(w == (ssize_t)sizeof(rec) && std::rename(tmp.c_str(), g_id_file.c_str()) == 0,
                     "cannot publish rendezvous file ", g_id_file);
        if (kutacc_check_err_set) ::unlink(tmp.c_str());
        return !kutacc_check_err_set;
    }
    const double timeout_s = env_seconds("KUTACC_RENDEZVOUS_TIMEOUT_S", 120.0);
    const int64_t slack = (int64_t)env_seconds("KUTACC_RENDEZVOUS_SLACK_S", 60.0);
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const int fd = ::open(g_id_file.c_str(), O_RDONLY | O_NOFOLLOW | O_CLOEXEC);
        if (fd >= 0) {
            IdRecord rec;
            struct stat st;
            const bool mine = ::fstat(fd, &st) == 0 && S_ISREG(st.st_mode) && st.st_uid == getuid() &&
                              (st.st_mode & (S_IWGRP | S_IWOTH)) == 0;
            const ssize_t r = mine ? ::read(fd, &rec, sizeof(rec)) : -1;
            ::close(fd);
            if (r == (ssize_t)sizeof(rec) && rec.world == nranks && rec.stamp >= now - slack) {
                id = rec.id;
                return true;
            }
        }
        const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (waited > timeout_s) {
            KUTACC_CHECK(false, "rank ", me, ": no fresh rendezvous record at ", g_id_file, " after ", waited, " s");
            return false;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
}

// strided byte gather/scatter between a [a, o, len] view and a dense buffer
__global__ void copy_rows_kernel(const uint8_t *__restrict__ src, int64_t s_a, int64_t s_o, uint8_t *__restrict__ dst,
                                 int64_t d_a, int64_t d_o, int64_t na, int64_t no, int64_t len)
{
    const int64_t total = na * no;
    for (int64_t row = blockIdx.x; row < total; row += gridDim.x) {
        const int64_t a = row / no, o = row % no;
        const uint8_t *s = src + a * s_a + o * s_o;
        uint8_t *d = dst + a * d_a + o * d_o;
        if (((((uintptr_t)s) | ((uintptr_t)d) | (uintptr_t)len) & 15u) == 0) {
            for (int64_t i = threadIdx.x; i < len / 16; i += blockDim.x)
                reinterpret_cast<uint4 *>(d)[i] = reinterpret_cast<const uint4 *>(s)[i];
        } else {
            for (int64_t i = threadIdx.x; i < len; i += blockDim.x) d[i] = s[i];
        }
    }
}

void copy_rows(cudaStream_t stream, const void *src, int64_t s_a, int64_t s_o, void *dst, int64_t d_a, int64_t d_o,
               int64_t na, int64_t no, int64_t len)
{
    if (na <= 0 || no <= 0 || len <= 0) return;
    const unsigned grid = (unsigned)std::min<int64_t>(na * no, 148 * 8);
    const unsigned block = len >= 4096 ? 256 : (len >= 512 ? 128 : 32);
    copy_rows_kernel<<<grid, block, 0, stream>>>((const uint8_t *)src, s_a, s_o, (uint8_t *)dst, d_a, d_o, na, no, len);
    count_launch();
}

}  // namespace

static void init_common(int64_t nranks, int64_t me, int64_t bufsz, const ncclUniqueId *given)
{
    KUTACC_CHECK(nranks > 0 && me >= 0 && me < nranks && bufsz >= 0, "kutacc_comm_init: invalid arguments ", nranks,
                 " ", me, " ", bufsz);
    if (kutacc_check_err_set) return;
    world_size = nranks;
    rank = me;
    buffer_size = bufsz;
    if (nranks == 1) return;
    if (const char *dev = std::getenv("KUTACC_DEVICE")) KUTACC_CUDA(cudaSetDevice(std::atoi(dev)));
    if (!load_nccl()) return;
    ncclUniqueId id;
    if (given) {
        id = *given;
    } else if (!exchange_id(nranks, me, id)) {
        return;
    }
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;
    // KUTACC_NCCL_MAX_CTAS bounds the CTAs a collective of this communicator launches. The persistent kernels fill
    // every SM with one CTA each; a collective that runs beside them takes whole SMs away, and the CTAs that find no
    // SM start late and finish late. With the collective bounded to n CTAs and kutacc_b200_set_sm_margin(n) the
    // kernels size their grids to the SMs that are left.
    const int max_ctas = (int)env_seconds("KUTACC_NCCL_MAX_CTAS", 0.0);
    if (max_ctas > 0) config.maxCTAs = max_ctas;
    const ncclResult_t r = g_nccl.CommInitRankConfig(&g_comm, (int)nranks, id, (int)me, &config);
    if (r != ncclSuccess && r != ncclInProgress) {
        KUTACC_CHECK(false, "NCCL error: ", g_nccl.GetErrorString(r), " (ncclCommInitRankConfig)");
        g_comm = nullptr;
        return;
    }
    const ncclResult_t done = settle(ncclInProgress);
    KUTACC_CHECK(done == ncclSuccess, "kutacc_comm_init: the communicator of ", nranks, " ranks was not built (",
                 g_comm == nullptr ? "set-up ran out of time and was aborted" : g_nccl.GetErrorString(done), ")");
    if (done != ncclSuccess && g_comm != nullptr) {
        g_nccl.CommAbort(g_comm);
        g_comm = nullptr;
    }
}

}  // namespace kutacc

extern "C" {

void kutacc_comm_init(int64_t world_size_, int64_t rank_, int64_t buffer_size_)
{
    kutacc::init_common(world_size_, rank_, buffer_size_, nullptr);
}

// Variant for callers that already have a way to broadcast 128 bytes between ranks.
KUTACC_B200_API void kutacc_b200_comm_unique_id(void *id128)
{
    using namespace kutacc;
    KUTACC_CHECK(id128 != nullptr, "kutacc_b200_comm_unique_id: nullptr");
    if (kutacc_check_err_set || !load_nccl()) return;
    ncclUniqueId id;
    KUTACC_NCCL(g_nccl.GetUniqueId(&id));
    std::memcpy(id128, &id, sizeof(id));
}
KUTACC_B200_API void kutacc_b200_comm_init_with_id(int64_t world_size_, int64_t rank_, const void *id128)
{
    using namespace kutacc;
    KUTACC_CHECK(id128 != nullptr, "kutacc_b200_comm_init_with_id: nullptr");
    if (kutacc_check_err_set) return;
    ncclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    init_common(world_size_, rank_, 0, &id);
}

void kutacc_comm_fini(void)
{
    using namespace kutacc;
    if (g_comm) {
        cudaStreamSynchronize((cudaStream_t)runtime().stream);
        // a non-blocking communicator is finalized (polled to completion) before it is destroyed
        if (g_nccl.CommFinalize) KUTACC_NCCL(g_nccl.CommFinalize(g_comm));
        if (g_comm) {                                       // still there: the poll did not have to abort it
            const ncclResult_t r = g_nccl.CommDestroy(g_comm);
            KUTACC_CHECK(r == ncclSuccess || r == ncclInProgress, "NCCL error: ", g_nccl.GetErrorString(r), " (ncclCommDestroy)");
        }
        g_comm = nullptr;
    }
    if (rank == 0 && !g_id_file.empty()) std::remove(g_id_file.c_str());
    g_id_file.clear();
    world_size = 1;
    rank = 0;
}

void kutacc_af2_all_gather(kutacc_tensor_h data_h, kutacc_tensor_h out_h)
{
    using namespace kutacc;
    if (data_h == nullptr || out_h == nullptr) {  // all_gather.cpp:88-92
        KUTACC_CHECK(data_h != nullptr, "all_gather: data is null");
        KUTACC_CHECK(out_h != nullptr, "all_gather: out is null");
        return;
    }
    if (kutacc_check_err_set) return;
    Tensor &data = *as_tensor(data_h), &out = *as_tensor(out_h);
    KUTACC_CHECK(data.dim() == 3 && out.dim() == 3 && data.data_ptr() && out.data_ptr(),
                 "all_gather: [m, n, len] byte tensors expected");
    if (kutacc_check_err_set) return;
    const int64_t m = out.sizes()[0], n = out.sizes()[1], len = data.sizes()[2];
    KUTACC_CHECK(data.strides()[2] == 1, data.strides()[2]);  // all_gather.cpp:37-38
    KUTACC_CHECK(out.strides()[2] == 1, out.strides()[2]);
    KUTACC_CHECK(m > 0 && n > 0 && len > 0 && out.sizes()[2] == len, "all_gather: shape invalid");
    if (kutacc_check_err_set) return;
    // sharded axis: dim 1 when the leading sizes agree (all_gather.cpp:27-33); a = sharded, o = whole
    const bool dim1 = data.sizes()[0] == m;
    const int64_t full = dim1 ? n : m, other = dim1 ? m : n;
    const int64_t ds_a = dim1 ? data.strides()[1] : data.strides()[0], ds_o = dim1 ? data.strides()[0] : data.strides()[1];
    const int64_t os_a = dim1 ? out.strides()[1] : out.strides()[0], os_o = dim1 ? out.strides()[0] : out.strides()[1];
    const int64_t block = (full + world_size - 1) / world_size;
    const int64_t mine = std::max<int64_t>(0, std::min(block, full - rank * block));
    KUTACC_CHECK((dim1 ? data.sizes()[1] : data.sizes()[0]) >= mine && (dim1 ? data.sizes()[0] : data.sizes()[1]) == other,
                 "all_gather: data shape does not match this rank's chunk");
    if (kutacc_check_err_set) return;

    auto span = [&](const Tensor &t) {
        return (size_t)((t.sizes()[0] - 1) * t.strides()[0] + (t.sizes()[1] - 1) * t.strides()[1] + len);
    };
    const size_t data_bytes = mine > 0 ? span(data) : 0, out_bytes = span(out);
    const size_t slot = (size_t)block * other * len;  // dense bytes per rank

    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    if (!rt.reserve_stage(staged_bytes_needed(data.data_ptr(), data_bytes) + staged_bytes_needed(out.data_ptr(), out_bytes)))
        return;
    DeviceArg d_in = data_bytes ? resolve_in(data.data_ptr(), data_bytes) : DeviceArg{};
    // a staged (host) output is rebuilt whole on the device and copied back; one whose strides leave gaps is
    // brought in first, so that the bytes between its elements come back unchanged
    const bool out_dense = out.strides()[1] == len && out.strides()[0] == n * len;
    DeviceArg d_out = out_dense ? resolve_out(out.data_ptr(), out_bytes) : resolve_in(out.data_ptr(), out_bytes);
    if (kutacc_check_err_set) return;

    const bool dense_dim0 = !dim1 && ds_o == len && ds_a == other * len && os_o == len && os_a == other * len;
    if (world_size == 1 || g_comm == nullptr) {
        KUTACC_CHECK(world_size == 1, "all_gather: kutacc_comm_init has not built a communicator");
        if (kutacc_check_err_set) return;
        copy_rows(stream, d_in.dev, ds_a, ds_o, d_out.dev, os_a, os_o, mine, other, len);
    } else if (dense_dim0 && full % world_size == 0) {
        // every rank's rows are one contiguous slab of out: gather in place
        KUTACC_NCCL(g_nccl.AllGather(d_in.dev, d_out.dev, slot, ncclUint8, g_comm, stream));
    } else if (dim1 && ds_a == len && os_a == len && full % world_size == 0 && other <= 64) {
        // sharded on dim 1 with dense strips (the pair bias [H, rows, keys]): for each of the few leading indices
        // every rank's rows are one contiguous slab of that strip of out: one group of in-place gathers, no copies
        KUTACC_NCCL(g_nccl.GroupStart());
        for (int64_t o = 0; o < other; ++o)
            KUTACC_NCCL(g_nccl.AllGather((const uint8_t *)d_in.dev + o * ds_o, (uint8_t *)d_out.dev + o * os_o,
                                         (size_t)block * len, ncclUint8, g_comm, stream));
        KUTACC_NCCL(g_nccl.GroupEnd());
    } else {
        if (!rt.reserve_workspace((size_t)(world_size + 1) * (slot + 256))) return;
        uint8_t *send = (uint8_t *)rt.take_workspace(slot);
        uint8_t *recv = (uint8_t *)rt.take_workspace((size_t)world_size * slot);
        if (kutacc_check_err_set) return;
        copy_rows(stream, d_in.dev, ds_a, ds_o, send, other * len, len, mine, other, len);
        KUTACC_NCCL(g_nccl.AllGather(send, recv, slot, ncclUint8, g_comm, stream));
        for (int64_t r = 0; r < world_size; ++r) {
            const int64_t have = std::max<int64_t>(0, std::min(block, full - r * block));
            copy_rows(stream, recv + (size_t)r * slot, other * len, len, (uint8_t *)d_out.dev + r * block * os_a, os_a,
                      os_o, have, other, len);
        }
    }
    finish_out(d_out);
    end_of_call();
}

// Re-shard a byte matrix between "rows split over the ranks" and "columns split over the ranks"
// (replaces src/comm/transpose.cpp:21-100, include/kutacc.h:58-65): data [chunk(m), n, len] -> out
// [m, chunk(n), len], or data [m, chunk(n), len] -> out [chunk(m), n, len]; block(x) = ceil(x / world),
// chunk_r(x) = min(block, x - r * block). Element (i, j) moves from the rank that owns row i to the rank that
// owns column j. Here: the block for every peer is packed into the library's workspace, the blocks are
// exchanged with one group of ncclSend/ncclRecv, and the received blocks are scattered into out; the block
// that stays on this rank is copied directly. buffer_size (the reference's shared-memory window) is not used.
void kutacc_af2_transpose(kutacc_tensor_h data_h, kutacc_tensor_h out_h)
{
    using namespace kutacc;
    if (data_h == nullptr || out_h == nullptr) {  // transpose.cpp:92-96
        KUTACC_CHECK(data_h != nullptr, "transpose: data is null");
        KUTACC_CHECK(out_h != nullptr, "transpose: out is null");
        return;
    }
    if (kutacc_check_err_set) return;
    Tensor &data = *as_tensor(data_h), &out = *as_tensor(out_h);
    KUTACC_CHECK(data.dim() == 3 && out.dim() == 3 && data.data_ptr() && out.data_ptr(),
                 "transpose: [m, n, len] byte tensors expected");
    if (kutacc_check_err_set) return;
    KUTACC_CHECK(data.strides()[2] == 1, data.strides()[2]);  // transpose.cpp:38-39
    KUTACC_CHECK(out.strides()[2] == 1, out.strides()[2]);
    if (kutacc_check_err_set) return;
    // local copies of the views; when data holds the whole of dim 0 the roles of dims 0 and 1 swap (:27-33)
    int64_t dsz[2] = {data.sizes()[0], data.sizes()[1]}, dst_[2] = {data.strides()[0], data.strides()[1]};
    int64_t osz[2] = {out.sizes()[0], out.sizes()[1]}, ost[2] = {out.strides()[0], out.strides()[1]};
    int64_t m = std::max(dsz[0], osz[0]), n = std::max(dsz[1], osz[1]);
    const int64_t len = data.sizes()[2];
    KUTACC_CHECK(m > 0 && n > 0 && len > 0 && out.sizes()[2] == len, "transpose: shape invalid");
    if (kutacc_check_err_set) return;
    const size_t data_bytes = (size_t)((dsz[0] - 1) * dst_[0] + (dsz[1] - 1) * dst_[1] + len);
    const size_t out_bytes = (size_t)((osz[0] - 1) * ost[0] + (osz[1] - 1) * ost[1] + len);
    if (dsz[0] == m) {
        std::swap(m, n);
        std::swap(dsz[0], dsz[1]);
        std::swap(dst_[0], dst_[1]);
        std::swap(osz[0], osz[1]);
        std::swap(ost[0], ost[1]);
    }
    // now: data [chunk(m), n], out [m, chunk(n)]
    const int64_t bm = (m + world_size - 1) / world_size, bn = (n + world_size - 1) / world_size;
    auto chunk_m = [&](int64_t r) { return std::max<int64_t>(0, std::min(bm, m - r * bm)); };
    auto chunk_n = [&](int64_t r) { return std::max<int64_t>(0, std::min(bn, n - r * bn)); };
    KUTACC_CHECK(dsz[0] >= chunk_m(rank) && dsz[1] == n && osz[0] == m && osz[1] >= chunk_n(rank),
                 "transpose: shapes do not match this rank's chunks");
    if (kutacc_check_err_set) return;

    Runtime &rt = runtime();
    cudaStream_t stream = (cudaStream_t)rt.stream;
    if (!rt.reserve_stage(staged_bytes_needed(data.data_ptr(), data_bytes) + staged_bytes_needed(out.data_ptr(), out_bytes)))
        return;
    DeviceArg d_in = resolve_in(data.data_ptr(), data_bytes);
    // a strided host output keeps the bytes around its elements: bring it in before it is copied back whole
    const bool out_dense = ost[1] == len && ost[0] == osz[1] * len;
    DeviceArg d_out = out_dense ? resolve_out(out.data_ptr(), out_bytes) : resolve_in(out.data_ptr(), out_bytes);
    if (kutacc_check_err_set) return;
    const uint8_t *src = (const uint8_t *)d_in.dev;
    uint8_t *dst = (uint8_t *)d_out.dev;
    const int64_t my_m = chunk_m(rank), my_n = chunk_n(rank);
    // the block that stays: rows of this rank, columns of this rank
    copy_rows(stream, src + rank * bn * dst_[1], dst_[0], dst_[1], dst + rank * bm * ost[0], ost[0], ost[1], my_m, my_n, len);
    if (world_size > 1) {
        KUTACC_CHECK(g_comm != nullptr, "transpose: kutacc_comm_init has not built a communicator");
        if (kutacc_check_err_set) return;
        const size_t slot = (size_t)bm * bn * len;
        if (!rt.reserve_workspace((size_t)2 * world_size * (slot + 256))) return;
        uint8_t *send = (uint8_t *)rt.take_workspace((size_t)world_size * slot);
        uint8_t *recv = (uint8_t *)rt.take_workspace((size_t)world_size * slot);
        if (kutacc_check_err_set) return;
        for (int64_t p = 0; p < world_size; ++p)
            if (p != rank)
                copy_rows(stream, src + p * bn * dst_[1], dst_[0], dst_[1], send + p * slot, chunk_n(p) * len, len, my_m,
                          chunk_n(p), len);
        KUTACC_NCCL(g_nccl.GroupStart());
        for (int64_t p = 0; p < world_size; ++p) {
            if (p == rank) continue;
            const size_t ns = (size_t)my_m * chunk_n(p) * len, nr = (size_t)chunk_m(p) * my_n * len;
            if (ns) KUTACC_NCCL(g_nccl.Send(send + p * slot, ns, ncclUint8, (int)p, g_comm, stream));
            if (nr) KUTACC_NCCL(g_nccl.Recv(recv + p * slot, nr, ncclUint8, (int)p, g_comm, stream));
        }
        KUTACC_NCCL(g_nccl.GroupEnd());
        for (int64_t p = 0; p < world_size; ++p)
            if (p != rank)
                copy_rows(stream, recv + p * slot, my_n * len, len, dst + p * bm * ost[0], ost[0], ost[1], chunk_m(p), my_n,
                          len);
    }
    finish_out(d_out);
    end_of_call();
}

}  // extern "C"
