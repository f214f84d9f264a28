/* Stand-in for libnccl used by the CPU tests of the communicator set-up (loaded through KUTACC_NCCL_LIB).
 * It has the symbols the library looks up and no transport: set-up never completes (every state query
 * answers "in progress"), which is what a rank sees when a peer never arrives. Calls are logged to the
 * file named by FAKE_NCCL_LOG so that a test can see that the communicator was aborted. */
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void *ncclComm_t;
typedef int ncclResult_t;
enum { ncclSuccess = 0, ncclSystemError = 2, ncclInProgress = 7 };

static int g_fake_comm;

static void note(const char *what)
{
    const char *path = getenv("FAKE_NCCL_LOG");
    if (!path) return;
    FILE *f = fopen(path, "a");
    if (f) {
        fprintf(f, "%s\n", what);
        fclose(f);
    }
}

ncclResult_t ncclGetUniqueId(ncclUniqueId *id)
{
    memset(id, 0x5a, sizeof(*id));
    note("ncclGetUniqueId");
    return ncclSuccess;
}
ncclResult_t ncclCommInitRankConfig(ncclComm_t *comm, int nranks, ncclUniqueId id, int rank, void *config)
{
    (void)nranks; (void)id; (void)rank; (void)config;
    *comm = &g_fake_comm;
    note("ncclCommInitRankConfig");
    return ncclInProgress;
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t *state)
{
    (void)comm;
    *state = ncclInProgress;
    return ncclSuccess;
}
ncclResult_t ncclCommAbort(ncclComm_t comm) { (void)comm; note("ncclCommAbort"); return ncclSuccess; }
ncclResult_t ncclCommFinalize(ncclComm_t comm) { (void)comm; note("ncclCommFinalize"); return ncclSuccess; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; note("ncclCommDestroy"); return ncclSuccess; }
ncclResult_t ncclAllGather(const void *s, void *r, size_t n, int t, ncclComm_t c, void *st)
{
    (void)s; (void)r; (void)n; (void)t; (void)c; (void)st;
    return ncclSystemError;
}
ncclResult_t ncclSend(const void *s, size_t n, int t, int p, ncclComm_t c, void *st)
{
    (void)s; (void)n; (void)t; (void)p; (void)c; (void)st;
    return ncclSystemError;
}
ncclResult_t ncclRecv(void *r, size_t n, int t, int p, ncclComm_t c, void *st)
{
    (void)r; (void)n; (void)t; (void)p; (void)c; (void)st;
    return ncclSystemError;
}
ncclResult_t ncclGroupStart(void) { return ncclSuccess; }
ncclResult_t ncclGroupEnd(void) { return ncclSuccess; }
const char *ncclGetErrorString(ncclResult_t r) { return r == ncclSuccess ? "no error" : "fake nccl error"; }
