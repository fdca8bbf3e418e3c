/* Stand-in for libnccl used only by the host-side failure tests: a communicator whose peers never arrive.
 * ncclCommInitRankConfig answers "in progress" and ncclCommGetAsyncError keeps saying so, which is what the real
 * library reports while a rank waits for the others; ncclCommAbort records that it was called.
 * Enum values as in nccl.h: ncclSuccess 0, ncclInProgress 7. */
#include <stddef.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef struct fake_comm { int aborted; } *ncclComm_t;
typedef int ncclResult_t;
static struct fake_comm g_comm;
int fake_nccl_aborts = 0;

ncclResult_t ncclGetUniqueId(ncclUniqueId *id) { memset(id, 0x5a, sizeof *id); return 0; }
ncclResult_t ncclCommInitRankConfig(ncclComm_t *comm, int nranks, ncclUniqueId id, int rank, void *config)
{
    (void)nranks; (void)id; (void)rank; (void)config;
    *comm = &g_comm;
    return 7;
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t *st) { (void)comm; *st = 7; return 0; }
ncclResult_t ncclCommAbort(ncclComm_t comm) { comm->aborted = 1; fake_nccl_aborts++; return 0; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; return 0; }
ncclResult_t ncclAllReduce(const void *s, void *r, size_t n, int dt, int op, ncclComm_t c, void *stream) { (void)s; (void)r; (void)n; (void)dt; (void)op; (void)c; (void)stream; return 7; }
ncclResult_t ncclAllGather(const void *s, void *r, size_t n, int dt, ncclComm_t c, void *stream) { (void)s; (void)r; (void)n; (void)dt; (void)c; (void)stream; return 7; }
ncclResult_t ncclBroadcast(const void *s, void *r, size_t n, int dt, int root, ncclComm_t c, void *stream) { (void)s; (void)r; (void)n; (void)dt; (void)root; (void)c; (void)stream; return 7; }
const char *ncclGetErrorString(ncclResult_t r) { return r == 7 ? "in progress" : "fake"; }
