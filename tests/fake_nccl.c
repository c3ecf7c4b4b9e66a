/* Test infrastructure: a stand-in for libnccl.so.2 that exports every symbol the kernel library resolves.  It moves
 * no data.  Its asynchronous error state is scripted through the environment:
 *   FAKE_NCCL_ERROR_AFTER unset or 0 : ncclCommGetAsyncError reports "in progress" for ever (a hung peer);
 *   FAKE_NCCL_ERROR_AFTER = n        : the n-th query reports ncclRemoteError (a peer that died).
 * fake_nccl_aborts() / fake_nccl_queries() tell the test what the library did. */
#include <stdlib.h>
#include <string.h>

enum { ncclSuccess = 0, ncclRemoteError = 6, ncclInProgress = 7 };
typedef struct { char internal[128]; } ncclUniqueId;
static int g_aborts, g_queries, g_comm;

int fake_nccl_aborts(void) { return g_aborts; }
int fake_nccl_queries(void) { return g_queries; }

int ncclGetUniqueId(ncclUniqueId *id) { memset(id, 7, sizeof(*id)); return ncclSuccess; }
int ncclCommInitRank(void **comm, int n, ncclUniqueId id, int rank) { (void)n; (void)id; (void)rank; *comm = &g_comm; return ncclSuccess; }
int ncclCommDestroy(void *c) { (void)c; return ncclSuccess; }
int ncclCommAbort(void *c) { (void)c; g_aborts++; return ncclSuccess; }
int ncclCommGetAsyncError(void *c, int *state) {
    (void)c;
    const char *e = getenv("FAKE_NCCL_ERROR_AFTER");
    const int after = e ? atoi(e) : 0;
    g_queries++;
    *state = (after > 0 && g_queries >= after) ? ncclRemoteError : ncclInProgress;
    return ncclSuccess;
}
const char *ncclGetErrorString(int r) { (void)r; return "fake"; }
int ncclBroadcast(const void *a, void *b, size_t n, int t, int root, void *c, void *s) { (void)a; (void)b; (void)n; (void)t; (void)root; (void)c; (void)s; return ncclSuccess; }
int ncclAllReduce(const void *a, void *b, size_t n, int t, int op, void *c, void *s) { (void)a; (void)b; (void)n; (void)t; (void)op; (void)c; (void)s; return ncclSuccess; }
int ncclReduce(const void *a, void *b, size_t n, int t, int op, int root, void *c, void *s) { (void)a; (void)b; (void)n; (void)t; (void)op; (void)root; (void)c; (void)s; return ncclSuccess; }
int ncclReduceScatter(const void *a, void *b, size_t n, int t, int op, void *c, void *s) { (void)a; (void)b; (void)n; (void)t; (void)op; (void)c; (void)s; return ncclSuccess; }
int ncclAllGather(const void *a, void *b, size_t n, int t, void *c, void *s) { (void)a; (void)b; (void)n; (void)t; (void)c; (void)s; return ncclSuccess; }
int ncclSend(const void *a, size_t n, int t, int peer, void *c, void *s) { (void)a; (void)n; (void)t; (void)peer; (void)c; (void)s; return ncclSuccess; }
int ncclRecv(void *a, size_t n, int t, int peer, void *c, void *s) { (void)a; (void)n; (void)t; (void)peer; (void)c; (void)s; return ncclSuccess; }
int ncclGroupStart(void) { return ncclSuccess; }
int ncclGroupEnd(void) { return ncclSuccess; }
