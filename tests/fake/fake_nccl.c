/* A stand-in for libnccl.so.2 used by tests/test_comm_failure_gpu.py: every collective
 * "succeeds" without moving data, and ncclCommGetAsyncError starts reporting a remote
 * error once the environment variable FAKE_NCCL_FAIL_AFTER says so. It lets the library's
 * handling of a failed communicator (a peer that died) be exercised on one GPU, with the
 * failure made on the host and nothing faulting on the device. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;
typedef void* cudaStream_t;

static int g_polls = 0;
static int g_aborted = 0;

int ncclGetVersion(int* v) { *v = 22809; return 0; }
const char* ncclGetErrorString(int r) { return r == 6 ? "remote process exited or there was a network error" : "fake"; }
int ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return 0; }
int ncclCommInitRank(ncclComm_t* c, int n, ncclUniqueId id, int rank) { (void)n; (void)id; (void)rank; *c = (void*)&g_polls; return 0; }
int ncclCommDestroy(ncclComm_t c) { (void)c; return 0; }
int ncclCommAbort(ncclComm_t c) {
  (void)c;
  g_aborted = 1;
  const char* f = getenv("FAKE_NCCL_ABORT_FILE");
  if (f) { FILE* fp = fopen(f, "w"); if (fp) { fputs("aborted\n", fp); fclose(fp); } }
  return 0;
}
int ncclAllReduce(const void* s, void* r, size_t n, int t, int op, ncclComm_t c, cudaStream_t st) {
  (void)s; (void)r; (void)n; (void)t; (void)op; (void)c; (void)st; return g_aborted ? 5 : 0;
}
int ncclReduceScatter(const void* s, void* r, size_t n, int t, int op, ncclComm_t c, cudaStream_t st) {
  (void)s; (void)r; (void)n; (void)t; (void)op; (void)c; (void)st; return g_aborted ? 5 : 0;
}
int ncclAllGather(const void* s, void* r, size_t n, int t, ncclComm_t c, cudaStream_t st) {
  (void)s; (void)r; (void)n; (void)t; (void)c; (void)st; return g_aborted ? 5 : 0;
}
int ncclCommGetAsyncError(ncclComm_t c, int* e) {
  (void)c;
  const char* after = getenv("FAKE_NCCL_FAIL_AFTER");
  ++g_polls;
  *e = (after && g_polls > atoi(after)) ? 6 /* ncclRemoteError */ : 0;
  return 0;
}
