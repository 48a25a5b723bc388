/* A stand-in for libnccl used ONLY by tests/test_comm_failures.py: the handful of entry points the attention
 * library resolves with dlsym, with behaviour chosen by the FAKE_NCCL_MODE environment variable, so that the
 * library's own waiting and error paths can be driven on a machine without any GPU or peer.
 *   never  the communicator stays "in progress" for ever (a rank that never joins)
 *   error  the communicator reports an asynchronous error after a few polls
 *   ready  the communicator becomes ready after a few polls
 * Every call is appended to the file named by FAKE_NCCL_LOG.  No data moves: collectives return success at once.
 */
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef enum { ncclSuccess = 0, ncclUnhandledCudaError = 1, ncclSystemError = 2, ncclInternalError = 3,
               ncclInvalidArgument = 4, ncclInvalidUsage = 5, ncclRemoteError = 6, ncclInProgress = 7 } ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;

static int polls = 0;

static void note(const char* what) {
  const char* path = getenv("FAKE_NCCL_LOG");
  if (!path) return;
  FILE* f = fopen(path, "a");
  if (!f) return;
  fprintf(f, "%s\n", what);
  fclose(f);
}

static const char* mode(void) {
  const char* m = getenv("FAKE_NCCL_MODE");
  return m ? m : "never";
}

ncclResult_t ncclGetUniqueId(ncclUniqueId* id) {
  note("GetUniqueId");
  memset(id, 0x5a, sizeof(*id));
  return ncclSuccess;
}

ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config) {
  (void)nranks; (void)id; (void)rank; (void)config;
  note("CommInitRankConfig");
  *comm = (ncclComm_t)&polls;
  polls = 0;
  return ncclInProgress;
}

ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* state) {
  (void)comm;
  ++polls;
  if (strcmp(mode(), "ready") == 0 && polls > 5) *state = ncclSuccess;
  else if (strcmp(mode(), "error") == 0 && polls > 5) *state = ncclRemoteError;
  else *state = ncclInProgress;
  return ncclSuccess;
}

ncclResult_t ncclCommAbort(ncclComm_t comm) { (void)comm; note("CommAbort"); return ncclSuccess; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; note("CommDestroy"); return ncclSuccess; }

ncclResult_t ncclAllGather(const void* s, void* r, size_t n, int t, ncclComm_t c, void* stream) {
  (void)s; (void)r; (void)n; (void)t; (void)c; (void)stream;
  note("AllGather");
  return ncclSuccess;
}

ncclResult_t ncclAllReduce(const void* s, void* r, size_t n, int t, int op, ncclComm_t c, void* stream) {
  (void)s; (void)r; (void)n; (void)t; (void)op; (void)c; (void)stream;
  note("AllReduce");
  return ncclSuccess;
}
