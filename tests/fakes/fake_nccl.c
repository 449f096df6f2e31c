/* A scripted stand-in for the NCCL entry points librt_b200.so resolves at run time, for the failure-handling tests:
 * the failing call is faked on the host, no GPU work is involved.  FAKE_NCCL_MODE selects the script:
 *   ok                  every call succeeds at once
 *   init_never          ncclCommInitRankConfig answers "in progress" and the communicator never settles
 *   init_slow           ... settles after 5 polls
 *   async_error         the communicator reports ncclRemoteError from the 4th poll after initialisation on
 *   allreduce_progress  ncclAllReduce answers "in progress"; settles after 3 polls
 * fake_nccl_counts() returns how often abort / destroy / all-reduce / poll were called. */
#include <stdlib.h>
#include <string.h>

enum { kSuccess = 0, kRemoteError = 6, kInProgress = 7 };
static int dummy_comm;
static int n_abort, n_destroy, n_allreduce, n_poll, pending;
static int mode_is(const char* m) {
  const char* e = getenv("FAKE_NCCL_MODE");
  return e && strcmp(e, m) == 0;
}
int ncclGetUniqueId(void* id) {
  memset(id, 7, 128);
  return kSuccess;
}
int ncclCommInitRank(void** comm, int n, char id[128], int rank) {
  (void)n; (void)id; (void)rank;
  *comm = &dummy_comm;
  return kSuccess;
}
int ncclCommInitRankConfig(void** comm, int n, char id[128], int rank, void* config) {
  (void)n; (void)id; (void)rank; (void)config;
  *comm = &dummy_comm;
  n_poll = 0;
  if (mode_is("init_never")) { pending = 1 << 30; return kInProgress; }
  if (mode_is("init_slow")) { pending = 5; return kInProgress; }
  pending = 0;
  return kSuccess;
}
int ncclCommGetAsyncError(void* comm, int* state) {
  (void)comm;
  ++n_poll;
  if (pending > 0) { --pending; *state = kInProgress; return kSuccess; }
  if (mode_is("async_error") && n_poll >= 4) { *state = kRemoteError; return kSuccess; }
  *state = kSuccess;
  return kSuccess;
}
int ncclCommAbort(void* comm) { (void)comm; ++n_abort; return kSuccess; }
int ncclCommDestroy(void* comm) { (void)comm; ++n_destroy; return kSuccess; }
int ncclAllReduce(const void* s, void* r, size_t count, int dtype, int op, void* comm, void* stream) {
  (void)s; (void)r; (void)count; (void)dtype; (void)op; (void)comm; (void)stream;
  ++n_allreduce;
  if (mode_is("allreduce_progress")) { pending = 3; return kInProgress; }
  return kSuccess;
}
const char* ncclGetErrorString(int code) {
  switch (code) {
    case kSuccess: return "no error";
    case kRemoteError: return "remote process exited or there was a network error";
    case kInProgress: return "NCCL operation in progress";
    default: return "some other error";
  }
}
void fake_nccl_counts(int out[4]) { out[0] = n_abort; out[1] = n_destroy; out[2] = n_allreduce; out[3] = n_poll; }
