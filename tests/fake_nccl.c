/* A stand-in for libnccl.so.2 that the failure-detection test loads through JAXCUDA_NCCL_LIB: the
 * calls the runtime binds, doing nothing, plus an asynchronous error state that the test sets from
 * the host through a file.  No GPU work is made to fail. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } uid_t128;

static int flag_value(void) {
  const char* path = getenv("FAKE_NCCL_FLAG");
  int v = 0;
  if (!path) return 0;
  FILE* f = fopen(path, "r");
  if (!f) return 0;
  if (fscanf(f, "%d", &v) != 1) v = 0;
  fclose(f);
  return v;
}

int ncclGetUniqueId(uid_t128* id) { memset(id, 7, sizeof *id); return 0; }
int ncclCommInitRank(void** comm, int nranks, uid_t128 id, int rank) { (void)nranks; (void)id; (void)rank; *comm = malloc(16); return 0; }
int ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, void* comm, void* stream) {
  (void)s; (void)r; (void)n; (void)dt; (void)op; (void)comm; (void)stream;
  return 0;
}
int ncclGroupStart(void) { return 0; }
int ncclGroupEnd(void) { return 0; }
const char* ncclGetErrorString(int code) { return code == 6 ? "remote process exited or there was a network error" : "some error"; }
int ncclCommGetAsyncError(void* comm, int* state) { (void)comm; *state = flag_value(); return 0; }
int ncclCommAbort(void* comm) {
  const char* path = getenv("FAKE_NCCL_ABORTED");
  if (path) { FILE* f = fopen(path, "w"); if (f) { fputs("aborted", f); fclose(f); } }
  free(comm);
  return 0;
}
int ncclCommDestroy(void* comm) { free(comm); return 0; }
