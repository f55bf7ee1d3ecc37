/* Stand-in for libnccl used by the failure-detection tests: the library under test binds NCCL
 * with dlopen and takes this file's entry points instead when STRICTB200_NCCL_LIB names the
 * built shared object. Collectives do nothing and succeed; the asynchronous error state and the
 * abort counter are set and read by the test through the fake_nccl_* functions. Nothing here
 * touches a GPU. */
#include <stddef.h>
#include <string.h>

typedef struct { char internal[128]; } uid_t128;
static int g_async_error = 0, g_aborts = 0, g_destroys = 0, g_allreduces = 0;
static int g_comm_storage;

int ncclGetUniqueId(uid_t128* id) { memset(id, 7, sizeof(*id)); return 0; }
int ncclCommInitRank(void** comm, int nranks, uid_t128 id, int rank) { (void)nranks; (void)id; (void)rank; *comm = &g_comm_storage; return 0; }
int ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, void* comm, void* stream) {
  (void)s; (void)r; (void)n; (void)dt; (void)op; (void)comm; (void)stream; g_allreduces++; return 0;
}
int ncclAllGather(const void* s, void* r, size_t n, int dt, void* comm, void* stream) { (void)s; (void)r; (void)n; (void)dt; (void)comm; (void)stream; return 0; }
int ncclCommDestroy(void* comm) { (void)comm; g_destroys++; return 0; }
int ncclCommAbort(void* comm) { (void)comm; g_aborts++; return 0; }
int ncclCommGetAsyncError(void* comm, int* async_error) { (void)comm; *async_error = g_async_error; return 0; }
const char* ncclGetErrorString(int rc) { (void)rc; return "fake nccl error"; }

void fake_nccl_set_async_error(int code) { g_async_error = code; }
int fake_nccl_aborts(void) { return g_aborts; }
int fake_nccl_destroys(void) { return g_destroys; }
int fake_nccl_allreduces(void) { return g_allreduces; }
