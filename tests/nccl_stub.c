/* A stand-in for libnccl.so.2 whose exchanges fail, for the test of the library's failure surface (named by
 * TSM_NCCL_LIBRARY).  The group can be joined; every collective then reports a remote error, as NCCL does when a peer has
 * died, and the communicator says the same when polled. */
#include <stddef.h>
#include <string.h>

typedef struct { char bytes[128]; } id_t;
static int comm_token;

int ncclGetUniqueId(id_t* id) { memset(id, 7, sizeof *id); return 0; }
int ncclCommInitRank(void** comm, int world, id_t id, int rank) { (void)world, (void)id, (void)rank; *comm = &comm_token; return 0; }
int ncclAllGather(const void* s, void* r, size_t n, int t, void* c, void* stream) { (void)s, (void)r, (void)n, (void)t, (void)c, (void)stream; return 6; }
int ncclAllReduce(const void* s, void* r, size_t n, int t, int op, void* c, void* stream) { (void)s, (void)r, (void)n, (void)t, (void)op, (void)c, (void)stream; return 6; }
int ncclReduceScatter(const void* s, void* r, size_t n, int t, int op, void* c, void* stream) { (void)s, (void)r, (void)n, (void)t, (void)op, (void)c, (void)stream; return 6; }
int ncclCommDestroy(void* c) { (void)c; return 0; }
int ncclCommAbort(void* c) { (void)c; return 0; }
int ncclCommGetAsyncError(void* c, int* e) { (void)c; *e = 6; return 0; }
const char* ncclGetErrorString(int rc) { return rc == 6 ? "remote process exited or there was a network error" : "error"; }
