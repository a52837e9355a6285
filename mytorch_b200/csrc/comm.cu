// NCCL reached through dlopen: communicator set-up and the four collectives the
// data-parallel training step uses (broadcast, all-reduce, barrier, abort).
// The library therefore loads on machines without NCCL; the first mt_comm_*
// call fails with a clear message if libnccl.so.2 cannot be found.
#include "common.cuh"
#include <dlfcn.h>
#include <mutex>
#include <string.h>

namespace mt {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
// enums as defined by nccl.h (stable across NCCL 2.x)
enum { ncclInt8 = 0, ncclChar = 0, ncclUint8 = 1, ncclInt32 = 2, ncclUint32 = 3, ncclInt64 = 4, ncclUint64 = 5,
       ncclFloat16 = 6, ncclFloat32 = 7, ncclFloat64 = 8, ncclBfloat16 = 9 };
enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclAvg = 4 };

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommAbort)(ncclComm_t);
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
  const char* (*GetErrorString)(ncclResult_t);
  bool ok = false;
};
static NcclApi g_nccl;
static std::once_flag g_nccl_once;

static bool load_nccl() {
  std::call_once(g_nccl_once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
#define MT_SYM(field, name) *(void**)(&g_nccl.field) = dlsym(h, name); if (!g_nccl.field) return;
    MT_SYM(GetUniqueId, "ncclGetUniqueId")
    MT_SYM(CommInitRank, "ncclCommInitRank")
    MT_SYM(CommDestroy, "ncclCommDestroy")
    MT_SYM(CommAbort, "ncclCommAbort")
    MT_SYM(AllReduce, "ncclAllReduce")
    MT_SYM(Broadcast, "ncclBroadcast")
    MT_SYM(GetErrorString, "ncclGetErrorString")
#undef MT_SYM
    g_nccl.ok = true;
  });
  if (!g_nccl.ok) set_error("NCCL (libnccl.so.2) could not be loaded: %s", dlerror() ? dlerror() : "symbols missing");
  return g_nccl.ok;
}

#define MT_CHECK_NCCL(expr)                                                                     \
  do {                                                                                          \
    ncclResult_t _r = (expr);                                                                   \
    if (_r != 0) {                                                                              \
      set_error("%s failed: %s", #expr, g_nccl.GetErrorString ? g_nccl.GetErrorString(_r) : "?"); \
      return MT_ERR_NCCL;                                                                       \
    }                                                                                           \
  } while (0)

static int nccl_dtype(int dt) { return dt == MT_F32 ? ncclFloat32 : dt == MT_F16 ? ncclFloat16 : ncclBfloat16; }

struct Comm {
  ncclComm_t comm;
  int rank, world;
  float* scratch;  // one device float for the barrier
};

}  // namespace mt

using namespace mt;

extern "C" {

int mt_comm_unique_id(void* id128) {
  if (!load_nccl()) return MT_ERR_NCCL;
  ncclUniqueId id;
  MT_CHECK_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(id128, &id, 128);
  return MT_OK;
}

int mt_comm_init(void** comm, const void* id128, int rank, int world_size) {
  MT_REQUIRE(comm && id128 && rank >= 0 && rank < world_size, "comm_init: bad arguments");
  if (!load_nccl()) return MT_ERR_NCCL;
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  Comm* c = new Comm();
  c->rank = rank; c->world = world_size; c->scratch = nullptr;
  ncclResult_t r = g_nccl.CommInitRank(&c->comm, world_size, id, rank);
  if (r != 0) {
    set_error("ncclCommInitRank failed: %s", g_nccl.GetErrorString(r));
    delete c;
    return MT_ERR_NCCL;
  }
  if (cudaMalloc(&c->scratch, 256) != cudaSuccess) { set_error("comm_init: scratch allocation failed"); delete c; return MT_ERR_CUDA; }
  cudaMemset(c->scratch, 0, 256);
  *comm = c;
  return MT_OK;
}

int mt_comm_broadcast(void* comm, void* buf, int64_t count, int dtype, int root, void* stream) {
  MT_REQUIRE(comm && buf && count >= 0, "comm_broadcast: bad arguments");
  Comm* c = (Comm*)comm;
  MT_CHECK_NCCL(g_nccl.Broadcast(buf, buf, (size_t)count, nccl_dtype(dtype), root, c->comm, as_stream(stream)));
  return MT_OK;
}

int mt_comm_allreduce(void* comm, const void* send, void* recv, int64_t count, int dtype, int op, void* stream) {
  MT_REQUIRE(comm && send && recv && count >= 0, "comm_allreduce: bad arguments");
  Comm* c = (Comm*)comm;
  int nop = op == 0 ? ncclSum : op == 1 ? ncclMax : ncclAvg;
  MT_CHECK_NCCL(g_nccl.AllReduce(send, recv, (size_t)count, nccl_dtype(dtype), nop, c->comm, as_stream(stream)));
  return MT_OK;
}

int mt_comm_barrier(void* comm, void* stream) {
  MT_REQUIRE(comm, "comm_barrier: bad arguments");
  Comm* c = (Comm*)comm;
  MT_CHECK_NCCL(g_nccl.AllReduce(c->scratch, c->scratch, 1, ncclFloat32, ncclSum, c->comm, as_stream(stream)));
  MT_CHECK_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return MT_OK;
}

int mt_comm_abort(void* comm) {
  if (!comm) return MT_OK;
  Comm* c = (Comm*)comm;
  if (g_nccl.ok) g_nccl.CommAbort(c->comm);
  if (c->scratch) cudaFree(c->scratch);
  delete c;
  return MT_OK;
}

int mt_comm_destroy(void* comm) {
  if (!comm) return MT_OK;
  Comm* c = (Comm*)comm;
  if (g_nccl.ok) g_nccl.CommDestroy(c->comm);
  if (c->scratch) cudaFree(c->scratch);
  delete c;
  return MT_OK;
}

}  // extern "C"
