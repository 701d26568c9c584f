// Collective communication for tensor-parallel execution: NCCL all-reduce on the library's stream.
//
// The reference has no distributed code at all; tensor parallelism over attention heads and MLP
// columns with a sum all-reduce after o_proj and down_proj is an addition.  NCCL is loaded at run
// time (dlopen) so that the library has no link-time dependency on it; one process drives one GPU
// and owns one communicator.  The all-reduce is enqueued on the same stream as the kernels, so it
// is ordered with them and can be captured into the decode graph.
#include <dlfcn.h>
#include <nccl.h>

#include "common.cuh"

namespace kd {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi g_nccl;
static ncclComm_t g_comm = nullptr;
static int g_nranks = 1, g_rank = 0;

static int load_nccl(const char* path) {
  if (g_nccl.handle) return KD_OK;
  const char* candidates[3] = {path, "libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* c : candidates) {
    if (c == nullptr || c[0] == 0) continue;
    h = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) return fail(KD_ERR_UNSUPPORTED, "could not load NCCL (%s)", dlerror());
  NcclApi a;
  a.handle = h;
#define KD_SYM(field, name)                                                        \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(h, name));                   \
  if (!a.field) return fail(KD_ERR_UNSUPPORTED, "NCCL symbol %s is missing", name)
  KD_SYM(GetUniqueId, "ncclGetUniqueId");
  KD_SYM(CommInitRank, "ncclCommInitRank");
  KD_SYM(AllReduce, "ncclAllReduce");
  KD_SYM(CommDestroy, "ncclCommDestroy");
  KD_SYM(CommAbort, "ncclCommAbort");
  KD_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
  KD_SYM(GetErrorString, "ncclGetErrorString");
#undef KD_SYM
  g_nccl = a;
  return KD_OK;
}

#define KD_NCCL_CHECK(expr)                                                                        \
  do {                                                                                             \
    ncclResult_t _r = (expr);                                                                      \
    if (_r != ncclSuccess) return fail(KD_ERR_CUDA, "%s failed: %s", #expr, g_nccl.GetErrorString(_r)); \
  } while (0)

}  // namespace kd

using namespace kd;

KD_API int kd_comm_unique_id(const char* nccl_path, char* id_out, size_t id_bytes) {
  KD_TRY(load_nccl(nccl_path));
  KD_REQUIRE(id_out && id_bytes >= sizeof(ncclUniqueId), "id buffer must hold %zu bytes", sizeof(ncclUniqueId));
  ncclUniqueId id;
  KD_NCCL_CHECK(g_nccl.GetUniqueId(&id));
  memcpy(id_out, &id, sizeof(id));
  return KD_OK;
}

KD_API int kd_comm_init(const char* nccl_path, int nranks, int rank, const char* id, size_t id_bytes) {
  KD_TRY(require_init());
  KD_TRY(load_nccl(nccl_path));
  KD_REQUIRE(g_comm == nullptr, "communicator already initialised");
  KD_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "bad rank %d of %d", rank, nranks);
  KD_REQUIRE(id && id_bytes >= sizeof(ncclUniqueId), "id buffer must hold %zu bytes", sizeof(ncclUniqueId));
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  KD_CUDA_CHECK(cudaSetDevice(ctx().device));
  KD_NCCL_CHECK(g_nccl.CommInitRank(&g_comm, nranks, uid, rank));
  g_nranks = nranks;
  g_rank = rank;
  return KD_OK;
}

KD_API int kd_comm_info(int* nranks, int* rank) {
  if (nranks) *nranks = g_comm ? g_nranks : 1;
  if (rank) *rank = g_comm ? g_rank : 0;
  return KD_OK;
}

KD_API int kd_allreduce_sum(const kd_tensor* t) {
  KD_TRY(require_init());
  KD_REQUIRE(t, "null tensor");
  KD_REQUIRE(is_contiguous(t), "all-reduce needs a contiguous tensor");
  KD_REQUIRE(t->dtype == KD_BF16 || t->dtype == KD_F32, "all-reduce supports bf16 and fp32");
  if (g_comm == nullptr || g_nranks == 1) return KD_OK;  // single rank: the sum over ranks is the tensor itself
  void* p = nullptr;
  KD_TRY(tensor_ptr(t, &p));
  const int64_t n = numel(t);
  if (n == 0) return KD_OK;
  KD_NCCL_CHECK(g_nccl.AllReduce(p, p, (size_t)n, t->dtype == KD_BF16 ? ncclBfloat16 : ncclFloat32, ncclSum, g_comm,
                                 ctx().stream));
  ctx().launches++;
  return KD_OK;
}

// Polls the communicator for an asynchronous error (a peer that died, a network fault).  Returns
// KD_OK when healthy; otherwise the communicator is aborted so that no later call blocks on it.
KD_API int kd_comm_check(void) {
  if (g_comm == nullptr) return KD_OK;
  ncclResult_t async = ncclSuccess;
  KD_NCCL_CHECK(g_nccl.CommGetAsyncError(g_comm, &async));
  if (async != ncclSuccess && async != ncclInProgress) {
    g_nccl.CommAbort(g_comm);
    g_comm = nullptr;
    g_nranks = 1;
    return fail(KD_ERR_DEVICE, "NCCL reported an asynchronous error (%s); communicator aborted", g_nccl.GetErrorString(async));
  }
  return KD_OK;
}

KD_API int kd_comm_destroy(void) {
  if (g_comm == nullptr) return KD_OK;
  cudaStreamSynchronize(ctx().stream);
  g_nccl.CommDestroy(g_comm);
  g_comm = nullptr;
  g_nranks = 1;
  g_rank = 0;
  return KD_OK;
}
