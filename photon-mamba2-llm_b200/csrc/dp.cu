// Data-parallel gradient averaging behind the C ABI: one NCCL communicator per GPU rank, one all-reduce per layer
// bucket on a communication stream of the library's own, enqueued as soon as that layer's gradient kernels are in
// the compute stream, so the transfer over NVLink overlaps the recompute / backward of the layers below.
// The reference has no distributed code (crates/pm-cli/src/train_cmd.rs:50 drives device 0 only); this is what a
// Rust trainer binds to run the path on 2 / 4 / 8 GPUs.
//
// NCCL is resolved at run time with dlopen("libnccl.so.2") (PMB_NCCL_LIB overrides the name), so the library has no
// link-time dependency on it and a process that already carries a copy of NCCL (e.g. a PyTorch host) shares it.
// Only local memory is handed to NCCL; none of this library's kernels reads a peer's memory.
#include <dlfcn.h>
#include <nccl.h>
#include <mutex>
#include "common.cuh"
#include "kernels.h"

namespace pmb {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;   // optional
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi g_nccl;
static std::mutex g_nccl_mu;

static pmb_status load_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle) return PMB_OK;
  const char* name = getenv("PMB_NCCL_LIB");
  void* h = dlopen(name ? name : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
  if (!h) return fail(PMB_ERR_UNSUPPORTED, "data parallel: cannot load %s: %s", name ? name : "libnccl.so.2", dlerror());
  NcclApi a;
  a.handle = h;
  a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
  a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
  a.CommInitRankConfig = reinterpret_cast<decltype(a.CommInitRankConfig)>(dlsym(h, "ncclCommInitRankConfig"));
  a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
  a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
  a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
  a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
  a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
  if (!a.GetUniqueId || !a.CommInitRank || !a.AllReduce || !a.AllGather || !a.CommDestroy || !a.GetErrorString)
    return fail(PMB_ERR_UNSUPPORTED, "data parallel: the NCCL library lacks a required symbol");
  g_nccl = a;
  return PMB_OK;
}

#define PMB_NCCL(expr)                                                                                          \
  do {                                                                                                          \
    ncclResult_t r__ = (expr);                                                                                  \
    if (r__ != ncclSuccess) return pmb::fail(PMB_ERR_CUDA, "%s failed: %s", #expr, pmb::g_nccl.GetErrorString(r__)); \
  } while (0)

}  // namespace pmb

using namespace pmb;

struct pmb_dp {
  ncclComm_t comm = nullptr;
  int nranks = 1, rank = 0, device = 0;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ready = nullptr, done = nullptr;   // compute -> comm, comm -> compute
};

extern "C" pmb_status pmb_dp_unique_id(void* h_id128) {
  if (!h_id128) return fail(PMB_ERR_ARG, "dp_unique_id: NULL argument");
  static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id size");
  PMB_TRY(load_nccl());
  ncclUniqueId id;
  PMB_NCCL(g_nccl.GetUniqueId(&id));
  memcpy(h_id128, &id, sizeof(id));
  return PMB_OK;
}

extern "C" pmb_status pmb_dp_init(int32_t nranks, int32_t rank, const void* h_id128, pmb_dp** out) {
  if (!out || !h_id128 || nranks < 1 || rank < 0 || rank >= nranks) return fail(PMB_ERR_ARG, "dp_init: bad argument");
  *out = nullptr;
  PMB_TRY(load_nccl());
  pmb_dp* dp = new pmb_dp();
  dp->nranks = nranks; dp->rank = rank;
  auto cleanup = [&](pmb_status s) { pmb_dp_destroy(dp); return s; };
  if (cudaGetDevice(&dp->device) != cudaSuccess) return cleanup(fail(PMB_ERR_CUDA, "dp_init: no current CUDA device"));
  ncclUniqueId id;
  memcpy(&id, h_id128, sizeof(id));
  // The all-reduces run beside compute kernels that want whole SMs (persistent GEMMs, one-CTA-per-SM scan kernels), so
  // the CTAs NCCL may take are capped where that was measured to pay: with two ranks a bucket needs few channels to fill
  // the links (8: 0.2 ms of a 13.6 ms step); with four the cap cost time, so larger worlds keep NCCL's own choice.
  // PMB_DP_MAX_CTAS overrides (0 = NCCL's default).
  int max_ctas = nranks == 2 ? 8 : 0;
  if (const char* e = getenv("PMB_DP_MAX_CTAS")) max_ctas = atoi(e);
  ncclResult_t r;
  if (max_ctas > 0 && g_nccl.CommInitRankConfig) {
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.maxCTAs = max_ctas;
    r = g_nccl.CommInitRankConfig(&dp->comm, nranks, id, rank, &cfg);
  } else {
    r = g_nccl.CommInitRank(&dp->comm, nranks, id, rank);
  }
  if (r != ncclSuccess) return cleanup(fail(PMB_ERR_CUDA, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(r)));
  int least = 0, greatest = 0;
  cudaDeviceGetStreamPriorityRange(&least, &greatest);
  // the communication stream gets the highest priority: an all-reduce's few CTAs should never queue behind compute
  if (cudaStreamCreateWithPriority(&dp->comm_stream, cudaStreamNonBlocking, greatest) != cudaSuccess ||
      cudaEventCreateWithFlags(&dp->ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&dp->done, cudaEventDisableTiming) != cudaSuccess)
    return cleanup(fail(PMB_ERR_CUDA, "dp_init: stream / event creation failed: %s", cudaGetErrorString(cudaGetLastError())));
  *out = dp;
  return PMB_OK;
}

extern "C" void pmb_dp_destroy(pmb_dp* dp) {
  if (!dp) return;
  if (dp->comm_stream) { cudaStreamSynchronize(dp->comm_stream); cudaStreamDestroy(dp->comm_stream); }
  if (dp->ready) cudaEventDestroy(dp->ready);
  if (dp->done) cudaEventDestroy(dp->done);
  if (dp->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(dp->comm);
  delete dp;
}

extern "C" int32_t pmb_dp_world_size(const pmb_dp* dp) { return dp ? dp->nranks : 0; }

extern "C" pmb_status pmb_dp_allreduce_async(pmb_dp* dp, void* stream, float* d_buf, int64_t count) {
  if (!dp || !d_buf || count <= 0) return fail(PMB_ERR_ARG, "dp_allreduce_async: bad argument");
  if (dp->nranks == 1) return PMB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // everything enqueued on `stream` so far (the bucket's gradient kernels) precedes the all-reduce
  PMB_CUDA(cudaEventRecord(dp->ready, st));
  PMB_CUDA(cudaStreamWaitEvent(dp->comm_stream, dp->ready, 0));
  PMB_NCCL(g_nccl.AllReduce(d_buf, d_buf, (size_t)count, ncclFloat, ncclAvg, dp->comm, dp->comm_stream));
  return PMB_OK;
}

extern "C" pmb_status pmb_dp_allgather_async(pmb_dp* dp, void* stream, const void* d_send, void* d_recv, int64_t bytes) {
  if (!dp || !d_send || !d_recv || bytes <= 0) return fail(PMB_ERR_ARG, "dp_allgather_async: bad argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PMB_CUDA(cudaEventRecord(dp->ready, st));
  PMB_CUDA(cudaStreamWaitEvent(dp->comm_stream, dp->ready, 0));
  if (dp->nranks == 1) {
    PMB_CUDA(cudaMemcpyAsync(d_recv, d_send, (size_t)bytes, cudaMemcpyDeviceToDevice, dp->comm_stream));
    return PMB_OK;
  }
  PMB_NCCL(g_nccl.AllGather(d_send, d_recv, (size_t)bytes, ncclChar, dp->comm, dp->comm_stream));
  return PMB_OK;
}

extern "C" pmb_status pmb_dp_sync(pmb_dp* dp, void* stream) {
  if (!dp) return fail(PMB_ERR_ARG, "dp_sync: NULL handle");
  if (dp->nranks == 1) return PMB_OK;
  PMB_CUDA(cudaEventRecord(dp->done, dp->comm_stream));
  PMB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), dp->done, 0));
  if (g_nccl.CommGetAsyncError) {
    ncclResult_t async = ncclSuccess;
    PMB_NCCL(g_nccl.CommGetAsyncError(dp->comm, &async));
    if (async != ncclSuccess && async != ncclInProgress) return fail(PMB_ERR_CUDA, "NCCL reported an asynchronous error: %s", g_nccl.GetErrorString(async));
  }
  return PMB_OK;
}
