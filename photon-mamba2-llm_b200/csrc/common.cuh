// Shared host/device helpers for the pm_b200 library.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>
#include "../../include/pm_b200.h"

namespace pmb {

extern thread_local char g_err[512];
extern std::atomic<long long> g_launches;

inline pmb_status fail(pmb_status st, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return st;
}

#define PMB_CUDA(expr)                                                                         \
  do {                                                                                         \
    cudaError_t e__ = (expr);                                                                  \
    if (e__ != cudaSuccess)                                                                    \
      return pmb::fail(PMB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),  \
                       __FILE__, __LINE__);                                                    \
  } while (0)

#define PMB_TRY(expr)                   \
  do {                                  \
    pmb_status s__ = (expr);            \
    if (s__ != PMB_OK) return s__;      \
  } while (0)

// Call after every kernel launch: counts it and surfaces launch-configuration errors.
#define PMB_LAUNCHED()                                                                          \
  do {                                                                                          \
    pmb::g_launches.fetch_add(1, std::memory_order_relaxed);                                    \
    cudaError_t e__ = cudaGetLastError();                                                       \
    if (e__ != cudaSuccess)                                                                     \
      return pmb::fail(PMB_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(e__), \
                       __FILE__, __LINE__);                                                     \
  } while (0)

// ---- optional per-kernel timing (off by default; pmb_profile_start/stop) -------------------------
// A scope records one CUDA event before and one after the launches it brackets, on the launching
// stream; pmb_profile_stop() synchronises and aggregates elapsed time, algorithmic FLOPs and bytes by name.
struct ProfRec { const char* name; double flops, bytes; cudaEvent_t e0, e1; };
extern bool g_prof_on;
extern std::vector<ProfRec> g_prof;
struct ProfScope {
  cudaStream_t st; ProfRec r; bool on;
  ProfScope(cudaStream_t s, const char* name, double flops, double bytes) : st(s), on(g_prof_on) {
    if (!on) return;
    r.name = name; r.flops = flops; r.bytes = bytes;
    cudaEventCreate(&r.e0); cudaEventCreate(&r.e1);
    cudaEventRecord(r.e0, st);
  }
  ~ProfScope() {
    if (!on) return;
    cudaEventRecord(r.e1, st);
    g_prof.push_back(r);
  }
};

// "Done once per device" flags.  Function attributes such as the opt-in dynamic shared-memory size belong to
// the (kernel, device) pair, so a process that drives several GPUs has to set them on each; the table is indexed
// by device ordinal like the library's other per-device state.  claim() returns true exactly once per ordinal
// (always true for ordinals outside the table, which costs a repeated call but never skips one).
constexpr int PMB_MAX_DEVICES = 64;
struct DeviceOnce {
  bool done[PMB_MAX_DEVICES] = {};
  bool pending(int dev) const { return dev < 0 || dev >= PMB_MAX_DEVICES || !done[dev]; }
  void mark(int dev) { if (dev >= 0 && dev < PMB_MAX_DEVICES) done[dev] = true; }
};
// Sets the dynamic shared-memory limit of `kernel` (given last, so template arguments with commas are fine)
// the first time the calling site runs on the current device.
#define PMB_SMEM_OPT_IN(bytes, ...)                                                                              \
  do {                                                                                                           \
    static pmb::DeviceOnce once__;                                                                               \
    int dev__ = 0;                                                                                               \
    PMB_CUDA(cudaGetDevice(&dev__));                                                                             \
    if (once__.pending(dev__)) {                                                                                 \
      PMB_CUDA(cudaFuncSetAttribute(__VA_ARGS__, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes)));    \
      once__.mark(dev__);                                                                                        \
    }                                                                                                            \
  } while (0)

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Bump allocator over a caller-provided workspace.
struct Arena {
  char* base;
  size_t size;
  size_t off = 0;
  bool ok = true;
  Arena(void* p, size_t n) : base(static_cast<char*>(p)), size(n) {}
  template <class T>
  T* take(size_t count) {
    off = align_up(off, 256);
    size_t bytes = count * sizeof(T);
    if (base != nullptr && off + bytes > size) ok = false;
    T* r = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += bytes;
    return r;
  }
  size_t used() const { return align_up(off, 256); }
};

struct Dims {
  int B, T, D, N, P, H, G, K, Q, I, X, J, nc;
  int64_t M;  // tokens
  float eps;
};

inline pmb_status make_dims(const pmb_mamba2_config* c, int batch, int seqlen, Dims* d) {
  if (!c) return fail(PMB_ERR_ARG, "config is NULL");
  if (c->d_model <= 0 || c->d_state <= 0 || c->d_head <= 0 || c->n_heads <= 0 || batch <= 0 || seqlen <= 0)
    return fail(PMB_ERR_SHAPE, "non-positive dimension in config/batch/seqlen");
  if (!(c->n_groups == 1 || c->n_groups == c->n_heads))
    return fail(PMB_ERR_SHAPE, "n_groups must be 1 or n_heads (got %d, H=%d)", c->n_groups, c->n_heads);
  if (c->d_conv < 2 || c->d_conv > 8) return fail(PMB_ERR_SHAPE, "d_conv must be in 2..8 (got %d)", c->d_conv);
  d->B = batch; d->T = seqlen; d->D = c->d_model; d->N = c->d_state; d->P = c->d_head; d->H = c->n_heads;
  d->G = c->n_groups; d->K = c->d_conv;
  // The reference routes block_len == 0, >= T or not dividing T to its dense path (ssd_ops.rs:70-78):
  // one chunk spanning the whole sequence computes the same quantity.
  int q = c->block_len;
  if (q <= 0 || q >= seqlen || seqlen % q != 0) q = seqlen;
  d->Q = q;
  d->nc = seqlen / q;
  d->I = d->H * d->P;
  d->X = d->I + 2 * d->G * d->N;
  d->J = d->I + d->X + d->H;
  d->M = (int64_t)batch * seqlen;
  d->eps = c->rmsnorm_eps;
  return PMB_OK;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_acc(float x) { return 1.0f / (1.0f + expf(-x)); }
// softplus in the reference's stable form max(x,0)+log(1+exp(-|x|)) (pm-candle ops_impl.rs:123-133)
__device__ __forceinline__ float softplus_acc(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum for blockDim.x <= 1024 (multiple of 32); `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) red[0] = r;
  __syncthreads();
  return red[0];
}

// (hi, lo) bf16 pair of an fp32 value: hi = bf16(v), lo = bf16(v - hi), both rounded to nearest even.
__device__ __forceinline__ void split_bf16_pair(float v, uint32_t& h, uint32_t& l) {
  const uint32_t u = __float_as_uint(v);
  h = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
  const uint32_t ul = __float_as_uint(v - __uint_as_float(h << 16));
  l = (ul + 0x7fffu + ((ul >> 16) & 1u)) >> 16;
}
// four consecutive values to the pair arrays (8-byte aligned destinations); lo == NULL: plain bf16 rounding into hi.
// Callers that index into the arrays pass `lo ? lo + offset : nullptr`, never an offset added to a null pointer.
__device__ __forceinline__ void store_pair4(uint16_t* hi, uint16_t* lo, float a, float b, float c, float d) {
  uint32_t h[4], l[4];
  split_bf16_pair(a, h[0], l[0]); split_bf16_pair(b, h[1], l[1]); split_bf16_pair(c, h[2], l[2]); split_bf16_pair(d, h[3], l[3]);
  *reinterpret_cast<uint2*>(hi) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
  if (lo) *reinterpret_cast<uint2*>(lo) = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
}

}  // namespace pmb
