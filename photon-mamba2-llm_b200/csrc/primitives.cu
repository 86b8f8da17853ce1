// Primitive ops of pm_core::Ops that the fused block path does not absorb (crates/pm-core/src/ops.rs:54-352):
// elementwise arithmetic and activations, strided copies (narrow / transpose / broadcast_as / concat are views over
// one copy kernel), embedding, gather, log-softmax, full reductions and cumulative sums.  An adaptor falls back to
// these for any op sequence it does not recognise as the block; they are correctness plumbing (plain HBM-bound
// kernels, fp32), not the measured hot path, and they run on the device like everything else: there is no CPU path.
#include "common.cuh"
#include "kernels.h"

namespace pmb {

__device__ __forceinline__ float apply_unary(int op, float x, float s) {
  switch (op) {
    case PMB_OP_NEG: return -x;
    case PMB_OP_EXP: return expf(x);
    case PMB_OP_SQRT: return sqrtf(x);
    case PMB_OP_SILU: return x * sigmoid_acc(x);
    case PMB_OP_SIGMOID: return sigmoid_acc(x);
    case PMB_OP_SOFTPLUS: return softplus_acc(x);
    case PMB_OP_MUL_SCALAR: return x * s;
    case PMB_OP_ADD_SCALAR: return x + s;
    default: return x;    // PMB_OP_COPY
  }
}
__device__ __forceinline__ float apply_binary(int op, float a, float b) {
  switch (op) {
    case PMB_OP_ADD: return a + b;
    case PMB_OP_SUB: return a - b;
    case PMB_OP_MUL: return a * b;
    default: return a / b;   // PMB_OP_DIV
  }
}

__global__ void unary_kernel(int op, const float* __restrict__ x, float s, float* __restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = apply_unary(op, x[i], s);
}
__global__ void binary_kernel(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = apply_binary(op, a[i], b[i]);
}

// out (contiguous, `shape`) [i] = src[offset + sum_d idx_d * stride_d]; a stride of 0 broadcasts, permuted strides
// transpose, an offset with shortened extents narrows.
struct StridedView { int64_t shape[PMB_MAX_RANK]; int64_t stride[PMB_MAX_RANK]; int rank; int64_t offset; };
__global__ void strided_copy_kernel(const float* __restrict__ src, StridedView v, float* __restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, at = v.offset;
    for (int d = v.rank - 1; d >= 0; --d) { at += (rem % v.shape[d]) * v.stride[d]; rem /= v.shape[d]; }
    out[i] = src[at];
  }
}

__global__ void gather_rows_kernel(const float* __restrict__ table, const int64_t* __restrict__ ids, float* __restrict__ out,
                                   int64_t rows, int64_t width, int64_t vocab, unsigned int* __restrict__ bad) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * width; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / width, c = i % width;
    const int64_t id = ids[r];
    if (id < 0 || id >= vocab) { if (c == 0) atomicOr(bad, 1u); out[i] = 0.0f; }
    else out[i] = table[id * width + c];
  }
}

// out[r] = x[r, idx[r]] (gather along the last axis with one index per row: the cross-entropy pick, pm-train/src/loss.rs:39-69)
__global__ void gather_last_kernel(const float* __restrict__ x, const int64_t* __restrict__ idx, float* __restrict__ out,
                                   int64_t rows, int64_t width, unsigned int* __restrict__ bad) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int64_t j = idx[r];
  if (j < 0 || j >= width) { atomicOr(bad, 1u); out[r] = 0.0f; }
  else out[r] = x[r * width + j];
}

// one block per row: out = x - logsumexp(x) over the last axis
__global__ void __launch_bounds__(256) log_softmax_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t width) {
  __shared__ float red[32];
  __shared__ float bc;
  const float* row = x + (int64_t)blockIdx.x * width;
  float* orow = out + (int64_t)blockIdx.x * width;
  float m = -INFINITY;
  for (int64_t i = threadIdx.x; i < width; i += blockDim.x) m = fmaxf(m, row[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) { float v = red[0]; for (int i = 1; i < (int)(blockDim.x >> 5); ++i) v = fmaxf(v, red[i]); bc = v; }
  __syncthreads();
  m = bc;
  float s = 0.0f;
  for (int64_t i = threadIdx.x; i < width; i += blockDim.x) s += expf(row[i] - m);
  const float lse = m + logf(block_sum(s, red));
  for (int64_t i = threadIdx.x; i < width; i += blockDim.x) orow[i] = row[i] - lse;
}

// two fixed-order passes: per-block partial sums, then one block over the partials
__global__ void __launch_bounds__(256) sum_partial_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ part) {
  __shared__ float red[32];
  float s = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) s += x[i];
  const float t = block_sum(s, red);
  if (threadIdx.x == 0) part[blockIdx.x] = t;
}
__global__ void __launch_bounds__(256) sum_final_kernel(const float* __restrict__ part, int nparts, float scale, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.0f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += part[i];
  const float t = block_sum(s, red);
  if (threadIdx.x == 0) *out = t * scale;
}

// inclusive cumulative sum along an axis of length `len` with `inner` contiguous elements below it: one thread per
// (outer, inner) pair walks the axis (Ops::cumsum serves the scan's short chunk axis, ssd_ops.rs:101-110)
__global__ void cumsum_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t outer, int64_t len, int64_t inner) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= outer * inner) return;
  const int64_t o = i / inner, j = i % inner;
  const float* p = x + o * len * inner + j;
  float* q = out + o * len * inner + j;
  float run = 0.0f;
  for (int64_t k = 0; k < len; ++k) { run += p[k * inner]; q[k * inner] = run; }
}

static unsigned grid_for(int64_t n) { int64_t b = cdiv(n, 256); return (unsigned)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b)); }

}  // namespace pmb

using namespace pmb;

extern "C" pmb_status pmb_unary_f32(void* stream, int32_t op, const float* d_x, float scalar, float* d_out, int64_t n) {
  if (!d_x || !d_out || n <= 0) return fail(PMB_ERR_ARG, "unary: bad argument");
  if (op < PMB_OP_COPY || op > PMB_OP_ADD_SCALAR) return fail(PMB_ERR_UNSUPPORTED, "unary: unknown op %d", op);
  unary_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(op, d_x, scalar, d_out, n);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" pmb_status pmb_binary_f32(void* stream, int32_t op, const float* d_a, const float* d_b, float* d_out, int64_t n) {
  if (!d_a || !d_b || !d_out || n <= 0) return fail(PMB_ERR_ARG, "binary: bad argument");
  if (op < PMB_OP_ADD || op > PMB_OP_DIV) return fail(PMB_ERR_UNSUPPORTED, "binary: unknown op %d", op);
  binary_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(op, d_a, d_b, d_out, n);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" pmb_status pmb_strided_copy_f32(void* stream, const float* d_src, int32_t rank, const int64_t* h_shape,
                                           const int64_t* h_strides, int64_t offset, float* d_out) {
  if (!d_src || !d_out || !h_shape || !h_strides || rank < 1 || rank > PMB_MAX_RANK) return fail(PMB_ERR_ARG, "strided_copy: bad argument (rank 1..%d)", PMB_MAX_RANK);
  StridedView v{};
  v.rank = rank; v.offset = offset;
  int64_t n = 1;
  for (int d = 0; d < rank; ++d) {
    if (h_shape[d] <= 0 || h_strides[d] < 0) return fail(PMB_ERR_SHAPE, "strided_copy: extents must be positive and strides non-negative");
    v.shape[d] = h_shape[d]; v.stride[d] = h_strides[d]; n *= h_shape[d];
  }
  strided_copy_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_src, v, d_out, n);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" pmb_status pmb_embedding_f32(void* stream, const float* d_table, int64_t vocab, int64_t width, const int64_t* d_ids,
                                        int64_t rows, float* d_out, uint32_t* d_bad_flag) {
  if (!d_table || !d_ids || !d_out || !d_bad_flag || vocab <= 0 || width <= 0 || rows <= 0) return fail(PMB_ERR_ARG, "embedding: bad argument");
  gather_rows_kernel<<<grid_for(rows * width), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_table, d_ids, d_out, rows, width, vocab, d_bad_flag);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" pmb_status pmb_gather_last_f32(void* stream, const float* d_x, const int64_t* d_index, int64_t rows, int64_t width,
                                          float* d_out, uint32_t* d_bad_flag) {
  if (!d_x || !d_index || !d_out || !d_bad_flag || rows <= 0 || width <= 0) return fail(PMB_ERR_ARG, "gather: bad argument");
  gather_last_kernel<<<(unsigned)cdiv(rows, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_index, d_out, rows, width, d_bad_flag);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" pmb_status pmb_log_softmax_f32(void* stream, const float* d_x, int64_t rows, int64_t width, float* d_out) {
  if (!d_x || !d_out || rows <= 0 || width <= 0 || rows > 0x7fffffff) return fail(PMB_ERR_ARG, "log_softmax: bad argument");
  log_softmax_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_out, width);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" size_t pmb_sum_workspace_bytes(void) { return 1024 * sizeof(float); }

extern "C" pmb_status pmb_sum_all_f32(void* stream, const float* d_x, int64_t n, int32_t mean, float* d_out, void* d_ws, size_t ws_bytes) {
  if (!d_x || !d_out || !d_ws || n <= 0) return fail(PMB_ERR_ARG, "sum_all: bad argument");
  if (ws_bytes < pmb_sum_workspace_bytes()) return fail(PMB_ERR_WORKSPACE, "sum_all: workspace too small");
  int64_t blocks = cdiv(n, 256 * 8);
  const int nparts = (int)(blocks > 1024 ? 1024 : blocks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  sum_partial_kernel<<<(unsigned)nparts, 256, 0, st>>>(d_x, n, static_cast<float*>(d_ws));
  PMB_LAUNCHED();
  sum_final_kernel<<<1, 256, 0, st>>>(static_cast<const float*>(d_ws), nparts, mean ? 1.0f / (float)n : 1.0f, d_out);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" pmb_status pmb_cumsum_f32(void* stream, const float* d_x, int64_t outer, int64_t len, int64_t inner, float* d_out) {
  if (!d_x || !d_out || outer <= 0 || len <= 0 || inner <= 0) return fail(PMB_ERR_ARG, "cumsum: bad argument");
  cumsum_kernel<<<(unsigned)cdiv(outer * inner, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_out, outer, len, inner);
  PMB_LAUNCHED();
  return PMB_OK;
}
