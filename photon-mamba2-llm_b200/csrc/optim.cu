// Fused global-norm gradient clipping + AdamW over a flat fp32 parameter buffer.
// Mirrors crates/pm-train/src/clip.rs:13-53 (global L2 norm, scale by max_norm / norm when above it) and
// crates/pm-train/src/optim.rs:104-157 (decoupled weight decay applied to the parameter first, then the moment
// updates, bias corrections as 1/(1-beta^t) factors, update = m_hat / (sqrt(v_hat) + eps)).
// The reference spends ~12 Ops calls and two assigns per parameter tensor and one host sync for the norm; here the
// norm stays on the device (two-pass, fixed order) and one kernel updates every parameter.
#include "common.cuh"
#include "kernels.h"

namespace pmb {

constexpr int SUMSQ_BLOCKS = 1024;

__global__ void __launch_bounds__(256) sumsq_partial_kernel(const float* __restrict__ g, int64_t n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) s = fmaf(g[i], g[i], s);
  float tot = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = tot;
}

__global__ void __launch_bounds__(256) sumsq_final_kernel(const float* __restrict__ partial, int nblocks, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.0f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) s += partial[i];
  float tot = block_sum(s, red);
  if (threadIdx.x == 0) *out = tot;
}

__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, int64_t n,
                             float lr, float beta1, float beta2, float eps, float wd, float inv_bc1, float inv_bc2,
                             float max_norm, const float* __restrict__ sumsq) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float scale = 1.0f;
  if (max_norm > 0.0f && sumsq) {
    float norm = sqrtf(*sumsq);
    if (norm > max_norm && norm > 0.0f) scale = max_norm / norm;
  }
  float gi = g[i] * scale;
  float pi = p[i];
  if (wd > 0.0f) pi *= (1.0f - lr * wd);
  float mi = beta1 * m[i] + (1.0f - beta1) * gi;
  float vi = beta2 * v[i] + (1.0f - beta2) * (gi * gi);
  m[i] = mi; v[i] = vi;
  float update = (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
  p[i] = pi - lr * update;
}

}  // namespace pmb

using namespace pmb;

extern "C" size_t pmb_grad_sumsq_workspace_bytes(void) { return SUMSQ_BLOCKS * sizeof(float); }

extern "C" pmb_status pmb_grad_sumsq(void* stream, int64_t n, const float* d_grads, float* d_sumsq_out, void* d_ws, size_t ws_bytes) {
  if (n <= 0 || !d_grads || !d_sumsq_out || !d_ws) return fail(PMB_ERR_ARG, "grad_sumsq: bad argument");
  if (ws_bytes < SUMSQ_BLOCKS * sizeof(float)) return fail(PMB_ERR_WORKSPACE, "grad_sumsq: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int blocks = (int)(cdiv(n, 256) < SUMSQ_BLOCKS ? cdiv(n, 256) : SUMSQ_BLOCKS);
  ProfScope prof(st, "grad_sumsq", 0.0, 4.0 * n);
  sumsq_partial_kernel<<<blocks, 256, 0, st>>>(d_grads, n, static_cast<float*>(d_ws));
  PMB_LAUNCHED();
  sumsq_final_kernel<<<1, 256, 0, st>>>(static_cast<float*>(d_ws), blocks, d_sumsq_out);
  PMB_LAUNCHED();
  return PMB_OK;
}

extern "C" pmb_status pmb_adamw_step(void* stream, int64_t n, float* d_params, const float* d_grads, float* d_m, float* d_v,
                                     float lr, float beta1, float beta2, float eps, float weight_decay, int32_t step,
                                     float max_norm, const float* d_sumsq) {
  if (n <= 0 || !d_params || !d_grads || !d_m || !d_v || step <= 0) return fail(PMB_ERR_ARG, "adamw_step: bad argument");
  if (max_norm > 0.0f && !d_sumsq) return fail(PMB_ERR_ARG, "adamw_step: clipping needs the squared gradient norm (pmb_grad_sumsq)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float bc1 = 1.0f - powf(beta1, (float)step), bc2 = 1.0f - powf(beta2, (float)step);
  ProfScope prof(st, "adamw_step", 0.0, 28.0 * n);
  adamw_kernel<<<(unsigned)cdiv(n, 256), 256, 0, st>>>(d_params, d_grads, d_m, d_v, n, lr, beta1, beta2, eps, weight_decay,
                                                        1.0f / bc1, 1.0f / bc2, max_norm, d_sumsq);
  PMB_LAUNCHED();
  return PMB_OK;
}
