// One-token recurrent decode (Mamba2Block::step, crates/pm-core/src/mamba2/block.rs:278-417):
// rolling conv window + h <- exp(A dt) h + dt (B (x) x), y = C h + D x, gate, norm, out_proj.
// The SSM update is HBM-bound: the (B,H,N,P) fp32 state is read and written once per token.
#include "common.cuh"
#include "kernels.h"

namespace pmb {

// conv window (B,X,K-1) fp32: oldest column first (state.rs:31-51).
__global__ void conv_step_kernel(const float* __restrict__ xzd, int J, int col0, const float* __restrict__ w,
                                 const float* __restrict__ bias, float* __restrict__ window, float* __restrict__ act,
                                 int B, int X, int K) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * X) return;
  int b = i / X, c = i % X;
  float* win = window + (int64_t)i * (K - 1);
  float xn = xzd[(int64_t)b * J + col0 + c];
  float u = bias ? bias[c] : 0.0f;
  for (int k = 0; k < K - 1; ++k) {
    float v = win[k];
    u = fmaf(w[c * K + k], v, u);
    if (k > 0) win[k - 1] = v;
  }
  u = fmaf(w[c * K + K - 1], xn, u);
  win[K - 2] = xn;
  act[i] = u * sigmoid_acc(u);
}

// One block per (b,h); thread = (p, n-slice).  state layout (B,H,N,P).
constexpr int STEP_THREADS = 256;
__global__ void __launch_bounds__(STEP_THREADS) ssm_step_kernel(const float* __restrict__ act, int X, int I, int G,
                                                                const float* __restrict__ xzd, int J,
                                                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                                const float* __restrict__ Dskip, float* __restrict__ state,
                                                                float* __restrict__ y, int H, int N, int P) {
  extern __shared__ float sh[];  // N (B vector) + N (C vector) + nslices*P partial outputs
  int bh = blockIdx.x, h = bh % H, b = bh / H;
  int g = h / (H / G);
  float* Bs = sh; float* Cs = sh + N; float* part = sh + 2 * N;
  const float* arow = act + (int64_t)b * X;
  for (int n = threadIdx.x; n < N; n += STEP_THREADS) {
    Bs[n] = arow[I + g * N + n];
    Cs[n] = arow[I + G * N + g * N + n];
  }
  __syncthreads();
  float dt = softplus_acc(xzd[(int64_t)b * J + I + X + h] + dt_bias[h]);
  float decay = expf(-expf(a_log[h]) * dt);
  int pw = P < STEP_THREADS ? P : STEP_THREADS;  // threads along p
  int nsl = STEP_THREADS / pw;                   // n-slices
  int p0 = threadIdx.x % pw, sl = threadIdx.x / pw;
  float* st = state + (int64_t)bh * N * P;
  for (int p = p0; p < P; p += pw) {
    float xv = arow[h * P + p];
    float acc = 0.0f;
    if (sl < nsl) {
      for (int n = sl; n < N; n += nsl) {
        float hv = fmaf(decay, st[(int64_t)n * P + p], dt * Bs[n] * xv);
        st[(int64_t)n * P + p] = hv;
        acc = fmaf(Cs[n], hv, acc);
      }
      part[sl * P + p] = acc;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += STEP_THREADS) {
    float s = 0.0f;
    for (int k = 0; k < nsl; ++k) s += part[k * P + p];
    y[(int64_t)b * I + h * P + p] = fmaf(Dskip[h], arow[h * P + p], s);
  }
}

// Vectorised variant (P % 4 == 0): a thread owns 4 adjacent p and every (256 / (P/4))-th state row, so each state
// row is read and written with 16-byte accesses; the B/C vectors and dt live in shared memory / registers.
__global__ void __launch_bounds__(STEP_THREADS) ssm_step_vec4_kernel(const float* __restrict__ act, int X, int I, int G,
                                                                     const float* __restrict__ xzd, int J,
                                                                     const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                                     const float* __restrict__ Dskip, float* __restrict__ state,
                                                                     float* __restrict__ y, int H, int N, int P) {
  extern __shared__ float sh[];  // N (B) + N (C) + nsl * P partial outputs
  int bh = blockIdx.x, h = bh % H, b = bh / H;
  int g = h / (H / G);
  float* Bs = sh; float* Cs = sh + N; float* part = sh + 2 * N;
  const float* arow = act + (int64_t)b * X;
  for (int n = threadIdx.x; n < N; n += STEP_THREADS) {
    Bs[n] = arow[I + g * N + n];
    Cs[n] = arow[I + G * N + g * N + n];
  }
  __syncthreads();
  const float dt = softplus_acc(xzd[(int64_t)b * J + I + X + h] + dt_bias[h]);
  const float decay = expf(-expf(a_log[h]) * dt);
  const int pw = P / 4;                    // threads along p
  const int nsl = STEP_THREADS / pw;       // state rows in flight
  const int p4 = threadIdx.x % pw, sl = threadIdx.x / pw;
  float4* st = reinterpret_cast<float4*>(state + (int64_t)bh * N * P);
  if (sl < nsl) {
    const float4 xv = *reinterpret_cast<const float4*>(arow + h * P + 4 * p4);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int n = sl; n < N; n += nsl) {
      float4 hv = st[(int64_t)n * pw + p4];
      const float bx = dt * Bs[n], cn = Cs[n];
      hv.x = fmaf(decay, hv.x, bx * xv.x); hv.y = fmaf(decay, hv.y, bx * xv.y);
      hv.z = fmaf(decay, hv.z, bx * xv.z); hv.w = fmaf(decay, hv.w, bx * xv.w);
      st[(int64_t)n * pw + p4] = hv;
      acc.x = fmaf(cn, hv.x, acc.x); acc.y = fmaf(cn, hv.y, acc.y); acc.z = fmaf(cn, hv.z, acc.z); acc.w = fmaf(cn, hv.w, acc.w);
    }
    *reinterpret_cast<float4*>(part + sl * P + 4 * p4) = acc;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += STEP_THREADS) {
    float s = 0.0f;
    for (int k = 0; k < nsl; ++k) s += part[k * P + p];
    y[(int64_t)b * I + h * P + p] = fmaf(Dskip[h], arow[h * P + p], s);
  }
}

}  // namespace pmb

using namespace pmb;

struct StepWs { float *xzd, *act, *y, *normed, *rstd; };

static size_t step_ws_layout(const Dims& d, void* base, size_t bytes, StepWs* out) {
  Arena ar(base, bytes);
  StepWs w;
  w.xzd = ar.take<float>((size_t)d.B * d.J);
  w.act = ar.take<float>((size_t)d.B * d.X);
  w.y = ar.take<float>((size_t)d.B * d.I);
  w.normed = ar.take<float>((size_t)d.B * d.I);
  w.rstd = ar.take<float>((size_t)d.B);
  if (out) *out = w;
  return ar.ok ? ar.used() : 0;
}

extern "C" size_t pmb_mamba2_step_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch) {
  Dims d;
  if (make_dims(cfg, batch, 1, &d) != PMB_OK) return 0;
  return step_ws_layout(d, nullptr, 0, nullptr);
}

extern "C" pmb_status pmb_mamba2_step(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* p,
                                      int32_t batch, const float* d_x_t, float* d_ssm_state, float* d_conv_window,
                                      float* d_y_t, void* d_ws, size_t ws_bytes) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, 1, &d));
  if (!p || !d_x_t || !d_ssm_state || !d_conv_window || !d_y_t || !d_ws) return fail(PMB_ERR_ARG, "mamba2_step: NULL argument");
  StepWs w;
  if (step_ws_layout(d, d_ws, ws_bytes, &w) == 0) return fail(PMB_ERR_WORKSPACE, "mamba2_step: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PMB_TRY(gemm(st, 0, 0, d.B, d.J, d.D, d_x_t, d.D, p->in_proj_weight, d.J, w.xzd, d.J, nullptr, 0));
  { ProfScope prof(st, "decode_conv_step", 0.0, 4.0 * d.B * d.X * (2.0 * d.K));
  conv_step_kernel<<<(unsigned)cdiv((int64_t)d.B * d.X, 256), 256, 0, st>>>(w.xzd, d.J, d.I, p->conv1d_weight, p->conv1d_bias,
                                                                            d_conv_window, w.act, d.B, d.X, d.K);
  PMB_LAUNCHED(); }
  const bool vec4 = (d.P % 4 == 0) && (d.P / 4 <= STEP_THREADS) && (STEP_THREADS % (d.P / 4) == 0) && (d.X % 4 == 0) &&
                    (reinterpret_cast<uintptr_t>(d_ssm_state) % 16 == 0);
  int pw = vec4 ? d.P / 4 : (d.P < STEP_THREADS ? d.P : STEP_THREADS);
  size_t shm = (size_t)(2 * d.N + (STEP_THREADS / pw) * d.P) * sizeof(float);
  if (shm > 48 * 1024) return fail(PMB_ERR_SHAPE, "mamba2_step: d_state/d_head too large for the step kernel");
  { ProfScope prof(st, "decode_ssm_step", 0.0, 8.0 * d.B * d.H * d.N * d.P);
  if (vec4) ssm_step_vec4_kernel<<<(unsigned)(d.B * d.H), STEP_THREADS, shm, st>>>(w.act, d.X, d.I, d.G, w.xzd, d.J, p->dt_bias, p->a_log, p->d_skip,
                                                                             d_ssm_state, w.y, d.H, d.N, d.P);
  else ssm_step_kernel<<<(unsigned)(d.B * d.H), STEP_THREADS, shm, st>>>(w.act, d.X, d.I, d.G, w.xzd, d.J, p->dt_bias, p->a_log, p->d_skip,
                                                                   d_ssm_state, w.y, d.H, d.N, d.P);
  PMB_LAUNCHED(); }
  PMB_TRY(gated_rmsnorm_fwd(st, d.B, d.I, d.eps, w.y, w.xzd, d.J, p->norm_weight, w.normed, w.rstd));
  PMB_TRY(gemm(st, 0, 0, d.B, d.D, d.I, w.normed, d.I, p->out_proj_weight, d.D, d_y_t, d.D, nullptr, 0));
  return PMB_OK;
}
