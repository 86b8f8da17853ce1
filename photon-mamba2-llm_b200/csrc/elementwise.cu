// HBM-bound kernels of the Mamba2 block: causal depthwise conv1d + bias + SiLU, dt softplus,
// gated RMSNorm, their backward passes, and small deterministic reductions.
#include "common.cuh"
#include "kernels.h"

namespace pmb {

__global__ void column_sum_kernel(const float* __restrict__ partial, int64_t rows, int cols, float* __restrict__ out);

// ---------------------------------------------------------------------------------------------
// conv1d (causal, depthwise) + bias + SiLU, forward.   u[t,c] = b[c] + sum_k w[c,k] * xbc[t-(K-1)+k, c]
// Layout stays (B,T,channels): a thread owns VEC adjacent channels and walks TT consecutive time steps
// with the K-1 previous inputs in registers, so every global access is a coalesced vector access and
// each input row is read (TT+K-1)/TT times.
// ---------------------------------------------------------------------------------------------
template <int K, int VEC, int TT>
// (eight CTAs per SM: the 1024 CTAs of a 2048-token launch are then resident at once instead of 1.15 waves)
__global__ void __launch_bounds__(128, 8) conv_silu_fwd_kernel(const float* __restrict__ xzd, int64_t ldx, int col0,
                                                            const float* __restrict__ w, const float* __restrict__ bias,
                                                            float* __restrict__ act, int X, int T, ConvPairOut po) {
  int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= X) return;
  int tblocks = (T + TT - 1) / TT;
  int b = blockIdx.y / tblocks;
  int t0 = (blockIdx.y % tblocks) * TT;
  int t1 = min(t0 + TT, T);
  float wr[VEC][K], br[VEC], win[VEC][K];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    br[v] = bias ? bias[c + v] : 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) wr[v][k] = w[(c + v) * K + k];
  }
  const float* src = xzd + (int64_t)b * T * ldx + col0 + c;
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    int t = t0 - (K - 1) + k;
    if (VEC == 4) {
      float4 q = t >= 0 ? *reinterpret_cast<const float4*>(src + (int64_t)t * ldx) : make_float4(0, 0, 0, 0);
      win[0][k] = q.x; win[1 % VEC][k] = q.y; win[2 % VEC][k] = q.z; win[3 % VEC][k] = q.w;
    } else {
      win[0][k] = t >= 0 ? src[(int64_t)t * ldx] : 0.0f;
    }
  }
  float* dst = act + (int64_t)b * T * X + c;
  // TT is a compile-time constant: all TT rows are requested before the first one is used
  float cur[TT][VEC];
#pragma unroll
  for (int i = 0; i < TT; ++i) {
    const int t = t0 + i;
    if (VEC == 4) {
      float4 q = t < t1 ? *reinterpret_cast<const float4*>(src + (int64_t)t * ldx) : make_float4(0, 0, 0, 0);
      cur[i][0] = q.x; cur[i][1 % VEC] = q.y; cur[i][2 % VEC] = q.z; cur[i][3 % VEC] = q.w;
    } else {
      cur[i][0] = t < t1 ? src[(int64_t)t * ldx] : 0.0f;
    }
  }
#pragma unroll
  for (int i = 0; i < TT; ++i) {
    const int t = t0 + i;
    float o[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      win[v][K - 1] = cur[i][v];
      float u = br[v];
#pragma unroll
      for (int k = 0; k < K; ++k) u = fmaf(wr[v][k], win[v][k], u);
      o[v] = u * sigmoid_acc(u);
#pragma unroll
      for (int k = 0; k < K - 1; ++k) win[v][k] = win[v][k + 1];
    }
    if (t < t1) {
      if (VEC == 4) {
        *reinterpret_cast<float4*>(dst + (int64_t)t * X) = make_float4(o[0], o[1 % VEC], o[2 % VEC], o[3 % VEC]);
        // the B | C columns also go out as a bf16 pair (operands of the fused scan kernels)
        if (po.hi && c >= po.col0) {
          const int64_t o16 = ((int64_t)b * T + t) * po.width + (c - po.col0);
          store_pair4(po.hi + o16, po.lo ? po.lo + o16 : nullptr, o[0], o[1 % VEC], o[2 % VEC], o[3 % VEC]);
        }
      }
      else dst[(int64_t)t * X] = o[0];
    }
  }
}

__global__ void dt_softplus_kernel(const float* __restrict__ xzd, int64_t ldx, int col0, const float* __restrict__ dt_bias,
                                   float* __restrict__ dt, int64_t rows, int H) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * H) return;
  int64_t r = i / H;
  int h = (int)(i % H);
  dt[i] = softplus_acc(xzd[r * ldx + col0 + h] + dt_bias[h]);
}

template <int K>
static pmb_status launch_conv_fwd_k(cudaStream_t st, const Dims& d, const float* xzd, const float* w, const float* b, float* act,
                                    ConvPairOut* pair) {
  // time steps per thread: short runs keep enough threads in flight for small token counts
  const bool long_runs = d.M >= 32768;
  const int TT = long_runs ? 16 : 8;
  bool vec = (d.X % 4 == 0) && (d.J % 4 == 0) && (d.I % 4 == 0) && ((reinterpret_cast<uintptr_t>(xzd) | reinterpret_cast<uintptr_t>(act)) % 16 == 0);
  int tblocks = (d.T + TT - 1) / TT;
  ConvPairOut po{};
  if (pair) {
    if (vec && pair->hi && ((reinterpret_cast<uintptr_t>(pair->hi) | reinterpret_cast<uintptr_t>(pair->lo)) % 8 == 0) && pair->width % 4 == 0) po = *pair;
    else pair->hi = nullptr;       // tells the caller that the pair was not written
  }
  if (vec) {
    dim3 grid((unsigned)cdiv(d.X / 4, 128), (unsigned)(d.B * tblocks));
    if (long_runs) conv_silu_fwd_kernel<K, 4, 16><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, act, d.X, d.T, po);
    else conv_silu_fwd_kernel<K, 4, 8><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, act, d.X, d.T, po);
  } else {
    dim3 grid((unsigned)cdiv(d.X, 128), (unsigned)(d.B * tblocks));
    if (long_runs) conv_silu_fwd_kernel<K, 1, 16><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, act, d.X, d.T, po);
    else conv_silu_fwd_kernel<K, 1, 8><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, act, d.X, d.T, po);
  }
  PMB_LAUNCHED();
  return PMB_OK;
}

pmb_status conv_silu_dt_fwd(cudaStream_t st, const Dims& d, const float* xzd, const float* w, const float* b,
                            const float* dt_bias, float* act, float* dt, ConvPairOut* pair) {
  ProfScope prof(st, "conv_silu_dt_fwd", 0.0, 4.0 * d.M * (2.0 * d.X + 2.0 * d.H));
  switch (d.K) {
    case 2: PMB_TRY(launch_conv_fwd_k<2>(st, d, xzd, w, b, act, pair)); break;
    case 3: PMB_TRY(launch_conv_fwd_k<3>(st, d, xzd, w, b, act, pair)); break;
    case 4: PMB_TRY(launch_conv_fwd_k<4>(st, d, xzd, w, b, act, pair)); break;
    case 5: PMB_TRY(launch_conv_fwd_k<5>(st, d, xzd, w, b, act, pair)); break;
    case 6: PMB_TRY(launch_conv_fwd_k<6>(st, d, xzd, w, b, act, pair)); break;
    case 7: PMB_TRY(launch_conv_fwd_k<7>(st, d, xzd, w, b, act, pair)); break;
    case 8: PMB_TRY(launch_conv_fwd_k<8>(st, d, xzd, w, b, act, pair)); break;
    default: return fail(PMB_ERR_SHAPE, "d_conv %d unsupported", d.K);
  }
  if (dt) {
    int64_t n = d.M * d.H;
    dt_softplus_kernel<<<(unsigned)cdiv(n, 256), 256, 0, st>>>(xzd, d.J, d.I + d.X, dt_bias, dt, d.M, d.H);
    PMB_LAUNCHED();
  }
  return PMB_OK;
}

// ---------------------------------------------------------------------------------------------
// conv backward.  du = dact * silu'(u) with u recomputed from the pre-conv window;
// dxbc[t',c] = sum_k w[c,k] du[t'+(K-1)-k, c];  dw[c,k] = sum_{b,t} du[t,c] xbc[t-(K-1)+k,c];  db = sum du.
// A thread owns one channel and TT time steps; per-(block-row) partial dw/db go to `partial`
// (rows = gridDim.y, K+1 values per channel) and are summed by column_sum_kernel (fixed order).
// ---------------------------------------------------------------------------------------------
// The work of one thread: channels [c, c + VEC) of batch b, time steps [t0, t1); writes its rows of the data gradient
// and leaves its share of the parameter gradients in dwacc / dbacc.
template <int K, int VEC, int TT>
__device__ __forceinline__ void conv_bwd_thread(const float* __restrict__ xzd, int64_t ldx, int col0, const float* __restrict__ w,
                                                const float* __restrict__ bias, const float* __restrict__ dact,
                                                float* __restrict__ dxzd, int X, int T, uint16_t* __restrict__ pair_hi,
                                                uint16_t* __restrict__ pair_lo, int c, int b, int t0, int t1,
                                                float (&dwacc)[VEC][K], float (&dbacc)[VEC]) {
  float wr[VEC][K], br[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    br[v] = bias ? bias[c + v] : 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) wr[v][k] = w[(c + v) * K + k];
  }
  const float* src = xzd + (int64_t)b * T * ldx + col0 + c;
  const float* dsrc = dact + (int64_t)b * T * X + c;
  float* ddst = dxzd + (int64_t)b * T * ldx + col0 + c;
  // xin holds xbc[t-(K-1) .. t]; dus holds du[t-(K-1) .. t] for the current t.
  float xin[VEC][K], dus[VEC][K];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    dbacc[v] = 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) { dwacc[v][k] = 0.0f; dus[v][k] = 0.0f; xin[v][k] = 0.0f; }
  }
  auto load = [&](const float* p, float (&o)[VEC]) {
    if (VEC == 4) { float4 q = *reinterpret_cast<const float4*>(p); o[0] = q.x; o[1 % VEC] = q.y; o[2 % VEC] = q.z; o[3 % VEC] = q.w; }
    else o[0] = *p;
  };
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    int t = t0 - (K - 1) + k;
    float o[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) o[v] = 0.0f;
    if (t >= 0) load(src + (int64_t)t * ldx, o);
#pragma unroll
    for (int v = 0; v < VEC; ++v) xin[v][k + 1] = o[v];
  }
  // Walk t from t0 to t1-1+(K-1): du[t] is needed by dxbc[t-(K-1) .. t]; du beyond the sequence end is 0.
  int tend = min(t1 + K - 1, T + K - 1);
  // all rows of the run are requested before the first one is used (TT is a compile-time constant)
  float xall[TT + K - 1][VEC], dall[TT + K - 1][VEC];
#pragma unroll
  for (int i = 0; i < TT + K - 1; ++i) {
    const int t = t0 + i;
#pragma unroll
    for (int v = 0; v < VEC; ++v) { xall[i][v] = 0.0f; dall[i][v] = 0.0f; }
    if (t < tend && t < T) { load(src + (int64_t)t * ldx, xall[i]); load(dsrc + (int64_t)t * X, dall[i]); }
  }
#pragma unroll
  for (int i = 0; i < TT + K - 1; ++i) {
    const int t = t0 + i;
    float xn[VEC], dn[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) { xn[v] = xall[i][v]; dn[v] = dall[i][v]; }
    float g[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
#pragma unroll
      for (int k = 0; k < K - 1; ++k) { xin[v][k] = xin[v][k + 1]; dus[v][k] = dus[v][k + 1]; }
      float du = 0.0f;
      if (t < T) {
        xin[v][K - 1] = xn[v];
        float u = br[v];
#pragma unroll
        for (int k = 0; k < K; ++k) u = fmaf(wr[v][k], xin[v][k], u);
        float s = sigmoid_acc(u);
        du = dn[v] * (s + u * s * (1.0f - s));
        if (t < t1) {  // this block owns the parameter-gradient contribution of t in [t0,t1)
          dbacc[v] += du;
#pragma unroll
          for (int k = 0; k < K; ++k) dwacc[v][k] = fmaf(du, xin[v][k], dwacc[v][k]);
        }
      }
      dus[v][K - 1] = du;
      float acc = 0.0f;   // dxbc[tp] = sum_k w[k] * du[tp + (K-1) - k] = sum_k w[k] * dus[K-1-k]
#pragma unroll
      for (int k = 0; k < K; ++k) acc = fmaf(wr[v][k], dus[v][K - 1 - k], acc);
      g[v] = acc;
    }
    int tp = t - (K - 1);
    if (t < tend && tp >= t0 && tp < t1) {
      const int64_t off = ((int64_t)b * T + tp) * ldx + col0 + c;
      if (pair_hi) {       // the gradient is only a GEMM operand: write it as a (hi, lo) bf16 pair with the same pitch
        if (VEC == 4) store_pair4(pair_hi + off, pair_lo ? pair_lo + off : nullptr, g[0], g[1 % VEC], g[2 % VEC], g[3 % VEC]);
        else { uint32_t h, l; split_bf16_pair(g[0], h, l); pair_hi[off] = (uint16_t)h; if (pair_lo) pair_lo[off] = (uint16_t)l; }
      } else if (VEC == 4) *reinterpret_cast<float4*>(ddst + (int64_t)tp * ldx) = make_float4(g[0], g[1 % VEC], g[2 % VEC], g[3 % VEC]);
      else ddst[(int64_t)tp * ldx] = g[0];
    }
  }
}

// partial = [gridDim.y rows of X*K weight partials][gridDim.y rows of X bias partials]
// One thread = one channel group and TT time steps, its own partial row (any shape, any alignment).
template <int K, int VEC, int TT>
__global__ void __launch_bounds__(128) conv_silu_bwd_kernel(const float* __restrict__ xzd, int64_t ldx, int col0,
                                                            const float* __restrict__ w, const float* __restrict__ bias,
                                                            const float* __restrict__ dact, float* __restrict__ dxzd,
                                                            float* __restrict__ partial, int X, int T,
                                                            uint16_t* __restrict__ pair_hi, uint16_t* __restrict__ pair_lo) {
  int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= X) return;
  int tblocks = (T + TT - 1) / TT;
  int b = blockIdx.y / tblocks;
  int t0 = (blockIdx.y % tblocks) * TT;
  int t1 = min(t0 + TT, T);
  float dwacc[VEC][K], dbacc[VEC];
  conv_bwd_thread<K, VEC, TT>(xzd, ldx, col0, w, bias, dact, dxzd, X, T, pair_hi, pair_lo, c, b, t0, t1, dwacc, dbacc);
  float* prow = partial + (int64_t)blockIdx.y * X * K;
  float* pbias = partial + (int64_t)gridDim.y * X * K + (int64_t)blockIdx.y * X;
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
#pragma unroll
    for (int k = 0; k < K; ++k) prow[(int64_t)(c + v) * K + k] = dwacc[v][k];
    pbias[c + v] = dbacc[v];
  }
}

// The same work with the parameter-gradient partials summed inside the CTA: 128 threads = 16 time slices x 8 channel
// quads (a 128-byte strip of every row), so a CTA covers 16 TT time steps of 32 channels and writes ONE partial row
// entry per channel instead of one per thread: 16 times fewer partial bytes than the kernel above, which at a few
// thousand tokens moved more partial sums than data.  Sums run in a fixed order (shuffles, then the warps in order).
// (The thread keeps TT + K - 1 rows of two tensors in registers, about 170 of them: small CTAs let three share an SM.)
constexpr int CONV_SLICES = 16;
constexpr int CONV_STRIP_THREADS = CONV_SLICES * 8;
template <int K, int TT>
__global__ void __launch_bounds__(CONV_STRIP_THREADS) conv_silu_bwd_strip_kernel(const float* __restrict__ xzd, int64_t ldx, int col0,
                                                                  const float* __restrict__ w, const float* __restrict__ bias,
                                                                  const float* __restrict__ dact, float* __restrict__ dxzd,
                                                                  float* __restrict__ partial, int X, int T,
                                                                  uint16_t* __restrict__ pair_hi, uint16_t* __restrict__ pair_lo) {
  constexpr int NV = 4 * K + 4, NW = CONV_STRIP_THREADS / 32;
  __shared__ float red[NW][8][NV];
  const int tx = threadIdx.x & 7, slice = threadIdx.x >> 3, warp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 8 + tx) * 4;
  const int tblocks = (T + CONV_SLICES * TT - 1) / (CONV_SLICES * TT);
  const int b = blockIdx.y / tblocks;
  const int t0 = (blockIdx.y % tblocks) * (CONV_SLICES * TT) + slice * TT;
  const int t1 = min(t0 + TT, T);
  float dwacc[4][K], dbacc[4];
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    dbacc[v] = 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) dwacc[v][k] = 0.0f;
  }
  if (c < X && t0 < T) conv_bwd_thread<K, 4, TT>(xzd, ldx, col0, w, bias, dact, dxzd, X, T, pair_hi, pair_lo, c, b, t0, t1, dwacc, dbacc);
  float vals[NV];
#pragma unroll
  for (int v = 0; v < 4; ++v) {
#pragma unroll
    for (int k = 0; k < K; ++k) vals[v * K + k] = dwacc[v][k];
    vals[4 * K + v] = dbacc[v];
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {          // the four time slices of a warp that share a channel quad
    vals[i] += __shfl_xor_sync(0xffffffffu, vals[i], 8);
    vals[i] += __shfl_xor_sync(0xffffffffu, vals[i], 16);
  }
  if ((threadIdx.x & 31) < 8) {
#pragma unroll
    for (int i = 0; i < NV; ++i) red[warp][tx][i] = vals[i];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 8 * NV; e += CONV_STRIP_THREADS) {
    const int q = e / NV, i = e % NV;
    const int cc = (blockIdx.x * 8 + q) * 4;
    if (cc < X) {
      float tot = 0.0f;
#pragma unroll
      for (int wv = 0; wv < NW; ++wv) tot += red[wv][q][i];
      if (i < 4 * K) partial[(int64_t)blockIdx.y * X * K + (int64_t)cc * K + i] = tot;      // (cc + v) * K + k with i = v * K + k
      else partial[(int64_t)gridDim.y * X * K + (int64_t)blockIdx.y * X + cc + (i - 4 * K)] = tot;
    }
  }
}

// time steps per thread: long runs recompute fewer halo rows (K - 1 per run) and write fewer partial sums; measured at
// 2048 tokens with the strip kernel: 4 steps 49 us, 8 steps 42 us, 16 steps 55 us per launch (PMB_CONV_TT overrides)
static int conv_bwd_tt(const Dims& d) {
  static const int forced = [] { const char* e = getenv("PMB_CONV_TT"); return e ? atoi(e) : 0; }();
  if (forced == 4 || forced == 8 || forced == 16) return forced;
  return d.M >= 32768 ? 16 : 8;
}

size_t conv_bwd_ws_bytes(const Dims& d) {
  const int CONV_BWD_TT = conv_bwd_tt(d);
  int tblocks = (d.T + CONV_BWD_TT - 1) / CONV_BWD_TT;
  return align_up((size_t)d.B * tblocks * d.X * (d.K + 1) * sizeof(float), 256);
}

// Rows of `partial` the launch below writes (what column_sum has to add up).
static int64_t conv_bwd_partial_rows(const Dims& d, bool strip) {
  const int tt = conv_bwd_tt(d);
  return (int64_t)d.B * (strip ? cdiv(d.T, CONV_SLICES * tt) : cdiv(d.T, tt));
}
static bool conv_bwd_strip_ok(const Dims& d, const float* xzd, const float* dact, const float* dxzd) {
  return (d.X % 4 == 0) && (d.J % 4 == 0) && (d.I % 4 == 0) && d.K <= 4 &&
         ((reinterpret_cast<uintptr_t>(xzd) | reinterpret_cast<uintptr_t>(dact) | reinterpret_cast<uintptr_t>(dxzd)) % 16 == 0);
}

template <int K>
static pmb_status launch_conv_bwd_k(cudaStream_t st, const Dims& d, const float* xzd, const float* w, const float* b,
                                    const float* dact, float* dxzd, float* partial, uint16_t* pair_hi, uint16_t* pair_lo) {
  const int tt = conv_bwd_tt(d);
  int tblocks = (d.T + tt - 1) / tt;
  bool vec = (d.X % 4 == 0) && (d.J % 4 == 0) && (d.I % 4 == 0) &&
             ((reinterpret_cast<uintptr_t>(xzd) | reinterpret_cast<uintptr_t>(dact) | reinterpret_cast<uintptr_t>(dxzd)) % 16 == 0);
  if (conv_bwd_strip_ok(d, xzd, dact, dxzd)) {
    if constexpr (K <= 4) {
      dim3 grid((unsigned)cdiv(d.X, 32), (unsigned)conv_bwd_partial_rows(d, true));
      if (tt == 16) conv_silu_bwd_strip_kernel<K, 16><<<grid, CONV_STRIP_THREADS, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
      else if (tt == 8) conv_silu_bwd_strip_kernel<K, 8><<<grid, CONV_STRIP_THREADS, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
      else conv_silu_bwd_strip_kernel<K, 4><<<grid, CONV_STRIP_THREADS, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
    }
  } else if (vec) {
    dim3 grid((unsigned)cdiv(d.X / 4, 128), (unsigned)(d.B * tblocks));
    if (tt == 16) conv_silu_bwd_kernel<K, 4, 16><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
    else if (tt == 8) conv_silu_bwd_kernel<K, 4, 8><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
    else conv_silu_bwd_kernel<K, 4, 4><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
  } else {
    dim3 grid((unsigned)cdiv(d.X, 128), (unsigned)(d.B * tblocks));
    if (tt == 16) conv_silu_bwd_kernel<K, 1, 16><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
    else if (tt == 8) conv_silu_bwd_kernel<K, 1, 8><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
    else conv_silu_bwd_kernel<K, 1, 4><<<grid, 128, 0, st>>>(xzd, d.J, d.I, w, b, dact, dxzd, partial, d.X, d.T, pair_hi, pair_lo);
  }
  PMB_LAUNCHED();
  return PMB_OK;
}

pmb_status conv_silu_bwd(cudaStream_t st, const Dims& d, const float* xzd, const float* w, const float* b,
                         const float* dact, float* dxzd, float* dw, float* db, void* ws, size_t ws_bytes, SideLane* red,
                         uint16_t* pair_hi, uint16_t* pair_lo) {
  if (ws_bytes < conv_bwd_ws_bytes(d)) return fail(PMB_ERR_WORKSPACE, "conv bwd workspace too small");
  float* partial = static_cast<float*>(ws);
  ProfScope prof(st, "conv_silu_bwd", 0.0, 4.0 * d.M * 3.0 * d.X);
  switch (d.K) {
    case 2: PMB_TRY(launch_conv_bwd_k<2>(st, d, xzd, w, b, dact, dxzd, partial, pair_hi, pair_lo)); break;
    case 3: PMB_TRY(launch_conv_bwd_k<3>(st, d, xzd, w, b, dact, dxzd, partial, pair_hi, pair_lo)); break;
    case 4: PMB_TRY(launch_conv_bwd_k<4>(st, d, xzd, w, b, dact, dxzd, partial, pair_hi, pair_lo)); break;
    case 5: PMB_TRY(launch_conv_bwd_k<5>(st, d, xzd, w, b, dact, dxzd, partial, pair_hi, pair_lo)); break;
    case 6: PMB_TRY(launch_conv_bwd_k<6>(st, d, xzd, w, b, dact, dxzd, partial, pair_hi, pair_lo)); break;
    case 7: PMB_TRY(launch_conv_bwd_k<7>(st, d, xzd, w, b, dact, dxzd, partial, pair_hi, pair_lo)); break;
    case 8: PMB_TRY(launch_conv_bwd_k<8>(st, d, xzd, w, b, dact, dxzd, partial, pair_hi, pair_lo)); break;
    default: return fail(PMB_ERR_SHAPE, "d_conv %d unsupported", d.K);
  }
  const int64_t rows = conv_bwd_partial_rows(d, conv_bwd_strip_ok(d, xzd, dact, dxzd));
  cudaStream_t rs = st;
  if (red) { PMB_TRY(order_after(st, red->ev[4], red->s)); rs = red->s; }
  column_sum_kernel<<<(unsigned)cdiv(d.X * d.K, 32), 256, 0, rs>>>(partial, rows, d.X * d.K, dw);
  PMB_LAUNCHED();
  column_sum_kernel<<<(unsigned)cdiv(d.X, 32), 256, 0, rs>>>(partial + rows * d.X * d.K, rows, d.X, db);
  PMB_LAUNCHED();
  return PMB_OK;
}

// ---------------------------------------------------------------------------------------------
// gated RMSNorm.  g = y * z * sigmoid(z); r = rsqrt(mean(g^2)+eps); out = g * r * w.
// One 256-thread block per row; the row stays in registers between the two passes.
// ---------------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_PER_THREAD = 8;   // width <= 2048 (registers hold a whole row)

__global__ void __launch_bounds__(NORM_THREADS) gated_rmsnorm_fwd_kernel(const float* __restrict__ y, const float* __restrict__ z,
                                                                         int64_t ldz, const float* __restrict__ w,
                                                                         float* __restrict__ out, float* __restrict__ rstd,
                                                                         int width, float eps, uint16_t* __restrict__ out_hi,
                                                                         uint16_t* __restrict__ out_lo) {
  __shared__ float red[32];
  int64_t row = blockIdx.x;
  const float* yr = y + row * width;
  const float* zr = z + row * ldz;
  float g[NORM_MAX_PER_THREAD];
  float ss = 0.0f;
#pragma unroll
  for (int n = 0; n < NORM_MAX_PER_THREAD; ++n) {
    int i = threadIdx.x + n * NORM_THREADS;
    if (i < width) {
      float zv = zr[i];
      float gv = yr[i] * zv * sigmoid_acc(zv);
      g[n] = gv;
      ss = fmaf(gv, gv, ss);
    }
  }
  float tot = block_sum(ss, red);
  float r = 1.0f / sqrtf(tot / (float)width + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int n = 0; n < NORM_MAX_PER_THREAD; ++n) {
    int i = threadIdx.x + n * NORM_THREADS;
    if (i < width) {
      float v = g[n] * r * w[i];
      if (out) out[row * width + i] = v;
      if (out_hi) {   // (hi, lo) bf16 pair of v for the pair GEMM: hi = bf16(v), lo = bf16(v - hi), round to nearest even
        uint32_t u = __float_as_uint(v);
        uint32_t h = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
        float rem = v - __uint_as_float(h << 16);
        uint32_t ul = __float_as_uint(rem);
        out_hi[row * width + i] = (uint16_t)h;
        if (out_lo) out_lo[row * width + i] = (uint16_t)((ul + 0x7fffu + ((ul >> 16) & 1u)) >> 16);
      }
    }
  }
}

// float4 variant: width % 4 == 0, 16-byte aligned rows.  PER float4 per thread, blockDim.x * PER >= width / 4.
template <int PER>
__global__ void __launch_bounds__(NORM_THREADS) gated_rmsnorm_fwd_vec_kernel(const float* __restrict__ y, const float* __restrict__ z,
                                                                             int64_t ldz, const float* __restrict__ w,
                                                                             float* __restrict__ out, float* __restrict__ rstd,
                                                                             int width, float eps, uint16_t* __restrict__ out_hi,
                                                                             uint16_t* __restrict__ out_lo) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int nvec = width >> 2;
  const float4* y4 = reinterpret_cast<const float4*>(y + row * width);
  const float4* z4 = reinterpret_cast<const float4*>(z + row * ldz);
  float4 g[PER];
  float ss = 0.0f;
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = threadIdx.x + n * blockDim.x;
    g[n] = make_float4(0, 0, 0, 0);
    if (i < nvec) {
      const float4 yv = y4[i], zv = z4[i];
      g[n] = make_float4(yv.x * zv.x * sigmoid_acc(zv.x), yv.y * zv.y * sigmoid_acc(zv.y), yv.z * zv.z * sigmoid_acc(zv.z),
                         yv.w * zv.w * sigmoid_acc(zv.w));
      ss = fmaf(g[n].x, g[n].x, fmaf(g[n].y, g[n].y, fmaf(g[n].z, g[n].z, fmaf(g[n].w, g[n].w, ss))));
    }
  }
  const float tot = block_sum(ss, red);
  const float r = 1.0f / sqrtf(tot / (float)width + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  auto split = [](float v, uint32_t& h, uint32_t& l) {   // (hi, lo) bf16 pair, round to nearest even
    const uint32_t u = __float_as_uint(v);
    h = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
    const uint32_t ul = __float_as_uint(v - __uint_as_float(h << 16));
    l = (ul + 0x7fffu + ((ul >> 16) & 1u)) >> 16;
  };
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = threadIdx.x + n * blockDim.x;
    if (i < nvec) {
      const float4 wv = reinterpret_cast<const float4*>(w)[i];
      const float4 v = make_float4(g[n].x * r * wv.x, g[n].y * r * wv.y, g[n].z * r * wv.z, g[n].w * r * wv.w);
      if (out) reinterpret_cast<float4*>(out + row * width)[i] = v;
      if (out_hi) {
        uint32_t h[4], l[4];
        split(v.x, h[0], l[0]); split(v.y, h[1], l[1]); split(v.z, h[2], l[2]); split(v.w, h[3], l[3]);
        reinterpret_cast<uint2*>(out_hi + row * width)[i] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
        if (out_lo) reinterpret_cast<uint2*>(out_lo + row * width)[i] = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
      }
    }
  }
}

// threads per block for the float4 kernels: every thread owns exactly `per` float4 when width/4 divides evenly
static inline int norm_vec_threads(int width, int* per) {
  const int nvec = width / 4;
  *per = (nvec + NORM_THREADS - 1) / NORM_THREADS;
  int t = (nvec + *per - 1) / *per;
  return ((t + 31) / 32) * 32;
}
static inline bool norm_vec_ok(int width, int64_t ldz, const void* a, const void* b, const void* c, const void* d2 = nullptr, const void* e2 = nullptr) {
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return (width % 4 == 0) && (ldz % 4 == 0) && width / 4 <= 2 * NORM_THREADS && al(a) && al(b) && al(c) && al(d2) && al(e2);
}

pmb_status gated_rmsnorm_fwd(cudaStream_t st, int64_t rows, int width, float eps, const float* y, const float* z, int64_t ldz,
                             const float* w, float* out, float* rstd, uint16_t* out_hi, uint16_t* out_lo) {
  if (width > NORM_THREADS * NORM_MAX_PER_THREAD) return fail(PMB_ERR_SHAPE, "rmsnorm width %d > %d", width, NORM_THREADS * NORM_MAX_PER_THREAD);
  ProfScope prof(st, "gated_rmsnorm_fwd", 0.0, 4.0 * rows * 3.0 * width);
  if (norm_vec_ok(width, ldz, y, z, w, out, out_hi) && (!out_lo || (reinterpret_cast<uintptr_t>(out_lo) & 15) == 0)) {
    int per = 1;
    const int threads = norm_vec_threads(width, &per);
    if (per == 1) gated_rmsnorm_fwd_vec_kernel<1><<<(unsigned)rows, threads, 0, st>>>(y, z, ldz, w, out, rstd, width, eps, out_hi, out_lo);
    else gated_rmsnorm_fwd_vec_kernel<2><<<(unsigned)rows, threads, 0, st>>>(y, z, ldz, w, out, rstd, width, eps, out_hi, out_lo);
    PMB_LAUNCHED();
    return PMB_OK;
  }
  gated_rmsnorm_fwd_kernel<<<(unsigned)rows, NORM_THREADS, 0, st>>>(y, z, ldz, w, out, rstd, width, eps, out_hi, out_lo);
  PMB_LAUNCHED();
  return PMB_OK;
}

// Backward.  dg = w r dout - g r^3 (sum_j dout_j g_j w_j)/I;  dy = dg z sig(z);
// dz = dg y (sig + z sig (1-sig));  dw_i = sum_rows dout_i g_i r.
// A block handles NORM_ROWS consecutive rows so the dw partial stays in registers across them.
constexpr int NORM_ROWS = 4;

__global__ void __launch_bounds__(NORM_THREADS) gated_rmsnorm_bwd_kernel(const float* __restrict__ dout, const float* __restrict__ y,
                                                                         const float* __restrict__ z, int64_t ldz,
                                                                         const float* __restrict__ w, const float* __restrict__ rstd,
                                                                         float* __restrict__ dy, float* __restrict__ dz, int64_t lddz,
                                                                         float* __restrict__ dw_partial, int64_t rows, int width) {
  __shared__ float red[32];
  float dwacc[NORM_MAX_PER_THREAD];
#pragma unroll
  for (int n = 0; n < NORM_MAX_PER_THREAD; ++n) dwacc[n] = 0.0f;
  int64_t r0 = (int64_t)blockIdx.x * NORM_ROWS;
  for (int rr = 0; rr < NORM_ROWS; ++rr) {
    int64_t row = r0 + rr;
    if (row >= rows) break;  // uniform across the block
    float r = rstd[row];
    // pass 1: load the row once, keep it in registers
    float zv[NORM_MAX_PER_THREAD], yv[NORM_MAX_PER_THREAD], dn[NORM_MAX_PER_THREAD];
    float dot = 0.0f;
#pragma unroll
    for (int n = 0; n < NORM_MAX_PER_THREAD; ++n) {
      int i = threadIdx.x + n * NORM_THREADS;
      if (i < width) {
        zv[n] = z[row * ldz + i]; yv[n] = y[row * width + i]; dn[n] = dout[row * width + i];
        float gv = yv[n] * zv[n] * sigmoid_acc(zv[n]);
        dot = fmaf(dn[n] * gv, w[i], dot);
      }
    }
    float tot = block_sum(dot, red);
    float coef = r * r * r * tot / (float)width;
#pragma unroll
    for (int n = 0; n < NORM_MAX_PER_THREAD; ++n) {
      int i = threadIdx.x + n * NORM_THREADS;
      if (i < width) {
        float s = sigmoid_acc(zv[n]);
        float gv = yv[n] * zv[n] * s;
        float dg = w[i] * r * dn[n] - gv * coef;
        dwacc[n] = fmaf(dn[n] * gv, r, dwacc[n]);
        dy[row * width + i] = dg * zv[n] * s;
        dz[row * lddz + i] = dg * yv[n] * (s + zv[n] * s * (1.0f - s));
      }
    }
  }
#pragma unroll
  for (int n = 0; n < NORM_MAX_PER_THREAD; ++n) {
    int i = threadIdx.x + n * NORM_THREADS;
    if (i < width) dw_partial[(int64_t)blockIdx.x * width + i] = dwacc[n];
  }
}

// float4 variant of the backward (same row blocking and partial layout).  Optional extras (see NormBwdExtra):
// dz as a (hi, lo) bf16 pair instead of fp32, and dY exp(S) for the scan backward.
template <int PER>
__global__ void __launch_bounds__(NORM_THREADS, 3) gated_rmsnorm_bwd_vec_kernel(const float* __restrict__ dout, const float* __restrict__ y,
                                                                             const float* __restrict__ z, int64_t ldz,
                                                                             const float* __restrict__ w, const float* __restrict__ rstd,
                                                                             float* __restrict__ dy, float* __restrict__ dz, int64_t lddz,
                                                                             float* __restrict__ dw_partial, int64_t rows, int width,
                                                                             NormBwdExtra ex) {
  __shared__ float red[32];
  const int nvec = width >> 2;
  float4 dwacc[PER], wv[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = threadIdx.x + n * blockDim.x;
    dwacc[n] = make_float4(0, 0, 0, 0);
    wv[n] = i < nvec ? reinterpret_cast<const float4*>(w)[i] : make_float4(0, 0, 0, 0);
  }
  const int64_t r0 = (int64_t)blockIdx.x * NORM_ROWS;
  for (int rr = 0; rr < NORM_ROWS; ++rr) {
    const int64_t row = r0 + rr;
    if (row >= rows) break;  // uniform across the block
    const float r = rstd[row];
    float4 zv[PER], yv[PER], dn[PER], gv[PER], sv[PER];
    float dot = 0.0f;
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = threadIdx.x + n * blockDim.x;
      zv[n] = yv[n] = dn[n] = gv[n] = sv[n] = make_float4(0, 0, 0, 0);
      if (i < nvec) {
        zv[n] = reinterpret_cast<const float4*>(z + row * ldz)[i];
        yv[n] = reinterpret_cast<const float4*>(y + row * width)[i];
        dn[n] = reinterpret_cast<const float4*>(dout + row * width)[i];
      }
    }
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      sv[n] = make_float4(sigmoid_acc(zv[n].x), sigmoid_acc(zv[n].y), sigmoid_acc(zv[n].z), sigmoid_acc(zv[n].w));
      gv[n] = make_float4(yv[n].x * zv[n].x * sv[n].x, yv[n].y * zv[n].y * sv[n].y, yv[n].z * zv[n].z * sv[n].z, yv[n].w * zv[n].w * sv[n].w);
      dot = fmaf(dn[n].x * gv[n].x, wv[n].x, fmaf(dn[n].y * gv[n].y, wv[n].y, fmaf(dn[n].z * gv[n].z, wv[n].z, fmaf(dn[n].w * gv[n].w, wv[n].w, dot))));
    }
    const float tot = block_sum(dot, red);
    const float coef = r * r * r * tot / (float)width;
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = threadIdx.x + n * blockDim.x;
      if (i < nvec) {
        float4 dg, o_dy, o_dz;
#define PMB_NORM_LANE(c)                                                        \
        dg.c = wv[n].c * r * dn[n].c - gv[n].c * coef;                           \
        dwacc[n].c = fmaf(dn[n].c * gv[n].c, r, dwacc[n].c);                     \
        o_dy.c = dg.c * zv[n].c * sv[n].c;                                       \
        o_dz.c = dg.c * yv[n].c * (sv[n].c + zv[n].c * sv[n].c * (1.0f - sv[n].c));
        PMB_NORM_LANE(x) PMB_NORM_LANE(y) PMB_NORM_LANE(z) PMB_NORM_LANE(w)
#undef PMB_NORM_LANE
        reinterpret_cast<float4*>(dy + row * width)[i] = o_dy;
        if (ex.dz_hi) store_pair4(ex.dz_hi + row * lddz + 4 * i, ex.dz_lo ? ex.dz_lo + row * lddz + 4 * i : nullptr, o_dz.x, o_dz.y, o_dz.z, o_dz.w);
        else reinterpret_cast<float4*>(dz + row * lddz)[i] = o_dz;
        if (ex.dy_hi) store_pair4(ex.dy_hi + row * width + 4 * i, ex.dy_lo ? ex.dy_lo + row * width + 4 * i : nullptr, o_dy.x, o_dy.y, o_dy.z, o_dy.w);
        if (ex.dys_hi) {   // the same, as a bf16 pair (operand of the pair contractions of the scan backward)
          const int h = (4 * i) / ex.P;
          const int64_t bb = row / ex.T, tt = row % ex.T;
          const float f = __expf(ex.S[(bb * ex.H + h) * ex.T + tt]);
          store_pair4(ex.dys_hi + row * width + 4 * i, ex.dys_lo ? ex.dys_lo + row * width + 4 * i : nullptr, o_dy.x * f, o_dy.y * f, o_dy.z * f, o_dy.w * f);
        }
        if (ex.dys) {    // dys[t, h, :] = dy[t, h, :] * exp(S[b, h, t]) for the scan backward (head width ex.P is a multiple of 4)
          const int h = (4 * i) / ex.P;
          const int64_t bb = row / ex.T, tt = row % ex.T;
          const float f = __expf(ex.S[(bb * ex.H + h) * ex.T + tt]);
          reinterpret_cast<float4*>(ex.dys + row * width)[i] = make_float4(o_dy.x * f, o_dy.y * f, o_dy.z * f, o_dy.w * f);
        }
      }
    }
  }
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = threadIdx.x + n * blockDim.x;
    if (i < nvec) reinterpret_cast<float4*>(dw_partial + (int64_t)blockIdx.x * width)[i] = dwacc[n];
  }
}

// out[j] = sum_r partial[r*cols + j].  Block = 32 columns x 8 row lanes; each lane sums rows ty, ty+8, ...
// and the 8 lane sums are added in a fixed order (deterministic).
__global__ void __launch_bounds__(256) column_sum_kernel(const float* __restrict__ partial, int64_t rows, int cols, float* __restrict__ out) {
  __shared__ float sh[8][33];
  int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  int j = blockIdx.x * 32 + tx;
  float s = 0.0f;
  if (j < cols)
    for (int64_t r = ty; r < rows; r += 8) s += partial[r * cols + j];
  sh[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < cols) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sh[k][tx];
    out[j] = t;
  }
}

size_t gated_rmsnorm_bwd_ws_bytes(int64_t rows, int width) {
  return align_up((size_t)cdiv(rows, NORM_ROWS) * width * sizeof(float), 256);
}

pmb_status gated_rmsnorm_bwd(cudaStream_t st, int64_t rows, int width, const float* dout, const float* y, const float* z, int64_t ldz,
                             const float* w, const float* rstd, float* dy, float* dz, int64_t lddz, float* dw, void* ws, size_t ws_bytes,
                             SideLane* red, const NormBwdExtra* extra) {
  NormBwdExtra ex{};
  if (extra) ex = *extra;
  if (width > NORM_THREADS * NORM_MAX_PER_THREAD) return fail(PMB_ERR_SHAPE, "rmsnorm width %d too large", width);
  if (ws_bytes < gated_rmsnorm_bwd_ws_bytes(rows, width)) return fail(PMB_ERR_WORKSPACE, "rmsnorm bwd workspace too small");
  float* partial = static_cast<float*>(ws);
  int64_t nblk = cdiv(rows, NORM_ROWS);
  ProfScope prof(st, "gated_rmsnorm_bwd", 0.0, 4.0 * rows * 5.0 * width);
  const bool vec_ok = norm_vec_ok(width, ldz, dout, y, z, w, dy) && (lddz % 4 == 0) &&
                      ((reinterpret_cast<uintptr_t>(dz) | reinterpret_cast<uintptr_t>(partial)) & 15) == 0;
  if ((ex.dz_hi || ex.dys || ex.dy_hi || ex.dys_hi) && !vec_ok) return fail(PMB_ERR_UNSUPPORTED, "gated_rmsnorm_bwd: pair / scaled outputs need the vector kernel's alignment");
  if (vec_ok) {
    int per = 1;
    const int threads = norm_vec_threads(width, &per);
    if (per == 1) gated_rmsnorm_bwd_vec_kernel<1><<<(unsigned)nblk, threads, 0, st>>>(dout, y, z, ldz, w, rstd, dy, dz, lddz, partial, rows, width, ex);
    else gated_rmsnorm_bwd_vec_kernel<2><<<(unsigned)nblk, threads, 0, st>>>(dout, y, z, ldz, w, rstd, dy, dz, lddz, partial, rows, width, ex);
  } else {
    gated_rmsnorm_bwd_kernel<<<(unsigned)nblk, NORM_THREADS, 0, st>>>(dout, y, z, ldz, w, rstd, dy, dz, lddz, partial, rows, width);
  }
  PMB_LAUNCHED();
  cudaStream_t rs = st;
  if (red) { PMB_TRY(order_after(st, red->ev[4], red->s)); rs = red->s; }
  column_sum_kernel<<<(unsigned)cdiv(width, 32), 256, 0, rs>>>(partial, nblk, width, dw);
  PMB_LAUNCHED();
  return PMB_OK;
}

// ---------------------------------------------------------------------------------------------
// Gated RMSNorm backward for callers that cannot allocate device memory.
//
// Some hosts may not call cudaMalloc at the point where they need this kernel: a trainer that handed the
// whole device to its own pool at start-up and has nothing left to carve a workspace from, or a
// latency-bound serving loop that must stay out of the driver's allocator.  For them the per-row-block
// weight-gradient partials live in the array below, which is part of the library image: every GPU that
// loads the library holds these 4 MiB until the process exits.
//
// In host code `g_static_scratch` names a host-side shadow of the symbol, not device memory; the device
// address is looked up once per device with cudaGetSymbolAddress (with that device current) and cached.
// That lookup happens on the first call on a device, so make that first call outside any stream capture.
// Nothing has to be zeroed between calls: each call overwrites the rows of the array it later reads.
// All calls share the one array, so two calls whose kernels may overlap on the GPU (different streams
// without an ordering between them) race on it; serialise them.
// ---------------------------------------------------------------------------------------------
constexpr size_t STATIC_SCRATCH_BYTES = 4u << 20;
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_BYTES / sizeof(float)];
constexpr int STATIC_SCRATCH_MAX_DEVICES = 64;
static float* g_static_scratch_addr[STATIC_SCRATCH_MAX_DEVICES] = {nullptr};

static pmb_status static_scratch_for_current_device(float** out) {
  int dev = -1;
  PMB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= STATIC_SCRATCH_MAX_DEVICES) return fail(PMB_ERR_UNSUPPORTED, "device ordinal %d is outside 0..%d", dev, STATIC_SCRATCH_MAX_DEVICES - 1);
  if (!g_static_scratch_addr[dev]) {
    void* p = nullptr;
    PMB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    g_static_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_static_scratch_addr[dev];
  return PMB_OK;
}

pmb_status gated_rmsnorm_bwd_static(cudaStream_t st, int64_t rows, int width, const float* dout, const float* y, const float* z,
                                    int64_t ldz, const float* w, const float* rstd, float* dy, float* dz, int64_t lddz, float* dw) {
  size_t need = gated_rmsnorm_bwd_ws_bytes(rows, width);
  if (need > STATIC_SCRATCH_BYTES)
    return fail(PMB_ERR_SHAPE, "gated_rmsnorm_bwd_static: rows=%lld x width=%d needs %zu bytes of scratch, the built-in array holds %zu "
                "(ceil(rows/%d) * width * 4 must not exceed it); use pmb_gated_rmsnorm_bwd with a caller workspace",
                (long long)rows, width, need, STATIC_SCRATCH_BYTES, NORM_ROWS);
  float* scratch = nullptr;
  PMB_TRY(static_scratch_for_current_device(&scratch));
  return gated_rmsnorm_bwd(st, rows, width, dout, y, z, ldz, w, rstd, dy, dz, lddz, dw, scratch, STATIC_SCRATCH_BYTES);
}

pmb_status column_sum(cudaStream_t st, const float* partial, int64_t rows, int cols, float* out) {
  column_sum_kernel<<<(unsigned)cdiv(cols, 32), 256, 0, st>>>(partial, rows, cols, out);
  PMB_LAUNCHED();
  return PMB_OK;
}

}  // namespace pmb

extern "C" size_t pmb_gated_rmsnorm_bwd_static_max_bytes(void) { return pmb::STATIC_SCRATCH_BYTES; }

extern "C" pmb_status pmb_gated_rmsnorm_bwd_static(void* stream, int64_t rows, int32_t width,
                                                   const float* d_dout, const float* d_y, const float* d_z, int64_t ldz,
                                                   const float* d_w, const float* d_rstd,
                                                   float* d_dy, float* d_dz, int64_t lddz, float* d_dw) {
  using namespace pmb;
  if (rows <= 0 || width <= 0 || ldz < width || lddz < width) return fail(PMB_ERR_SHAPE, "gated_rmsnorm_bwd_static: bad shape");
  if (!d_dout || !d_y || !d_z || !d_w || !d_rstd || !d_dy || !d_dz || !d_dw) return fail(PMB_ERR_ARG, "gated_rmsnorm_bwd_static: NULL argument");
  return gated_rmsnorm_bwd_static(static_cast<cudaStream_t>(stream), rows, width, d_dout, d_y, d_z, ldz, d_w, d_rstd, d_dy, d_dz, lddz, d_dw);
}
