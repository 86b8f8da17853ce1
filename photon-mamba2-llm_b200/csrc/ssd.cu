// Chunked SSD scan (forward and fused-recompute backward) as a set of batched tile contractions.
//
// Per (batch b, chunk c, head h), with S = inclusive cumsum of a inside the chunk, L[t,s] = exp(S_t - S_s) (s <= t),
// x~ = x * dt:
//   forward   CB = C B^T                                   (per group)
//             states = sum_q exp(S_end - S_q) B_q (x) x~_q  -> exclusive scan over chunks -> h_prev
//             Y = (CB o L) x~ + diag(exp S) C h_prev (+ D x)
//   backward  dh_prev = sum_t exp(S_t) C_t (x) dY_t + exp(S_end) dh   (reverse scan over chunks)
//             dx~ = (CB o L)^T dY + exp(S_end - S_s) B_s dh
//             dG = sum_heads L o (dY x~^T);  dC = dG B + sum_h exp(S_t) dY_t h_prev^T;
//             dB = dG^T C + sum_h exp(S_end - S_s) x~_s dh^T
//             dS_t = <dY_t, Y_t> - <x~_t, dx~_t>, dS_{Q-1} += <dh, h_next>;  da = reverse cumsum(dS)
// The reference computes the same quantities with ~40 primitive ops and autograd
// (crates/pm-core/src/mamba2/ssd_ops.rs:167-284); nothing of size (Q,Q) per head is stored here.
//
// This file holds the SIMT (fp32 FMA) engine: one 64x64-tile kernel template, specialised by small functor
// structs that say how to read operand elements and where results go.
#include <cstdlib>
#include <cuda_bf16.h>
#include "common.cuh"
#include "kernels.h"
#include "bgemm.cuh"
#include "ssd_tc.h"
#include "ssd_fused.h"

namespace pmb {

struct SsdP {
  int B, T, H, P, N, G, Q, nc, hpg;
  const float* x; int64_t ldx;
  const float* dt; const float* A; const float* a;
  const float* b; const float* c; int64_t ldbc;
  const float* D;
  float* S; float* hprev; float* hlast; float* CB; float* dh; float* dG; float* dxt;
  const float* y; int64_t ldy;
  const float* dy; int64_t lddy;
  float* yout; int64_t ldyo;
  float* db; float* dc; int64_t lddbc;

  __device__ __forceinline__ int64_t tok(int bb, int cc, int q) const { return (int64_t)bb * T + (int64_t)cc * Q + q; }
  __device__ __forceinline__ float Sv(int bb, int h, int cc, int q) const { return S[((int64_t)bb * H + h) * T + (int64_t)cc * Q + q]; }
  __device__ __forceinline__ float dtv(int64_t tk, int h) const { return dt ? dt[tk * H + h] : 1.0f; }
};

// ---- F1: CB[t,s] = sum_n C[t,n] B[s,n], per (b,c,g) --------------------------------------------
struct OpCB {
  static constexpr bool SEG_SCALE = false;
  SsdP p; int Mdim, Ndim;
  int bb, cc, g; const float* cp; const float* bp; float* out;
  __device__ bool init(int batch, int m0, int n0) {
    if (n0 > m0 + BM - 1) return false;  // strictly above the diagonal: never read
    g = batch % p.G; int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    cp = p.c + p.tok(bb, cc, 0) * p.ldbc + g * p.N;
    bp = p.b + p.tok(bb, cc, 0) * p.ldbc + g * p.N;
    out = p.CB + (int64_t)batch * p.Q * p.Q;
    return true;
  }
  __device__ int nseg() const { return 1; }
  __device__ void krange(int, int, int, int& k0, int& k1) const { k0 = 0; k1 = p.N; }
  __device__ bool a_kcontig(int) const { return true; }
  __device__ bool b_kcontig(int) const { return true; }
  __device__ float a(int, int m, int k) const { return cp[(int64_t)m * p.ldbc + k]; }
  __device__ float b(int, int k, int n) const { return bp[(int64_t)n * p.ldbc + k]; }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ bool seg_active(int) const { return true; }
  __device__ void store(int m, int n, float v) const { out[(int64_t)m * p.Q + n] = v; }
};

// Common context for per-(b,c,h) ops.
struct HeadCtx {
  int bb, cc, h, g; int64_t t0;  // first token of the chunk
  __device__ void set(const SsdP& p, int batch) {
    h = batch % p.H; int bc = batch / p.H; cc = bc % p.nc; bb = bc / p.nc; g = h / p.hpg;
    t0 = p.tok(bb, cc, 0);
  }
};

// ---- F2: states[n,p] = sum_q B[q,n] exp(S_end - S_q) x~[q,p], per (b,c,h) -----------------------
struct OpState {
  static constexpr bool SEG_SCALE = false;
  SsdP p; int Mdim, Ndim;
  HeadCtx cx; float send; const float* sp; float* out;
  __device__ bool init(int batch, int, int) {
    cx.set(p, batch);
    sp = p.S + ((int64_t)cx.bb * p.H + cx.h) * p.T + (int64_t)cx.cc * p.Q;
    send = sp[p.Q - 1];
    out = p.hprev + (int64_t)batch * p.N * p.P;
    return true;
  }
  __device__ int nseg() const { return 1; }
  __device__ void krange(int, int, int, int& k0, int& k1) const { k0 = 0; k1 = p.Q; }
  __device__ bool a_kcontig(int) const { return false; }
  __device__ bool b_kcontig(int) const { return false; }
  __device__ float a(int, int m, int k) const {
    int64_t tk = cx.t0 + k;
    return p.b[tk * p.ldbc + cx.g * p.N + m] * expf(send - sp[k]) * p.dtv(tk, cx.h);
  }
  __device__ float b(int, int k, int n) const { return p.x[(cx.t0 + k) * p.ldx + cx.h * p.P + n]; }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ bool seg_active(int) const { return true; }
  __device__ void store(int m, int n, float v) const { out[(int64_t)m * p.P + n] = v; }
};

// ---- F4: Y[t,p] = sum_{s<=t} CB[t,s] L[t,s] x~[s,p] + exp(S_t) sum_n C[t,n] h_prev[n,p] (+ D x) --
struct OpScan {
  static constexpr bool SEG_SCALE = false;
  SsdP p; int Mdim, Ndim;
  HeadCtx cx; const float* sp; const float* cb; const float* hp;
  __device__ bool init(int batch, int, int) {
    cx.set(p, batch);
    sp = p.S + ((int64_t)cx.bb * p.H + cx.h) * p.T + (int64_t)cx.cc * p.Q;
    cb = p.CB + (((int64_t)cx.bb * p.nc + cx.cc) * p.G + cx.g) * p.Q * p.Q;
    hp = p.hprev + (int64_t)batch * p.N * p.P;
    return true;
  }
  __device__ int nseg() const { return 2; }
  __device__ void krange(int seg, int m0, int, int& k0, int& k1) const {
    k0 = 0; k1 = seg == 0 ? min(p.Q, m0 + BM) : p.N;
  }
  __device__ bool a_kcontig(int) const { return true; }
  __device__ bool b_kcontig(int) const { return false; }
  __device__ float a(int seg, int m, int k) const {
    if (seg == 0) {
      if (k > m) return 0.0f;
      return cb[(int64_t)m * p.Q + k] * expf(sp[m] - sp[k]) * p.dtv(cx.t0 + k, cx.h);
    }
    return p.c[(cx.t0 + m) * p.ldbc + cx.g * p.N + k] * expf(sp[m]);
  }
  __device__ float b(int seg, int k, int n) const {
    if (seg == 0) return p.x[(cx.t0 + k) * p.ldx + cx.h * p.P + n];
    return hp[(int64_t)k * p.P + n];
  }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ bool seg_active(int) const { return true; }
  __device__ void store(int m, int n, float v) const {
    if (p.D) v = fmaf(p.D[cx.h], p.x[(cx.t0 + m) * p.ldx + cx.h * p.P + n], v);
    p.yout[(cx.t0 + m) * p.ldyo + cx.h * p.P + n] = v;
  }
};

// ---- B1: contrib[n,p] = sum_t C[t,n] exp(S_t) dY[t,p], per (b,c,h) ------------------------------
struct OpDstate {
  static constexpr bool SEG_SCALE = false;
  SsdP p; int Mdim, Ndim;
  HeadCtx cx; const float* sp; float* out;
  __device__ bool init(int batch, int, int) {
    cx.set(p, batch);
    sp = p.S + ((int64_t)cx.bb * p.H + cx.h) * p.T + (int64_t)cx.cc * p.Q;
    out = p.dh + (int64_t)batch * p.N * p.P;
    return true;
  }
  __device__ int nseg() const { return 1; }
  __device__ void krange(int, int, int, int& k0, int& k1) const { k0 = 0; k1 = p.Q; }
  __device__ bool a_kcontig(int) const { return false; }
  __device__ bool b_kcontig(int) const { return false; }
  __device__ float a(int, int m, int k) const { return p.c[(cx.t0 + k) * p.ldbc + cx.g * p.N + m] * expf(sp[k]); }
  __device__ float b(int, int k, int n) const { return p.dy[(cx.t0 + k) * p.lddy + cx.h * p.P + n]; }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ bool seg_active(int) const { return true; }
  __device__ void store(int m, int n, float v) const { out[(int64_t)m * p.P + n] = v; }
};

// ---- B3: dx~[s,p] = sum_{t>=s} CB[t,s] L[t,s] dY[t,p] + exp(S_end - S_s) sum_n B[s,n] dh[n,p] ----
struct OpDx {
  static constexpr bool SEG_SCALE = false;
  SsdP p; int Mdim, Ndim;
  HeadCtx cx; const float* sp; const float* cb; const float* dhp; float send;
  __device__ bool init(int batch, int, int) {
    cx.set(p, batch);
    sp = p.S + ((int64_t)cx.bb * p.H + cx.h) * p.T + (int64_t)cx.cc * p.Q;
    send = sp[p.Q - 1];
    cb = p.CB + (((int64_t)cx.bb * p.nc + cx.cc) * p.G + cx.g) * p.Q * p.Q;
    dhp = p.dh + (int64_t)batch * p.N * p.P;
    return true;
  }
  __device__ int nseg() const { return 2; }
  __device__ void krange(int seg, int m0, int, int& k0, int& k1) const {
    if (seg == 0) { k0 = m0; k1 = p.Q; } else { k0 = 0; k1 = p.N; }
  }
  __device__ bool a_kcontig(int seg) const { return seg != 0; }
  __device__ bool b_kcontig(int) const { return false; }
  __device__ float a(int seg, int m, int k) const {
    if (seg == 0) {
      if (k < m) return 0.0f;
      return cb[(int64_t)k * p.Q + m] * expf(sp[k] - sp[m]);
    }
    return p.b[(cx.t0 + m) * p.ldbc + cx.g * p.N + k] * expf(send - sp[m]);
  }
  __device__ float b(int seg, int k, int n) const {
    if (seg == 0) return p.dy[(cx.t0 + k) * p.lddy + cx.h * p.P + n];
    return dhp[(int64_t)k * p.P + n];
  }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ bool seg_active(int) const { return true; }
  __device__ void store(int m, int n, float v) const { p.dxt[(cx.t0 + m) * (int64_t)(p.H * p.P) + cx.h * p.P + n] = v; }
};

// ---- B5: dG[t,s] = sum_{h in group} L_h[t,s] sum_p dY_h[t,p] x~_h[s,p], per (b,c,g) --------------
struct OpDG {
  static constexpr bool SEG_SCALE = true;
  SsdP p; int Mdim, Ndim;
  int nsplit; float* part;      // split-K over heads: partial tiles go to `part`, summed by splitk_reduce_kernel
  int bb, cc, g, split; int64_t t0; float* out;
  __device__ bool init(int batch, int m0, int n0) {
    if (n0 > m0 + BM - 1) return false;
    split = batch % nsplit; batch /= nsplit;
    g = batch % p.G; int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    t0 = p.tok(bb, cc, 0);
    out = nsplit > 1 ? part + (int64_t)blockIdx.z * p.Q * p.Q : p.dG + (int64_t)batch * p.Q * p.Q;
    return true;
  }
  __device__ bool seg_active(int seg) const { return seg % nsplit == split; }
  __device__ int nseg() const { return p.hpg; }
  __device__ void krange(int, int, int, int& k0, int& k1) const { k0 = 0; k1 = p.P; }
  __device__ bool a_kcontig(int) const { return true; }
  __device__ bool b_kcontig(int) const { return true; }
  __device__ float a(int seg, int m, int k) const { return p.dy[(t0 + m) * p.lddy + (g * p.hpg + seg) * p.P + k]; }
  __device__ float b(int seg, int k, int n) const {
    int h = g * p.hpg + seg;
    return p.x[(t0 + n) * p.ldx + h * p.P + k] * p.dtv(t0 + n, h);
  }
  __device__ float seg_scale(int seg, int m, int n) const {
    if (n > m) return 0.0f;
    int h = g * p.hpg + seg;
    const float* sp = p.S + ((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q;
    return expf(sp[m] - sp[n]);
  }
  __device__ void store(int m, int n, float v) const { out[(int64_t)m * p.Q + n] = v; }
};

// ---- B6a: dC[t,n] = sum_{s<=t} dG[t,s] B[s,n] + sum_h exp(S_h,t) sum_p dY_h[t,p] h_prev_h[n,p] ----
struct OpDC {
  static constexpr bool SEG_SCALE = false;
  SsdP p; int Mdim, Ndim;
  int nsplit; float* part;
  int bb, cc, g, split; int64_t t0; const float* dg; float* pout;
  __device__ bool init(int batch, int, int) {
    split = batch % nsplit; batch /= nsplit;
    g = batch % p.G; int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    t0 = p.tok(bb, cc, 0);
    dg = p.dG + (int64_t)batch * p.Q * p.Q;
    pout = part + (int64_t)blockIdx.z * Mdim * Ndim;
    return true;
  }
  __device__ bool seg_active(int seg) const { return seg == 0 ? split == 0 : (seg - 1) % nsplit == split; }
  __device__ int nseg() const { return 1 + p.hpg; }
  __device__ void krange(int seg, int m0, int, int& k0, int& k1) const {
    k0 = 0; k1 = seg == 0 ? min(p.Q, m0 + BM) : p.P;
  }
  __device__ bool a_kcontig(int) const { return true; }
  __device__ bool b_kcontig(int seg) const { return seg != 0; }
  __device__ float a(int seg, int m, int k) const {
    if (seg == 0) return dg[(int64_t)m * p.Q + k];
    int h = g * p.hpg + seg - 1;
    return p.dy[(t0 + m) * p.lddy + h * p.P + k] * expf(p.Sv(bb, h, cc, m));
  }
  __device__ float b(int seg, int k, int n) const {
    if (seg == 0) return p.b[(t0 + k) * p.ldbc + g * p.N + n];
    int h = g * p.hpg + seg - 1;
    return p.hprev[((((int64_t)bb * p.nc + cc) * p.H + h) * p.N + n) * p.P + k];
  }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ void store(int m, int n, float v) const {
    if (nsplit > 1) pout[(int64_t)m * Ndim + n] = v; else p.dc[(t0 + m) * p.lddbc + g * p.N + n] = v;
  }
};

// ---- B6b: dB[s,n] = sum_{t>=s} dG[t,s] C[t,n] + sum_h exp(S_end - S_s) sum_p x~_h[s,p] dh_h[n,p] --
struct OpDB {
  static constexpr bool SEG_SCALE = false;
  SsdP p; int Mdim, Ndim;
  int nsplit; float* part;
  int bb, cc, g, split; int64_t t0; const float* dg; float* pout;
  __device__ bool init(int batch, int, int) {
    split = batch % nsplit; batch /= nsplit;
    g = batch % p.G; int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    t0 = p.tok(bb, cc, 0);
    dg = p.dG + (int64_t)batch * p.Q * p.Q;
    pout = part + (int64_t)blockIdx.z * Mdim * Ndim;
    return true;
  }
  __device__ bool seg_active(int seg) const { return seg == 0 ? split == 0 : (seg - 1) % nsplit == split; }
  __device__ int nseg() const { return 1 + p.hpg; }
  __device__ void krange(int seg, int m0, int, int& k0, int& k1) const {
    if (seg == 0) { k0 = m0; k1 = p.Q; } else { k0 = 0; k1 = p.P; }
  }
  __device__ bool a_kcontig(int seg) const { return seg != 0; }
  __device__ bool b_kcontig(int seg) const { return seg != 0; }
  __device__ float a(int seg, int m, int k) const {
    if (seg == 0) return dg[(int64_t)k * p.Q + m];
    int h = g * p.hpg + seg - 1;
    float send = p.Sv(bb, h, cc, p.Q - 1);
    return p.x[(t0 + m) * p.ldx + h * p.P + k] * p.dtv(t0 + m, h) * expf(send - p.Sv(bb, h, cc, m));
  }
  __device__ float b(int seg, int k, int n) const {
    if (seg == 0) return p.c[(t0 + k) * p.ldbc + g * p.N + n];
    int h = g * p.hpg + seg - 1;
    return p.dh[((((int64_t)bb * p.nc + cc) * p.H + h) * p.N + n) * p.P + k];
  }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ void store(int m, int n, float v) const {
    if (nsplit > 1) pout[(int64_t)m * Ndim + n] = v; else p.db[(t0 + m) * p.lddbc + g * p.N + n] = v;
  }
};

// ---------------------------------------------------------------------------------------------
// Small kernels
// ---------------------------------------------------------------------------------------------

// S[b,h,c*Q+q] = inclusive cumsum over q of a.  One warp per (b,c,h).  With raw.dt_raw the warp first forms
// dt = softplus(dt_raw + bias) (written out for the later kernels) and A = -exp(a_log).
struct CumsumRaw { const float* dt_raw; int64_t ld_raw; const float* dt_bias; const float* a_log; float* dt_out; float* A_out; };
__global__ void chunk_cumsum_kernel(SsdP p, CumsumRaw raw) {
  int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int total = p.B * p.nc * p.H;
  if (w >= total) return;
  int h = w % p.H, bc = w / p.H, cc = bc % p.nc, bb = bc / p.nc;
  float carry = 0.0f;
  float* out = p.S + ((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q;
  // the strided loads of up to 8 rounds are requested together, ahead of the dependent scan chain
  constexpr int AHEAD = 8;
  const float Ah = raw.dt_raw ? -expf(raw.a_log[h]) : (p.dt ? p.A[h] : 1.0f);
  const float bias = raw.dt_raw ? raw.dt_bias[h] : 0.0f;
  if (raw.dt_raw && bc == 0 && lane == 0) raw.A_out[h] = Ah;
  const float* srcv = p.dt ? p.dt : p.a;
  float pre[AHEAD];
  for (int q0 = 0; q0 < p.Q; q0 += 32) {
    const int r = (q0 >> 5) % AHEAD;
    if (r == 0) {
#pragma unroll
      for (int j = 0; j < AHEAD; ++j) {
        const int qq = q0 + 32 * j + lane;
        pre[j] = 0.0f;
        if (qq < p.Q) {
          const int64_t tk = p.tok(bb, cc, qq);
          if (raw.dt_raw) {
            const float dtv = softplus_acc(raw.dt_raw[tk * raw.ld_raw + h] + bias);
            raw.dt_out[tk * p.H + h] = dtv;
            pre[j] = Ah * dtv;
          } else {
            pre[j] = Ah * srcv[tk * p.H + h];
          }
        }
      }
    }
    int q = q0 + lane;
    float v = 0.0f;
#pragma unroll
    for (int j = 0; j < AHEAD; ++j) if (j == r) v = pre[j];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    v += carry;
    if (q < p.Q) out[q] = v;
    carry = __shfl_sync(0xffffffffu, v, 31);
  }
}

// Fused variant for the tensor-core path, one 256-thread block per (b,c,h): the same cumsum (with dt and A formed
// here when raw inputs are given), then xs[t,:] = x[t,:] * dt_t * exp(S_end - S_t), the operand that the chunk-state
// and dB contractions share.  S and dt of the chunk stay in shared memory between the two phases.
constexpr int PREP_THREADS = 256, PREP_MAX_Q = 1024;
__global__ void __launch_bounds__(PREP_THREADS) chunk_prepare_kernel(SsdP p, CumsumRaw raw, float* __restrict__ xs,
                                                                     uint16_t* __restrict__ xt_hi, uint16_t* __restrict__ xt_lo,
                                                                     uint16_t* __restrict__ xs_hi, uint16_t* __restrict__ xs_lo) {
  __shared__ float sS[PREP_MAX_Q], sdt[PREP_MAX_Q], wsum[PREP_THREADS / 32];
  // gridDim.y CTAs share one (b,c,h): each repeats the short cumulative sum (same order, same values) and takes its
  // slice of the rows in the second phase; the first of them writes dt, A and S
  const int w = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const bool writer = blockIdx.y == 0;
  const int h = w % p.H, bc = w / p.H, cc = bc % p.nc, bb = bc / p.nc;
  const float Ah = raw.dt_raw ? -expf(raw.a_log[h]) : (p.dt ? p.A[h] : 1.0f);
  const float bias = raw.dt_raw ? raw.dt_bias[h] : 0.0f;
  if (raw.dt_raw && bc == 0 && tid == 0 && writer) raw.A_out[h] = Ah;
  float* Sout = p.S + ((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q;
  float carry = 0.0f;
  for (int q0 = 0; q0 < p.Q; q0 += PREP_THREADS) {
    const int q = q0 + tid;
    float v = 0.0f, dtv = 1.0f;
    if (q < p.Q) {
      const int64_t tk = p.tok(bb, cc, q);
      if (raw.dt_raw) { dtv = softplus_acc(raw.dt_raw[tk * raw.ld_raw + h] + bias); if (writer) raw.dt_out[tk * p.H + h] = dtv; v = Ah * dtv; }
      else if (p.dt) { dtv = p.dt[tk * p.H + h]; v = Ah * dtv; }
      else v = p.a[tk * p.H + h];
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
    if (lane == 31) wsum[wid] = v;
    __syncthreads();
    float off = carry;
    for (int j = 0; j < wid; ++j) off += wsum[j];          // fixed order: the same sums for every launch
    v += off;
    if (q < p.Q) { sS[q] = v; sdt[q] = dtv; if (writer) Sout[q] = v; }
    float tot = carry;
    for (int j = 0; j < PREP_THREADS / 32; ++j) tot += wsum[j];
    carry = tot;
    __syncthreads();
  }
  const float send = sS[p.Q - 1];
  const int P4 = p.P >> 2;
  const int rows_per = (p.Q + (int)gridDim.y - 1) / (int)gridDim.y;        // this CTA's rows [r0, r1) of the chunk
  const int r0 = (int)blockIdx.y * rows_per, r1 = min(p.Q, r0 + rows_per);
  const int total = r1 * P4;
  const int64_t tok0 = p.tok(bb, cc, 0);
  constexpr int U = 4;
  for (int i0 = r0 * P4 + tid; i0 < total; i0 += U * PREP_THREADS) {
    float4 v[U]; float f[U], fd[U]; int tt[U], jj[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * PREP_THREADS;
      tt[u] = i / P4; jj[u] = i % P4;
      if (i < total) {
        v[u] = reinterpret_cast<const float4*>(p.x + (tok0 + tt[u]) * p.ldx + h * p.P)[jj[u]];
        fd[u] = sdt[tt[u]];
        f[u] = __expf(send - sS[tt[u]]) * fd[u];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * PREP_THREADS;
      if (i < total) {
        const int64_t o = (tok0 + tt[u]) * (int64_t)(p.H * p.P) + h * p.P + 4 * jj[u];
        if (xs_hi) store_pair4(xs_hi + o, xs_lo ? xs_lo + o : nullptr, v[u].x * f[u], v[u].y * f[u], v[u].z * f[u], v[u].w * f[u]);
        else *reinterpret_cast<float4*>(xs + o) = make_float4(v[u].x * f[u], v[u].y * f[u], v[u].z * f[u], v[u].w * f[u]);
        // x~ = x dt as a bf16 pair: the V operand of the fused intra-chunk kernel
        if (xt_hi) store_pair4(xt_hi + o, xt_lo ? xt_lo + o : nullptr, v[u].x * fd[u], v[u].y * fd[u], v[u].z * fd[u], v[u].w * fd[u]);
      }
    }
  }
}

// Exclusive scan over chunks, in place, forward or reverse.  One thread owns VEC adjacent p of one (b,h,n).
//   forward: buf[c] holds states[c] on entry and h_prev[c] (state entering chunk c) on exit; last = final state.
//            run_{c+1} = exp(S_end[c]) run_c + states[c],  run_0 = init (or 0)
//   reverse: buf[c] holds contrib[c] on entry and dh[c] (adjoint of the state leaving chunk c) on exit.
//            run_{c-1} = exp(S_end[c]) run_c + contrib[c], run_{nc-1} = 0
// The chunk values are fetched four at a time before the dependent chain so the loads overlap.
template <int VEC>
__global__ void __launch_bounds__(256) state_scan_kernel(SsdP p, float* __restrict__ buf, const float* __restrict__ init,
                                                         float* __restrict__ last, int reverse,
                                                         uint16_t* __restrict__ pair_hi, uint16_t* __restrict__ pair_lo) {
  const int64_t NP = (int64_t)p.N * p.P;
  const int64_t per = NP / VEC;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)p.B * p.H * per) return;
  const int64_t e = (i % per) * VEC; const int64_t bh = i / per; const int h = (int)(bh % p.H); const int bb = (int)(bh / p.H);
  float run[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) run[v] = (init && !reverse) ? init[bh * NP + e + v] : 0.0f;
  const float* send = p.S + ((int64_t)bb * p.H + h) * p.T + p.Q - 1;
  for (int c0 = 0; c0 < p.nc; c0 += 4) {
    float tmp[4][VEC]; float dec[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cc = reverse ? p.nc - 1 - (c0 + j) : c0 + j;
      if (c0 + j < p.nc) {
        const float* slot = buf + (((int64_t)bb * p.nc + cc) * p.H + h) * NP + e;
        if (VEC == 4) { float4 q = *reinterpret_cast<const float4*>(slot); tmp[j][0] = q.x; tmp[j][1 % VEC] = q.y; tmp[j][2 % VEC] = q.z; tmp[j][3 % VEC] = q.w; }
        else tmp[j][0] = slot[0];
        dec[j] = expf(send[(int64_t)cc * p.Q]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cc = reverse ? p.nc - 1 - (c0 + j) : c0 + j;
      if (c0 + j < p.nc) {
        float* slot = buf + (((int64_t)bb * p.nc + cc) * p.H + h) * NP + e;
        if (VEC == 4) {
          *reinterpret_cast<float4*>(slot) = make_float4(run[0], run[1 % VEC], run[2 % VEC], run[3 % VEC]);
          // the same values as a bf16 pair: the state operand of the fused intra-chunk kernel
          if (pair_hi) store_pair4(pair_hi + (slot - buf), pair_lo ? pair_lo + (slot - buf) : nullptr, run[0], run[1 % VEC], run[2 % VEC], run[3 % VEC]);
        }
        else slot[0] = run[0];
#pragma unroll
        for (int v = 0; v < VEC; ++v) run[v] = fmaf(dec[j], run[v], tmp[j][v]);
      }
    }
  }
  if (last && !reverse) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) last[bh * NP + e + v] = run[v];
  }
}

// dsend[b,c,h] = <dh[c], h_next[c]> with h_next[c] = h_prev[c+1], or the final state for the last chunk.
// own_state != 0: <dh[c], h_prev[c]> instead (the fused backward adds the other part of <dh, h_next> from the very
// values that enter dS, see chunk_rows_finish_w_kernel).
__global__ void __launch_bounds__(256) state_dot_kernel(SsdP p, float* __restrict__ dsend, int own_state) {
  __shared__ float red[32];
  const int bch = blockIdx.x;
  const int h = bch % p.H; const int bc = bch / p.H; const int cc = bc % p.nc; const int bb = bc / p.nc;
  const int NP = p.N * p.P;
  const float* a = p.dh + (int64_t)bch * NP;
  const float* b = own_state ? p.hprev + (int64_t)bch * NP : (cc + 1 < p.nc) ? p.hprev + (((int64_t)bb * p.nc + cc + 1) * p.H + h) * NP : p.hlast + ((int64_t)bb * p.H + h) * NP;
  float dot = 0.0f;
  for (int e = threadIdx.x; e < NP; e += blockDim.x) dot = fmaf(a[e], b[e], dot);
  float tot = block_sum(dot, red);
  if (threadIdx.x == 0) dsend[bch] = tot;
}

// Reverse scan and d[b,c,h] = <dh[c], h_prev[c]> in one launch for the pair path: one CTA per (b,h), a thread owns
// ITEMS groups of four adjacent p; the chunk values are fetched four chunks at a time before the dependent chain.
// Per-chunk dot products: warp sums into shared memory, then one thread per chunk adds the warps in order.
constexpr int SCAN_DOT_MAX_NC = 64;
template <int ITEMS>
__global__ void __launch_bounds__(1024) state_scan_rev_dot_kernel(SsdP p, float* __restrict__ buf, uint16_t* __restrict__ pair_hi,
                                                                  uint16_t* __restrict__ pair_lo, float* __restrict__ dsend) {
  __shared__ float wdot[SCAN_DOT_MAX_NC][32];
  const int bh = blockIdx.x, h = bh % p.H, bb = bh / p.H;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nth = blockDim.x;
  const int64_t NP = (int64_t)p.N * p.P;
  const float* send = p.S + ((int64_t)bb * p.H + h) * p.T + p.Q - 1;
  float4 run[ITEMS];
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) run[it] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int c0 = 0; c0 < p.nc; c0 += 4) {
    float4 q[4][ITEMS], hv[4][ITEMS]; float dec[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cc = p.nc - 1 - (c0 + j);
      if (cc >= 0) {
        const int64_t base = (((int64_t)bb * p.nc + cc) * p.H + h) * NP;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          const int64_t e = ((int64_t)it * nth + tid) * 4;
          if (e < NP) { q[j][it] = *reinterpret_cast<const float4*>(buf + base + e); hv[j][it] = *reinterpret_cast<const float4*>(p.hprev + base + e); }
        }
        dec[j] = expf(send[(int64_t)cc * p.Q]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cc = p.nc - 1 - (c0 + j);
      if (cc >= 0) {
        const int64_t base = (((int64_t)bb * p.nc + cc) * p.H + h) * NP;
        float dot = 0.0f;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          const int64_t e = ((int64_t)it * nth + tid) * 4;
          if (e < NP) {
            const float4 r = run[it];
            *reinterpret_cast<float4*>(buf + base + e) = r;
            store_pair4(pair_hi + base + e, pair_lo ? pair_lo + base + e : nullptr, r.x, r.y, r.z, r.w);
            dot = fmaf(r.x, hv[j][it].x, fmaf(r.y, hv[j][it].y, fmaf(r.z, hv[j][it].z, fmaf(r.w, hv[j][it].w, dot))));
            run[it] = make_float4(fmaf(dec[j], r.x, q[j][it].x), fmaf(dec[j], r.y, q[j][it].y), fmaf(dec[j], r.z, q[j][it].z), fmaf(dec[j], r.w, q[j][it].w));
          }
        }
        dot = warp_sum(dot);
        if (lane == 0) wdot[cc][wid] = dot;
      }
    }
  }
  __syncthreads();
  if (tid < p.nc) {
    float tot = 0.0f;
    for (int j = 0; j < (nth >> 5); ++j) tot += wdot[tid][j];
    dsend[((int64_t)bb * p.nc + tid) * p.H + h] = tot;
  }
}

// true when the merged kernel took the launch
static bool launch_state_scan_rev_dot(cudaStream_t st, const SsdP& p, float* buf, uint16_t* pair_hi, uint16_t* pair_lo, float* dsend) {
  const int64_t quads = (int64_t)p.N * p.P / 4;
  if ((p.P & 3) || !pair_hi || !p.hprev || p.nc > SCAN_DOT_MAX_NC || quads > 4 * 1024) return false;
  const int items = quads <= 1024 ? 1 : (quads <= 2048 ? 2 : 4);
  const unsigned threads = (unsigned)(((quads + items - 1) / items + 31) / 32 * 32);
  const unsigned grid = (unsigned)(p.B * p.H);
  if (items == 1) state_scan_rev_dot_kernel<1><<<grid, threads, 0, st>>>(p, buf, pair_hi, pair_lo, dsend);
  else if (items == 2) state_scan_rev_dot_kernel<2><<<grid, threads, 0, st>>>(p, buf, pair_hi, pair_lo, dsend);
  else state_scan_rev_dot_kernel<4><<<grid, threads, 0, st>>>(p, buf, pair_hi, pair_lo, dsend);
  return true;
}

static pmb_status launch_state_scan(cudaStream_t st, const SsdP& p, float* buf, const float* init, float* last, int reverse,
                                    uint16_t* pair_hi = nullptr, uint16_t* pair_lo = nullptr) {
  const int64_t NP = (int64_t)p.N * p.P;
  const bool vec = (p.P % 4 == 0);
  const int64_t n = (int64_t)p.B * p.H * (vec ? NP / 4 : NP);
  if (vec) state_scan_kernel<4><<<(unsigned)cdiv(n, 256), 256, 0, st>>>(p, buf, init, last, reverse, pair_hi, pair_lo);
  else state_scan_kernel<1><<<(unsigned)cdiv(n, 256), 256, 0, st>>>(p, buf, init, last, reverse, nullptr, nullptr);
  PMB_LAUNCHED();
  return PMB_OK;
}

// One warp per (b,t,h): row dot products and dx.
//   ddt_x = <dx~, x>;  dS = <dY, Y - D x> - dt * ddt_x;  dDrow = <dY, x>;  dx = dx~ * dt + D * dY
__global__ void ssd_rowdots_kernel(SsdP p, float* __restrict__ dx, int64_t lddx, float* __restrict__ ddt_x,
                                   float* __restrict__ dS, float* __restrict__ dDrow) {
  int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  int64_t total = (int64_t)p.B * p.T * p.H;
  if (w >= total) return;
  int h = (int)(w % p.H); int64_t tk = w / p.H;
  float dtv = p.dtv(tk, h), Dv = p.D ? p.D[h] : 0.0f;
  float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
  for (int pp = lane; pp < p.P; pp += 32) {
    float xv = p.x[tk * p.ldx + h * p.P + pp];
    float dxt = p.dxt[tk * (int64_t)(p.H * p.P) + h * p.P + pp];
    float dyv = p.dy[tk * p.lddy + h * p.P + pp];
    float yv = p.y[tk * p.ldy + h * p.P + pp] - Dv * xv;
    s1 = fmaf(dxt, xv, s1);
    s2 = fmaf(dyv, yv, s2);
    s3 = fmaf(dyv, xv, s3);
    dx[tk * lddx + h * p.P + pp] = fmaf(dxt, dtv, Dv * dyv);
  }
  s1 = warp_sum(s1); s2 = warp_sum(s2); s3 = warp_sum(s3);
  if (lane == 0) {
    ddt_x[w] = s1;
    dS[w] = s2 - dtv * s1;
    dDrow[w] = s3;
  }
}

// One warp per (b,c,h): da = reverse inclusive cumsum of dS (dS[Q-1] += dsend).
// a-mode (dt == NULL): writes da.  dt-mode: ddt = ddt_x + A da; partial sums of da*dt and dDrow per chunk.
__global__ void ssd_chunk_finish_kernel(SsdP p, const float* __restrict__ ddt_x, const float* __restrict__ dS,
                                        const float* __restrict__ dDrow, const float* __restrict__ dsend,
                                        float* __restrict__ da_out, float* __restrict__ ddt_out, float* __restrict__ part) {
  int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int total = p.B * p.nc * p.H;
  if (w >= total) return;
  int h = w % p.H, bc = w / p.H, cc = bc % p.nc, bb = bc / p.nc;
  float carry = 0.0f, pA = 0.0f, pD = 0.0f;
  float Ah = p.dt ? p.A[h] : 0.0f;
  int nblk = (p.Q + 31) / 32;
  // the strided loads of up to 8 rounds are requested together, ahead of the dependent scan chain
  constexpr int AHEAD = 8;
  float pre[AHEAD];
  const float send = dsend[w];
  for (int blk = nblk - 1; blk >= 0; --blk) {
    const int r = (nblk - 1 - blk) % AHEAD;
    if (r == 0) {
#pragma unroll
      for (int j = 0; j < AHEAD; ++j) {
        const int qq = (blk - j) * 32 + lane;
        pre[j] = (blk - j >= 0 && qq < p.Q) ? dS[p.tok(bb, cc, qq) * p.H + h] : 0.0f;
      }
    }
    int q = blk * 32 + lane;
    float v = 0.0f;
    int64_t idx = 0;
#pragma unroll
    for (int j = 0; j < AHEAD; ++j) if (j == r) v = pre[j];
    if (q < p.Q) {
      idx = p.tok(bb, cc, q) * p.H + h;
      if (q == p.Q - 1) v += send;
    } else {
      v = 0.0f;
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float u = __shfl_down_sync(0xffffffffu, v, o);
      if (lane + o < 32) v += u;
    }
    v += carry;
    if (q < p.Q) {
      if (p.dt) {
        ddt_out[idx] = fmaf(Ah, v, ddt_x[idx]);
        pA = fmaf(v, p.dt[idx], pA);
        pD += dDrow[idx];
      } else {
        da_out[idx] = v;
      }
    }
    carry = __shfl_sync(0xffffffffu, v, 0);
  }
  if (p.dt) {
    pA = warp_sum(pA); pD = warp_sum(pD);
    if (lane == 0) {
      part[(int64_t)bc * p.H + h] = pA;
      part[(int64_t)p.B * p.nc * p.H + (int64_t)bc * p.H + h] = pD;
    }
  }
}

// Fused variant of the two kernels above, one 256-thread block per (b,c,h), for launches whose blocks fit the
// machine at once: the row dot products stay in shared memory and feed the reverse cumsum directly.
__global__ void __launch_bounds__(PREP_THREADS) chunk_rows_finish_kernel(SsdP p, float* __restrict__ dx, int64_t lddx,
                                                                         const float* __restrict__ dsend, float* __restrict__ da_out,
                                                                         float* __restrict__ ddt_out, float* __restrict__ part) {
  __shared__ float s_ddtx[PREP_MAX_Q], s_dS[PREP_MAX_Q], s_dD[PREP_MAX_Q], s_dt[PREP_MAX_Q], wsum[PREP_THREADS / 32], red[32];
  const int w = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int h = w % p.H, bc = w / p.H, cc = bc % p.nc, bb = bc / p.nc;
  const float Dv = p.D ? p.D[h] : 0.0f;
  const int64_t tok0 = p.tok(bb, cc, 0);
  const int P4 = p.P >> 2;
  // phase 1: a half-warp per row, float4 lanes (P <= 64) or strided lanes beyond
  const int sub = lane >> 4, l16 = lane & 15;
  for (int t0 = wid * 2; t0 < p.Q; t0 += (PREP_THREADS / 32) * 2) {
    const int t = t0 + sub;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f, dtv = 1.0f;
    if (t < p.Q) {
      const int64_t tk = tok0 + t;
      dtv = p.dtv(tk, h);
      for (int j = l16; j < P4; j += 16) {
        const float4 xv = reinterpret_cast<const float4*>(p.x + tk * p.ldx + h * p.P)[j];
        const float4 dxt = reinterpret_cast<const float4*>(p.dxt + tk * (int64_t)(p.H * p.P) + h * p.P)[j];
        const float4 dyv = reinterpret_cast<const float4*>(p.dy + tk * p.lddy + h * p.P)[j];
        float4 yv = reinterpret_cast<const float4*>(p.y + tk * p.ldy + h * p.P)[j];
        yv.x -= Dv * xv.x; yv.y -= Dv * xv.y; yv.z -= Dv * xv.z; yv.w -= Dv * xv.w;
        s1 = fmaf(dxt.x, xv.x, fmaf(dxt.y, xv.y, fmaf(dxt.z, xv.z, fmaf(dxt.w, xv.w, s1))));
        s2 = fmaf(dyv.x, yv.x, fmaf(dyv.y, yv.y, fmaf(dyv.z, yv.z, fmaf(dyv.w, yv.w, s2))));
        s3 = fmaf(dyv.x, xv.x, fmaf(dyv.y, xv.y, fmaf(dyv.z, xv.z, fmaf(dyv.w, xv.w, s3))));
        reinterpret_cast<float4*>(dx + tk * lddx + h * p.P)[j] =
            make_float4(fmaf(dxt.x, dtv, Dv * dyv.x), fmaf(dxt.y, dtv, Dv * dyv.y), fmaf(dxt.z, dtv, Dv * dyv.z), fmaf(dxt.w, dtv, Dv * dyv.w));
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {        // sums within each half-warp
      s1 += __shfl_xor_sync(0xffffffffu, s1, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); s3 += __shfl_xor_sync(0xffffffffu, s3, o);
    }
    if (t < p.Q && l16 == 0) { s_ddtx[t] = s1; s_dS[t] = s2 - dtv * s1; s_dD[t] = s3; s_dt[t] = dtv; }
  }
  __syncthreads();
  if (tid == 0) s_dS[p.Q - 1] += dsend[w];
  __syncthreads();
  // phase 2: reverse inclusive cumsum of dS over the chunk, rounds of 256 from the end
  const float Ah = p.dt ? p.A[h] : 0.0f;
  float carry = 0.0f, pA = 0.0f, pD = 0.0f;
  for (int r0 = 0; r0 < p.Q; r0 += PREP_THREADS) {
    const int q = p.Q - 1 - (r0 + tid);                 // thread 0 owns the last element of the chunk
    float v = q >= 0 ? s_dS[q] : 0.0f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
    if (lane == 31) wsum[wid] = v;
    __syncthreads();
    float off = carry;
    for (int j = 0; j < wid; ++j) off += wsum[j];
    v += off;
    if (q >= 0) {
      const int64_t idx = (tok0 + q) * p.H + h;
      if (p.dt) { ddt_out[idx] = fmaf(Ah, v, s_ddtx[q]); pA = fmaf(v, s_dt[q], pA); pD += s_dD[q]; }
      else da_out[idx] = v;
    }
    float tot = carry;
    for (int j = 0; j < PREP_THREADS / 32; ++j) tot += wsum[j];
    carry = tot;
    __syncthreads();
  }
  if (p.dt) {
    const float tA = block_sum(pA, red);
    const float tD = block_sum(pD, red);
    if (tid == 0) {
      part[(int64_t)bc * p.H + h] = tA;
      part[(int64_t)p.B * p.nc * p.H + (int64_t)bc * p.H + h] = tD;
    }
  }
}

// Row sums and the reverse cumulative sum for the fused backward, one 256-thread block per (b,c,h).
// The gradient w.r.t. the in-chunk cumulative sum S is assembled from terms that were each formed once:
//   dS_t = r_t - c_t + f_t - e_t,      dS_{Q-1} += sum_s e_s + exp(S_end) <dh, h_prev>
//   r_t = sum_{s<t} W[t,s], c_t = sum_{u>t} W[u,t]   (W = dM o G o L, both sums from the same registers of the fused kernel)
//   f_t = <dY_t, exp(S_t) C_t h_prev>                 (the carried-state part of y, kept by the forward kernel)
//   e_s = exp(S_end - S_s) <x~_s, B_s dh>             (from the fused kernel's epilogue)
// so the cancellation inside sum_t S_t dS_t (the gradient of A) is between identically rounded numbers and never
// goes through y - D x or through two separately rounded matrix products.  da = reverse cumsum(dS);
// ddt = <dx~, x> + A da;  dx = dx~ dt + D dY;  per-chunk partials of dA and dD.
struct WSums { const float* rpart; const float* csum; const float* esum; const float* yoff; int nb; };
// Each half-warp has two rows in flight per pass (all loads of both rows are issued before the first use), and two
// CTAs fit on an SM, so that the 192 CTAs of a 2048-token launch at 24 heads are resident at once (one CTA per SM
// meant a second wave of 44 CTAs).
constexpr int ROWS_THREADS = 256;
// LEAN16 (the bf16-input scan: no dt, no skip term, dx = dx~ already written by the fused kernel): only <dY, y_off>
// is formed per row, dY (dy16) and y_off (ws.yoff, reinterpreted) both read as bf16 rows of H*P.
template <bool LEAN16>
__global__ void __launch_bounds__(ROWS_THREADS, LEAN16 ? 3 : 2) chunk_rows_finish_w_kernel(SsdP p, WSums ws, float* __restrict__ dx, int64_t lddx,
                                                                           const float* __restrict__ dd, float* __restrict__ da_out,
                                                                           float* __restrict__ ddt_out, float* __restrict__ part,
                                                                           SsdGrads::RawDt raw, const uint16_t* __restrict__ dy16) {
  __shared__ float s_ddtx[PREP_MAX_Q], s_dS[PREP_MAX_Q], s_dD[PREP_MAX_Q], s_dt[PREP_MAX_Q], s_e[PREP_MAX_Q], wsum[ROWS_THREADS / 32], red[32];
  constexpr int NHW = ROWS_THREADS / 16;
  const int w = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int h = w % p.H, bc = w / p.H, cc = bc % p.nc, bb = bc / p.nc;
  const float Dv = p.D ? p.D[h] : 0.0f;
  const int64_t tok0 = p.tok(bb, cc, 0);
  const int P4 = p.P >> 2;
  const int hw = tid >> 4, l16 = lane & 15;
  const int64_t hp = (int64_t)p.H * p.P;
  if (LEAN16) {
    // eight lanes per row (16 bytes of dY and of y_off each per pass), four rows per warp and four such groups in
    // flight per thread; y_off was written as bf16 by the fused forward kernel
    const uint16_t* yoff16 = reinterpret_cast<const uint16_t*>(ws.yoff);
    const int P8 = p.P >> 3, l8 = lane & 7, sub = lane >> 3;
    constexpr int NW = ROWS_THREADS / 32, U = 4;
    for (int tb = 0; tb < p.Q; tb += NW * 4 * U) {
      int t[U]; float s2[U], rr[U], cs[U], es[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        t[u] = tb + (u * NW + wid) * 4 + sub; s2[u] = 0.0f; rr[u] = 0.0f; cs[u] = 0.0f; es[u] = 0.0f;
        if (t[u] < p.Q && l8 == 0) {
          const int64_t idx = (tok0 + t[u]) * p.H + h;
          for (int rb = 0; rb <= t[u] / 128; ++rb) rr[u] += ws.rpart[((int64_t)w * ws.nb + rb) * p.Q + t[u]];
          cs[u] = ws.csum[idx]; es[u] = ws.esum[idx];
        }
      }
      for (int j = l8; j < P8; j += 8) {
        uint4 d[U], y[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (t[u] < p.Q) {
            const int64_t o = (tok0 + t[u]) * hp + h * p.P + 8 * j;
            d[u] = *reinterpret_cast<const uint4*>(dy16 + o);
            y[u] = *reinterpret_cast<const uint4*>(yoff16 + o);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (t[u] < p.Q) {
            const uint32_t dw[4] = {d[u].x, d[u].y, d[u].z, d[u].w}, yw[4] = {y[u].x, y[u].y, y[u].z, y[u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              s2[u] = fmaf(__uint_as_float(dw[e] << 16), __uint_as_float(yw[e] << 16), s2[u]);
              s2[u] = fmaf(__uint_as_float(dw[e] & 0xffff0000u), __uint_as_float(yw[e] & 0xffff0000u), s2[u]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) s2[u] += __shfl_xor_sync(0xffffffffu, s2[u], o);
        if (t[u] < p.Q && l8 == 0) { s_e[t[u]] = es[u]; s_dS[t[u]] = ((rr[u] - cs[u]) + s2[u]) - es[u]; }
      }
    }
  }
  for (int tb = 0; !LEAN16 && tb < p.Q; tb += 2 * NHW) {
    const int t[2] = {tb + hw, tb + NHW + hw};
    float s1[2] = {0.0f, 0.0f}, s2[2] = {0.0f, 0.0f}, s3[2] = {0.0f, 0.0f}, dtv[2] = {1.0f, 1.0f};
    float rr[2] = {0.0f, 0.0f}, cs[2] = {0.0f, 0.0f}, es[2] = {0.0f, 0.0f};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (t[u] < p.Q) {
        const int64_t tk = tok0 + t[u];
        dtv[u] = p.dtv(tk, h);
        if (l16 == 0) {
          const int64_t idx = tk * p.H + h;
          for (int rb = 0; rb <= t[u] / 128; ++rb) rr[u] += ws.rpart[((int64_t)w * ws.nb + rb) * p.Q + t[u]];   // row blocks whose rows s can be < t
          cs[u] = ws.csum[idx]; es[u] = ws.esum[idx];
        }
      }
    }
    for (int j = l16; j < P4; j += 16) {
      float4 xv[2], dxt[2], dyv[2], yo[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (t[u] < p.Q) {
          const int64_t tk = tok0 + t[u];
          xv[u] = reinterpret_cast<const float4*>(p.x + tk * p.ldx + h * p.P)[j];
          dxt[u] = reinterpret_cast<const float4*>(p.dxt + tk * hp + h * p.P)[j];
          dyv[u] = reinterpret_cast<const float4*>(p.dy + tk * p.lddy + h * p.P)[j];
          yo[u] = reinterpret_cast<const float4*>(ws.yoff + tk * hp + h * p.P)[j];
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (t[u] < p.Q) {
          const int64_t tk = tok0 + t[u];
          s1[u] = fmaf(dxt[u].x, xv[u].x, fmaf(dxt[u].y, xv[u].y, fmaf(dxt[u].z, xv[u].z, fmaf(dxt[u].w, xv[u].w, s1[u]))));
          s2[u] = fmaf(dyv[u].x, yo[u].x, fmaf(dyv[u].y, yo[u].y, fmaf(dyv[u].z, yo[u].z, fmaf(dyv[u].w, yo[u].w, s2[u]))));
          s3[u] = fmaf(dyv[u].x, xv[u].x, fmaf(dyv[u].y, xv[u].y, fmaf(dyv[u].z, xv[u].z, fmaf(dyv[u].w, xv[u].w, s3[u]))));
          reinterpret_cast<float4*>(dx + tk * lddx + h * p.P)[j] =
              make_float4(fmaf(dxt[u].x, dtv[u], Dv * dyv[u].x), fmaf(dxt[u].y, dtv[u], Dv * dyv[u].y), fmaf(dxt[u].z, dtv[u], Dv * dyv[u].z),
                          fmaf(dxt[u].w, dtv[u], Dv * dyv[u].w));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        s1[u] += __shfl_xor_sync(0xffffffffu, s1[u], o); s2[u] += __shfl_xor_sync(0xffffffffu, s2[u], o); s3[u] += __shfl_xor_sync(0xffffffffu, s3[u], o);
      }
      if (t[u] < p.Q && l16 == 0) {
        s_ddtx[t[u]] = s1[u]; s_dD[t[u]] = s3[u]; s_dt[t[u]] = dtv[u]; s_e[t[u]] = es[u];
        s_dS[t[u]] = ((rr[u] - cs[u]) + s2[u]) - es[u];
      }
    }
  }
  __syncthreads();
  // sum of e over the chunk in a fixed order, then the terms that belong to the last position
  float ep = 0.0f;
  for (int q = tid; q < p.Q; q += ROWS_THREADS) ep += s_e[q];
  const float esum = block_sum(ep, red);
  if (tid == 0) {
    const float send = p.S[((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q + p.Q - 1];
    s_dS[p.Q - 1] += esum + expf(send) * dd[w];
  }
  __syncthreads();
  const float Ah = p.dt ? p.A[h] : 0.0f;
  float carry = 0.0f, pA = 0.0f, pD = 0.0f, pB = 0.0f;
  for (int r0 = 0; r0 < p.Q; r0 += ROWS_THREADS) {
    const int q = p.Q - 1 - (r0 + tid);
    float v = q >= 0 ? s_dS[q] : 0.0f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
    if (lane == 31) wsum[wid] = v;
    __syncthreads();
    float off = carry;
    for (int j = 0; j < wid; ++j) off += wsum[j];
    v += off;
    if (q >= 0) {
      const int64_t idx = (tok0 + q) * p.H + h;
      if (p.dt) {
        const float ddt = fmaf(Ah, v, s_ddtx[q]);
        ddt_out[idx] = ddt; pA = fmaf(v, s_dt[q], pA); pD += s_dD[q];
        if (raw.hi) {      // through the softplus: d softplus(u) / du = sigmoid(u) = 1 - exp(-softplus(u))
          const float gr = ddt * (-expm1f(-s_dt[q]));
          const int64_t o = (tok0 + q) * raw.ld + raw.col0 + h;
          uint32_t hh, ll;
          split_bf16_pair(gr, hh, ll);
          raw.hi[o] = (uint16_t)hh;
          if (raw.lo) raw.lo[o] = (uint16_t)ll;
          pB += gr;
        }
      }
      else da_out[idx] = v;
    }
    float tot = carry;
    for (int j = 0; j < ROWS_THREADS / 32; ++j) tot += wsum[j];
    carry = tot;
    __syncthreads();
  }
  if (p.dt) {
    const float tA = block_sum(pA, red);
    const float tD = block_sum(pD, red);
    const float tB = block_sum(pB, red);
    if (tid == 0) {
      part[(int64_t)bc * p.H + h] = tA;
      part[(int64_t)p.B * p.nc * p.H + (int64_t)bc * p.H + h] = tD;
      part[2 * (int64_t)p.B * p.nc * p.H + (int64_t)bc * p.H + h] = tB;
    }
  }
}

// The per-head sums of the pair path in one launch: thread h adds the per-(b,c) partials of dA, dD and (when asked
// for) d_dt_bias in a fixed order; d_a_log = A dA.
__global__ void head_finish_kernel(const float* __restrict__ part, int rows, int H, const float* __restrict__ A, float* __restrict__ dA,
                                   float* __restrict__ dD, float* __restrict__ d_dt_bias, float* __restrict__ d_a_log) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float a = 0.0f, d = 0.0f, b = 0.0f;
  for (int r = 0; r < rows; ++r) {
    a += part[(int64_t)r * H + h];
    d += part[((int64_t)rows + r) * H + h];
    b += part[(2 * (int64_t)rows + r) * H + h];
  }
  dA[h] = a;
  if (dD) dD[h] = d;
  if (d_dt_bias) d_dt_bias[h] = b;
  if (d_a_log) d_a_log[h] = A[h] * a;
}

// Sums the split-K partial tiles in a fixed order.  mode 0: dG (lower-triangular 64x64 tiles only, the
// others were never produced); mode 1/2: dC/dB rows go to out + token * ld + g * cols.
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int nsplit, int rows, int cols, int mode, int G, int Q,
                                     float* __restrict__ out, int64_t ld, int64_t total, int tile, int accumulate,
                                     uint16_t* __restrict__ pair_hi, uint16_t* __restrict__ pair_lo) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  int64_t mn = (int64_t)rows * cols;
  int64_t batch = i / mn; int64_t r = i % mn; int m = (int)(r / cols), n = (int)(r % cols);
  if (mode == 0 && n / tile > m / tile) return;   // tiles above the diagonal were never produced
  float s = 0.0f;
  for (int k = 0; k < nsplit; ++k) s += part[(batch * nsplit + k) * mn + r];
  if (mode == 0 && pair_hi) {       // dG as a bf16 pair: it is only ever an operand of the dC / dB contractions
    uint32_t h, l;
    split_bf16_pair(s, h, l);
    pair_hi[batch * mn + r] = (uint16_t)h;
    if (pair_lo) pair_lo[batch * mn + r] = (uint16_t)l;
  } else if (mode == 0) {
    out[batch * mn + r] = accumulate ? out[batch * mn + r] + s : s;
  } else {
    int g = (int)(batch % G); int64_t bc = batch / G;
    out[(bc * Q + m) * ld + g * cols + n] = s;
  }
}

static int pick_nsplit(int batches, int tiles, int hpg) {
  int want = (int)cdiv(2 * 148, (int64_t)batches * tiles);
  if (want < 1) want = 1;
  return want > hpg ? hpg : want;
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static bool fused_enabled();

// Buffers of one scan.  part bit 0: what the forward writes and the backward reads (kept per forward slot by the
// block workspace); bit 1: what only the backward touches (one copy).  Fields of the other part are left alone.
void ssd_ws_take(Arena& ar, int B, int T, int H, int P, int N, int G, int Q, SsdWs* wp, int part) {
  SsdWs& w = *wp;
  const int nc = T / Q;
  const bool tcshape = Q % 64 == 0 && N % 32 == 0 && P % 64 == 0;
  const bool fz = ssd_fused_supported(P, N, Q, true) && fused_enabled();
  const size_t hp = (size_t)B * T * H * P, gn = (size_t)B * T * 2 * G * N, stn = (size_t)B * nc * H * N * P, qq = (size_t)B * nc * G * Q * Q;
  if (part & 1) {
    w.S = ar.take<float>((size_t)B * H * T);
    w.hprev = ar.take<float>(stn);
    w.hlast = ar.take<float>((size_t)B * H * N * P);
    if (!fz) w.CB = ar.take<float>(qq);
    w.xs = ar.take<float>((tcshape && !fz) ? hp : 0);
    w.xs_hi = fz ? ar.take<uint16_t>(hp) : nullptr; w.xs_lo = fz ? ar.take<uint16_t>(hp) : nullptr;
    // bf16 (hi, lo) pairs of the operands of the fused intra-chunk kernels, and the carried-state part of y
    w.xt_hi = fz ? ar.take<uint16_t>(hp) : nullptr; w.xt_lo = fz ? ar.take<uint16_t>(hp) : nullptr;
    w.bc_hi = fz ? ar.take<uint16_t>(gn) : nullptr; w.bc_lo = fz ? ar.take<uint16_t>(gn) : nullptr;
    w.hp_hi = fz ? ar.take<uint16_t>(stn) : nullptr; w.hp_lo = fz ? ar.take<uint16_t>(stn) : nullptr;
    w.yoff = fz ? ar.take<float>(hp) : nullptr;
  }
  if (part & 2) {
    if (fz) w.CB = ar.take<float>(qq);     // only for a backward that cannot take the fused kernel after a forward that did
    w.dh = ar.take<float>(stn);
    w.dG = ar.take<float>(qq);
    w.dxt = ar.take<float>(hp);
    w.rows = ar.take<float>((size_t)4 * B * T * H);
    w.part = ar.take<float>((size_t)B * nc * 3 * H);
    {
      int nbcg = B * nc * G, hpg = H / G, qt = (int)cdiv(Q, BM);
      size_t a = (size_t)pick_nsplit(nbcg, qt * (qt + 1) / 2, hpg) * nbcg * Q * Q;
      size_t b = (size_t)pick_nsplit(nbcg, qt * (int)cdiv(N, BN), hpg) * nbcg * Q * N;
      size_t need = a > b ? a : b;
      if (tcshape) {
        // tensor-core path: the head-split dB / dC partial tiles
        size_t dbc = (size_t)ssd_tc_dbc_nsplit_dims(B, T, H, N, G, Q) * nbcg * Q * N;
        if (dbc > need) need = dbc;
        size_t dgp = (size_t)ssd_tc_dg_nsplit_dims(B, T, H, G, Q) * nbcg * Q * Q;
        if (dgp > need) need = dgp;
      }
      if (fz) {
        // pair path: dC and dB run side by side, each with its own partial tiles
        size_t dbc2 = (size_t)2 * ssd_pairs_dbc_nsplit(B, T, H, N, G, Q) * nbcg * Q * N;
        if (dbc2 > need) need = dbc2;
        size_t dgp2 = (size_t)ssd_pairs_dg_nsplit(B, T, H, G, Q) * nbcg * Q * Q;
        if (dgp2 > need) need = dgp2;
      }
      w.splitk = ar.take<float>(need);
    }
    w.dys = ar.take<float>((tcshape && !fz) ? hp : 0);
    w.dys_hi = fz ? ar.take<uint16_t>(hp) : nullptr; w.dys_lo = fz ? ar.take<uint16_t>(hp) : nullptr;
    w.dg_hi = fz ? ar.take<uint16_t>(qq) : nullptr; w.dg_lo = fz ? ar.take<uint16_t>(qq) : nullptr;
    w.dy_hi = fz ? ar.take<uint16_t>(hp) : nullptr; w.dy_lo = fz ? ar.take<uint16_t>(hp) : nullptr;
    w.dh_hi = fz ? ar.take<uint16_t>(stn) : nullptr; w.dh_lo = fz ? ar.take<uint16_t>(stn) : nullptr;
    // the sums of W that the fused backward kernel leaves for the row-sum kernel
    w.csum = fz ? ar.take<float>((size_t)B * T * H) : nullptr;
    w.esum = fz ? ar.take<float>((size_t)B * T * H) : nullptr;
    w.rpart = fz ? ar.take<float>((size_t)B * T * H * (Q / 128)) : nullptr;
  }
}

size_t ssd_ws_layout(int B, int T, int H, int P, int N, int G, int Q, void* base, size_t bytes, SsdWs* out) {
  Arena ar(base, bytes);
  SsdWs w{};
  ssd_ws_take(ar, B, T, H, P, N, G, Q, &w, 3);
  if (out) *out = w;
  return ar.ok ? ar.used() : 0;
}

static pmb_status fill_params(const SsdIn& in, const SsdWs& ws, SsdP* pp) {
  if (in.Q <= 0 || in.T % in.Q != 0) return fail(PMB_ERR_SHAPE, "ssd: T=%d is not a multiple of block_len=%d", in.T, in.Q);
  if (!(in.G == 1 || in.G == in.H)) return fail(PMB_ERR_SHAPE, "ssd: n_groups must be 1 or n_heads");
  SsdP p{};
  p.B = in.B; p.T = in.T; p.H = in.H; p.P = in.P; p.N = in.N; p.G = in.G; p.Q = in.Q; p.nc = in.T / in.Q; p.hpg = in.H / in.G;
  p.x = in.x; p.ldx = in.ldx; p.dt = in.dt; p.A = in.A; p.a = in.a; p.b = in.b; p.c = in.c; p.ldbc = in.ldbc; p.D = in.D;
  p.S = ws.S; p.hprev = ws.hprev; p.hlast = ws.hlast; p.CB = ws.CB; p.dh = ws.dh; p.dG = ws.dG; p.dxt = ws.dxt;
  *pp = p;
  return PMB_OK;
}

template <class Op>
static pmb_status run_op(cudaStream_t st, const char* name, const Op& op, int batches, double flops) {
  ProfScope prof(st, name, flops, 0.0);
  return launch_bgemm(st, op, batches);
}

template <class Op>
static Op make_op(const SsdP& p, int Mdim, int Ndim) {
  Op op{};
  op.p = p; op.Mdim = Mdim; op.Ndim = Ndim;
  return op;
}

// ---------------------------------------------------------------------------------------------
// Independent kernels of one scan run side by side.  At training sizes of a few thousand tokens every kernel
// of the scan occupies the GPU for tens of microseconds with one or two ragged waves of latency-bound CTAs, so
// the chains that do not depend on each other (forward: C B^T next to x~ -> chunk states -> state pass;
// backward: dG -> dC -> dB next to dstates -> reverse pass -> dx~ -> row sums) go to two streams joined by events.
// One side stream and a handful of events per device, created on first use (make the first call outside stream
// capture).  PMB_SSD_CONCURRENT=0 keeps everything on the caller's stream.
// ---------------------------------------------------------------------------------------------
// lane 0 serves the backward, lane 2 the forward: a recompute may be in flight on another stream while the
// backward of the block above it runs, and the two must not share events
static pmb_status side_lane(int idx, SideLane** out) {
  static const int on = [] { const char* e = getenv("PMB_SSD_CONCURRENT"); return (e && e[0] == '0') ? 0 : 1; }();
  *out = nullptr;
  if (!on) return PMB_OK;
  return get_side_lane(idx, out);
}
static bool fused_enabled() {
  static const int on = [] { const char* e = getenv("PMB_SSD_FUSED"); return (e && e[0] == '0') ? 0 : 1; }();
  return on != 0;
}

// x~[b,t,h,:] = x[b,t,h,:] * dt[b,t,h] as a bf16 pair (only when the fused cumsum kernel did not already write it)
__global__ void __launch_bounds__(256) xt_pair_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ dt,
                                                      uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, int64_t rows, int H, int P,
                                                      const float* __restrict__ S, int T, int Q, uint16_t* __restrict__ xs_hi, uint16_t* __restrict__ xs_lo) {
  const int P4 = P >> 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * H * P4) return;
  const int j = (int)(i % P4); const int64_t w = i / P4; const int h = (int)(w % H); const int64_t tk = w / H;
  const float f = dt ? dt[tk * H + h] : 1.0f;
  const float4 v = reinterpret_cast<const float4*>(x + tk * ldx + h * P)[j];
  const int64_t o = (tk * H + h) * (int64_t)P + 4 * j;
  store_pair4(hi + o, lo ? lo + o : nullptr, v.x * f, v.y * f, v.z * f, v.w * f);      // (lo == NULL: the hi halves alone are read)
  // xs = x~ exp(S_end - S_t): the operand of the chunk-state and dB contractions
  const int b = (int)(tk / T), t = (int)(tk % T);
  const float* sp = S + ((int64_t)b * H + h) * T;
  const float f2 = f * __expf(sp[(t / Q) * Q + Q - 1] - sp[t]);
  store_pair4(xs_hi + o, xs_lo ? xs_lo + o : nullptr, v.x * f2, v.y * f2, v.z * f2, v.w * f2);
}

// The B and C columns (adjacent in the caller's buffer when it is the block's activation buffer, else two arrays)
// as bf16 pairs with row pitch 2*G*N: B in columns [0, G*N), C in [G*N, 2*G*N).
static pmb_status fused_operand_pairs(cudaStream_t st, const SsdIn& in, const SsdWs& ws, bool want_xt) {
  const int64_t rows = (int64_t)in.B * in.T;
  const int gn = in.G * in.N;
  if (in.bc_pair_ready) {
    // written by the producer of B and C
  } else if (in.c == in.b + gn) {
    PMB_TRY(split_pair16(st, in.b, rows, 2 * gn, in.ldbc, ws.bc_hi, ws.bc_lo, 2 * gn));
  } else {
    ProfScope prof(st, "split_f32_bf16x2", 0.0, 16.0 * rows * gn);
    PMB_TRY(split_pair16_strided(st, in.b, rows, gn, in.ldbc, ws.bc_hi, ws.bc_lo, 2 * gn));
    PMB_TRY(split_pair16_strided(st, in.c, rows, gn, in.ldbc, ws.bc_hi + gn, ws.bc_lo + gn, 2 * gn));
  }
  if (want_xt) {
    ProfScope prof(st, "ssd_xt_pair", 0.0, (in.plain16 ? 8.0 : 12.0) * rows * in.H * in.P);
    xt_pair_kernel<<<(unsigned)cdiv(rows * in.H * (in.P / 4), 256), 256, 0, st>>>(in.x, in.ldx, in.dt, ws.xt_hi, in.plain16 ? nullptr : ws.xt_lo, rows,
                                                                                  in.H, in.P, ws.S, in.T, in.Q, ws.xs_hi, in.plain16 ? nullptr : ws.xs_lo);
    PMB_LAUNCHED();
  }
  return PMB_OK;
}

static FusedArgs fused_args(const SsdIn& in, const SsdWs& ws) {
  FusedArgs fa{};
  fa.B = in.B; fa.T = in.T; fa.H = in.H; fa.P = in.P; fa.N = in.N; fa.G = in.G; fa.Q = in.Q;
  fa.S = ws.S;
  const int64_t pitch = 2 * (int64_t)in.G * in.N;
  const bool pairs = ws.bc_lo && !in.plain16;
  fa.b = Op16{ws.bc_hi, pairs ? ws.bc_lo : nullptr, pitch};
  fa.c = Op16{ws.bc_hi + in.G * in.N, pairs ? ws.bc_lo + in.G * in.N : nullptr, pitch};
  return fa;
}

pmb_status ssd_fwd(cudaStream_t st, const SsdIn& in, const float* init_state, float* y, int64_t ldy, float* final_state,
                   const SsdWs& ws) {
  SsdP p;
  PMB_TRY(fill_params(in, ws, &p));
  p.yout = y; p.ldyo = ldy;
  int nbch = p.B * p.nc * p.H, nbcg = p.B * p.nc * p.G;
  const double tok = (double)p.B * p.T;
  const bool tc = ssd_tc_supported(in) && (ldy % 4 == 0) && (reinterpret_cast<uintptr_t>(y) % 16 == 0);
  // the intra-chunk chain C B^T -> mask -> x x~ (+ the carried-state term) as one tcgen05 kernel on bf16 pairs
  const bool fz = tc && fused_enabled() && ssd_fused_supported(p.P, p.N, p.Q, true);
  SsdIn in_tc = in;
  bool xt_ready = false;
  {
    CumsumRaw raw{in.dt_raw, in.ld_raw, in.dt_bias, in.a_log, const_cast<float*>(in.dt), const_cast<float*>(in.A)};
    if (in.dt_raw && (!in.dt || !in.A || !in.dt_bias || !in.a_log)) return fail(PMB_ERR_ARG, "ssd: dt_raw needs dt, A, dt_bias and a_log");
    // (one block per (b,c,h): worth it while those blocks fit the machine at once; beyond that the two separate,
    // finer-grained kernels use the memory system better)
    if (tc && nbch <= 4 * 148 && p.Q <= PREP_MAX_Q && (in.ldx % 4 == 0) && (reinterpret_cast<uintptr_t>(in.x) % 16 == 0)) {
      ProfScope prof(st, "ssd_chunk_prepare", 0.0, 8.0 * tok * p.H * (1.0 + p.P));
      // at a few hundred (b,c,h) the second phase (the only one with real traffic) is short of threads: split its rows
      const unsigned ysplit = nbch <= 148 ? 4u : (nbch <= 2 * 148 ? 2u : 1u);
      chunk_prepare_kernel<<<dim3((unsigned)nbch, ysplit), PREP_THREADS, 0, st>>>(p, raw, ws.xs, fz ? ws.xt_hi : nullptr, in.plain16 ? nullptr : ws.xt_lo, fz ? ws.xs_hi : nullptr,
                                                                                  in.plain16 ? nullptr : ws.xs_lo);
      PMB_LAUNCHED();
      in_tc.xs_ready = true;
      xt_ready = fz;
    } else {
      ProfScope prof(st, "ssd_chunk_cumsum", 0.0, 8.0 * tok * p.H);
      chunk_cumsum_kernel<<<(unsigned)cdiv((int64_t)nbch * 32, 256), 256, 0, st>>>(p, raw);
      PMB_LAUNCHED();
    }
  }
  SideLane* lane = nullptr;
  if (tc && !fz) PMB_TRY(side_lane(2, &lane));      // (the pair path is one chain: nothing to run beside it)
  if (fz) {
    // every contraction reads bf16 pairs: B | C and x~ / xs come from their producers, or are split here
    if (!in.bc_pair_ready || !xt_ready) PMB_TRY(fused_operand_pairs(st, in, ws, !xt_ready));
    PMB_TRY(ssd_pairs_state(st, in, ws, 0));
  } else if (tc) {
    cudaStream_t sb = lane ? lane->s : st;
    if (lane) PMB_TRY(order_after(st, lane->ev[0], sb));     // S is ready
    PMB_TRY(ssd_tc_cb(sb, in, ws));
    PMB_TRY(ssd_tc_state(st, in_tc, ws));
  } else {
    PMB_TRY(run_op(st, "ssd_cb", make_op<OpCB>(p, p.Q, p.Q), nbcg, 2.0 * tok * p.Q * p.N * p.G));
    PMB_TRY(run_op(st, "ssd_chunk_state", make_op<OpState>(p, p.N, p.P), nbch, 2.0 * tok * p.H * p.N * p.P));
  }
  int64_t nel = (int64_t)p.B * p.H * p.N * p.P;
  {
    ProfScope prof(st, "ssd_state_pass", 0.0, 8.0 * nel * p.nc);
    PMB_TRY(launch_state_scan(st, p, p.hprev, init_state, p.hlast, 0, fz ? ws.hp_hi : nullptr, in.plain16 ? nullptr : ws.hp_lo));
  }
  if (lane) PMB_TRY(order_after(lane->s, lane->ev[1], st));   // C B^T (or the operand pairs) are ready
  if (fz) {
    FusedArgs fa = fused_args(in, ws);
    fa.v = Op16{ws.xt_hi, in.plain16 ? nullptr : ws.xt_lo, (int64_t)p.H * p.P};
    fa.state = Op16{ws.hp_hi, in.plain16 ? nullptr : ws.hp_lo, p.P};
    fa.out = y; fa.ldo = ldy; fa.x = in.x; fa.ldx = in.ldx; fa.D = in.D;
    fa.off_out = ws.yoff;
    PMB_TRY(ssd_fused(st, 0, fa));
  }
  else if (tc) PMB_TRY(ssd_tc_scan(st, in, y, ldy, ws));
  else PMB_TRY(run_op(st, "ssd_chunk_scan", make_op<OpScan>(p, p.Q, p.P), nbch, 2.0 * tok * p.H * p.P * (p.Q + p.N)));
  if (final_state) PMB_CUDA(cudaMemcpyAsync(final_state, ws.hlast, (size_t)nel * sizeof(float), cudaMemcpyDeviceToDevice, st));
  return PMB_OK;
}

// dYs[b,t,h,:] = dY[b,t,h,:] exp(S[b,h,t]) as a bf16 pair (when the producer of dY did not already write it)
__global__ void __launch_bounds__(256) dys_pair_kernel(const float* __restrict__ dy, int64_t lddy, const float* __restrict__ S,
                                                       uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, int64_t rows, int T, int H, int P) {
  const int P4 = P >> 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * H * P4) return;
  const int j = (int)(i % P4); const int64_t w = i / P4; const int h = (int)(w % H); const int64_t tk = w / H;
  const float f = __expf(S[((tk / T) * H + h) * T + tk % T]);
  const float4 v = reinterpret_cast<const float4*>(dy + tk * lddy + h * P)[j];
  const int64_t o = (tk * H + h) * (int64_t)P + 4 * j;
  store_pair4(hi + o, lo ? lo + o : nullptr, v.x * f, v.y * f, v.z * f, v.w * f);
}

bool ssd_bwd_takes_pairs(const SsdIn& in, const float* dy, int64_t lddy, const SsdGrads& g) {
  const bool tc = ssd_tc_supported(in) && (lddy % 4 == 0) && (reinterpret_cast<uintptr_t>(dy) % 16 == 0) && (g.lddbc % 4 == 0) &&
                  ((reinterpret_cast<uintptr_t>(g.db) | reinterpret_cast<uintptr_t>(g.dc)) % 16 == 0);
  return tc && fused_enabled() && ssd_fused_supported(in.P, in.N, in.Q, true) && (g.lddx % 4 == 0) && (reinterpret_cast<uintptr_t>(g.dx) % 16 == 0);
}

pmb_status ssd_bwd(cudaStream_t st, const SsdIn& in, const float* y, int64_t ldy, const float* dy, int64_t lddy,
                   const SsdGrads& g, const SsdWs& ws) {
  SsdP p;
  PMB_TRY(fill_params(in, ws, &p));
  p.y = y; p.ldy = ldy; p.dy = dy; p.lddy = lddy; p.db = g.db; p.dc = g.dc; p.lddbc = g.lddbc;
  int nbch = p.B * p.nc * p.H, nbcg = p.B * p.nc * p.G;
  int64_t rows = (int64_t)p.B * p.T * p.H;
  float* ddt_x = ws.rows; float* dS = ws.rows + rows; float* dDrow = ws.rows + 2 * rows; float* dsend = ws.rows + 3 * rows;
  const double tok = (double)p.B * p.T;
  const bool tc = ssd_tc_supported(in) && (lddy % 4 == 0) && (reinterpret_cast<uintptr_t>(dy) % 16 == 0) && (g.lddbc % 4 == 0) &&
                  ((reinterpret_cast<uintptr_t>(g.db) | reinterpret_cast<uintptr_t>(g.dc)) % 16 == 0);
  const bool tc_group = tc;
  const bool fz = ssd_bwd_takes_pairs(in, dy, lddy, g);
  SideLane* lane = nullptr;
  if (tc) PMB_TRY(side_lane(0, &lane));
  cudaStream_t sb = lane ? lane->s : st;                      // stream of the dG -> dC -> dB chain
  if (fz) {
    // both chains read dY (and dY exp(S)) as bf16 pairs: written by the producer of dY, or here
    const int64_t tokens = (int64_t)p.B * p.T;
    if (!in.dy_pair_ready) PMB_TRY(split_pair16(st, dy, tokens, p.H * p.P, lddy, ws.dy_hi, ws.dy_lo, (int64_t)p.H * p.P));
    if (!in.dys_ready) {
      ProfScope prof(st, "ssd_prescale_dy", 0.0, 8.0 * tokens * p.H * p.P);
      dys_pair_kernel<<<(unsigned)cdiv(tokens * p.H * (p.P / 4), 256), 256, 0, st>>>(dy, lddy, ws.S, ws.dys_hi, ws.dys_lo, tokens, p.T, p.H, p.P);
      PMB_LAUNCHED();
    }
  }
  if (lane) PMB_TRY(order_after(st, lane->ev[0], sb));        // inputs of the scan are ready
  if (fz) {
    PMB_TRY(ssd_pairs_state(st, in, ws, 1));
  } else if (tc) {
    PMB_TRY(ssd_tc_dstate(st, in, dy, lddy, ws));
  } else {
    PMB_TRY(run_op(st, "ssd_bwd_dstate", make_op<OpDstate>(p, p.N, p.P), nbch, 2.0 * tok * p.H * p.N * p.P));
  }
  if (lane) PMB_CUDA(cudaEventRecord(lane->ev[1], st));       // dY exp(S) is ready (dC reads it)
  {
    ProfScope prof(st, "ssd_bwd_state_pass", 0.0, 12.0 * p.B * p.H * p.N * p.P * p.nc);
    uint16_t* const dh_lo = in.plain16 ? nullptr : ws.dh_lo;
    if (fz && launch_state_scan_rev_dot(st, p, p.dh, ws.dh_hi, dh_lo, dsend)) {
      PMB_LAUNCHED();
    } else {
      PMB_TRY(launch_state_scan(st, p, p.dh, nullptr, nullptr, 1, fz ? ws.dh_hi : nullptr, dh_lo));
      state_dot_kernel<<<(unsigned)nbch, 256, 0, st>>>(p, dsend, fz ? 1 : 0);
      PMB_LAUNCHED();
    }
  }
  if (lane) PMB_CUDA(cudaEventRecord(lane->ev[2], st));       // dh is ready (dB reads it)
  if (fz) {
    // dY as a bf16 pair (the B / C / x~ pairs were written by the forward of this scan and are still in the workspace)
    FusedArgs fa = fused_args(in, ws);
    fa.v = Op16{ws.dy_hi, in.plain16 ? nullptr : ws.dy_lo, (int64_t)p.H * p.P};
    fa.state = Op16{ws.dh_hi, in.plain16 ? nullptr : ws.dh_lo, p.P};
    fa.out = p.dxt; fa.ldo = (int64_t)p.H * p.P;
    fa.xt = Op16{ws.xt_hi, in.plain16 ? nullptr : ws.xt_lo, (int64_t)p.H * p.P};
    fa.csum = ws.csum; fa.esum = ws.esum; fa.rpart = ws.rpart;
    PMB_TRY(ssd_fused(st, 1, fa));
  }
  else if (tc) {
    // (a forward that took the fused kernel left no C B^T behind: form it now)
    if (fused_enabled() && ssd_fused_supported(p.P, p.N, p.Q, true)) PMB_TRY(ssd_tc_cb(st, in, ws));
    PMB_TRY(ssd_tc_dx(st, in, dy, lddy, ws));
  }
  else PMB_TRY(run_op(st, "ssd_bwd_dx", make_op<OpDx>(p, p.Q, p.P), nbch, 2.0 * tok * p.H * p.P * (p.Q + p.N)));
  {
    ProfScope prof(st, "ssd_bwd_rows", 0.0, 4.0 * tok * p.H * (5.0 * p.P + 8.0));
    const bool vec_ok = (p.P % 4 == 0) && (p.ldx % 4 == 0) && (p.ldy % 4 == 0) && (p.lddy % 4 == 0) && (g.lddx % 4 == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.y) | reinterpret_cast<uintptr_t>(p.dy) |
                          reinterpret_cast<uintptr_t>(g.dx) | reinterpret_cast<uintptr_t>(p.dxt)) % 16 == 0);
    if (fz) {
      WSums wsm{ws.rpart, ws.csum, ws.esum, ws.yoff, p.Q / 128};
      chunk_rows_finish_w_kernel<false><<<(unsigned)nbch, ROWS_THREADS, 0, st>>>(p, wsm, g.dx, g.lddx, dsend, g.da, g.ddt, ws.part, in.dt ? g.raw : SsdGrads::RawDt{}, nullptr);
      PMB_LAUNCHED();
    } else if (vec_ok && nbch <= 4 * 148 && p.Q <= PREP_MAX_Q) {
      chunk_rows_finish_kernel<<<(unsigned)nbch, PREP_THREADS, 0, st>>>(p, g.dx, g.lddx, dsend, g.da, g.ddt, ws.part);
      PMB_LAUNCHED();
    } else {
      ssd_rowdots_kernel<<<(unsigned)cdiv(rows * 32, 256), 256, 0, st>>>(p, g.dx, g.lddx, ddt_x, dS, dDrow);
      PMB_LAUNCHED();
      ssd_chunk_finish_kernel<<<(unsigned)cdiv((int64_t)nbch * 32, 256), 256, 0, st>>>(p, ddt_x, dS, dDrow, dsend, g.da, g.ddt, ws.part);
      PMB_LAUNCHED();
    }
  }
  auto head_sums = [&](cudaStream_t s) -> pmb_status {   // part = [dA partials (B*nc,H)] [dD partials (B*nc,H)] [d_dt_bias partials]
    if (!in.dt) return PMB_OK;
    if (fz) {
      head_finish_kernel<<<(unsigned)cdiv(p.H, 128), 128, 0, s>>>(ws.part, p.B * p.nc, p.H, in.A, g.dA, g.dD, g.raw.hi ? g.raw.d_dt_bias : nullptr,
                                                                  g.raw.hi ? g.raw.d_a_log : nullptr);
      PMB_LAUNCHED();
      return PMB_OK;
    }
    PMB_TRY(column_sum(s, ws.part, (int64_t)p.B * p.nc, p.H, g.dA));
    if (g.dD) PMB_TRY(column_sum(s, ws.part + (int64_t)p.B * p.nc * p.H, (int64_t)p.B * p.nc, p.H, g.dD));
    return PMB_OK;
  };
  // the two tiny per-head reductions ride at the end of the side chain instead of holding up the caller's stream
  if (lane && tc_group) PMB_CUDA(cudaEventRecord(lane->ev[4], st));
  else PMB_TRY(head_sums(st));
  // The three per-group contractions sum over the heads of the group; with few (batch, chunk) pairs the
  // head loop is split across CTAs and the partial tiles are summed in a fixed order afterwards.
  const int qt = (int)cdiv(p.Q, BM);
  auto reduce = [&](int nsplit, int cols, int mode, float* out, int64_t ld, int tile = BM, cudaStream_t rs = nullptr,
                    const float* part = nullptr) -> pmb_status {
    if (nsplit <= 1) return PMB_OK;
    int64_t total = (int64_t)nbcg * p.Q * cols;
    splitk_reduce_kernel<<<(unsigned)cdiv(total, 256), 256, 0, rs ? rs : (tc_group ? sb : st)>>>(part ? part : ws.splitk, nsplit, p.Q, cols, mode, p.G, p.Q, out, ld, total, tile, 0,
                                                                                     (mode == 0 && fz) ? ws.dg_hi : nullptr, ws.dg_lo);
    PMB_LAUNCHED();
    return PMB_OK;
  };
  if (fz) {
    {
      ProfScope prof(sb, "ssd_bwd_dg_pair", 2.0 * tok * p.H * p.Q * p.P, 0.0);
      const int nsg = ssd_pairs_dg_nsplit(p.B, p.T, p.H, p.G, p.Q);
      PMB_TRY(ssd_pairs_dg(sb, in, ws, nsg));
      PMB_TRY(reduce(nsg, p.Q, 0, ws.dG, 0, 128));
    }
    const int ns = ssd_pairs_dbc_nsplit(p.B, p.T, p.H, p.N, p.G, p.Q);
    // dC and dB both wait for dG only: they run side by side, each with its own partial tiles
    SideLane* lane_b = nullptr;
    if (lane) PMB_TRY(side_lane(5, &lane_b));
    if (lane_b) PMB_CUDA(cudaEventRecord(lane->ev[5], sb));               // dG and its pair are ready
    {
      if (lane) PMB_CUDA(cudaStreamWaitEvent(sb, lane->ev[1], 0));       // (the forward's h_prev pair is long there)
      ProfScope prof(sb, "ssd_bwd_dc_pair", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
      PMB_TRY(ssd_pairs_dbc(sb, in, ws, 0, g.dc, g.lddbc, ns, ws.splitk));
      PMB_TRY(reduce(ns, p.N, 1, g.dc, g.lddbc));
    }
    {
      cudaStream_t sdb = lane_b ? lane_b->s : sb;
      float* part_b = lane_b ? ws.splitk + (size_t)ns * nbcg * p.Q * p.N : ws.splitk;
      if (lane_b) PMB_CUDA(cudaStreamWaitEvent(sdb, lane->ev[5], 0));
      if (lane) PMB_CUDA(cudaStreamWaitEvent(sdb, lane->ev[2], 0));      // dh and its pair are ready
      ProfScope prof(sdb, "ssd_bwd_db_pair", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
      PMB_TRY(ssd_pairs_dbc(sdb, in, ws, 1, g.db, g.lddbc, ns, part_b));
      PMB_TRY(reduce(ns, p.N, 2, g.db, g.lddbc, BM, sdb, part_b));
    }
    if (lane_b) PMB_TRY(order_after(lane_b->s, lane_b->ev[0], sb));
    if (lane) {
      PMB_CUDA(cudaStreamWaitEvent(sb, lane->ev[4], 0));
      PMB_TRY(head_sums(sb));
      PMB_TRY(order_after(sb, lane->ev[3], st));               // join
    }
    return PMB_OK;
  }
  if (tc_group) {
    {
      ProfScope prof(sb, "ssd_bwd_dg_tc", 2.0 * tok * p.H * p.Q * p.P, 0.0);
      const int nsg = ssd_tc_dg_nsplit_dims(p.B, p.T, p.H, p.G, p.Q);
      PMB_TRY(ssd_tc_dg(sb, in, dy, lddy, ws, nsg));
      PMB_TRY(reduce(nsg, p.Q, 0, ws.dG, 0, 128));
    }
    const int ns = ssd_tc_dbc_nsplit(in);
    {
      if (lane) PMB_CUDA(cudaStreamWaitEvent(sb, lane->ev[1], 0));
      ProfScope prof(sb, "ssd_bwd_dc_tc", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
      PMB_TRY(ssd_tc_dc(sb, in, g.dc, g.lddbc, ws, ns));
      PMB_TRY(reduce(ns, p.N, 1, g.dc, g.lddbc));
    }
    {
      if (lane) PMB_CUDA(cudaStreamWaitEvent(sb, lane->ev[2], 0));
      ProfScope prof(sb, "ssd_bwd_db_tc", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
      PMB_TRY(ssd_tc_db(sb, in, g.db, g.lddbc, ws, ns));
      PMB_TRY(reduce(ns, p.N, 2, g.db, g.lddbc));
    }
    if (lane) {
      PMB_CUDA(cudaStreamWaitEvent(sb, lane->ev[4], 0));
      PMB_TRY(head_sums(sb));
      PMB_TRY(order_after(sb, lane->ev[3], st));               // join
    }
    return PMB_OK;
  }
  {
    OpDG op = make_op<OpDG>(p, p.Q, p.Q);
    op.nsplit = pick_nsplit(nbcg, qt * (qt + 1) / 2, p.hpg); op.part = ws.splitk;
    ProfScope prof(st, "ssd_bwd_dg", 2.0 * tok * p.H * p.Q * p.P, 0.0);
    PMB_TRY(launch_bgemm(st, op, nbcg * op.nsplit));
    PMB_TRY(reduce(op.nsplit, p.Q, 0, ws.dG, 0));
  }
  {
    OpDC op = make_op<OpDC>(p, p.Q, p.N);
    op.nsplit = pick_nsplit(nbcg, qt * (int)cdiv(p.N, BN), p.hpg); op.part = ws.splitk;
    ProfScope prof(st, "ssd_bwd_dc", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
    PMB_TRY(launch_bgemm(st, op, nbcg * op.nsplit));
    PMB_TRY(reduce(op.nsplit, p.N, 1, g.dc, g.lddbc));
  }
  {
    OpDB op = make_op<OpDB>(p, p.Q, p.N);
    op.nsplit = pick_nsplit(nbcg, qt * (int)cdiv(p.N, BN), p.hpg); op.part = ws.splitk;
    ProfScope prof(st, "ssd_bwd_db", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
    PMB_TRY(launch_bgemm(st, op, nbcg * op.nsplit));
    PMB_TRY(reduce(op.nsplit, p.N, 2, g.db, g.lddbc));
  }
  return PMB_OK;
}

// ---------------------------------------------------------------------------------------------
// The scan on bf16 inputs as they are (the bf16-storage mode of the block, mamba2/block.rs:203-208: x, B, C in
// bf16, the recurrence in fp32).  x, B, C and dY go to the tensor cores as plain bf16 operands (one MMA per
// product instead of the three of an fp32 pair), a, S, the chunk states and every accumulator stay fp32, y and dx
// leave the fused kernels as bf16.  No fp32 copy of any (B,T,H,P) tensor is made.
// ---------------------------------------------------------------------------------------------

// dst[tk,h,:] = bf16(src[tk,h,:] * f):  mode 0: f = exp(S_end - S_t) (operand of the chunk states and of dB),
// mode 1: f = exp(S_t) (operand of d(states) and of dC).  Eight elements per thread.  `keep` (optional) receives a copy of src.
__global__ void __launch_bounds__(256) scale_rows16_kernel(const uint16_t* __restrict__ src, const float* __restrict__ S,
                                                           uint16_t* __restrict__ dst, uint16_t* __restrict__ keep, int64_t rows, int T, int H,
                                                           int P, int Q, int mode) {
  const int P8 = P >> 3;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * H * P8) return;
  const int j = (int)(i % P8); const int64_t w = i / P8; const int h = (int)(w % H); const int64_t tk = w / H;
  const int t = (int)(tk % T);
  const float* sp = S + ((tk / T) * H + h) * T;
  const float f = mode == 0 ? __expf(sp[(t / Q) * Q + Q - 1] - sp[t]) : __expf(sp[t]);
  const int64_t o = (tk * H + h) * (int64_t)P + 8 * j;
  const uint4 v = *reinterpret_cast<const uint4*>(src + o);
  if (keep) *reinterpret_cast<uint4*>(keep + o) = v;      // the unscaled values, for the backward
  const uint32_t in[4] = {v.x, v.y, v.z, v.w};
  uint32_t out[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(__uint_as_float(in[e] << 16) * f, __uint_as_float(in[e] & 0xffff0000u) * f);
    out[e] = *reinterpret_cast<const uint32_t*>(&r);
  }
  *reinterpret_cast<uint4*>(dst + o) = make_uint4(out[0], out[1], out[2], out[3]);
}

bool ssd16_supported(int B, int T, int H, int P, int N, int G, int Q) {
  if (!fused_enabled() || !ssd_fused_supported(P, N, Q, false) || P != 64) return false;
  if (Q <= 0 || T % Q != 0 || Q > PREP_MAX_Q || !(G == 1 || G == H)) return false;
  if (T / Q > SCAN_DOT_MAX_NC || (int64_t)N * P / 4 > 4 * 1024) return false;        // the one-launch reverse scan
  return (int64_t)B * T < (1LL << 31) && (int64_t)B * (T / Q) * H * N < (1LL << 31);
}

// Workspace of the bf16-input scan: the fields of SsdWs that its kernels touch (every *_lo stays NULL, which is how the
// contractions know that the operands are plain bf16), plus fp32 landing buffers for dB and dC.
size_t ssd16_ws_layout(int B, int T, int H, int P, int N, int G, int Q, void* base, size_t bytes, SsdWs* out, float** db32, float** dc32) {
  Arena ar(base, bytes);
  SsdWs w{};
  const int nc = T / Q;
  const size_t hp = (size_t)B * T * H * P, gn = (size_t)B * T * G * N, stn = (size_t)B * nc * H * N * P, qq = (size_t)B * nc * G * Q * Q;
  const size_t bth = (size_t)B * T * H;
  w.S = ar.take<float>(bth);
  w.hprev = ar.take<float>(stn);
  w.hlast = ar.take<float>((size_t)B * H * N * P);
  w.xs_hi = ar.take<uint16_t>(hp);
  w.xt_hi = ar.take<uint16_t>(hp);
  w.bc_hi = ar.take<uint16_t>(2 * gn);
  w.hp_hi = ar.take<uint16_t>(stn);
  w.yoff = reinterpret_cast<float*>(ar.take<uint16_t>(hp));      // holds bf16 here
  w.dh = ar.take<float>(stn);
  w.rows = ar.take<float>(bth);
  w.part = ar.take<float>((size_t)B * nc * 3 * H);
  {
    const size_t nbcg = (size_t)B * nc * G;
    const size_t dbc = (size_t)ssd_pairs_dbc_nsplit(B, T, H, N, G, Q) * nbcg * Q * N;
    const size_t dgp = (size_t)ssd_pairs_dg_nsplit(B, T, H, G, Q) * nbcg * Q * Q;
    w.splitk = ar.take<float>(dbc > dgp ? dbc : dgp);
  }
  w.dys_hi = ar.take<uint16_t>(hp);
  w.dg_hi = ar.take<uint16_t>(qq);
  w.dh_hi = ar.take<uint16_t>(stn);
  w.csum = ar.take<float>(bth);
  w.esum = ar.take<float>(bth);
  w.rpart = ar.take<float>(bth * (Q / 128));
  float* b32 = ar.take<float>(gn);
  float* c32 = ar.take<float>(gn);
  if (out) *out = w;
  if (db32) *db32 = b32;
  if (dc32) *dc32 = c32;
  return ar.ok ? ar.used() : 0;
}

static SsdIn ssd16_in(int B, int T, int H, int P, int N, int G, int Q, const float* a) {
  SsdIn in{};
  in.B = B; in.T = T; in.H = H; in.P = P; in.N = N; in.G = G; in.Q = Q;
  in.ldx = (int64_t)H * P; in.a = a; in.ldbc = (int64_t)G * N;
  return in;
}

pmb_status ssd16_fwd(cudaStream_t st, int B, int T, int H, int P, int N, int G, int Q, const uint16_t* x, const float* a,
                     const uint16_t* b, const uint16_t* c, const float* init_state, uint16_t* y, float* final_state, const SsdWs& ws) {
  const SsdIn in = ssd16_in(B, T, H, P, N, G, Q, a);
  SsdP p;
  PMB_TRY(fill_params(in, ws, &p));
  const int nbch = p.B * p.nc * p.H;
  const int64_t tok = (int64_t)B * T, hp = (int64_t)H * P, gn = (int64_t)G * N;
  {
    ProfScope prof(st, "ssd_chunk_cumsum", 0.0, 8.0 * tok * p.H);
    chunk_cumsum_kernel<<<(unsigned)cdiv((int64_t)nbch * 32, 256), 256, 0, st>>>(p, CumsumRaw{});
    PMB_LAUNCHED();
  }
  {
    // B | C side by side (the layout every contraction's tensor maps describe)
    ProfScope prof(st, "ssd16_keep_bc", 0.0, 8.0 * tok * gn);
    PMB_CUDA(cudaMemcpy2DAsync(ws.bc_hi, (size_t)(4 * gn), b, (size_t)(2 * gn), (size_t)(2 * gn), (size_t)tok, cudaMemcpyDeviceToDevice, st));
    PMB_CUDA(cudaMemcpy2DAsync(ws.bc_hi + gn, (size_t)(4 * gn), c, (size_t)(2 * gn), (size_t)(2 * gn), (size_t)tok, cudaMemcpyDeviceToDevice, st));
  }
  {
    ProfScope prof(st, "ssd16_prescale_x", 0.0, 6.0 * tok * hp);      // (also keeps x for the backward, which is not handed x again)
    scale_rows16_kernel<<<(unsigned)cdiv(tok * H * (P / 8), 256), 256, 0, st>>>(x, ws.S, ws.xs_hi, ws.xt_hi, tok, T, H, P, Q, 0);
    PMB_LAUNCHED();
  }
  PMB_TRY(ssd_pairs_state(st, in, ws, 0));
  {
    ProfScope prof(st, "ssd_state_pass", 0.0, 8.0 * (double)p.B * p.H * p.N * p.P * p.nc);
    PMB_TRY(launch_state_scan(st, p, p.hprev, init_state, p.hlast, 0, ws.hp_hi, nullptr));
  }
  FusedArgs fa = fused_args(in, ws);
  fa.v = Op16{ws.xt_hi, nullptr, hp};
  fa.state = Op16{ws.hp_hi, nullptr, p.P};
  fa.out16 = y; fa.ldo = hp;
  fa.off_out16 = reinterpret_cast<uint16_t*>(ws.yoff);
  PMB_TRY(ssd_fused(st, 0, fa));
  if (final_state) PMB_CUDA(cudaMemcpyAsync(final_state, ws.hlast, (size_t)p.B * p.H * p.N * p.P * sizeof(float), cudaMemcpyDeviceToDevice, st));
  return PMB_OK;
}

pmb_status ssd16_bwd(cudaStream_t st, int B, int T, int H, int P, int N, int G, int Q, const float* a, const uint16_t* dy,
                     uint16_t* dx, float* da, uint16_t* db, uint16_t* dc, const SsdWs& ws_in, float* db32, float* dc32) {
  const SsdIn in = ssd16_in(B, T, H, P, N, G, Q, a);
  SsdWs ws = ws_in;
  ws.dy_hi = const_cast<uint16_t*>(dy); ws.dy_lo = nullptr;
  SsdP p;
  PMB_TRY(fill_params(in, ws, &p));
  const int nbch = p.B * p.nc * p.H, nbcg = p.B * p.nc * p.G;
  const int64_t tok = (int64_t)B * T, hp = (int64_t)H * P, gn = (int64_t)G * N;
  float* dsend = ws.rows;
  {
    ProfScope prof(st, "ssd16_prescale_dy", 0.0, 4.0 * tok * hp);
    scale_rows16_kernel<<<(unsigned)cdiv(tok * H * (P / 8), 256), 256, 0, st>>>(dy, ws.S, ws.dys_hi, nullptr, tok, T, H, P, Q, 1);
    PMB_LAUNCHED();
  }
  PMB_TRY(ssd_pairs_state(st, in, ws, 1));
  {
    ProfScope prof(st, "ssd_bwd_state_pass", 0.0, 12.0 * p.B * p.H * p.N * p.P * p.nc);
    if (!launch_state_scan_rev_dot(st, p, p.dh, ws.dh_hi, nullptr, dsend)) return fail(PMB_ERR_UNSUPPORTED, "ssd16: reverse scan shape");
    PMB_LAUNCHED();
  }
  {
    FusedArgs fa = fused_args(in, ws);
    fa.v = Op16{dy, nullptr, hp};
    fa.state = Op16{ws.dh_hi, nullptr, p.P};
    fa.out16 = dx; fa.ldo = hp;
    fa.xt = Op16{ws.xt_hi, nullptr, hp};
    fa.csum = ws.csum; fa.esum = ws.esum; fa.rpart = ws.rpart;
    PMB_TRY(ssd_fused(st, 1, fa));
  }
  {
    ProfScope prof(st, "ssd_bwd_rows", 0.0, tok * p.H * (6.0 * p.P + 32.0));
    WSums wsm{ws.rpart, ws.csum, ws.esum, ws.yoff, p.Q / 128};
    chunk_rows_finish_w_kernel<true><<<(unsigned)nbch, ROWS_THREADS, 0, st>>>(p, wsm, nullptr, 0, dsend, da, nullptr, ws.part, SsdGrads::RawDt{}, dy);
    PMB_LAUNCHED();
  }
  auto reduce = [&](int nsplit, int cols, int mode, float* out, int64_t ld, int tile) -> pmb_status {
    if (nsplit <= 1) return PMB_OK;
    const int64_t total = (int64_t)nbcg * p.Q * cols;
    splitk_reduce_kernel<<<(unsigned)cdiv(total, 256), 256, 0, st>>>(ws.splitk, nsplit, p.Q, cols, mode, p.G, p.Q, out, ld, total, tile, 0,
                                                                     mode == 0 ? ws.dg_hi : nullptr, nullptr);
    PMB_LAUNCHED();
    return PMB_OK;
  };
  {
    ProfScope prof(st, "ssd_bwd_dg_pair", 2.0 * tok * p.H * p.Q * p.P, 0.0);
    const int nsg = ssd_pairs_dg_nsplit(p.B, p.T, p.H, p.G, p.Q);
    PMB_TRY(ssd_pairs_dg(st, in, ws, nsg));
    PMB_TRY(reduce(nsg, p.Q, 0, nullptr, 0, 128));
  }
  const int ns = ssd_pairs_dbc_nsplit(p.B, p.T, p.H, p.N, p.G, p.Q);
  {
    ProfScope prof(st, "ssd_bwd_dc_pair", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
    PMB_TRY(ssd_pairs_dbc(st, in, ws, 0, dc32, gn, ns, ws.splitk));
    PMB_TRY(reduce(ns, p.N, 1, dc32, gn, BM));
  }
  PMB_TRY(cast_f32_bf16(st, dc32, dc, tok * gn));
  {
    ProfScope prof(st, "ssd_bwd_db_pair", 2.0 * tok * p.N * (p.G * p.Q + (double)p.H * p.P), 0.0);
    PMB_TRY(ssd_pairs_dbc(st, in, ws, 1, db32, gn, ns, ws.splitk));
    PMB_TRY(reduce(ns, p.N, 2, db32, gn, BM));
  }
  return cast_f32_bf16(st, db32, db, tok * gn);
}

}  // namespace pmb
