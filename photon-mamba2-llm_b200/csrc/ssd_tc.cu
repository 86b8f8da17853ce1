// Tensor-core (tcgen05, 3xTF32) versions of the chunked SSD contractions, built on tc_bgemm_kernel.
// Operands are read in place from the block's activation buffers through rank-3 tensor maps
// (contiguous axis, token axis, head/group axis); decay factors, dt and the causal mask are applied to the
// landed tiles in shared memory by the transform warps, never materialised in HBM.
// Shapes taken here: block_len % 64 == 0, d_state % 32 == 0, d_head % 64 == 0 (the production shapes);
// other shapes run on the fp32 FMA tile engine of ssd.cu.
#include <unordered_map>
#include <mutex>
#include <cstdlib>
#include "common.cuh"
#include "kernels.h"
#include "tc_bgemm.cuh"
#include "ssd_tc.h"

namespace pmb {

static __device__ unsigned int g_ssd_tc_status = 0;

pmb_status read_clear_device_status_ssd(unsigned int* word) {
  unsigned int zero = 0;
  PMB_CUDA(cudaMemcpyFromSymbol(word, g_ssd_tc_status, sizeof(unsigned int)));
  if (*word) PMB_CUDA(cudaMemcpyToSymbol(g_ssd_tc_status, &zero, sizeof(unsigned int)));
  return PMB_OK;
}

namespace {

using tcb::MapSet;

struct TcP {
  int B, T, H, P, N, G, Q, nc, hpg;
  const float* x; int64_t ldx;
  const float* dt; const float* D;
  const float* S;
  const float* dy; int64_t lddy;
  float* y; int64_t ldy;
  float* hprev; float* dh; float* CB; float* dG; float* dxt; float* part;
  const float* xs;   // (B,T,H,P)  x * dt * exp(S_end - S_t)
  const float* dys;  // (B,T,H,P)  dY * exp(S_t)
  int nsplit;
  float* dc; float* db; int64_t lddbc;
  __device__ __forceinline__ float dtv(int64_t tk, int h) const { return dt ? dt[tk * H + h] : 1.0f; }
};

// ------------------------------------------------------------------------------------------------
// CB[t,s] = sum_n C[t,n] B[s,n] per (b,c,g).  maps: 0 = C (K-major rows), 1 = B (K-major rows)
// ------------------------------------------------------------------------------------------------
struct TcCB {
  static constexpr int BN = 128;
  static constexpr bool A_SCALE = false, B_SCALE = false, SEG_EPI = false;
  static constexpr int AUX_FLOATS = 0;
  float* aux;
  __device__ void stage(int, int) {}
  TcP p; int Mdim, Ndim;
  int g; int64_t tok0; float* out;
  __device__ bool init(int batch, int m0, int n0) {
    if (n0 > m0 + tcb::BM - 1) return false;
    g = batch % p.G; int bc = batch / p.G;
    tok0 = (int64_t)bc * p.Q;
    out = p.CB + (int64_t)batch * p.Q * p.Q;
    return true;
  }
  __device__ int nseg() const { return 1; }
  __device__ void seg(int, int, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const {
    kt0 = 0; kt1 = p.N / 32; am = 0; bm = 1; amn = 0; bmn = 0;
  }
  __device__ void a_coord(int, int kt, int m0, int& c0, int& c1, int& c2) const { c0 = kt * 32; c1 = (int)(tok0 + m0); c2 = g; }
  __device__ void b_coord(int, int kt, int n0, int& c0, int& c1, int& c2) const { c0 = kt * 32; c1 = (int)(tok0 + n0); c2 = g; }
  __device__ void a_scale4(int, int, int, int, float (&)[4]) const {}
  __device__ float b_scale(int, int, int) const { return 1.0f; }
  __device__ void seg_accumulate(int, int, int, const float (&)[32], float (&)[32]) const {}
  __device__ void stage_seg(int, int, int) {}
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    float4* dst = reinterpret_cast<float4*>(out + (int64_t)m * p.Q + nb);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
};

constexpr int TC_MAX_Q = 1024;

struct HeadTile {
  int bb, cc, h, g; int64_t tok0; const float* sp; float send;
  __device__ void set(const TcP& p, int batch) {
    h = batch % p.H; int bc = batch / p.H; cc = bc % p.nc; bb = bc / p.nc; g = h / p.hpg;
    tok0 = (int64_t)bc * p.Q;
    sp = p.S + ((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q;
    send = sp[p.Q - 1];
  }
};

// ------------------------------------------------------------------------------------------------
// states[n,p]  = sum_q B[q,n] xs[q,p]    (MODE 0; xs = x dt exp(S_end - S_q); maps: 0 = B MN-major, 1 = xs MN-major)
// contrib[n,p] = sum_t C[t,n] dYs[t,p]   (MODE 1; dYs = dY exp(S_t);          maps: 0 = C MN-major, 1 = dYs MN-major)
// per (b,c,h); output (N,P) into hprev / dh.  The decay factors are folded into xs / dYs by one elementwise
// pass (they are reused by the per-group dB / dC contractions), so this is a plain contraction.
// ------------------------------------------------------------------------------------------------
template <int MODE>
struct TcState {
  static constexpr int BN = 64;
  static constexpr bool A_SCALE = false, B_SCALE = false, SEG_EPI = false;
  static constexpr int AUX_FLOATS = 0;
  float* aux;
  __device__ void stage(int, int) {}
  TcP p; int Mdim, Ndim;
  int h, g; int64_t tok0; float* out;
  __device__ bool init(int batch, int, int) {
    h = batch % p.H; int bc = batch / p.H; g = h / p.hpg;
    tok0 = (int64_t)bc * p.Q;
    out = (MODE == 0 ? p.hprev : p.dh) + (int64_t)batch * p.N * p.P;
    return true;
  }
  __device__ int nseg() const { return 1; }
  __device__ void seg(int, int, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const {
    kt0 = 0; kt1 = p.Q / 32; am = 0; bm = 1; amn = 1; bmn = 1;
  }
  __device__ void a_coord(int, int kt, int m0, int& c0, int& c1, int& c2) const { c0 = m0; c1 = (int)(tok0 + kt * 32); c2 = g; }
  __device__ void b_coord(int, int kt, int n0, int& c0, int& c1, int& c2) const { c0 = n0; c1 = (int)(tok0 + kt * 32); c2 = h; }
  __device__ void a_scale4(int, int, int, int, float (&)[4]) const {}
  __device__ float b_scale(int, int, int) const { return 1.0f; }
  __device__ void seg_accumulate(int, int, int, const float (&)[32], float (&)[32]) const {}
  __device__ void stage_seg(int, int, int) {}
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    float4* dst = reinterpret_cast<float4*>(out + (int64_t)m * p.P + nb);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
};

// ------------------------------------------------------------------------------------------------
// MODE 0 (forward):  Y[t,p]  = sum_{s<=t} CB[t,s] exp(S_t-S_s) dt_s x[s,p] + exp(S_t) sum_n C[t,n] h_prev[n,p] + D x[t,p]
//   maps: 0 = CB (K-major rows t), 1 = x (MN-major), 2 = C (K-major rows), 3 = h_prev (MN-major)
// MODE 1 (backward): dx~[s,p] = sum_{t>=s} CB[t,s] exp(S_t-S_s) dY[t,p] + exp(S_end-S_s) sum_n B[s,n] dh[n,p]
//   maps: 0 = CB (MN-major: rows t, contiguous s), 1 = dY (MN-major), 2 = B (K-major rows), 3 = dh (MN-major)
// per (b,c,h); output (Q,P).
// ------------------------------------------------------------------------------------------------
template <int MODE>
struct TcScan {
  static constexpr int BN = 64;
  static constexpr bool A_SCALE = true, B_SCALE = false, SEG_EPI = false;
  static constexpr int AUX_FLOATS = 2 * TC_MAX_Q;   // [0,Q): S of this (b,c,h);  [Q,2Q): dt (1 when absent)
  float* aux;
  __device__ void stage(int tid, int nthr) {
    for (int q = tid; q < p.Q; q += nthr) { aux[q] = t.sp[q]; aux[p.Q + q] = p.dtv(t.tok0 + q, t.h); }
  }
  TcP p; int Mdim, Ndim;
  HeadTile t; int64_t cbrow0; int batch_;
  __device__ bool init(int batch, int, int) {
    t.set(p, batch);
    batch_ = batch;
    cbrow0 = (((int64_t)t.bb * p.nc + t.cc) * p.G + t.g) * p.Q;
    return true;
  }
  __device__ int nseg() const { return 2; }
  __device__ void seg(int s, int m0, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const {
    if (s == 0) {
      am = 0; bm = 1; bmn = 1;
      if (MODE == 0) { kt0 = 0; kt1 = min(p.Q, m0 + tcb::BM) / 32; amn = 0; }
      else { kt0 = m0 / 32; kt1 = p.Q / 32; amn = 1; }
    } else {
      kt0 = 0; kt1 = p.N / 32; am = 2; bm = 3; amn = 0; bmn = 1;
    }
  }
  __device__ void a_coord(int s, int kt, int m0, int& c0, int& c1, int& c2) const {
    if (s == 0) {
      if (MODE == 0) { c0 = kt * 32; c1 = (int)(cbrow0 + m0); } else { c0 = m0; c1 = (int)(cbrow0 + kt * 32); }
      c2 = 0;
    } else { c0 = kt * 32; c1 = (int)(t.tok0 + m0); c2 = t.g; }
  }
  __device__ void b_coord(int s, int kt, int n0, int& c0, int& c1, int& c2) const {
    if (s == 0) { c0 = n0; c1 = (int)(t.tok0 + kt * 32); c2 = t.h; }
    else { c0 = n0; c1 = (int)((int64_t)batch_ * p.N + kt * 32); c2 = 0; }
  }
  // aux[0..Q) = S, aux[Q..2Q) = dt.  Branch-free: masked or out-of-chunk elements become exactly 0.
  __device__ void a_scale4(int s, int a_mn, int m, int k, float (&f)[4]) const {
    const int Q = p.Q;
    if (s == 0) {
      if (MODE == 0) {            // K-major: row t = m, columns s = k..k+3:  exp(S_t - S_s) dt_s [s <= t]
        const float sm = aux[min(m, Q - 1)];
        const float4 sk = *reinterpret_cast<const float4*>(aux + k);
        const float4 dk = *reinterpret_cast<const float4*>(aux + Q + k);
        const float ss[4] = {sk.x, sk.y, sk.z, sk.w}, dd[4] = {dk.x, dk.y, dk.z, dk.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float w = __expf(sm - ss[e]) * dd[e];
          f[e] = (k + e <= m && m < Q) ? f[e] * w : 0.0f;
        }
      } else {                    // MN-major: row t = k, columns s = m..m+3:  exp(S_t - S_s) [t >= s]
        const float st = aux[k];
        const int mc = min(m, Q - 4);
        const float4 sq = *reinterpret_cast<const float4*>(aux + mc);
        const float ss[4] = {sq.x, sq.y, sq.z, sq.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float w = __expf(st - ss[e]);
          f[e] = (k >= m + e && m + e < Q && mc == m) ? f[e] * w : 0.0f;
        }
      }
    } else {                      // K-major, one factor per row
      const float sm = aux[min(m, Q - 1)];
      const float w = MODE == 0 ? __expf(sm) : __expf(t.send - sm);
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = (m < Q) ? f[e] * w : 0.0f;
    }
  }
  __device__ float b_scale(int, int, int) const { return 1.0f; }
  __device__ void seg_accumulate(int, int, int, const float (&)[32], float (&)[32]) const {}
  __device__ void stage_seg(int, int, int) {}
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    if (MODE == 0) {
      const int64_t row = t.tok0 + m;
      float4* dst = reinterpret_cast<float4*>(p.y + row * p.ldy + t.h * p.P + nb);
      if (p.D) {
        const float dv = p.D[t.h];
        const float4* xs = reinterpret_cast<const float4*>(p.x + row * p.ldx + t.h * p.P + nb);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 q = xs[j];
          dst[j] = make_float4(fmaf(dv, q.x, v[4 * j]), fmaf(dv, q.y, v[4 * j + 1]), fmaf(dv, q.z, v[4 * j + 2]), fmaf(dv, q.w, v[4 * j + 3]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
    } else {
      float4* dst = reinterpret_cast<float4*>(p.dxt + (t.tok0 + m) * (int64_t)(p.H * p.P) + t.h * p.P + nb);
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  }
};

// ------------------------------------------------------------------------------------------------
// dG[t,s] = sum_{h in group} exp(S_h,t - S_h,s) dt_h,s [s<=t] sum_p dY_h[t,p] x_h[s,p]  per (b,c,g).
// One segment per head: its product lands in a fresh TMEM accumulator and is folded, scaled by that head's
// decay mask, into register sums while the tensor core computes the next head (SEG_EPI).
//   maps: 0 = dY (K-major rows t), 1 = x (K-major rows s)
// ------------------------------------------------------------------------------------------------
struct TcDG {
  static constexpr int BN = 128;
  static constexpr bool A_SCALE = false, B_SCALE = false, SEG_EPI = true;
  static constexpr int AUX_FLOATS = 4 * TC_MAX_Q;   // two halves of [S (Q) | dt (Q)], one per segment in flight
  float* aux;
  __device__ void stage(int, int) {}
  __device__ void stage_seg(int s, int tid, int nthr) {
    const int h = head_of(s);
    float* dst = aux + (s & 1) * 2 * p.Q;
    const float* sp = p.S + ((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q;
    for (int q = tid; q < p.Q; q += nthr) { dst[q] = sp[q]; dst[p.Q + q] = p.dtv(tok0 + q, h); }
  }
  TcP p; int Mdim, Ndim;
  int bb, cc, g, split; int64_t tok0; float* out;
  // with few (batch, chunk) pairs the heads of a group are dealt round-robin to p.nsplit CTAs whose partial
  // tiles are summed afterwards in a fixed order
  __device__ bool init(int batch, int m0, int n0) {
    if (n0 > m0 + tcb::BM - 1) return false;
    split = batch % p.nsplit; batch /= p.nsplit;
    g = batch % p.G; int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    tok0 = (int64_t)bc * p.Q;
    out = p.nsplit > 1 ? p.part + (int64_t)blockIdx.z * p.Q * p.Q : p.dG + (int64_t)batch * p.Q * p.Q;
    return true;
  }
  __device__ int nseg() const { return (p.hpg - split + p.nsplit - 1) / p.nsplit; }
  __device__ int head_of(int s) const { return g * p.hpg + split + s * p.nsplit; }
  __device__ void seg(int, int, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const {
    kt0 = 0; kt1 = p.P / 32; am = 0; bm = 1; amn = 0; bmn = 0;
  }
  __device__ void a_coord(int s, int kt, int m0, int& c0, int& c1, int& c2) const { c0 = kt * 32; c1 = (int)(tok0 + m0); c2 = head_of(s); }
  __device__ void b_coord(int s, int kt, int n0, int& c0, int& c1, int& c2) const { c0 = kt * 32; c1 = (int)(tok0 + n0); c2 = head_of(s); }
  __device__ void a_scale4(int, int, int, int, float (&)[4]) const {}
  __device__ float b_scale(int, int, int) const { return 1.0f; }
  __device__ void seg_accumulate(int s, int m, int nb, const float (&v)[32], float (&acc)[32]) const {
    if (m >= p.Q || nb > m) return;
    const float* sv = aux + (s & 1) * 2 * p.Q;
    const float* dv = sv + p.Q;
    const float sm = sv[m];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 s4 = *reinterpret_cast<const float4*>(sv + nb + j);
      const float4 d4 = *reinterpret_cast<const float4*>(dv + nb + j);
      const float ss[4] = {s4.x, s4.y, s4.z, s4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float w = (nb + j + e <= m) ? __expf(sm - ss[e]) * dd[e] : 0.0f;
        acc[j + e] = fmaf(v[j + e], w, acc[j + e]);
      }
    }
  }
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    float4* dst = reinterpret_cast<float4*>(out + (int64_t)m * p.Q + nb);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
};

// ------------------------------------------------------------------------------------------------
// MODE 0: dC[t,n] = sum_{s<=t} dG[t,s] B[s,n] + sum_h sum_p dYs_h[t,p] h_prev_h[n,p]      (dYs = dY exp(S_t))
//   maps: 0 = dG (K-major rows t), 1 = B (MN-major), 2 = dYs (K-major rows t), 3 = h_prev (K-major rows n)
// MODE 1: dB[s,n] = sum_{t>=s} dG[t,s] C[t,n] + sum_h sum_p xs_h[s,p] dh_h[n,p]           (xs = x dt exp(S_end - S_s))
//   maps: 0 = dG (MN-major), 1 = C (MN-major), 2 = xs (K-major rows s), 3 = dh (K-major rows n)
// per (b,c,g) and head split; output (Q,N) into the C / B columns of the activation-gradient buffer, or,
// when the head loop is split across CTAs, into partial tiles that ssd.cu's reduce kernel sums.
// ------------------------------------------------------------------------------------------------
template <int MODE, int BN_>
struct TcDBC {
  static constexpr int BN = BN_;
  static constexpr bool A_SCALE = false, B_SCALE = false, SEG_EPI = false;
  static constexpr int AUX_FLOATS = 0;
  float* aux;
  __device__ void stage(int, int) {}
  TcP p; int Mdim, Ndim;
  int bb, cc, g, split, nh; int64_t tok0, dgrow0; float* pout;
  __device__ bool init(int batch, int, int) {
    split = batch % p.nsplit; batch /= p.nsplit;
    g = batch % p.G; int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    tok0 = (int64_t)bc * p.Q;
    dgrow0 = (int64_t)batch * p.Q;
    nh = (p.hpg - split + p.nsplit - 1) / p.nsplit;       // heads split, split + nsplit, ...
    pout = p.part + (int64_t)blockIdx.z * Mdim * Ndim;
    return true;
  }
  // segment 0 (the dG term) belongs to split 0; the others own head segments only
  __device__ int nseg() const { return (split == 0 ? 1 : 0) + nh; }
  __device__ int head_of(int s) const { return g * p.hpg + split + (s - (split == 0 ? 1 : 0)) * p.nsplit; }
  __device__ void seg(int s, int m0, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const {
    if (split == 0 && s == 0) {
      am = 0; bm = 1; bmn = 1;
      if (MODE == 0) { kt0 = 0; kt1 = min(p.Q, m0 + tcb::BM) / 32; amn = 0; }
      else { kt0 = m0 / 32; kt1 = p.Q / 32; amn = 1; }
    } else { kt0 = 0; kt1 = p.P / 32; am = 2; bm = 3; amn = 0; bmn = 0; }
  }
  __device__ void a_coord(int s, int kt, int m0, int& c0, int& c1, int& c2) const {
    if (split == 0 && s == 0) {
      if (MODE == 0) { c0 = kt * 32; c1 = (int)(dgrow0 + m0); } else { c0 = m0; c1 = (int)(dgrow0 + kt * 32); }
      c2 = 0;
    } else { c0 = kt * 32; c1 = (int)(tok0 + m0); c2 = head_of(s); }
  }
  __device__ void b_coord(int s, int kt, int n0, int& c0, int& c1, int& c2) const {
    if (split == 0 && s == 0) { c0 = n0; c1 = (int)(tok0 + kt * 32); c2 = g; }
    else {
      int h = head_of(s);
      c0 = kt * 32; c1 = (int)((((int64_t)bb * p.nc + cc) * p.H + h) * p.N + n0); c2 = 0;
    }
  }
  __device__ void a_scale4(int, int, int, int, float (&)[4]) const {}
  __device__ float b_scale(int, int, int) const { return 1.0f; }
  __device__ void seg_accumulate(int, int, int, const float (&)[32], float (&)[32]) const {}
  __device__ void stage_seg(int, int, int) {}
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    float* base = p.nsplit > 1 ? pout + (int64_t)m * Ndim + nb
                               : (MODE == 0 ? p.dc : p.db) + (tok0 + m) * p.lddbc + g * p.N + nb;
    float4* dst = reinterpret_cast<float4*>(base);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
};

// ---- host-side tensor-map cache (the workspace pointers repeat every layer and step) -------------
struct MapKey {
  const void* base; int64_t d0, d1, d2, s0, s1; int b0, b1; bool mn;
  bool operator==(const MapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s0 == o.s0 && s1 == o.s1 && b0 == o.b0 && b1 == o.b1 && mn == o.mn;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    auto mix = [&](int64_t v) { h ^= std::hash<int64_t>()(v) + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2); };
    mix(k.d0); mix(k.d1); mix(k.d2); mix(k.s0); mix(k.s1); mix(k.b0); mix(k.b1); mix(k.mn);
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;   // shared by all devices and host threads
std::mutex g_maps_mu;

// rank-3 map: dims (d0 contiguous, d1 rows with pitch s0 floats, d2 with pitch s1 floats), box (b0, b1, 1)
pmb_status get_map(CUtensorMap* out, const float* base, int64_t d0, int64_t d1, int64_t d2, int64_t s0, int64_t s1, int b0, int b1, bool mn) {
  MapKey key{base, d0, d1, d2, s0, s1, b0, b1, mn};
  std::lock_guard<std::mutex> lock(g_maps_mu);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    if (g_maps.size() > 4096) g_maps.clear();
    CUtensorMap m;
    int64_t dims[3] = {d0, d1, d2}, strides[2] = {s0, s1};
    int box[3] = {b0, b1, 1};
    PMB_TRY(tcx::make_map(&m, base, 3, dims, strides, box, mn));
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return PMB_OK;
}

TcP make_p(const SsdIn& in, const SsdWs& ws) {
  TcP p{};
  p.B = in.B; p.T = in.T; p.H = in.H; p.P = in.P; p.N = in.N; p.G = in.G; p.Q = in.Q; p.nc = in.T / in.Q; p.hpg = in.H / in.G;
  p.x = in.x; p.ldx = in.ldx; p.dt = in.dt; p.D = in.D; p.S = ws.S;
  p.hprev = ws.hprev; p.dh = ws.dh; p.CB = ws.CB; p.dG = ws.dG; p.dxt = ws.dxt; p.part = ws.splitk;
  p.xs = ws.xs; p.dys = ws.dys; p.nsplit = 1;
  return p;
}

template <class Op>
Op mk(const TcP& p, int Mdim, int Ndim) { Op op{}; op.p = p; op.Mdim = Mdim; op.Ndim = Ndim; return op; }

// device address of this device's status word (looked up once per device)
unsigned int* status_ptr() {
  static unsigned int* ptr[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!ptr[dev]) cudaGetSymbolAddress((void**)&ptr[dev], g_ssd_tc_status);
  return ptr[dev];
}

}  // namespace

// Self-test of the bounded-wait path every tcgen05 kernel of this library relies on: one thread waits on an
// mbarrier that nothing ever arms, gives up after `polls` polls, raises bit 128 of the scan's device status word
// and returns.  No copy, no tensor-memory allocation and no other thread is involved, so the launch ends by itself.
__global__ void bounded_wait_selftest_kernel(unsigned int* __restrict__ status, uint32_t polls) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = tcx::smem_u32(&bar);
  tcx::mbar_init(b, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  if (!tcx::mbar_wait(b, 0, polls)) atomicOr(status, 128u);
}

pmb_status bounded_wait_selftest(cudaStream_t st, uint32_t polls) {
  bounded_wait_selftest_kernel<<<1, 1, 0, st>>>(status_ptr(), polls);
  PMB_LAUNCHED();
  return PMB_OK;
}

bool ssd_tc_supported(const SsdIn& in) {
  static const bool off = [] { const char* e = getenv("PMB_SSD_ENGINE"); return e && strcmp(e, "simt") == 0; }();
  if (off) return false;
  if (in.Q % 64 != 0 || in.N % 32 != 0 || in.P % 64 != 0) return false;
  if (in.N > 128 || in.Q > TC_MAX_Q || (in.ldx & 3) || (in.ldbc & 3)) return false;
  if ((reinterpret_cast<uintptr_t>(in.x) | reinterpret_cast<uintptr_t>(in.b) | reinterpret_cast<uintptr_t>(in.c)) & 15) return false;
  if ((int64_t)in.B * in.T >= (1LL << 31) / 4) return false;
  return true;
}

// Forward contractions.  chunk_cumsum and state_pass stay in ssd.cu (called by the dispatcher around these).
pmb_status ssd_tc_cb(cudaStream_t st, const SsdIn& in, const SsdWs& ws) {
  TcP p = make_p(in, ws);
  MapSet ms{};
  int64_t tok = (int64_t)p.B * p.T;
  PMB_TRY(get_map(&ms.m[0], in.c, p.N, tok, p.G, in.ldbc, p.N, 32, 128, false));
  PMB_TRY(get_map(&ms.m[1], in.b, p.N, tok, p.G, in.ldbc, p.N, 32, 128, false));
  ms.m[2] = ms.m[0]; ms.m[3] = ms.m[0];
  ProfScope prof(st, "ssd_cb_tc", 2.0 * tok * p.Q * p.N * p.G, 0.0);
  return tcb::launch(st, ms, mk<TcCB>(p, p.Q, p.Q), p.B * p.nc * p.G, status_ptr());
}

// xs[b,t,h,:] = x[b,t,h,:] * dt * exp(S_end - S_t)  (mode 0)   or   dYs[b,t,h,:] = dY[b,t,h,:] * exp(S_t)  (mode 1).
// A thread owns one float4 of four (b,t,h) rows a grid stride apart and requests all four before using any.
// HBM-bound: reads and writes (B,T,H,P) once.
constexpr int PRESCALE_UNROLL = 4;
__global__ void __launch_bounds__(256) prescale_rows_kernel(const float* __restrict__ src, int64_t ld, const float* __restrict__ S,
                                                            const float* __restrict__ dt, float* __restrict__ dst, int B, int T, int H, int P,
                                                            int Q, int mode) {
  const int P4 = P >> 2;
  const int64_t total = (int64_t)B * T * H * P4;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  float4 v[PRESCALE_UNROLL]; float f[PRESCALE_UNROLL]; float4* out[PRESCALE_UNROLL];
#pragma unroll
  for (int u = 0; u < PRESCALE_UNROLL; ++u) {
    const int64_t idx = i0 + u * stride;
    out[u] = nullptr; f[u] = 0.0f; v[u] = make_float4(0, 0, 0, 0);
    if (idx < total) {
      const int i = (int)(idx % P4); const int64_t w = idx / P4;
      const int h = (int)(w % H); const int64_t tk = w / H; const int b = (int)(tk / T); const int t = (int)(tk % T);
      const float* sp = S + ((int64_t)b * H + h) * T;
      if (mode == 0) {
        const int cend = (t / Q) * Q + Q - 1;
        f[u] = __expf(sp[cend] - sp[t]) * (dt ? dt[tk * H + h] : 1.0f);
      } else {
        f[u] = __expf(sp[t]);
      }
      v[u] = reinterpret_cast<const float4*>(src + tk * ld + h * P)[i];
      out[u] = reinterpret_cast<float4*>(dst + tk * (int64_t)(H * P) + h * P) + i;
    }
  }
#pragma unroll
  for (int u = 0; u < PRESCALE_UNROLL; ++u)
    if (out[u]) *out[u] = make_float4(v[u].x * f[u], v[u].y * f[u], v[u].z * f[u], v[u].w * f[u]);
}

static pmb_status prescale(cudaStream_t st, const char* name, const float* src, int64_t ld, const SsdIn& in, const SsdWs& ws, float* dst, int mode) {
  int64_t rows = (int64_t)in.B * in.T * in.H;
  ProfScope prof(st, name, 0.0, 8.0 * rows * in.P);
  prescale_rows_kernel<<<(unsigned)cdiv(rows * (in.P / 4), 256 * PRESCALE_UNROLL), 256, 0, st>>>(src, ld, ws.S, in.dt, dst, in.B, in.T, in.H, in.P, in.Q, mode);
  PMB_LAUNCHED();
  return PMB_OK;
}

pmb_status ssd_tc_state(cudaStream_t st, const SsdIn& in, const SsdWs& ws) {
  TcP p = make_p(in, ws);
  if (!in.xs_ready) PMB_TRY(prescale(st, "ssd_prescale_x", in.x, in.ldx, in, ws, ws.xs, 0));
  MapSet ms{};
  int64_t tok = (int64_t)p.B * p.T;
  PMB_TRY(get_map(&ms.m[0], in.b, p.N, tok, p.G, in.ldbc, p.N, 32, 32, true));
  PMB_TRY(get_map(&ms.m[1], ws.xs, p.P, tok, p.H, (int64_t)p.H * p.P, p.P, 32, 32, true));
  ms.m[2] = ms.m[0]; ms.m[3] = ms.m[0];
  ProfScope prof(st, "ssd_chunk_state_tc", 2.0 * tok * p.H * p.N * p.P, 0.0);
  return tcb::launch(st, ms, mk<TcState<0>>(p, p.N, p.P), p.B * p.nc * p.H, status_ptr());
}

pmb_status ssd_tc_scan(cudaStream_t st, const SsdIn& in, float* y, int64_t ldy, const SsdWs& ws) {
  TcP p = make_p(in, ws);
  p.y = y; p.ldy = ldy;
  MapSet ms{};
  int64_t tok = (int64_t)p.B * p.T;
  PMB_TRY(get_map(&ms.m[0], ws.CB, p.Q, (int64_t)p.B * p.nc * p.G * p.Q, 1, p.Q, (int64_t)p.Q * p.Q, 32, 128, false));
  PMB_TRY(get_map(&ms.m[1], in.x, p.P, tok, p.H, in.ldx, p.P, 32, 32, true));
  PMB_TRY(get_map(&ms.m[2], in.c, p.N, tok, p.G, in.ldbc, p.N, 32, 128, false));
  PMB_TRY(get_map(&ms.m[3], ws.hprev, p.P, (int64_t)p.B * p.nc * p.H * p.N, 1, p.P, (int64_t)p.N * p.P, 32, 32, true));
  ProfScope prof(st, "ssd_chunk_scan_tc", 2.0 * tok * p.H * p.P * (p.Q + p.N), 0.0);
  return tcb::launch(st, ms, mk<TcScan<0>>(p, p.Q, p.P), p.B * p.nc * p.H, status_ptr(), +1);
}

// Backward contractions.  Expects ws.xs from the forward of the same scan (it is recomputed here because
// the forward and the backward of a block may be separated by other layers reusing the workspace).
pmb_status ssd_tc_dstate(cudaStream_t st, const SsdIn& in, const float* dy, int64_t lddy, const SsdWs& ws) {
  TcP p = make_p(in, ws);
  if (!in.dys_ready) PMB_TRY(prescale(st, "ssd_prescale_dy", dy, lddy, in, ws, ws.dys, 1));
  MapSet ms{};
  int64_t tok = (int64_t)p.B * p.T;
  PMB_TRY(get_map(&ms.m[0], in.c, p.N, tok, p.G, in.ldbc, p.N, 32, 32, true));
  PMB_TRY(get_map(&ms.m[1], ws.dys, p.P, tok, p.H, (int64_t)p.H * p.P, p.P, 32, 32, true));
  ms.m[2] = ms.m[0]; ms.m[3] = ms.m[0];
  ProfScope prof(st, "ssd_bwd_dstate_tc", 2.0 * tok * p.H * p.N * p.P, 0.0);
  return tcb::launch(st, ms, mk<TcState<1>>(p, p.N, p.P), p.B * p.nc * p.H, status_ptr());
}

pmb_status ssd_tc_dx(cudaStream_t st, const SsdIn& in, const float* dy, int64_t lddy, const SsdWs& ws) {
  TcP p = make_p(in, ws);
  MapSet ms{};
  int64_t tok = (int64_t)p.B * p.T;
  PMB_TRY(get_map(&ms.m[0], ws.CB, p.Q, (int64_t)p.B * p.nc * p.G * p.Q, 1, p.Q, (int64_t)p.Q * p.Q, 32, 32, true));
  PMB_TRY(get_map(&ms.m[1], dy, p.P, tok, p.H, lddy, p.P, 32, 32, true));
  PMB_TRY(get_map(&ms.m[2], in.b, p.N, tok, p.G, in.ldbc, p.N, 32, 128, false));
  PMB_TRY(get_map(&ms.m[3], ws.dh, p.P, (int64_t)p.B * p.nc * p.H * p.N, 1, p.P, (int64_t)p.N * p.P, 32, 32, true));
  ProfScope prof(st, "ssd_bwd_dx_tc", 2.0 * tok * p.H * p.P * (p.Q + p.N), 0.0);
  return tcb::launch(st, ms, mk<TcScan<1>>(p, p.Q, p.P), p.B * p.nc * p.H, status_ptr());
}

int ssd_tc_dg_nsplit_dims(int B, int T, int H, int G, int Q) {
  int nbcg = B * (T / Q) * G, hpg = H / G;
  int qt = (int)cdiv(Q, tcb::BM);
  int want = (int)cdiv(2 * 148, (int64_t)nbcg * (qt * (qt + 1) / 2));
  if (want < 1) want = 1;
  return want > hpg ? hpg : want;
}

// dG for every (b,c,g): heads are summed inside the CTA (nsplit CTAs per group, partial tiles in ws.splitk when > 1).
pmb_status ssd_tc_dg(cudaStream_t st, const SsdIn& in, const float* dy, int64_t lddy, const SsdWs& ws, int nsplit) {
  TcP p = make_p(in, ws);
  p.nsplit = nsplit;
  MapSet ms{};
  int64_t tok = (int64_t)p.B * p.T;
  PMB_TRY(get_map(&ms.m[0], dy, p.P, tok, p.H, lddy, p.P, 32, 128, false));
  PMB_TRY(get_map(&ms.m[1], in.x, p.P, tok, p.H, in.ldx, p.P, 32, 128, false));
  ms.m[2] = ms.m[0]; ms.m[3] = ms.m[0];
  return tcb::launch(st, ms, mk<TcDG>(p, p.Q, p.Q), p.B * p.nc * p.G * nsplit, status_ptr());
}

// Number of head splits for the per-group dB / dC contractions: enough CTAs to fill the GPU twice.
int ssd_tc_dbc_nsplit_dims(int B, int T, int H, int N, int G, int Q) {
  int nbcg = B * (T / Q) * G, hpg = H / G;
  int tiles = (int)(cdiv(Q, tcb::BM) * cdiv(N, N <= 64 ? 64 : 128));
  int want = (int)cdiv(2 * 148, (int64_t)nbcg * tiles);
  if (want < 1) want = 1;
  return want > hpg ? hpg : want;
}
int ssd_tc_dbc_nsplit(const SsdIn& in) { return ssd_tc_dbc_nsplit_dims(in.B, in.T, in.H, in.N, in.G, in.Q); }

template <int MODE, int BN>
static pmb_status dbc_launch(cudaStream_t st, const SsdIn& in, const SsdWs& ws, float* out, int64_t lddbc, int nsplit) {
  TcP p = make_p(in, ws);
  p.dc = out; p.db = out; p.lddbc = lddbc; p.nsplit = nsplit;
  MapSet ms{};
  int64_t tok = (int64_t)p.B * p.T;
  int64_t nbcg = (int64_t)p.B * p.nc * p.G, nbch = (int64_t)p.B * p.nc * p.H;
  int64_t hp = (int64_t)p.H * p.P;
  if (MODE == 0) {
    PMB_TRY(get_map(&ms.m[0], ws.dG, p.Q, nbcg * p.Q, 1, p.Q, (int64_t)p.Q * p.Q, 32, 128, false));
    PMB_TRY(get_map(&ms.m[1], in.b, p.N, tok, p.G, in.ldbc, p.N, 32, 32, true));
    PMB_TRY(get_map(&ms.m[2], ws.dys, p.P, tok, p.H, hp, p.P, 32, 128, false));
    PMB_TRY(get_map(&ms.m[3], ws.hprev, p.P, nbch * p.N, 1, p.P, (int64_t)p.N * p.P, 32, BN, false));
  } else {
    PMB_TRY(get_map(&ms.m[0], ws.dG, p.Q, nbcg * p.Q, 1, p.Q, (int64_t)p.Q * p.Q, 32, 32, true));
    PMB_TRY(get_map(&ms.m[1], in.c, p.N, tok, p.G, in.ldbc, p.N, 32, 32, true));
    PMB_TRY(get_map(&ms.m[2], ws.xs, p.P, tok, p.H, hp, p.P, 32, 128, false));
    PMB_TRY(get_map(&ms.m[3], ws.dh, p.P, nbch * p.N, 1, p.P, (int64_t)p.N * p.P, 32, BN, false));
  }
  return tcb::launch(st, ms, mk<TcDBC<MODE, BN>>(p, p.Q, p.N), (int)nbcg * nsplit, status_ptr());
}

// dC / dB: with nsplit > 1 the result is nsplit partial (Q,N) tiles per (b,c,g) in ws.splitk for the caller to reduce.
pmb_status ssd_tc_dc(cudaStream_t st, const SsdIn& in, float* dc, int64_t lddbc, const SsdWs& ws, int nsplit) {
  if (in.N <= 64) return dbc_launch<0, 64>(st, in, ws, dc, lddbc, nsplit);
  return dbc_launch<0, 128>(st, in, ws, dc, lddbc, nsplit);
}
pmb_status ssd_tc_db(cudaStream_t st, const SsdIn& in, float* db, int64_t lddbc, const SsdWs& ws, int nsplit) {
  if (in.N <= 64) return dbc_launch<1, 64>(st, in, ws, db, lddbc, nsplit);
  return dbc_launch<1, 128>(st, in, ws, db, lddbc, nsplit);
}

}  // namespace pmb
