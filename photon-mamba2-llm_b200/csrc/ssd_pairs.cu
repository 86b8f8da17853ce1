// The contractions of the chunked SSD scan other than the fused intra-chunk kernel, on bf16 pairs that their
// producers already wrote (pair_bgemm_kernel: TMA -> tensor core, no rescaling in shared memory):
//   states[n,p]  = sum_q B[q,n] xs[q,p]           xs  = x dt exp(S_end - S_q)   (chunk-prepare kernel)
//   dstate[n,p]  = sum_t C[t,n] dYs[t,p]          dYs = dY exp(S_t)             (gated-norm backward)
//   dG[t,s]      = sum_{h in group} exp(S_h,t - S_h,s) [s<=t] sum_p dY_h[t,p] x~_h[s,p]
//   dC[t,n]      = sum_{s<=t} dG[t,s] B[s,n] + sum_h sum_p dYs_h[t,p] h_prev_h[n,p]
//   dB[s,n]      = sum_{t>=s} dG[t,s] C[t,n] + sum_h sum_p xs_h[s,p]  dh_h[n,p]
// (mamba2/ssd_ops.rs:201-234 and its autograd compute the same quantities op by op.)
// Shapes: block_len % 128 == 0, d_state = d_head = 64 with (hi, lo) pairs; with plain bf16 operands (no lo arrays in
// the workspace: the bf16-input scan) d_state may also be 128.  Other shapes keep the 3xTF32 / FMA engines.
#include "common.cuh"
#include "kernels.h"
#include "pair_bgemm.cuh"
#include "ssd_fused.h"

namespace pmb {

static __device__ unsigned int g_pairs_status = 0;

pmb_status read_clear_device_status_pairs(unsigned int* word) {
  unsigned int zero = 0;
  PMB_CUDA(cudaMemcpyFromSymbol(word, g_pairs_status, sizeof(unsigned int)));
  if (*word) PMB_CUDA(cudaMemcpyToSymbol(g_pairs_status, &zero, sizeof(unsigned int)));
  return PMB_OK;
}

namespace {

using pbg::MapSet;

struct PP {
  int B, T, H, P, N, G, Q, nc, hpg, nsplit;
  const float* S;
  float* out; int64_t ld;          // dC / dB destination (token rows, group g at column g*N)
  float* part;                     // split partial tiles
  float* st_out;                   // states / dstates (B*nc*H, N, P)
  uint16_t* dg_hi; uint16_t* dg_lo;
};

constexpr int MAX_Q = 1024;

// ---- states (MODE 0) / dstates (MODE 1): maps 0 = B or C (MN-major: n contiguous, token rows), 1 = xs or dYs (MN-major)
template <int NS_>
struct PState {
  static constexpr int BN = 64, NS = NS_;
  static constexpr bool SEG_EPI = false;
  static constexpr int AUX_FLOATS = 0;
  float* aux;
  __device__ void stage(int, int) {}
  PP p; int Mdim, Ndim;
  int h, g, tok0; float* out;
  __device__ bool init(int batch, int, int) {
    h = batch % p.H; const int bc = batch / p.H; g = h / p.hpg;
    tok0 = bc * p.Q;
    out = p.st_out + (int64_t)batch * p.N * p.P;
    return true;
  }
  __device__ int nseg() const { return 1; }
  __device__ void seg(int, int, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const { kt0 = 0; kt1 = p.Q / 64; am = 0; bm = 1; amn = 1; bmn = 1; }
  __device__ void a_coord(int, int kt, int m0, int& c0, int& c1, int& c2) const { c0 = m0; c1 = tok0 + kt * 64; c2 = g; }
  __device__ void b_coord(int, int kt, int n0, int& c0, int& c1, int& c2) const { c0 = n0; c1 = tok0 + kt * 64; c2 = h; }
  __device__ void seg_accumulate(int, int, int, const float (&)[32], float (&)[32]) const {}
  __device__ void stage_seg(int, int, int) {}
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    float4* dst = reinterpret_cast<float4*>(out + (int64_t)m * p.P + nb);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
};

// ---- dG: one segment per head (K = d_head), folded with that head's decay mask in registers.
// maps 0 = dY (K-major rows t), 1 = x~ (K-major rows s)
template <int NS_>
struct PDG {
  static constexpr int BN = 128, NS = NS_;
  static constexpr bool SEG_EPI = true;
  static constexpr int AUX_FLOATS = 2 * MAX_Q;   // two halves of S (Q), one per segment in flight
  float* aux;
  __device__ void stage(int, int) {}
  PP p; int Mdim, Ndim;
  int bb, cc, g, split, tok0; int64_t obase;
  __device__ void stage_seg(int s, int tid, int nthr) {
    const int h = head_of(s);
    float* dst = aux + (s & 1) * p.Q;
    const float* sp = p.S + ((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q;
    for (int q = tid; q < p.Q; q += nthr) dst[q] = sp[q];
  }
  __device__ bool init(int batch, int m0, int n0) {
    if (n0 > m0 + pbg::BM - 1) return false;                  // above the diagonal
    split = batch % p.nsplit; batch /= p.nsplit;
    g = batch % p.G; const int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    tok0 = bc * p.Q;
    obase = (p.nsplit > 1 ? (int64_t)blockIdx.z : (int64_t)batch) * p.Q * p.Q;
    return true;
  }
  __device__ int nseg() const { return (p.hpg - split + p.nsplit - 1) / p.nsplit; }
  __device__ int head_of(int s) const { return g * p.hpg + split + s * p.nsplit; }
  __device__ void seg(int, int, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const { kt0 = 0; kt1 = p.P / 64; am = 0; bm = 1; amn = 0; bmn = 0; }
  __device__ void a_coord(int s, int kt, int m0, int& c0, int& c1, int& c2) const { c0 = kt * 64; c1 = tok0 + m0; c2 = head_of(s); }
  __device__ void b_coord(int s, int kt, int n0, int& c0, int& c1, int& c2) const { c0 = kt * 64; c1 = tok0 + n0; c2 = head_of(s); }
  __device__ void seg_accumulate(int s, int m, int nb, const float (&v)[32], float (&acc)[32]) const {
    if (m >= p.Q || nb > m) return;
    const float* sv = aux + (s & 1) * p.Q;
    const float sm = sv[m];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 s4 = *reinterpret_cast<const float4*>(sv + nb + j);
      const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float w = (nb + j + e <= m) ? __expf(sm - ss[e]) : 0.0f;
        acc[j + e] = fmaf(v[j + e], w, acc[j + e]);
      }
    }
  }
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    const int64_t o = obase + (int64_t)m * p.Q + nb;
    if (p.nsplit > 1) {
      float4* dst = reinterpret_cast<float4*>(p.part + o);
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        store_pair4(p.dg_hi + o + 4 * j, NS == 2 ? p.dg_lo + o + 4 * j : nullptr, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  }
};

// ---- dC (MODE 0) / dB (MODE 1).  maps: 0 = dG (MODE 0: K-major rows t; MODE 1: MN-major, s contiguous, t rows),
// 1 = B or C (MN-major), 2 = dYs or xs (K-major rows), 3 = h_prev or dh (K-major rows n)
template <int MODE, int NS_>
struct PDBC {
  static constexpr int BN = 64, NS = NS_;
  static constexpr bool SEG_EPI = false;
  static constexpr int AUX_FLOATS = 0;
  float* aux;
  __device__ void stage(int, int) {}
  PP p; int Mdim, Ndim;
  int bb, cc, g, split, nh, tok0, dgrow0; float* pout;
  __device__ bool init(int batch, int, int) {
    split = batch % p.nsplit; batch /= p.nsplit;
    g = batch % p.G; const int bc = batch / p.G; cc = bc % p.nc; bb = bc / p.nc;
    tok0 = bc * p.Q;
    dgrow0 = batch * p.Q;
    nh = (p.hpg - split + p.nsplit - 1) / p.nsplit;
    pout = p.part + (int64_t)blockIdx.z * Mdim * Ndim;
    return true;
  }
  // segment 0 (the dG term) belongs to split 0; the others own head segments only
  __device__ int nseg() const { return (split == 0 ? 1 : 0) + nh; }
  __device__ int head_of(int s) const { return g * p.hpg + split + (s - (split == 0 ? 1 : 0)) * p.nsplit; }
  __device__ void seg(int s, int m0, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const {
    if (split == 0 && s == 0) {
      am = 0; bm = 1; bmn = 1;
      if (MODE == 0) { kt0 = 0; kt1 = min(p.Q, m0 + pbg::BM) / 64; amn = 0; }
      else { kt0 = m0 / 64; kt1 = p.Q / 64; amn = 1; }
    } else { kt0 = 0; kt1 = p.P / 64; am = 2; bm = 3; amn = 0; bmn = 0; }
  }
  __device__ void a_coord(int s, int kt, int m0, int& c0, int& c1, int& c2) const {
    if (split == 0 && s == 0) {
      if (MODE == 0) { c0 = kt * 64; c1 = dgrow0 + m0; } else { c0 = m0; c1 = dgrow0 + kt * 64; }
      c2 = 0;
    } else { c0 = kt * 64; c1 = tok0 + m0; c2 = head_of(s); }
  }
  __device__ void b_coord(int s, int kt, int n0, int& c0, int& c1, int& c2) const {
    if (split == 0 && s == 0) { c0 = n0; c1 = tok0 + kt * 64; c2 = g; }
    else { c0 = kt * 64; c1 = ((bb * p.nc + cc) * p.H + head_of(s)) * p.N + n0; c2 = 0; }
  }
  __device__ void seg_accumulate(int, int, int, const float (&)[32], float (&)[32]) const {}
  __device__ void stage_seg(int, int, int) {}
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    float* base = p.nsplit > 1 ? pout + (int64_t)m * Ndim + nb : p.out + (int64_t)(tok0 + m) * p.ld + g * p.N + nb;
    float4* dst = reinterpret_cast<float4*>(base);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  }
};

PP make_pp(const SsdIn& in, const SsdWs& ws) {
  PP p{};
  p.B = in.B; p.T = in.T; p.H = in.H; p.P = in.P; p.N = in.N; p.G = in.G; p.Q = in.Q; p.nc = in.T / in.Q; p.hpg = in.H / in.G; p.nsplit = 1;
  p.S = ws.S; p.part = ws.splitk; p.dg_hi = ws.dg_hi; p.dg_lo = ws.dg_lo;
  return p;
}

template <class Op>
Op mk(const PP& p, int Mdim, int Ndim) { Op op{}; op.p = p; op.Mdim = Mdim; op.Ndim = Ndim; return op; }

unsigned int* status_ptr() {
  static unsigned int* ptr[PMB_MAX_DEVICES] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= PMB_MAX_DEVICES) dev = 0;
  if (!ptr[dev]) cudaGetSymbolAddress((void**)&ptr[dev], g_pairs_status);
  return ptr[dev];
}

// logical map i of the set <- the (hi, lo) arrays of one operand
pmb_status set_map(MapSet* ms, int i, const uint16_t* hi, const uint16_t* lo, int64_t d0, int64_t d1, int64_t d2, int64_t s0, int64_t s1, int b0, int b1) {
  PMB_TRY(sf::bf16_map3(&ms->m[2 * i], hi, d0, d1, d2, s0, s1, b0, b1));
  if (!lo) { ms->m[2 * i + 1] = ms->m[2 * i]; return PMB_OK; }      // plain bf16 operand: the lo map is never used
  return sf::bf16_map3(&ms->m[2 * i + 1], lo, d0, d1, d2, s0, s1, b0, b1);
}

}  // namespace

// plain16: the same workspace seen without its lo arrays, which is how the launchers below pick one MMA per product
static SsdWs hi_only(const SsdWs& w) {
  SsdWs v = w;
  v.xt_lo = v.xs_lo = v.dys_lo = v.dg_lo = v.bc_lo = v.dy_lo = v.hp_lo = v.dh_lo = nullptr;
  return v;
}

pmb_status ssd_pairs_state(cudaStream_t st, const SsdIn& in, const SsdWs& ws_in, int mode) {
  const SsdWs ws = in.plain16 ? hi_only(ws_in) : ws_in;
  PP p = make_pp(in, ws);
  p.st_out = mode == 0 ? ws.hprev : ws.dh;
  const int64_t tok = (int64_t)p.B * p.T, bcp = 2 * (int64_t)p.G * p.N, hp = (int64_t)p.H * p.P;
  const uint16_t* a_hi = mode == 0 ? ws.bc_hi : ws.bc_hi + p.G * p.N;
  const uint16_t* a_lo = !ws.bc_lo ? nullptr : (mode == 0 ? ws.bc_lo : ws.bc_lo + p.G * p.N);
  MapSet ms{};
  PMB_TRY(set_map(&ms, 0, a_hi, a_lo, p.N, tok, p.G, bcp, p.N, 64, 64));
  PMB_TRY(set_map(&ms, 1, mode == 0 ? ws.xs_hi : ws.dys_hi, mode == 0 ? ws.xs_lo : ws.dys_lo, p.P, tok, p.H, hp, p.P, 64, 64));
  for (int i = 4; i < 8; ++i) ms.m[i] = ms.m[0];
  ProfScope prof(st, mode == 0 ? "ssd_chunk_state_pair" : "ssd_bwd_dstate_pair", 2.0 * tok * p.H * p.N * p.P, 0.0);
  if (!ws.bc_lo) return pbg::launch(st, ms, mk<PState<1>>(p, p.N, p.P), p.B * p.nc * p.H, status_ptr());
  return pbg::launch(st, ms, mk<PState<2>>(p, p.N, p.P), p.B * p.nc * p.H, status_ptr());
}

// Head-split factor of a per-group contraction with `ctas` CTAs per split: as many splits as fit the machine in ONE wave
// (one CTA more than that costs a second wave), then the fewest splits that give the same number of heads per CTA
// (fewer partial tiles to write and add up).  The 128-wide dG tiles run one CTA per SM, the 64-wide ones two.
static int pick_head_split(int64_t ctas, int hpg, int ctas_per_sm) {
  int want = (int)((ctas_per_sm * 148) / (ctas > 0 ? ctas : 1));
  if (want < 1) want = 1;
  if (want > hpg) want = hpg;
  const int per = (hpg + want - 1) / want;        // heads per CTA at that split
  return (hpg + per - 1) / per;
}

int ssd_pairs_dg_nsplit(int B, int T, int H, int G, int Q) {
  const int nbcg = B * (T / Q) * G, hpg = H / G, qt = Q / pbg::BM;
  return pick_head_split((int64_t)nbcg * (qt * (qt + 1) / 2), hpg, pbg::Geometry<PDG<2>::BN, 2>::CTAS_PER_SM);
}

pmb_status ssd_pairs_dg(cudaStream_t st, const SsdIn& in, const SsdWs& ws_in, int nsplit) {
  const SsdWs ws = in.plain16 ? hi_only(ws_in) : ws_in;
  PP p = make_pp(in, ws);
  p.nsplit = nsplit;
  const int64_t tok = (int64_t)p.B * p.T, hp = (int64_t)p.H * p.P;
  MapSet ms{};
  PMB_TRY(set_map(&ms, 0, ws.dy_hi, ws.dy_lo, p.P, tok, p.H, hp, p.P, 64, 128));
  PMB_TRY(set_map(&ms, 1, ws.xt_hi, ws.xt_lo, p.P, tok, p.H, hp, p.P, 64, 128));
  for (int i = 4; i < 8; ++i) ms.m[i] = ms.m[0];
  if (!ws.dy_lo) return pbg::launch(st, ms, mk<PDG<1>>(p, p.Q, p.Q), p.B * p.nc * p.G * nsplit, status_ptr());
  return pbg::launch(st, ms, mk<PDG<2>>(p, p.Q, p.Q), p.B * p.nc * p.G * nsplit, status_ptr());
}

int ssd_pairs_dbc_nsplit(int B, int T, int H, int N, int G, int Q) {
  const int nbcg = B * (T / Q) * G, hpg = H / G;
  const int tiles = (Q / pbg::BM) * (int)cdiv(N, 64);
  return pick_head_split((int64_t)nbcg * tiles, hpg, pbg::Geometry<PDBC<0, 2>::BN, 2>::CTAS_PER_SM);
}

pmb_status ssd_pairs_dbc(cudaStream_t st, const SsdIn& in, const SsdWs& ws_in, int mode, float* out, int64_t ld, int nsplit, float* part) {
  const SsdWs ws = in.plain16 ? hi_only(ws_in) : ws_in;
  PP p = make_pp(in, ws);
  p.out = out; p.ld = ld; p.nsplit = nsplit; p.part = part;
  const int64_t tok = (int64_t)p.B * p.T, bcp = 2 * (int64_t)p.G * p.N, hp = (int64_t)p.H * p.P;
  const int64_t nbcg = (int64_t)p.B * p.nc * p.G, nbch = (int64_t)p.B * p.nc * p.H;
  MapSet ms{};
  if (mode == 0) {
    PMB_TRY(set_map(&ms, 0, ws.dg_hi, ws.dg_lo, p.Q, nbcg * p.Q, 1, p.Q, (int64_t)p.Q * p.Q, 64, 128));
    PMB_TRY(set_map(&ms, 1, ws.bc_hi, ws.bc_lo, p.N, tok, p.G, bcp, p.N, 64, 64));
    PMB_TRY(set_map(&ms, 2, ws.dys_hi, ws.dys_lo, p.P, tok, p.H, hp, p.P, 64, 128));
    PMB_TRY(set_map(&ms, 3, ws.hp_hi, ws.hp_lo, p.P, nbch * p.N, 1, p.P, (int64_t)p.N * p.P, 64, 64));
    if (!ws.bc_lo) return pbg::launch(st, ms, mk<PDBC<0, 1>>(p, p.Q, p.N), (int)nbcg * nsplit, status_ptr());
    return pbg::launch(st, ms, mk<PDBC<0, 2>>(p, p.Q, p.N), (int)nbcg * nsplit, status_ptr());
  }
  PMB_TRY(set_map(&ms, 0, ws.dg_hi, ws.dg_lo, p.Q, nbcg * p.Q, 1, p.Q, (int64_t)p.Q * p.Q, 64, 64));
  PMB_TRY(set_map(&ms, 1, ws.bc_hi + p.G * p.N, ws.bc_lo ? ws.bc_lo + p.G * p.N : nullptr, p.N, tok, p.G, bcp, p.N, 64, 64));
  PMB_TRY(set_map(&ms, 2, ws.xs_hi, ws.xs_lo, p.P, tok, p.H, hp, p.P, 64, 128));
  PMB_TRY(set_map(&ms, 3, ws.dh_hi, ws.dh_lo, p.P, nbch * p.N, 1, p.P, (int64_t)p.N * p.P, 64, 64));
  if (!ws.bc_lo) return pbg::launch(st, ms, mk<PDBC<1, 1>>(p, p.Q, p.N), (int)nbcg * nsplit, status_ptr());
  return pbg::launch(st, ms, mk<PDBC<1, 2>>(p, p.Q, p.N), (int)nbcg * nsplit, status_ptr());
}

}  // namespace pmb
