// Fused intra-chunk kernels of the chunked SSD scan (tcgen05 / TMEM); see ssd_fused.cu.  Internal to the library.
#pragma once
#include <cuda.h>
#include "kernels.h"

namespace pmb {

// A matrix operand stored as bf16: `hi` alone (lo == NULL: one MMA per product, the bf16-storage mode) or the
// (hi, lo) pair of an fp32 matrix (three MMAs per product).  `pitch` = elements between consecutive rows (tokens).
struct Op16 { const uint16_t* hi; const uint16_t* lo; int64_t pitch; };

struct FusedArgs {
  int B, T, H, P, N, G, Q;
  const float* S;          // (B,H,T) inclusive cumulative sums of a within each chunk
  Op16 c, b;               // (B*T, G*N) token rows; group g occupies columns [g*N, (g+1)*N)
  Op16 v;                  // mode 0: x~ = x*dt (B*T, H*P);  mode 1: dY (B*T, H*P)
  Op16 state;              // mode 0: h_prev (B*nc*H*N, P);  mode 1: dh (B*nc*H*N, P)   (rows of P, contiguous)
  float* out; int64_t ldo; // mode 0: y;  mode 1: dx~   (token rows, head h at column h*P)
  uint16_t* out16;         // when set, the result is written here as bf16 (row pitch ldo elements) and `out` is not used
  const float* x; int64_t ldx; const float* D;   // mode 0: skip term D[h] * x (D == NULL: none)
  float* off_out;          // mode 0, optional: (B,T,H,P) the carried-state part of y, exp(S_t) C_t h_prev
  uint16_t* off_out16;     // the same as bf16 (set one of the two at most)
  // mode 1 only: x~ (the rows of the CTA, for dM = dY x~^T) and the sums of W[t,s] = dM[t,s] G[t,s] exp(S_t - S_s), s < t
  Op16 xt;                 // (B*T, H*P)
  float* csum;             // (B,T,H)  c_s = sum_{t>s} W[t,s]
  float* esum;             // (B,T,H)  e_s = exp(S_end - S_s) <x~_s, B_s dh>
  float* rpart;            // (B*nc*H, Q/128, Q)  r_t = sum_{s<t} W[t,s], one partial per row block of s (valid for t >= 128*block)
};

// Shapes the fused kernels take: block_len a multiple of 128 (at most 1024); d_state and d_head in {64, 128} with
// plain bf16 operands, d_state = d_head = 64 with (hi, lo) pairs (what fits the shared-memory plan of both modes).
// The other contractions below take d_head = 64 only.
bool ssd_fused_supported(int P, int N, int Q, bool pairs);

// mode 0: Y[t,:]   = sum_{s<=t} (C_t.B_s) exp(S_t-S_s) x~_s + exp(S_t) C_t h_prev + D x_t          per (b, chunk, head)
// mode 1: dx~[s,:] = sum_{t>=s} (C_t.B_s) exp(S_t-S_s) dY_t  + exp(S_end-S_s) B_s dh               per (b, chunk, head)
//         plus csum, esum, rpart (see FusedArgs)
pmb_status ssd_fused(cudaStream_t st, int mode, const FusedArgs& a);

pmb_status read_clear_device_status_fused(unsigned int* word);
pmb_status read_clear_device_status_pairs(unsigned int* word);

// ---- the other contractions of the scan on the same bf16 pairs (ssd_pairs.cu; shapes of ssd_fused_supported(pairs)):
// states / dstates (per head), dG (summed over the heads of a group, decay mask folded in registers), dC / dB.
pmb_status ssd_pairs_state(cudaStream_t st, const SsdIn& in, const SsdWs& ws, int mode);      // 0: chunk states, 1: d(states)
int ssd_pairs_dg_nsplit(int B, int T, int H, int G, int Q);
pmb_status ssd_pairs_dg(cudaStream_t st, const SsdIn& in, const SsdWs& ws, int nsplit);       // -> ws.dg_hi/lo (nsplit == 1) or ws.splitk partials
int ssd_pairs_dbc_nsplit(int B, int T, int H, int N, int G, int Q);
// mode 0: dC, 1: dB; `part` = where the head-split partial tiles go (nsplit * B * nc * G * Q * N floats)
pmb_status ssd_pairs_dbc(cudaStream_t st, const SsdIn& in, const SsdWs& ws, int mode, float* out, int64_t ld, int nsplit, float* part);

namespace sf {
// cached rank-3 bf16 tensor map: dims (d0 contiguous, d1 rows with pitch s0 elements, d2 with pitch s1), box (b0, b1, 1)
pmb_status bf16_map3(CUtensorMap* out, const uint16_t* base, int64_t d0, int64_t d1, int64_t d2, int64_t s0, int64_t s1, int b0, int b1);
}

}  // namespace pmb
