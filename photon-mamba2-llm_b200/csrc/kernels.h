// Internal host-side launch interface shared by the translation units of the library.
#pragma once
#include "common.cuh"

namespace pmb {

// ---- abi.cu: side streams for kernels that do not depend on each other.  One stream and six events per (device,
// lane index), created on first use (so the first call should come before any stream capture).  lane 0: scan
// backward chains; 1: gradient GEMMs of a block that are off the critical path; 2: scan forward; 3: recompute-ahead;
// 4: embedding-table gradient of the LM head; 5: unused; 6: the gradient kernels of the stack backward (high priority,
// like lane 0).  *out stays NULL past device 63.
struct SideLane { cudaStream_t s = nullptr; cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr}; };
pmb_status get_side_lane(int idx, SideLane** out);
void set_lanes_enabled(int on);
// `to` waits for everything enqueued on `from` so far
pmb_status order_after(cudaStream_t from, cudaEvent_t ev, cudaStream_t to);

// ---- elementwise.cu
// optional second output of the conv forward: columns [col0, col0 + width) of `act` (the B | C columns) as a (hi, lo)
// bf16 pair with row pitch `width`.  Written only by the vector kernel; `hi` is reset to NULL when it was not.
struct ConvPairOut { uint16_t* hi = nullptr; uint16_t* lo = nullptr; int col0 = 0; int width = 0; };
pmb_status conv_silu_dt_fwd(cudaStream_t st, const Dims& d, const float* xzd, const float* w, const float* b,
                            const float* dt_bias, float* act, float* dt, ConvPairOut* pair = nullptr);
size_t conv_bwd_ws_bytes(const Dims& d);
pmb_status conv_silu_bwd(cudaStream_t st, const Dims& d, const float* xzd, const float* w, const float* b,
                         const float* dact, float* dxzd, float* dw, float* db, void* ws, size_t ws_bytes,
                         SideLane* red = nullptr,    // red: the two small column reductions go to this lane (caller joins it)
                         uint16_t* pair_hi = nullptr, uint16_t* pair_lo = nullptr);   // pair: dxBC as a bf16 pair (pitch J) instead of fp32
pmb_status gated_rmsnorm_fwd(cudaStream_t st, int64_t rows, int width, float eps, const float* y, const float* z,
                             int64_t ldz, const float* w, float* out, float* rstd, uint16_t* out_hi = nullptr,
                             uint16_t* out_lo = nullptr);   // out_hi/out_lo: optional (hi, lo) bf16 pair of the output; out may then be NULL
size_t gated_rmsnorm_bwd_ws_bytes(int64_t rows, int width);
// optional outputs of the gated RMSNorm backward: dz as a (hi, lo) bf16 pair (pitch lddz) instead of fp32, and
// dys = dy * exp(S[b,h,t]) (S laid out (B,H,T), heads of width P, rows = B*T) for the scan backward
struct NormBwdExtra { uint16_t* dz_hi = nullptr; uint16_t* dz_lo = nullptr; uint16_t* dy_hi = nullptr; uint16_t* dy_lo = nullptr; /* dy as a pair, contiguous rows */
                      uint16_t* dys_hi = nullptr; uint16_t* dys_lo = nullptr; /* dy * exp(S) as a pair */
                      float* dys = nullptr; const float* S = nullptr; int H = 0, P = 1, T = 1; };
pmb_status gated_rmsnorm_bwd(cudaStream_t st, int64_t rows, int width, const float* dout, const float* y, const float* z,
                             int64_t ldz, const float* w, const float* rstd, float* dy, float* dz, int64_t lddz,
                             float* dw, void* ws, size_t ws_bytes, SideLane* red = nullptr, const NormBwdExtra* extra = nullptr);
pmb_status column_sum(cudaStream_t st, const float* partial, int64_t rows, int cols, float* out);

// ---- ssd.cu
// Inputs of the scan in "block form": x (B,T,H,P) stride ldx; either (dt, A) with a = A[h]*dt and x~ = x*dt
// (dt != NULL), or `a` given directly and x~ = x (dt == NULL).  b/c (B,T,G,N) stride ldbc.
struct SsdIn {
  int B, T, H, P, N, G, Q;
  const float* x; int64_t ldx;
  const float* dt;        // (B,T,H) or NULL
  const float* A;         // (H) = -exp(a_log), used when dt != NULL
  const float* a;         // (B,T,H), used when dt == NULL
  const float* b; const float* c; int64_t ldbc;
  const float* D;         // (H) skip weights or NULL:  y += D[h] * x
  bool dys_ready = false; // backward: ws.dys = dY exp(S) was already written by the caller
  bool dy_pair_ready = false;  // backward: ws.dy_hi / dy_lo (the pair of dY) were already written by the caller
  bool bc_pair_ready = false;  // forward: ws.bc_hi / bc_lo (the pairs of B | C) were already written by the caller
  bool xs_ready = false;  // forward (internal): ws.xs was already written by the fused cumsum kernel
  // bf16-storage mode of the block: the scan's tensor-core products read the hi halves of the operand pairs alone
  // (one MMA per product); the producers still write both halves, the recurrence and all accumulators stay fp32
  bool plain16 = false;
  // forward only, optional: form dt and A inside the cumsum kernel.  dt = softplus(dt_raw[token*ld_raw + h] + dt_bias[h])
  // is written to `dt` and A[h] = -exp(a_log[h]) to `A` (both must then point at writable buffers).
  const float* dt_raw = nullptr; int64_t ld_raw = 0; const float* dt_bias = nullptr; const float* a_log = nullptr;
};
struct SsdWs {            // persistent between fwd and bwd of one scan
  float* S;               // (B,H,T) inclusive cumsum of a within each chunk
  float* hprev;           // (B,nc,H,N,P) state entering each chunk
  float* hlast;           // (B,H,N,P) state leaving the last chunk
  float* CB;              // (B,nc,G,Q,Q)
  // backward scratch
  float* dh;              // (B,nc,H,N,P)
  float* dG;              // (B,nc,G,Q,Q)
  float* dxt;             // (B,T,H,P) gradient w.r.t. x~
  float* rows;            // 4 x (B,T,H): ddt_x, dS, dDrow, dSend(padded)
  float* part;            // (B*nc, 2H) partial sums
  float* splitk;          // split-K partial tiles of the per-group backward contractions
  float* xs;              // (B,T,H,P) x * dt * exp(S_end - S_t)   (tensor-core path only)
  float* dys;             // (B,T,H,P) dY * exp(S_t)               (tensor-core path only)
  // (hi, lo) bf16 pairs of the fused intra-chunk kernels' operands (shapes those kernels take only)
  uint16_t *xt_hi, *xt_lo;   // (B,T,H,P)  x~ = x * dt
  uint16_t *xs_hi, *xs_lo;   // (B,T,H,P)  x~ exp(S_end - S_t)
  uint16_t *dys_hi, *dys_lo; // (B,T,H,P)  dY exp(S_t)
  uint16_t *dg_hi, *dg_lo;   // (B,nc,G,Q,Q) dG
  uint16_t *bc_hi, *bc_lo;   // (B,T,2*G*N) B | C
  uint16_t *dy_hi, *dy_lo;   // (B,T,H,P)  dY
  uint16_t *hp_hi, *hp_lo;   // (B,nc,H,N,P) state entering each chunk
  uint16_t *dh_hi, *dh_lo;   // (B,nc,H,N,P) adjoint of the state leaving each chunk
  float* yoff;               // (B,T,H,P) exp(S_t) C_t h_prev: the carried-state part of y (forward -> backward)
  float *csum, *esum;        // (B,T,H)   column sums of W and the dh term of dS (fused backward)
  float* rpart;              // (B,nc,H,Q/128,Q) partial row sums of W (fused backward)
};
size_t ssd_ws_layout(int B, int T, int H, int P, int N, int G, int Q, void* base, size_t bytes, SsdWs* out);
// the same buffers taken from a caller's arena in two parts: bit 0 = forward-written / backward-read, bit 1 = backward only
struct Arena;
void ssd_ws_take(Arena& ar, int B, int T, int H, int P, int N, int G, int Q, SsdWs* w, int part);
// The scan on bf16 inputs as they are (plain bf16 tensor-core operands, fp32 recurrence; no fp32 staging copies).
// Shapes: d_head 64, d_state 64 or 128, block_len % 128 == 0, at most 64 chunks per sequence.
bool ssd16_supported(int B, int T, int H, int P, int N, int G, int Q);
size_t ssd16_ws_layout(int B, int T, int H, int P, int N, int G, int Q, void* base, size_t bytes, SsdWs* out, float** db32, float** dc32);
pmb_status ssd16_fwd(cudaStream_t st, int B, int T, int H, int P, int N, int G, int Q, const uint16_t* x, const float* a,
                     const uint16_t* b, const uint16_t* c, const float* init_state, uint16_t* y, float* final_state, const SsdWs& ws);
pmb_status ssd16_bwd(cudaStream_t st, int B, int T, int H, int P, int N, int G, int Q, const float* a, const uint16_t* dy,
                     uint16_t* dx, float* da, uint16_t* db, uint16_t* dc, const SsdWs& ws, float* db32, float* dc32);
pmb_status ssd_fwd(cudaStream_t st, const SsdIn& in, const float* init_state, float* y, int64_t ldy,
                   float* final_state, const SsdWs& ws);
// Backward.  dy (stride lddy) is the gradient w.r.t. y (skip term included when in.D != NULL).
// Outputs: dx (stride lddx; gradient w.r.t. raw x when dt != NULL), db/dc (stride lddbc),
// and either `da` (B,T,H) when in.dt == NULL, or ddt (B,T,H), dA (H), dD (H) when in.dt != NULL.
struct SsdGrads {
  float* dx; int64_t lddx;
  float* db; float* dc; int64_t lddbc;
  float* da;    // dt == NULL mode
  float* ddt;   // dt != NULL mode: gradient w.r.t. dt (B,T,H)
  float* dA;    // (H) gradient w.r.t. A
  float* dD;    // (H) gradient w.r.t. D, or NULL
  // Optional, honoured only when ssd_bwd_takes_pairs() is true for the call (dt != NULL mode): the gradient w.r.t. the
  // pre-softplus dt, ddt_raw = ddt (1 - exp(-dt)), written at [token * ld + col0 + h] as a bf16 pair (lo may be NULL:
  // plain bf16 rounding), its sum over tokens d_dt_bias (H), and d_a_log (H) = A dA.
  struct RawDt { uint16_t* hi = nullptr; uint16_t* lo = nullptr; int64_t ld = 0; int col0 = 0; float* d_dt_bias = nullptr; float* d_a_log = nullptr; } raw;
};
// true when the backward with these arguments runs on bf16 pairs (fused intra-chunk kernel) and serves SsdGrads::raw
bool ssd_bwd_takes_pairs(const SsdIn& in, const float* dy, int64_t lddy, const SsdGrads& g);
pmb_status ssd_bwd(cudaStream_t st, const SsdIn& in, const float* y, int64_t ldy, const float* dy, int64_t lddy,
                   const SsdGrads& g, const SsdWs& ws);

// ---- gemm_simt.cu / gemm_tc.cu
pmb_status gemm_simt(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                     const float* B, int64_t ldb, float* C, int64_t ldc, const float* R);
// returns PMB_ERR_UNSUPPORTED (without touching the error text) when alignment rules are not met
pmb_status gemm_tc(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                   const float* B, int64_t ldb, float* C, int64_t ldc, const float* R);
pmb_status gemm_tc_small(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                         const float* B, int64_t ldb, float* C, int64_t ldc, const float* R);
pmb_status read_clear_device_status_small(unsigned int* word);
bool gemm_tc_supported(int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                       const float* B, int64_t ldb, const float* C, int64_t ldc);
pmb_status gemm(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                const float* B, int64_t ldb, float* C, int64_t ldc, const float* R, int engine);
pmb_status read_clear_device_status(unsigned int* word);

// ---- gemm_bf16.cu: bf16 operands, fp32 accumulation; C and R are fp32 or bf16 (out_bf16)
pmb_status gemm_bf16(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                     const void* B, int64_t ldb, void* C, int64_t ldc, const void* R, int out_bf16);
pmb_status read_clear_device_status_bf16(unsigned int* word);
// fp32 matrices as (hi, lo) bf16 pairs: hi = bf16(a), lo = bf16(a - hi); ld = row pitch in elements (multiple of 8)
struct Pair16 { const uint16_t* hi; const uint16_t* lo; int64_t ld; };
pmb_status split_pair16(cudaStream_t st, const float* src, int64_t rows, int64_t cols, int64_t ld, uint16_t* hi, uint16_t* lo,
                        int64_t ld16);
// same, but writes only columns [0, cols) of each destination row and leaves the rest of the pitch untouched
pmb_status split_pair16_strided(cudaStream_t st, const float* src, int64_t rows, int64_t cols, int64_t ld, uint16_t* hi, uint16_t* lo,
                                int64_t ld16);
// tile_mode: -1 = chosen by tile count, 0 = 128x128 single-CTA tiles, 1 = 256x128 / 2 = 256x256 CTA-pair tiles
pmb_status gemm_pairs(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const Pair16& A, const Pair16& B,
                      float* C, int64_t ldc, const float* R, int tile_mode = -1);
// `emit` (optional): the result is also written as a bf16 pair with row pitch emit.ld, for the product that reads it
// next as an operand (needs the TMA-store epilogue: C 16-byte aligned, ldc a multiple of 4; otherwise the call fails)
struct PairGemm { int ta, tb; int64_t M, N, K; Pair16 A, B; float* C; int64_t ldc; const float* R; Pair16 emit = Pair16{nullptr, nullptr, 0}; };
// up to four independent products in one launch (tiles of g[0] first: give it the longer K)
pmb_status gemm_pairs_group(cudaStream_t st, const PairGemm* g, int n, int tile_mode = -1);
bool gemm_pairs_enabled();   // false when PMB_GEMM_ENGINE is tf32 or simt
// fp32 operands of any alignment: split into the library's pair scratch (compacted row pitch), then gemm_pairs
pmb_status gemm_f32_via_bf16x2(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                               const float* B, int64_t ldb, float* C, int64_t ldc, const float* R, int tile_mode = -1);

// ---- block.cu.  w16 != NULL selects bf16 storage: x / residual / out / dout / dx are bf16 and the two
// projections use the bf16 weight copies; NULL = fp32 everywhere.
// With pairs == true the struct instead carries pre-split (hi, lo) bf16 pairs of the fp32 weights (hi in in_proj /
// out_proj, lo in in_lo / out_lo) and storage stays fp32.
struct Weights16 {
  const uint16_t* in_proj; const uint16_t* out_proj;
  const uint16_t* in_lo = nullptr; const uint16_t* out_lo = nullptr;
  bool pairs = false;
};
inline bool storage_is_bf16(const Weights16* w) { return w && !w->pairs; }
bool block_uses_pairs(const Dims& d);   // fp32 blocks route their four projections' GEMMs through bf16 pairs
size_t block_ws_bytes(const Dims& d, bool bf16 = false);
size_t stack_ws_bytes(const Dims& d, bool bf16 = false, bool presplit = false);   // two forward slots: lets stack_bwd recompute one block ahead
pmb_status cast_f32_bf16(cudaStream_t st, const float* src, uint16_t* dst, int64_t n);
pmb_status block_fwd(cudaStream_t st, const Dims& d, const pmb_block_params& p, const void* x, const void* residual,
                     void* out, void* ws, size_t ws_bytes, const Weights16* w16, bool x_pair_ready = false, bool emit_out_pair = false);
pmb_status block_bwd(cudaStream_t st, const Dims& d, const pmb_block_params& p, const void* x, const void* dout,
                     const void* dx_accum, void* dx, const pmb_block_grads& g, void* ws, size_t ws_bytes, const Weights16* w16,
                     bool dout_pair_ready = false, bool emit_dx_pair = false);

pmb_status stack_fwd(cudaStream_t st, const Dims& d, int n_layers, const pmb_block_params* layers, const Weights16* w16,
                     void* saved, void* ws, size_t ws_bytes);
pmb_status stack_bwd(cudaStream_t st, const Dims& d, int n_layers, const pmb_block_params* layers, const Weights16* w16,
                     const pmb_block_grads* grads, const void* saved, void* dhidden, void* ws, size_t ws_bytes,
                     pmb_layer_callback on_layer_done, void* user);

}  // namespace pmb
