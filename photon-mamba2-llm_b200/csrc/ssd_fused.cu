// Fused intra-chunk kernel of the chunked SSD scan on tcgen05 (mamba2/ssd_ops.rs:83-138,201-234 compute the same
// chain op by op: C B^T, the decay mask, the product with x, and the carried-state term).
//
// One CTA owns 128 rows of one (batch, chunk, head) and walks the 64-wide column blocks its causal mask allows:
//   1. G = R K^T on the tensor core into one of two TMEM buffers (R = the CTA's 128 rows of C, K = 64 rows of B in
//      mode 0; the roles of B and C swap in mode 1), K = d_state;
//   2. four warps read G from TMEM (thread = row), multiply by exp(S_row - S_col) with the causal test in fp32
//      registers, and write the masked tile into shared memory as a K-major bf16 operand (hi and lo halves of the
//      fp32 value in pair mode);
//   3. acc1 += masked tile x V (V = 64 rows of x~ in mode 0, of dY in mode 1; MN-major) on the tensor core;
// while step 2 of block j runs, the tensor core already computes step 1 of block j+1.  The carried-state term
// (C h_prev in mode 0, B dh in mode 1) goes to a second accumulator and is scaled per row in the epilogue, which
// also adds the skip term D x (mode 0).  C B^T never reaches HBM and no operand is rescaled in shared memory.
//
// Mode 1 (backward) also forms, from the same registers, the quantity the gradient of the decay needs.  With
// dM[t,s] = <dY_t, x~_s> (one more MMA per column block: the x~ rows of the CTA times the dY tile already in shared
// memory) and W[t,s] = dM[t,s] G[t,s] exp(S_t - S_s) for s < t, the gradient w.r.t. the in-chunk cumulative sum is
// dS_k = sum_s W[k,s] - sum_t W[t,k] (+ the carried-state terms).  Row sums over t (thread-private) and column sums
// over s (a fixed-order warp butterfly, then a fixed-order sum over the four warps) come from the SAME register
// values of W, so the near-total cancellation between the two in  sum_k S_k dS_k  (the gradient of A) is between
// identically rounded numbers.  Forming dS as <dY, Y> - <x~, dx~> from two separately rounded tensor-core products
// instead loses the gradient of a_log / dt_bias entirely when |S| is large (strong decay) or the scan's output is
// small next to the skip term.
//
// Operands are bf16 in HBM (TMA, 128-byte swizzle): either plain bf16 (NS = 1, bf16-storage mode) or the (hi, lo)
// pair of an fp32 tensor (NS = 2: lo*hi + hi*lo + hi*hi per product, 16 mantissa bits per operand).
// warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..9 = two mask + epilogue groups of four warps (even / odd
// column blocks), so the mask work of two blocks and the tensor-core work of a third overlap.  Every mbarrier wait is bounded; on
// expiry the CTA raises the status word, stops issuing work, and leaves through the common exit (TMEM freed).
#include <cuda_bf16.h>
#include <mutex>
#include <unordered_map>
#include "tc_common.cuh"
#include "kernels.h"
#include "ssd_fused.h"

namespace pmb {

static __device__ unsigned int g_fused_status = 0;

pmb_status read_clear_device_status_fused(unsigned int* word) {
  unsigned int zero = 0;
  PMB_CUDA(cudaMemcpyFromSymbol(word, g_fused_status, sizeof(unsigned int)));
  if (*word) PMB_CUDA(cudaMemcpyToSymbol(g_fused_status, &zero, sizeof(unsigned int)));
  return PMB_OK;
}

namespace sf {

using namespace tcx;

constexpr int RB = 128;                 // rows per CTA (the MMA's M)
constexpr int CW = 64;                  // columns per block of the masked tile
constexpr int NEPI = 4;                 // warps of one mask / epilogue group: one per TMEM lane quarter
constexpr int NGRP = 2;                 // two groups: one takes the even column blocks, the other the odd ones
constexpr int NMASK = 32 * NEPI * NGRP; // mask / epilogue threads
constexpr int NTHREADS = 64 + NMASK;
constexpr int T128 = RB * 128;          // bytes of a 128-row x 64-element bf16 tile (128-byte rows)
constexpr int T64 = CW * 128;           // bytes of a 64-row x 64-element bf16 tile
constexpr int MAXQ = 1024;

// Shared-memory plan.  NS = operand parts (1 plain bf16, 2 hi/lo), NK = d_state / 64, PB = d_head / 64.
//   ROP    the CTA's row operand, resident: NS x NK tiles of 128 x 64
//   ring   STAGES slots of [K operand: NS x NK tiles of 64 x 64 | V: NS x PB tiles of 64 x 64]; slot use 0 carries the
//          carried-state tile (NS x NK x PB tiles of 64 x 64, never larger than a slot) instead of a column block
//   MOP    MB buffers of the masked tile: NS tiles of 128 x 64
template <int MODE, int NS, int NK, int PB>
struct Geo {
  static constexpr int ROP = NS * NK * T128 + (MODE == 1 ? NS * PB * T128 : 0);   // mode 1: + the x~ rows of the CTA
  static constexpr int XR_OFF = NS * NK * T128;
  static constexpr int COP = NS * NK * T64;
  static constexpr int V = NS * PB * T64;
  static constexpr int STAGE = COP + V;
  static constexpr int ST = NS * NK * PB * T64;
  // TM: the masked tile goes back into TMEM over G and is the A operand of the second product from there, so there
  // are no masked-tile buffers in shared memory.  Mode 0: two CTAs then fit on an SM.  Mode 1 stays at one CTA per SM
  // (384 TMEM columns, two resident row operands) and gains only the shorter hand-over (measured: 3.5 % of the
  // kernel with pairs, nothing with plain bf16 operands, which keep the shared-memory tile).
  static constexpr bool TM = (MODE == 0) || (NS == 2);
  static constexpr int MOP1 = TM ? 0 : NS * T128;
  static constexpr int BUDGET = MODE == 0 ? 104 * 1024 : 218 * 1024;
  static constexpr int MB = (ROP + 2 * MOP1 + 2 * STAGE <= BUDGET) ? 2 : 1;
  static constexpr int REM = BUDGET - ROP - MB * MOP1;
  static constexpr int STAGES = REM / STAGE >= 4 ? 4 : REM / STAGE;
  static constexpr bool FITS = STAGES >= 2 && ST <= STAGE && MB == 2;   // (one masked-tile buffer per mask group)
  static constexpr int TILES = ROP + STAGES * STAGE + MB * MOP1;
  static constexpr int SMEM = TILES + 1024 /*alignment slack*/ + 256 /*barriers*/ + MAXQ * 4 /*S of the chunk*/ +
                              (MODE == 1 ? (2 * NGRP * NEPI * CW + 2 * RB) * 4 : 0) /*column sums of W, group exchange*/;
  static constexpr int TMEM_COLS = ((MODE == 1 ? 4 : 2) * CW + 2 * 64 * PB) <= 256 ? 256 : 512;
  static constexpr int CTAS = (TM && TMEM_COLS == 256) ? 2 : 1;      // CTAs per SM the plan is sized for
};

struct Maps { CUtensorMap rop[2], cop[2], v[2], st[2], xr[2]; };   // [0] = hi (or the plain bf16 tensor), [1] = lo

struct Params {
  int H, hpg, Q, nc, nb, T, N;
  const float* S;
  float* out; int64_t ldo;
  uint16_t* out16;          // when set: the result goes here as bf16 (same row pitch, in elements) instead of to `out`
  const float* x; int64_t ldx; const float* D;
  float* off_out;           // mode 0, optional: (B,T,H,P) the carried-state part of y, exp(S_t) C_t h_prev
  uint16_t* off_out16;      // the same as bf16 (one of the two at most)
  float* csum; float* esum; // mode 1: (B,T,H)  c_s = sum_{t>s} W[t,s];  e_s = exp(S_end - S_s) <x~_s, B_s dh>
  float* rpart;             // mode 1: (B*nc*H, nb, Q)  partial row sums r_t = sum_{s<t} W[t,s] over the s of one row block
  unsigned int* status;
};

// On entry every lane holds v[0..31]: its row's values for 32 consecutive columns.  On exit lane l holds the sum of
// column l over the warp's 32 rows.  Fixed order: the result does not depend on timing.
__device__ __forceinline__ float warp_column_sums(float (&v)[32], int lane) {
#pragma unroll
  for (int w = 16; w >= 1; w >>= 1) {
    const bool upper = (lane & w) != 0;
#pragma unroll
    for (int k = 0; k < w; ++k) {
      const float keep = upper ? v[k + w] : v[k];
      const float send = upper ? v[k] : v[k + w];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, w);
    }
  }
  return v[0];
}

// two fp32 values -> packed bf16x2 of their high parts (round to nearest even) and of the remainders
__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo, bool want_lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  if (want_lo) {
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(a - hf.x, b - hf.y);
    lo = *reinterpret_cast<const uint32_t*>(&l);
  }
}

template <int MODE, int NS, int NK, int PB>
__global__ void __launch_bounds__(NTHREADS, (Geo<MODE, NS, NK, PB>::CTAS))
ssd_fused_kernel(const __grid_constant__ Maps maps, const Params p) {
  using GE = Geo<MODE, NS, NK, PB>;
  constexpr int STAGES = GE::STAGES, MB = GE::MB, P = 64 * PB;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t rop_s = base;
  const uint32_t ring_s = rop_s + GE::ROP;
  const uint32_t mop_s = ring_s + STAGES * GE::STAGE;
  const uint32_t bars = mop_s + MB * GE::MOP1;
  enum { R_FULL = 0, LD_FULL = 1, LD_EMPTY = LD_FULL + STAGES, G_FULL = LD_EMPTY + STAGES, G_FREE = G_FULL + 2,
         M_READY = G_FREE + 2, M_FREE = M_READY + MB, ACC_FULL = M_FREE + MB, NBAR = ACC_FULL + 1 };
  static_assert(8 * NBAR + 8 <= 256, "barrier block");
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint8_t* bar_ptr = base_ptr + (bars - base);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * NBAR);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* sS = reinterpret_cast<float*>(bar_ptr + 256);
  float* rsum = sS + MAXQ;                              // mode 1: [NGRP][2][NEPI][CW] column sums of W per warp
  float* xchg = rsum + 2 * NGRP * NEPI * CW;            // mode 1: [2][RB] second group's row sums, handed to the first

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bch = (int)blockIdx.x;                      // (b * nc + chunk) * H + head
  // the row blocks with the most column blocks are scheduled first
  const int rb = MODE == 0 ? p.nb - 1 - (int)blockIdx.y : (int)blockIdx.y;
  const int h = bch % p.H, bc = bch / p.H, cc = bc % p.nc, bb = bc / p.nc;
  const int g = h / p.hpg;
  const int tok0 = bc * p.Q;                            // first token of the chunk (T = nc * Q)
  const int ncb = MODE == 0 ? 2 * (rb + 1) : (p.Q - RB * rb) / CW;
  const int cb0 = MODE == 0 ? 0 : 2 * rb;
  if (threadIdx.x == 0) {
    mbar_init(bar(R_FULL), 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(bar(LD_FULL + s), 1); mbar_init(bar(LD_EMPTY + s), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar(G_FULL + i), 1); mbar_init(bar(G_FREE + i), NEPI); }
    for (int i = 0; i < MB; ++i) { mbar_init(bar(M_READY + i), NEPI); mbar_init(bar(M_FREE + i), 1); }
    mbar_init(bar(ACC_FULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "n"(GE::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const uint32_t tG = tmem, tDM = tmem + 2 * CW, tA1 = tmem + (MODE == 1 ? 4 : 2) * CW, tA2 = tA1 + P;

  auto give_up = [&](unsigned int code) { atomicOr(p.status, code); *abort_flag = 1; };
  // bounded wait that also ends as soon as another role of the CTA has given up
  auto wait = [&](int b, uint32_t parity, unsigned int code) -> bool {
    if (*abort_flag) return false;
    if (mbar_wait(bar(b), parity)) return true;
    give_up(code);
    return false;
  };
  // the same for the mask warps, which sleep between polls (they share schedulers with the MMA issuer)
  auto wait_idle = [&](int b, uint32_t parity, unsigned int code) -> bool {
    if (*abort_flag) return false;
    if (mbar_wait_idle(bar(b), parity)) return true;
    give_up(code);
    return false;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(bar(R_FULL), GE::ROP);
#pragma unroll
      for (int sp = 0; sp < NS; ++sp)
#pragma unroll
        for (int kt = 0; kt < NK; ++kt)
          tma_load_3d(rop_s + (sp * NK + kt) * T128, &maps.rop[sp], 64 * kt, tok0 + RB * rb, g, bar(R_FULL));
      if (MODE == 1) {
#pragma unroll
        for (int sp = 0; sp < NS; ++sp)
#pragma unroll
          for (int pb = 0; pb < PB; ++pb)
            tma_load_3d(rop_s + GE::XR_OFF + (sp * PB + pb) * T128, &maps.xr[sp], 64 * pb, tok0 + RB * rb, h, bar(R_FULL));
      }
      int issued = 0;
      for (int it = 0; it <= ncb; ++it) {
        const int s = it % STAGES;
        if (!wait(LD_EMPTY + s, (uint32_t)(((it / STAGES) & 1) ^ 1), 1u)) break;
        const uint32_t dst = ring_s + s * GE::STAGE;
        if (it == 0) {
          mbar_expect_tx(bar(LD_FULL + s), GE::ST);
#pragma unroll
          for (int sp = 0; sp < NS; ++sp)
#pragma unroll
            for (int kt = 0; kt < NK; ++kt)
#pragma unroll
              for (int pb = 0; pb < PB; ++pb)
                tma_load_3d(dst + ((sp * NK + kt) * PB + pb) * T64, &maps.st[sp], 64 * pb, bch * p.N + 64 * kt, 0, bar(LD_FULL + s));
        } else {
          const int row0 = tok0 + CW * (cb0 + it - 1);
          mbar_expect_tx(bar(LD_FULL + s), GE::STAGE);
#pragma unroll
          for (int sp = 0; sp < NS; ++sp)
#pragma unroll
            for (int kt = 0; kt < NK; ++kt)
              tma_load_3d(dst + (sp * NK + kt) * T64, &maps.cop[sp], 64 * kt, row0, g, bar(LD_FULL + s));
#pragma unroll
          for (int sp = 0; sp < NS; ++sp)
#pragma unroll
            for (int pb = 0; pb < PB; ++pb)
              tma_load_3d(dst + GE::COP + (sp * PB + pb) * T64, &maps.v[sp], 64 * pb, row0, h, bar(LD_FULL + s));
        }
        issued = it + 1;
      }
      if (*abort_flag) {
        // give the copies already in flight a bounded chance to land before the CTA exits
        mbar_wait(bar(R_FULL), 0);
        for (int it = (issued > STAGES ? issued - STAGES : 0); it < issued; ++it) mbar_wait(bar(LD_FULL + it % STAGES), (uint32_t)((it / STAGES) & 1));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t id_g = idesc_bf16(0, 0, RB, CW);       // G: both operands K-major
      const uint32_t id_v = idesc_bf16(0, 1, RB, P);        // x V and x state: B operand MN-major
      // Operand descriptors as (lo, hi) halves: hi never changes, lo = address field | leading offset.  A product
      // walks its tiles by adding byte offsets >> 4 to lo, so one MMA costs the issuing thread a few integer adds.
      const uint32_t dh = desc_hi(1024, 2);
      auto lo_k = [](uint32_t a) { return desc_lo(a, 16); };          // K-major tile (128-byte rows)
      auto lo_mn = [](uint32_t a) { return desc_lo(a, T64); };        // MN-major: 64-wide blocks along N are T64 apart
      // one k-step (16) of a product whose operands are split NS ways: A parts `as` apart, B parts `bs` apart (16-byte units)
      auto kstep = [&](uint32_t d, uint32_t alo, uint32_t as, uint32_t blo, uint32_t bs, uint32_t idesc, uint32_t acc) {
        if (NS == 2) {
          mma_f16_h(d, alo + as, dh, blo, dh, idesc, acc);        // lo x hi
          mma_f16_h(d, alo, dh, blo + bs, dh, idesc, 1u);         // hi x lo
          mma_f16_h(d, alo, dh, blo, dh, idesc, 1u);              // hi x hi
        } else {
          mma_f16_h(d, alo, dh, blo, dh, idesc, acc);
        }
      };
      bool ok = wait(R_FULL, 0u, 2u) && wait(LD_FULL + 0, 0u, 2u);
      if (ok) {
        // carried-state term: acc2 = R x state  (K = d_state)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t r0 = lo_k(rop_s), s0 = lo_mn(ring_s);
#pragma unroll
        for (int kt = 0; kt < NK; ++kt)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            kstep(tA2, r0 + ((kt * T128 + k * 32) >> 4), (NK * T128) >> 4, s0 + ((kt * PB * T64 + k * 2048) >> 4), (NK * PB * T64) >> 4, id_v, (kt | k) ? 1u : 0u);
        umma_commit(bar(LD_EMPTY + 0));
      }
      // G of column block jj into TMEM buffer jj & 1
      auto mma_g = [&](int jj) -> bool {
        const int it = jj + 1, s = it % STAGES;
        if (!wait(LD_FULL + s, (uint32_t)((it / STAGES) & 1), 2u)) return false;
        // (TM: the buffer's previous content, masked tile jj - 2, was read by a product issued before this one)
        if (!GE::TM && jj >= 2 && !wait(G_FREE + (jj & 1), (uint32_t)(((jj >> 1) - 1) & 1), 4u)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t cop = ring_s + s * GE::STAGE;
        const uint32_t r0 = lo_k(rop_s), c0d = lo_k(cop);
#pragma unroll
        for (int kt = 0; kt < NK; ++kt)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            kstep(tG + (uint32_t)((jj & 1) * CW), r0 + ((kt * T128 + k * 32) >> 4), (NK * T128) >> 4, c0d + ((kt * T64 + k * 32) >> 4), (NK * T64) >> 4, id_g, (kt | k) ? 1u : 0u);
        if (MODE == 1) {
          // dM^T[s,t] = <x~_s, dY_t>: the resident x~ rows times the dY tile of this block read as a K-major operand
          // (its 64 rows of 128 bytes are the same bytes that the product with the masked tile reads MN-major)
#pragma unroll
          for (int pb = 0; pb < PB; ++pb)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              kstep(tDM + (uint32_t)((jj & 1) * CW), r0 + ((GE::XR_OFF + pb * T128 + k * 32) >> 4), (PB * T128) >> 4,
                    c0d + ((GE::COP + pb * T64 + k * 32) >> 4), (PB * T64) >> 4, id_g, (pb | k) ? 1u : 0u);
        }
        umma_commit(bar(G_FULL + (jj & 1)));
        return true;
      };
      // G runs two blocks ahead of the masked product: one block for each mask group
      ok = ok && mma_g(0);
      if (ok && ncb > 1) ok = mma_g(1);
      for (int jj = 0; jj < ncb && ok; ++jj) {
        const int mb = jj % MB, s = (jj + 1) % STAGES;
        if (!wait(M_READY + mb, (uint32_t)((jj / MB) & 1), 8u)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t m0d = lo_k(mop_s + mb * GE::MOP1), v0d = lo_mn(ring_s + s * GE::STAGE + GE::COP);
        if (GE::TM) {
          // masked tile in TMEM, in place of G: per 32 k of the block [hi: 16 columns | lo: 16 columns], 8 columns per k-step
          const uint32_t bs = (PB * T64) >> 4;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t ta = tG + (uint32_t)(mb * CW + (k >> 1) * 32 + (k & 1) * 8);
            const uint32_t vb = v0d + ((k * 2048) >> 4);
            const uint32_t acc = (jj | k) ? 1u : 0u;
            if (NS == 2) {
              mma_f16_ts_h(tA1, ta + 16u, vb, dh, id_v, acc);        // lo x hi
              mma_f16_ts_h(tA1, ta, vb + bs, dh, id_v, 1u);          // hi x lo
              mma_f16_ts_h(tA1, ta, vb, dh, id_v, 1u);               // hi x hi
            } else {
              mma_f16_ts_h(tA1, ta, vb, dh, id_v, acc);
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            kstep(tA1, m0d + ((k * 32) >> 4), T128 >> 4, v0d + ((k * 2048) >> 4), (PB * T64) >> 4, id_v, (jj | k) ? 1u : 0u);
        }
        umma_commit(bar(LD_EMPTY + s));
        umma_commit(bar(M_FREE + mb));
        if (jj + 2 < ncb && !mma_g(jj + 2)) { ok = false; break; }
      }
      umma_commit(bar(ACC_FULL));
    }
  } else {
    // ---------------- mask (TMEM -> registers -> shared-memory operand), then epilogue ----------------
    const int quarter = warp & 3;                       // the TMEM lane quarter this warp may read
    const int grp = (warp - 2) >> 2;                    // mask group: column blocks jj with jj % 2 == grp
    const int r_local = quarter * 32 + lane;
    const int row = rb * RB + r_local;                  // row within the chunk
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    // S of the chunk -> shared memory (the copies and the first G product are already under way)
    {
      const float* Sp = p.S + ((int64_t)bb * p.H + h) * p.T + (int64_t)cc * p.Q;
      for (int q = (int)threadIdx.x - 64; q < p.Q; q += NMASK) sS[q] = Sp[q];
      asm volatile("bar.sync 3, %0;" ::"n"(NMASK) : "memory");
    }
    const float S_row = sS[row];
    bool ok = true;
    float c_acc = 0.0f;                                 // mode 1: sum over t > s of W[t,s] for this thread's row s
    // Every iteration reaches the named barrier below whatever happened before it (a warp that gave up skips the
    // work, not the barrier), so the four warps of a group can never wait for one another unboundedly.
    for (int jj = grp; jj < ncb; jj += NGRP) {
      const int c0 = (cb0 + jj) * CW, mb = jj & 1, use = jj >> 1;       // use-th block of this group's buffers
      bool got = ok && wait_idle(G_FULL + mb, (uint32_t)(use & 1), 16u);
      if (!GE::TM && got && use >= 1) got = wait_idle(M_FREE + mb, (uint32_t)((use - 1) & 1), 32u);
      ok = __all_sync(0xffffffffu, got);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint8_t* mrow = base_ptr + (mop_s - base) + mb * GE::MOP1 + (r_local >> 3) * 1024 + (r_local & 7) * 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32(tG + lane_addr + (uint32_t)(mb * CW + half * 32), r);
          float wv[32];
          if (MODE == 1) {
            uint32_t d[32];
            tmem_ld32(tDM + lane_addr + (uint32_t)(mb * CW + half * 32), d);
#pragma unroll
            for (int e = 0; e < 32; ++e) wv[e] = __uint_as_float(d[e]);
          }
          uint32_t mh[16], ml[16];                  // TM: this half's packed hi / lo values
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint32_t hi[4], lo[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const int e = q8 * 8 + 2 * e2;
              const int col = c0 + half * 32 + e;
              const float2 sc = *reinterpret_cast<const float2*>(sS + col);
              float m0, m1;
              if (MODE == 0) {       // row = t, col = s: exp(S_t - S_s) for s <= t
                m0 = col <= row ? __uint_as_float(r[e]) * __expf(S_row - sc.x) : 0.0f;
                m1 = col + 1 <= row ? __uint_as_float(r[e + 1]) * __expf(S_row - sc.y) : 0.0f;
              } else {               // row = s, col = t: exp(S_t - S_s) for t >= s
                m0 = col >= row ? __uint_as_float(r[e]) * __expf(sc.x - S_row) : 0.0f;
                m1 = col + 1 >= row ? __uint_as_float(r[e + 1]) * __expf(sc.y - S_row) : 0.0f;
                // W[t,s] for t > s (the diagonal does not depend on S)
                wv[e] = col > row ? wv[e] * m0 : 0.0f;
                wv[e + 1] = col + 1 > row ? wv[e + 1] * m1 : 0.0f;
                c_acc += wv[e] + wv[e + 1];
              }
              split2(m0, m1, hi[e2], lo[e2], NS == 2);
            }
            if (GE::TM) {
#pragma unroll
              for (int e2 = 0; e2 < 4; ++e2) { mh[q8 * 4 + e2] = hi[e2]; ml[q8 * 4 + e2] = lo[e2]; }
            } else {
              const int sw = ((half * 4 + q8) ^ (r_local & 7)) << 4;     // 128-byte swizzle of the 16-byte chunk
              *reinterpret_cast<uint4*>(mrow + sw) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
              if (NS == 2) *reinterpret_cast<uint4*>(mrow + T128 + sw) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
          }
          if (GE::TM) {
            // over the 32 columns of G just read: [hi of these 32 k | lo of these 32 k]
            tmem_st16(tG + lane_addr + (uint32_t)(mb * CW + half * 32), mh);
            if (NS == 2) tmem_st16(tG + lane_addr + (uint32_t)(mb * CW + half * 32 + 16), ml);
          }
          if (MODE == 1) {
            // column sums of W over this warp's 32 rows: lane l ends up with column half*32 + l
            rsum[(((grp * 2) + (use & 1)) * NEPI + quarter) * CW + half * 32 + lane] = warp_column_sums(wv, lane);
          }
        }
        if (GE::TM) tmem_wait_st();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (!GE::TM) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) { if (!GE::TM) mbar_arrive(bar(G_FREE + mb)); mbar_arrive(bar(M_READY + mb)); }
      }
      if (MODE == 1) {
        if (grp == 0) asm volatile("bar.sync 1, %0;" ::"n"(32 * NEPI) : "memory");
        else asm volatile("bar.sync 2, %0;" ::"n"(32 * NEPI) : "memory");
        // r_t partial of this row block for the 64 columns t of the block: the four warps' sums in a fixed order
        if (r_local < CW && *abort_flag == 0) {
          const float* q = rsum + ((grp * 2) + (use & 1)) * NEPI * CW + r_local;
          p.rpart[((int64_t)bch * p.nb + rb) * p.Q + c0 + r_local] = ((q[0] + q[CW]) + q[2 * CW]) + q[3 * CW];
        }
      }
    }
    const int64_t trow = (int64_t)tok0 + row;
    // the skip term's x for this thread's first output piece is requested before the wait for the accumulators
    float4 xpre[8];
    if (MODE == 0 && p.D) {
      const float4* xs0 = reinterpret_cast<const float4*>(p.x + trow * p.ldx + h * P + 32 * grp);
#pragma unroll
      for (int j = 0; j < 8; ++j) xpre[j] = xs0[j];
    }
    const bool acc_ok = __all_sync(0xffffffffu, ok && wait_idle(ACC_FULL, 0u, 64u));
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool aborted = __any_sync(0xffffffffu, *abort_flag != 0);
    const bool run = acc_ok && !aborted;
    const float fac = MODE == 0 ? __expf(S_row) : __expf(sS[p.Q - 1] - S_row);
    float e_acc = 0.0f;       // mode 1: <x~_s, B_s dh> with x~ read back from the resident operand tile (hi + lo)
    if (run) {
      const float dv = (MODE == 0 && p.D) ? p.D[h] : 0.0f;
      // the two groups share the columns of the output: 32-column pieces alternate between them
#pragma unroll 1
      for (int c0 = 32 * grp; c0 < P; c0 += 32 * NGRP) {
        uint32_t a1[32], a2[32];
        tmem_ld32(tA1 + lane_addr + (uint32_t)c0, a1);
        tmem_ld32(tA2 + lane_addr + (uint32_t)c0, a2);
        if (MODE == 0 && p.off_out) {
          float4* od = reinterpret_cast<float4*>(p.off_out + (trow * p.H + h) * (int64_t)P + c0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            od[j] = make_float4(fac * __uint_as_float(a2[4 * j]), fac * __uint_as_float(a2[4 * j + 1]), fac * __uint_as_float(a2[4 * j + 2]),
                                fac * __uint_as_float(a2[4 * j + 3]));
        }
        if (MODE == 0 && p.off_out16) {
          uint2* od = reinterpret_cast<uint2*>(p.off_out16 + (trow * p.H + h) * (int64_t)P + c0);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const __nv_bfloat162 b0 = __floats2bfloat162_rn(fac * __uint_as_float(a2[4 * j]), fac * __uint_as_float(a2[4 * j + 1]));
            const __nv_bfloat162 b1 = __floats2bfloat162_rn(fac * __uint_as_float(a2[4 * j + 2]), fac * __uint_as_float(a2[4 * j + 3]));
            od[j] = make_uint2(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
          }
        }
        if (MODE == 1) {
          // this row of the x~ tile: 64-element block c0 / 64, 16-byte chunks (c0 % 64) / 8 .. + 3, swizzled
          const uint8_t* xrow = base_ptr + (rop_s - base) + GE::XR_OFF + (c0 >> 6) * T128 + (r_local >> 3) * 1024 + (r_local & 7) * 128;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const int sw = ((((c0 & 63) >> 3) + ch) ^ (r_local & 7)) << 4;
            const uint4 xh = *reinterpret_cast<const uint4*>(xrow + sw);
            const uint32_t hw[4] = {xh.x, xh.y, xh.z, xh.w};
            uint32_t lw[4] = {0u, 0u, 0u, 0u};
            if (NS == 2) { const uint4 xl = *reinterpret_cast<const uint4*>(xrow + PB * T128 + sw); lw[0] = xl.x; lw[1] = xl.y; lw[2] = xl.z; lw[3] = xl.w; }
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
              const float x0 = __uint_as_float(hw[e2] << 16) + __uint_as_float(lw[e2] << 16);
              const float x1 = __uint_as_float(hw[e2] & 0xffff0000u) + __uint_as_float(lw[e2] & 0xffff0000u);
              e_acc = fmaf(x0, __uint_as_float(a2[ch * 8 + 2 * e2]), e_acc);
              e_acc = fmaf(x1, __uint_as_float(a2[ch * 8 + 2 * e2 + 1]), e_acc);
            }
          }
        }
        float4* dst = reinterpret_cast<float4*>(p.out + trow * p.ldo + h * P + c0);
        uint2* dst16 = reinterpret_cast<uint2*>(p.out16 + trow * p.ldo + h * P + c0);
        const float4* xs = (MODE == 0 && p.D) ? reinterpret_cast<const float4*>(p.x + trow * p.ldx + h * P + c0) : nullptr;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o;
          o.x = fmaf(fac, __uint_as_float(a2[4 * j]), __uint_as_float(a1[4 * j]));
          o.y = fmaf(fac, __uint_as_float(a2[4 * j + 1]), __uint_as_float(a1[4 * j + 1]));
          o.z = fmaf(fac, __uint_as_float(a2[4 * j + 2]), __uint_as_float(a1[4 * j + 2]));
          o.w = fmaf(fac, __uint_as_float(a2[4 * j + 3]), __uint_as_float(a1[4 * j + 3]));
          if (xs) {
            const float4 q = (c0 == 32 * grp) ? xpre[j] : xs[j];
            o.x = fmaf(dv, q.x, o.x); o.y = fmaf(dv, q.y, o.y); o.z = fmaf(dv, q.z, o.z); o.w = fmaf(dv, q.w, o.w);
          }
          if (p.out16) {
            const __nv_bfloat162 b0 = __floats2bfloat162_rn(o.x, o.y), b1 = __floats2bfloat162_rn(o.z, o.w);
            dst16[j] = make_uint2(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
          } else {
            dst[j] = o;
          }
        }
      }
    }
    if (MODE == 1) {
      // the second group hands its partial row sums to the first (same rows, other column blocks / output pieces)
      if (grp == 1) { xchg[r_local] = c_acc; xchg[RB + r_local] = e_acc; }
      asm volatile("bar.sync 3, %0;" ::"n"(NMASK) : "memory");
      if (grp == 0 && run) {
        p.csum[trow * p.H + h] = c_acc + xchg[r_local];
        p.esum[trow * p.H + h] = fac * (e_acc + xchg[RB + r_local]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(GE::TMEM_COLS) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------------------
struct MapKey {
  const void* base; int64_t d0, d1, d2, s0, s1; int b0, b1;
  bool operator==(const MapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s0 == o.s0 && s1 == o.s1 && b0 == o.b0 && b1 == o.b1;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.base);
    auto mix = [&](int64_t v) { h ^= std::hash<int64_t>()(v) + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2); };
    mix(k.d0); mix(k.d1); mix(k.d2); mix(k.s0); mix(k.s1); mix(k.b0); mix(k.b1);
    return h;
  }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;   // shared by all devices and host threads
static std::mutex g_maps_mu;

// rank-3 bf16 map: dims (d0 contiguous, d1 rows with pitch s0 elements, d2 with pitch s1 elements), box (b0, b1, 1),
// 128-byte swizzle
pmb_status bf16_map3(CUtensorMap* out, const uint16_t* base, int64_t d0, int64_t d1, int64_t d2, int64_t s0, int64_t s1, int b0, int b1) {
  MapKey key{base, d0, d1, d2, s0, s1, b0, b1};
  std::lock_guard<std::mutex> lock(g_maps_mu);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    if (g_maps.size() > 8192) g_maps.clear();
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(PMB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)d2};
    cuuint64_t strides[2] = {(cuuint64_t)s0 * 2, (cuuint64_t)s1 * 2};
    cuuint32_t box[3] = {(cuuint32_t)b0, (cuuint32_t)b1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<uint16_t*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return fail(PMB_ERR_CUDA, "cuTensorMapEncodeTiled (bf16, rank 3) failed with code %d (dims %lld %lld %lld, pitches %lld %lld)", (int)r,
                  (long long)d0, (long long)d1, (long long)d2, (long long)s0, (long long)s1);
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return PMB_OK;
}

static unsigned int* status_ptr() {
  static unsigned int* ptr[PMB_MAX_DEVICES] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= PMB_MAX_DEVICES) dev = 0;
  if (!ptr[dev]) cudaGetSymbolAddress((void**)&ptr[dev], g_fused_status);
  return ptr[dev];
}

template <int MODE, int NS, int NK, int PB>
static pmb_status launch(cudaStream_t st, const FusedArgs& a) {
  using GE = Geo<MODE, NS, NK, PB>;
  if (!GE::FITS) return fail(PMB_ERR_UNSUPPORTED, "ssd_fused: this shape does not fit the shared-memory plan");
  const int nc = a.T / a.Q;
  const int64_t tok = (int64_t)a.B * a.T;
  const Op16& rop = MODE == 0 ? a.c : a.b;
  const Op16& cop = MODE == 0 ? a.b : a.c;
  Maps ms{};
  for (int sp = 0; sp < NS; ++sp) {
    const uint16_t* r = sp ? rop.lo : rop.hi; const uint16_t* c = sp ? cop.lo : cop.hi;
    const uint16_t* v = sp ? a.v.lo : a.v.hi; const uint16_t* s = sp ? a.state.lo : a.state.hi;
    PMB_TRY(bf16_map3(&ms.rop[sp], r, a.N, tok, a.G, rop.pitch, a.N, 64, RB));
    PMB_TRY(bf16_map3(&ms.cop[sp], c, a.N, tok, a.G, cop.pitch, a.N, 64, CW));
    PMB_TRY(bf16_map3(&ms.v[sp], v, a.P, tok, a.H, a.v.pitch, a.P, 64, CW));
    PMB_TRY(bf16_map3(&ms.st[sp], s, a.P, (int64_t)a.B * nc * a.H * a.N, 1, a.P, (int64_t)a.P * a.N, 64, CW));
    if (MODE == 1) PMB_TRY(bf16_map3(&ms.xr[sp], sp ? a.xt.lo : a.xt.hi, a.P, tok, a.H, a.xt.pitch, a.P, 64, RB));
    else ms.xr[sp] = ms.rop[sp];
  }
  if (NS == 1) { ms.rop[1] = ms.rop[0]; ms.cop[1] = ms.cop[0]; ms.v[1] = ms.v[0]; ms.st[1] = ms.st[0]; ms.xr[1] = ms.xr[0]; }
  Params p{};
  p.H = a.H; p.hpg = a.H / a.G; p.Q = a.Q; p.nc = nc; p.nb = a.Q / RB; p.T = a.T; p.N = a.N;
  p.S = a.S; p.out = a.out; p.out16 = a.out16; p.ldo = a.ldo; p.x = a.x; p.ldx = a.ldx; p.D = a.D;
  p.off_out = a.off_out; p.off_out16 = a.off_out16; p.csum = a.csum; p.esum = a.esum; p.rpart = a.rpart;
  p.status = status_ptr();
  PMB_SMEM_OPT_IN(GE::SMEM, ssd_fused_kernel<MODE, NS, NK, PB>);
  if (GE::CTAS > 1) {      // two CTAs per SM need the largest shared-memory carve-out
    static DeviceOnce once;
    int dev = 0;
    PMB_CUDA(cudaGetDevice(&dev));
    if (once.pending(dev)) {
      PMB_CUDA(cudaFuncSetAttribute(ssd_fused_kernel<MODE, NS, NK, PB>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
      once.mark(dev);
    }
  }
  dim3 grid((unsigned)(a.B * nc * a.H), (unsigned)p.nb);
  ssd_fused_kernel<MODE, NS, NK, PB><<<grid, NTHREADS, GE::SMEM, st>>>(ms, p);
  PMB_LAUNCHED();
  return PMB_OK;
}

template <int MODE, int NS>
static pmb_status pick(cudaStream_t st, const FusedArgs& a) {
  const int nk = a.N / 64, pb = a.P / 64;
  if (nk == 1 && pb == 1) return launch<MODE, NS, 1, 1>(st, a);
  if (NS == 1) {      // plain bf16 operands are half the size: the wider shapes fit as well
    if (nk == 2 && pb == 1) return launch<MODE, 1, 2, 1>(st, a);
    if (nk == 1 && pb == 2) return launch<MODE, 1, 1, 2>(st, a);
    if (nk == 2 && pb == 2) return launch<MODE, 1, 2, 2>(st, a);
  }
  return fail(PMB_ERR_UNSUPPORTED, "ssd_fused: d_state %d / d_head %d not supported", a.N, a.P);
}

}  // namespace sf

bool ssd_fused_supported(int P, int N, int Q, bool pairs) {
  if (Q % sf::RB != 0 || Q > sf::MAXQ) return false;
  if (!(N == 64 || N == 128) || !(P == 64 || P == 128)) return false;
  if (pairs && !(N == 64 && P == 64)) return false;     // the backward's plan (two resident row operands) fits pairs at 64 x 64 only
  return true;
}

pmb_status ssd_fused(cudaStream_t st, int mode, const FusedArgs& a) {
  const bool pairs = a.c.lo != nullptr;
  if (!ssd_fused_supported(a.P, a.N, a.Q, pairs) || a.T % a.Q != 0 || a.H % a.G != 0)
    return fail(PMB_ERR_UNSUPPORTED, "ssd_fused: unsupported shape (P=%d N=%d Q=%d)", a.P, a.N, a.Q);
  if ((a.b.lo != nullptr) != pairs || (a.v.lo != nullptr) != pairs || (a.state.lo != nullptr) != pairs || (mode == 1 && (a.xt.lo != nullptr) != pairs))
    return fail(PMB_ERR_ARG, "ssd_fused: operands must be all pairs or all plain bf16");
  if (mode == 1 && (!a.xt.hi || !a.csum || !a.esum || !a.rpart)) return fail(PMB_ERR_ARG, "ssd_fused: mode 1 needs x~ and the three sum outputs");
  if ((int64_t)a.B * a.T >= (1LL << 31) || (int64_t)a.B * (a.T / a.Q) * a.H * a.N >= (1LL << 31))
    return fail(PMB_ERR_SHAPE, "ssd_fused: too many rows for 32-bit tile coordinates");
  if (!a.out && !a.out16) return fail(PMB_ERR_ARG, "ssd_fused: no output");
  if ((a.ldo & 3) || ((reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.out16)) & 15) || (a.D && ((a.ldx & 3) || (reinterpret_cast<uintptr_t>(a.x) & 15))))
    return fail(PMB_ERR_SHAPE, "ssd_fused: output and x rows must be 16-byte aligned");
  const double tok = (double)a.B * a.T;
  // algorithmic work: G per head (2 Q N), masked product (2 Q P) over the causal half (counted in full), state term (2 N P)
  ProfScope prof(st, mode == 0 ? "ssd_fused_y" : "ssd_fused_dx", 2.0 * tok * a.H * ((double)a.Q * (a.N + a.P) + (double)a.N * a.P), 0.0);
  if (mode == 0) return pairs ? sf::pick<0, 2>(st, a) : sf::pick<0, 1>(st, a);
  return pairs ? sf::pick<1, 2>(st, a) : sf::pick<1, 1>(st, a);
}

}  // namespace pmb
