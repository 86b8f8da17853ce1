// Batched tile contraction on tcgen05 with operands that are already bf16 in HBM: plain bf16 (NS = 1) or the
// (hi, lo) pair of an fp32 tensor (NS = 2: lo*hi + hi*lo + hi*hi per k-step), specialised by an Op functor.
//
//   OUT[batch](m, n) = sum over segments s, k:  A_s[m,k] * B_s[k,n]
//
// Each CTA owns one 128 x BN output tile of one batch entry.  Operand tiles arrive by TMA (rank-3 bf16 tensor maps:
// contiguous axis, row axis, head/group axis; 128-byte swizzle) into a ring and go to the tensor core as they land:
// nothing rescales or splits a tile in shared memory (the producers of the operands wrote the scaled pairs).  One lane
// issues the MMAs into a TMEM accumulator that lives across all segments; eight warps then drain TMEM and hand
// 32-column row pieces to Op::store.  Operand majorness may differ per segment.  All mbarrier waits are bounded;
// expiry raises *status and the CTA leaves through the common exit.
//
// Op interface (device side; BN, NS, SEG_EPI are static constexpr):
//   int  Mdim, Ndim                                  output extents per batch entry
//   bool init(int batch, int m0, int n0)             false: tile not needed
//   int  nseg()
//   void seg(int s, int m0, int n0, int& kt0, int& kt1, int& amap, int& bmap, int& a_mn, int& b_mn)
//        k tiles [kt0, kt1) of 64; which of the 4 logical tensor maps feed A and B (map 2i = hi, 2i+1 = lo); majorness
//   void a_coord(int s, int kt, int m0, int& c0, int& c1, int& c2)   TMA coordinates of the A tile
//   void b_coord(int s, int kt, int n0, int& c0, int& c1, int& c2)   (K-major: (k, row, z); MN-major: (mn, k, z))
//   void store(int m, int nb, const float (&v)[32])  row m, columns nb..nb+31 (caller-checked m < Mdim)
//   SEG_EPI: every segment gets a fresh TMEM accumulator (two alternate) and the epilogue warps fold it into
//        per-thread registers with  void seg_accumulate(int s, int m, int nb, const float (&v)[32], float (&acc)[32])
//        while the tensor core works on the next segment; store() then receives the register sums;
//        void stage_seg(int s, int tid, int nthreads) fills the segment's half of `aux` (two halves alternate)
//   static constexpr int AUX_FLOATS; float* aux; void stage(int tid, int nthreads)   per-CTA vectors in shared memory
#pragma once
#include "tc_common.cuh"

namespace pmb {
namespace pbg {

using namespace tcx;

constexpr int BM = 128, BK = 64, NEW_WARPS = 8, NEW = NEW_WARPS * 32, NTHREADS = 64 + NEW;

struct MapSet { CUtensorMap m[8]; };   // logical map i: m[2i] = hi (or the plain tensor), m[2i+1] = lo

template <int BN, int NS>
struct Geometry {
  static constexpr int A_BYTES = BM * 128;            // 128 rows x 64 bf16
  static constexpr int B_BYTES = BN * 128;
  static constexpr int PART = A_BYTES + B_BYTES;      // the hi (or lo) tiles of one stage
  static constexpr int STAGE_BYTES = NS * PART;
  // 64-wide tiles: two stages, so that two CTAs share an SM (the per-(batch, chunk, head) problems are short chains
  // that leave the SM idle between dependent steps); wider tiles: as many stages as fit in ~190 KiB, at most four
  // (plain bf16 operands, NS = 1: every tile is half the size and the per-segment products are one or two k-tiles long,
  // so the 128-wide tiles take the two-stage, two-CTA plan as well)
  static constexpr int STAGES = (BN <= 64 || NS == 1) ? 2 : ((190 * 1024) / STAGE_BYTES > 4 ? 4 : (190 * 1024) / STAGE_BYTES);
  static constexpr int CTAS_PER_SM = ((BN <= 64 || NS == 1) && STAGES * STAGE_BYTES <= 100 * 1024) ? 2 : 1;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BASE = RING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <class Op>
__global__ void __launch_bounds__(NTHREADS, Geometry<Op::BN, Op::NS>::CTAS_PER_SM)
pair_bgemm_kernel(const __grid_constant__ MapSet maps, Op op, unsigned int* __restrict__ status, int grid_mode) {
  constexpr int BN = Op::BN, NS = Op::NS;
  using G = Geometry<BN, NS>;
  constexpr int STAGES = G::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles - raw);
  const uint32_t bars = tiles + G::RING_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t accum_bar = bars + 8u * (2 * STAGES);
  auto seg_bar = [&](int b) { return bars + 8u * (2 * STAGES + 1 + b); };    // segment's MMAs complete (SEG_EPI)
  auto free_bar = [&](int b) { return bars + 8u * (2 * STAGES + 3 + b); };   // TMEM buffer drained (SEG_EPI)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tiles_ptr + G::RING_BYTES + 8 * (2 * STAGES + 5));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  op.aux = reinterpret_cast<float*>(tiles_ptr + G::RING_BYTES + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid_mode 0: (n tile, m tile, batch).  1 / 2: (n tile, batch, m tile) with the m tiles in ascending / descending
  // order, so that the tiles with the most k-steps of every batch entry are scheduled first (causal operands).
  const int mt = grid_mode == 0 ? (int)blockIdx.y : (grid_mode == 1 ? (int)blockIdx.z : (int)(gridDim.z - 1 - blockIdx.z));
  const int batch_id = grid_mode == 0 ? (int)blockIdx.z : (int)blockIdx.y;
  const int m0 = mt * BM, n0 = blockIdx.x * BN;
  if (!op.init(batch_id, m0, n0)) return;   // uniform per CTA
  const int nseg = op.nseg();
  op.stage(threadIdx.x, NTHREADS);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(accum_bar, 1);
    for (int b = 0; b < 2; ++b) { mbar_init(seg_bar(b), 1); mbar_init(free_bar(b), NEW_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  constexpr int TMEM_COLS = (BN < 32 ? 32 : BN) * (Op::SEG_EPI ? 2 : 1);
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      bool stop = false;
      for (int sg = 0; sg < nseg && !stop; ++sg) {
        int kt0, kt1, amap, bmap, a_mn, b_mn;
        op.seg(sg, m0, n0, kt0, kt1, amap, bmap, a_mn, b_mn);
        for (int kt = kt0; kt < kt1; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) { atomicOr(status, 1u); *abort_flag = 1; stop = true; break; }
          if (*abort_flag) { stop = true; break; }
          mbar_expect_tx(full_bar(s), G::STAGE_BYTES);
          int a0, a1, a2, b0, b1, b2;
          op.a_coord(sg, kt, m0, a0, a1, a2);
          op.b_coord(sg, kt, n0, b0, b1, b2);
#pragma unroll
          for (int sp = 0; sp < NS; ++sp) {
            const uint32_t a_dst = tiles + s * G::STAGE_BYTES + sp * G::PART, b_dst = a_dst + G::A_BYTES;
            if (!a_mn) {
              tma_load_3d(a_dst, &maps.m[2 * amap + sp], a0, a1, a2, full_bar(s));
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_3d(a_dst + j * (BK * 128), &maps.m[2 * amap + sp], a0 + 64 * j, a1, a2, full_bar(s));
            }
            if (!b_mn) {
              tma_load_3d(b_dst, &maps.m[2 * bmap + sp], b0, b1, b2, full_bar(s));
            } else {
#pragma unroll
              for (int j = 0; j < (BN + 63) / 64; ++j) tma_load_3d(b_dst + j * (BK * 128), &maps.m[2 * bmap + sp], b0 + 64 * j, b1, b2, full_bar(s));
            }
          }
        }
      }
      if (*abort_flag) {
        // give copies already in flight a bounded chance to land before the CTA exits
        for (int k = (it > STAGES ? it - STAGES : 0); k < it; ++k) mbar_wait(full_bar(k % STAGES), (k / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int it = 0;
      bool stop = false;
      const uint32_t d_hi = desc_hi(1024, 2);
      for (int sg = 0; sg < nseg && !stop; ++sg) {
        int kt0, kt1, amap, bmap, a_mn, b_mn;
        op.seg(sg, m0, n0, kt0, kt1, amap, bmap, a_mn, b_mn);
        const uint32_t idesc = idesc_bf16(a_mn, b_mn, BM, BN);
        // K-major: 128-byte rows, 8-row groups 1024 B apart, a k-step (16) advances 32 B.
        // MN-major: 64-wide blocks BK*128 B apart, 8-k-row groups 1024 B apart, a k-step advances 2048 B.
        const uint32_t a_lbo = a_mn ? BK * 128 : 16, b_lbo = b_mn ? BK * 128 : 16;
        const uint32_t a_step = (a_mn ? 2048u : 32u) >> 4, b_step = (b_mn ? 2048u : 32u) >> 4;
        constexpr uint32_t LO = G::PART >> 4;
        uint32_t tmem_d = tmem_acc;
        if (Op::SEG_EPI) {
          tmem_d = tmem_acc + (uint32_t)((sg & 1) * BN);
          if (sg >= 2 && !mbar_wait(free_bar(sg & 1), (uint32_t)(((sg >> 1) - 1) & 1))) { atomicOr(status, 32u); *abort_flag = 1; stop = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        for (int kt = kt0; kt < kt1; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(full_bar(s), ph)) { atomicOr(status, 2u); *abort_flag = 1; stop = true; break; }
          if (*abort_flag) { stop = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_s = tiles + s * G::STAGE_BYTES;
          uint32_t al = desc_lo(a_s, a_lbo), bl = desc_lo(a_s + G::A_BYTES, b_lbo);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const bool first = Op::SEG_EPI ? (kt == kt0 && k == 0) : (it == 0 && k == 0);
            if (NS == 2) {
              mma_f16_h(tmem_d, al + LO, d_hi, bl, d_hi, idesc, first ? 0u : 1u);
              mma_f16_h(tmem_d, al, d_hi, bl + LO, d_hi, idesc, 1u);
              mma_f16_h(tmem_d, al, d_hi, bl, d_hi, idesc, 1u);
            } else {
              mma_f16_h(tmem_d, al, d_hi, bl, d_hi, idesc, first ? 0u : 1u);
            }
            al += a_step; bl += b_step;
          }
          umma_commit(empty_bar(s));
        }
        if (Op::SEG_EPI && !stop) umma_commit(seg_bar(sg & 1));
      }
      umma_commit(accum_bar);
    }
  } else {
    // ---------------- epilogue warps ----------------
    const int st = threadIdx.x - 64;
    bool ok = true;
    const int lane_base = (warp & 3) * 32;       // the TMEM lane quarter this warp may read
    const int grp = (warp - 2) >> 2;             // two warps share a quarter: they take alternate 32-column chunks
    const int m = m0 + lane_base + lane;
    constexpr int NCHUNK = BN / 32 > 0 ? BN / 32 : 1;
    constexpr int MYCH = (NCHUNK + 1) / 2;       // chunks per warp
    float racc[Op::SEG_EPI ? MYCH : 1][32];
    if (Op::SEG_EPI) {
#pragma unroll
      for (int c = 0; c < (Op::SEG_EPI ? MYCH : 1); ++c)
#pragma unroll
        for (int j = 0; j < 32; ++j) racc[c][j] = 0.0f;
      // folds the finished accumulator of segment j into the register sums and hands its TMEM buffer back
      // (a warp that gave up keeps reaching the named barriers below: it skips the work, not the barrier)
      for (int sg = 0; sg < nseg; ++sg) {
        // per-segment vectors for seg_accumulate go to one of two aux halves; the barriers (epilogue warps only) keep
        // a fast warp from overwriting a half that a slower warp still reads for segment sg - 2
        asm volatile("bar.sync 1, %0;" ::"n"(NEW) : "memory");
        if (ok) op.stage_seg(sg, st, NEW);
        asm volatile("bar.sync 1, %0;" ::"n"(NEW) : "memory");
        if (!ok) continue;
        const int b = sg & 1;
        const bool done = __all_sync(0xffffffffu, mbar_wait_idle(seg_bar(b), (uint32_t)((sg >> 1) & 1)));
        if (!done) { if (lane == 0) { atomicOr(status, 64u); *abort_flag = 1; } ok = false; continue; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int cc = 0; cc < (Op::SEG_EPI ? MYCH : 1); ++cc) {
          const int c = 2 * cc + grp;
          if (c < NCHUNK) {
            uint32_t r[32];
            tmem_ld32(tmem_acc + (uint32_t)(b * BN) + ((uint32_t)lane_base << 16) + (uint32_t)(c * 32), r);
            float v[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = __uint_as_float(r[q]);
            op.seg_accumulate(sg, m, n0 + c * 32, v, racc[cc]);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(free_bar(b));
      }
    }
    const bool acc_ok = __all_sync(0xffffffffu, mbar_wait_idle(accum_bar, 0));
    if (!acc_ok && lane == 0) { atomicOr(status, 8u); *abort_flag = 1; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool aborted = __any_sync(0xffffffffu, *abort_flag != 0);
    if (ok && acc_ok && !aborted) {
      if (Op::SEG_EPI) {
#pragma unroll
        for (int cc = 0; cc < (Op::SEG_EPI ? MYCH : 1); ++cc) {
          const int c = 2 * cc + grp;
          if (c < NCHUNK && m < op.Mdim && n0 + c * 32 < op.Ndim) op.store(m, n0 + c * 32, racc[cc]);
        }
      } else {
#pragma unroll 1
        for (int c0 = grp * 32; c0 < BN; c0 += 64) {
          uint32_t r[32];
          tmem_ld32(tmem_acc + ((uint32_t)lane_base << 16) + (uint32_t)c0, r);
          if (m < op.Mdim && n0 + c0 < op.Ndim) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            op.store(m, n0 + c0, v);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS) : "memory");
  }
}

// heavy_m: +1 = the last m tile of a batch entry has the most k-steps, -1 = the first one, 0 = all alike
template <class Op>
static pmb_status launch(cudaStream_t st, const MapSet& maps, const Op& op, int batches, unsigned int* status, int heavy_m = 0) {
  using G = Geometry<Op::BN, Op::NS>;
  PMB_SMEM_OPT_IN(G::SMEM_BASE + Op::AUX_FLOATS * 4, pair_bgemm_kernel<Op>);
  const unsigned mtiles = (unsigned)cdiv(op.Mdim, BM);
  const int mode = (heavy_m == 0 || batches > 65535 || mtiles < 2) ? 0 : (heavy_m > 0 ? 2 : 1);
  dim3 grid((unsigned)cdiv(op.Ndim, Op::BN), mode ? (unsigned)batches : mtiles, mode ? mtiles : (unsigned)batches);
  pair_bgemm_kernel<Op><<<grid, NTHREADS, G::SMEM_BASE + Op::AUX_FLOATS * 4, st>>>(maps, op, status, mode);
  PMB_LAUNCHED();
  return PMB_OK;
}

}  // namespace pbg
}  // namespace pmb
