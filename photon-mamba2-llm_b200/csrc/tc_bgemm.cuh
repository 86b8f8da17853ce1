// Batched tile contraction on tcgen05 with fp32 operands (3xTF32), specialised by an Op functor.
//
//   OUT[batch](m, n) = sum over segments s, k:  (A_s[m,k] * a_scale_s(m,k)) * (B_s[k,n] * b_scale_s(n,k))
//
// Each CTA owns one 128 x BN output tile of one batch entry.  Operand tiles arrive by TMA (rank-3 tensor
// maps: contiguous axis, token/row axis, head/group axis) into a 3-stage ring; eight "transform" warps
// rescale the landed tile in shared memory (decay factors, dt, causal mask) and split it into TF32-exact
// high and low parts; one lane issues three kind::tf32 MMAs per k-step into a TMEM accumulator that lives
// across all segments; the transform warps then drain TMEM and hand 32-column row pieces to Op::store.
// A zero scale forces the element to zero even if the landed value is not finite (masked regions).
// Operand majorness may differ per segment (K-major tiles use the 128-byte swizzle, MN-major tiles the
// 32-byte-atom variant).  All mbarrier waits are bounded; expiry raises *status and the CTA drains.
//
// Op interface (device side; BN, A_SCALE, B_SCALE are static constexpr):
//   int  Mdim, Ndim                                  output extents per batch entry
//   bool init(int batch, int m0, int n0)             false: tile not needed
//   int  nseg()
//   void seg(int s, int m0, int n0, int& kt0, int& kt1, int& amap, int& bmap, int& a_mn, int& b_mn)
//        k tiles [kt0, kt1) of 32; which of the 4 tensor maps feed A and B; operand majorness
//   void a_coord(int s, int kt, int m0, int& c0, int& c1, int& c2)   TMA coordinates of the A tile
//   void b_coord(int s, int kt, int n0, int& c0, int& c1, int& c2)   (K-major: (k, row, z); MN-major: (mn, k, z))
//   void a_scale4(int s, int a_mn, int m, int k, float (&f)[4])   (only if A_SCALE) rescales the four values of one
//        16-byte chunk in place: elements (m, k..k+3) of a K-major tile or (m..m+3, k) of an MN-major tile;
//        an element that must not contribute is set to exactly 0 whatever was loaded
//   float b_scale(int s, int n, int k)                            (only if B_SCALE)
//   void store(int m, int nb, const float (&v)[32])  row m, columns nb..nb+31 (caller-checked m < Mdim)
//   static constexpr bool SEG_EPI: when true every segment gets a fresh TMEM accumulator (two are alternated) and the
//        transform warps fold it into per-thread registers with
//        void seg_accumulate(int s, int m, int nb, const float (&v)[32], float (&acc)[32])
//        while the tensor core already works on the next segment; store() then receives the register sums;
//        void stage_seg(int s, int tid, int nthreads) fills the segment's half of `aux` (two halves alternate)
//   static constexpr int AUX_FLOATS; float* aux; void stage(int tid, int nthreads)
//        per-CTA vectors (cumulative sums, dt) copied once into shared memory at `aux` before the pipeline
//        starts, so that the scale functors and the epilogue read them with shared-memory latency
#pragma once
#include "tc_common.cuh"

namespace pmb {
namespace tcb {

using namespace tcx;

// warp 0: TMA producer, warp 1: MMA issuer, warps 2..9: transform + epilogue.  Eight transform warps (two per
// scheduler and CTA) because the scale/split work, not the tensor core, paces the small per-chunk problems.
constexpr int BM = 128, BK = 32, NXF_WARPS = 8, NXF = NXF_WARPS * 32, NTHREADS = 64 + NXF;
// Ring depth: 3 stages and one CTA per SM for 128-wide tiles; 2 stages for 64-wide tiles so that two CTAs share
// an SM (the small per-(batch,chunk,head) problems are latency-bound: a second resident CTA fills the bubbles).
template <int BN> struct RingDepth { static constexpr int STAGES = BN <= 64 ? 2 : 3; static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1; };

struct MapSet { CUtensorMap m[4]; };

template <int BN>
struct Geometry {
  static constexpr int STAGES = RingDepth<BN>::STAGES;
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int HALF = A_BYTES + B_BYTES;       // hi (or lo) part of one stage
  static constexpr int STAGE_BYTES = 2 * HALF;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BASE = RING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// logical (row, k) of the 4 floats held by 16-byte chunk `i` of a K-major tile (rows of 128 bytes)
__device__ __forceinline__ void decode_kmajor(int i, int& row, int& k) {
  row = i >> 3;
  k = (((i & 7) ^ (row & 7)) << 2);
}
// logical (mn, k) of chunk `i` of an MN-major tile: blocks of 32 floats along MN, BK rows of 128 bytes each,
// 32-byte units XOR-swizzled with (k row mod 4)
__device__ __forceinline__ void decode_mnmajor(int i, int& mn, int& k) {
  int blk = i / (BK * 8);
  int r = (i >> 3) & (BK - 1);
  int c32 = (i >> 1) & 3, half = i & 1;
  k = r;
  mn = blk * 32 + ((c32 ^ (r & 3)) << 3) + (half << 2);
}

template <class Op>
__global__ void __launch_bounds__(NTHREADS, RingDepth<Op::BN>::CTAS_PER_SM)
tc_bgemm_kernel(const __grid_constant__ MapSet maps, Op op, unsigned int* __restrict__ status, int grid_mode) {
  constexpr int BN = Op::BN;
  using G = Geometry<BN>;
  constexpr int STAGES = G::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles - raw);
  const uint32_t bars = tiles + STAGES * G::STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto split_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto empty_bar = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  const uint32_t accum_bar = bars + 8u * (3 * STAGES);
  auto seg_bar = [&](int b) { return bars + 8u * (3 * STAGES + 1 + b); };    // segment's MMAs complete (SEG_EPI)
  auto free_bar = [&](int b) { return bars + 8u * (3 * STAGES + 3 + b); };   // TMEM buffer drained (SEG_EPI)
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tiles_ptr + STAGES * G::STAGE_BYTES + 8 * (3 * STAGES + 5));
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
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(split_bar(s), NXF_WARPS);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(accum_bar, 1);
    for (int b = 0; b < 2; ++b) { mbar_init(seg_bar(b), 1); mbar_init(free_bar(b), NXF_WARPS); }
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
          const uint32_t a_dst = tiles + s * G::STAGE_BYTES, b_dst = a_dst + G::A_BYTES;
          mbar_expect_tx(full_bar(s), G::HALF);
          int c0, c1, c2;
          op.a_coord(sg, kt, m0, c0, c1, c2);
          if (!a_mn) {
            tma_load_3d(a_dst, &maps.m[amap], c0, c1, c2, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < BM / 32; ++j) tma_load_3d(a_dst + j * (BK * 128), &maps.m[amap], c0 + 32 * j, c1, c2, full_bar(s));
          }
          op.b_coord(sg, kt, n0, c0, c1, c2);
          if (!b_mn) {
            tma_load_3d(b_dst, &maps.m[bmap], c0, c1, c2, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j) tma_load_3d(b_dst + j * (BK * 128), &maps.m[bmap], c0 + 32 * j, c1, c2, full_bar(s));
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
      for (int sg = 0; sg < nseg && !stop; ++sg) {
        int kt0, kt1, amap, bmap, a_mn, b_mn;
        op.seg(sg, m0, n0, kt0, kt1, amap, bmap, a_mn, b_mn);
        const uint32_t idesc = idesc_tf32(a_mn, b_mn, BM, BN);
        const uint32_t a_lbo = a_mn ? BK * 128 : 16, b_lbo = b_mn ? BK * 128 : 16;
        const uint32_t a_kstep = a_mn ? 1024 : 32, b_kstep = b_mn ? 1024 : 32;
        const uint32_t a_sbo = a_mn ? 512 : 1024, b_sbo = b_mn ? 512 : 1024;
        const uint32_t a_lt = a_mn ? 1 : 2, b_lt = b_mn ? 1 : 2;
        uint32_t tmem_d = tmem_acc;
        if (Op::SEG_EPI) {
          tmem_d = tmem_acc + (uint32_t)((sg & 1) * BN);
          if (sg >= 2 && !mbar_wait(free_bar(sg & 1), (uint32_t)(((sg >> 1) - 1) & 1))) { atomicOr(status, 32u); *abort_flag = 1; stop = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        for (int kt = kt0; kt < kt1; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(split_bar(s), ph)) { atomicOr(status, 2u); *abort_flag = 1; stop = true; break; }
          if (*abort_flag) { stop = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_hi = tiles + s * G::STAGE_BYTES, b_hi = a_hi + G::A_BYTES, a_lo = a_hi + G::HALF, b_lo = b_hi + G::HALF;
#pragma unroll
          for (int k = 0; k < BK / 8; ++k) {
            const uint64_t dah = make_desc(a_hi + k * a_kstep, a_lbo, a_sbo, a_lt), dbh = make_desc(b_hi + k * b_kstep, b_lbo, b_sbo, b_lt);
            const uint64_t dal = make_desc(a_lo + k * a_kstep, a_lbo, a_sbo, a_lt), dbl = make_desc(b_lo + k * b_kstep, b_lbo, b_sbo, b_lt);
            const bool first = Op::SEG_EPI ? (kt == kt0 && k == 0) : (it == 0 && k == 0);
            mma_tf32(tmem_d, dal, dbh, idesc, first ? 0u : 1u);
            mma_tf32(tmem_d, dah, dbl, idesc, 1u);
            mma_tf32(tmem_d, dah, dbh, idesc, 1u);
          }
          umma_commit(empty_bar(s));
        }
        if (Op::SEG_EPI && !stop) umma_commit(seg_bar(sg & 1));
      }
      umma_commit(accum_bar);
    }
  } else {
    // ---------------- transform (scale + hi/lo split), then epilogue: warps 2..5 ----------------
    const int st = threadIdx.x - 64;
    bool ok = true;
    int it = 0;
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
    }
    // folds the finished accumulator of segment j into the register sums and hands its TMEM buffer back
    auto seg_epilogue = [&](int j) -> bool {
      const int b = j & 1;
      const bool done = __all_sync(0xffffffffu, mbar_wait(seg_bar(b), (uint32_t)((j >> 1) & 1)));
      if (!done) { if (lane == 0) { atomicOr(status, 64u); *abort_flag = 1; } return false; }
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
          op.seg_accumulate(j, m, n0 + c * 32, v, racc[cc]);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(free_bar(b));
      return true;
    };
    for (int sg = 0; sg < nseg && ok; ++sg) {
      int kt0, kt1, amap, bmap, a_mn, b_mn;
      op.seg(sg, m0, n0, kt0, kt1, amap, bmap, a_mn, b_mn);
      if (Op::SEG_EPI) {
        // per-segment vectors for seg_accumulate go to one of two aux buffers; the barriers (transform warps only)
        // keep a fast warp from overwriting a buffer that a slower warp still reads for segment sg-2
        asm volatile("bar.sync 1, %0;" ::"n"(NXF) : "memory");
        op.stage_seg(sg, st, NXF);
        asm volatile("bar.sync 1, %0;" ::"n"(NXF) : "memory");
      }
      for (int kt = kt0; kt < kt1; ++kt, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        const bool landed = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph));
        if (!landed) { if (lane == 0) { atomicOr(status, 4u); *abort_flag = 1; } ok = false; break; }
        if (__any_sync(0xffffffffu, *abort_flag != 0)) { ok = false; break; }
        uint4* hi = reinterpret_cast<uint4*>(tiles_ptr + s * G::STAGE_BYTES);
        uint4* lo = reinterpret_cast<uint4*>(tiles_ptr + s * G::STAGE_BYTES + G::HALF);
        const int kbase = kt * BK;
        // A tile
#pragma unroll 2
        for (int i = st; i < G::A_BYTES / 16; i += NXF) {
          uint4 v = hi[i];
          float f[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
          if (Op::A_SCALE) {
            int r, k;
            if (!a_mn) decode_kmajor(i, r, k); else decode_mnmajor(i, r, k);
            op.a_scale4(sg, a_mn, m0 + r, kbase + k, f);
          }
          uint4 h, l;
          h.x = __float_as_uint(f[0]) & 0xFFFFE000u; h.y = __float_as_uint(f[1]) & 0xFFFFE000u;
          h.z = __float_as_uint(f[2]) & 0xFFFFE000u; h.w = __float_as_uint(f[3]) & 0xFFFFE000u;
          l.x = __float_as_uint(f[0] - __uint_as_float(h.x)); l.y = __float_as_uint(f[1] - __uint_as_float(h.y));
          l.z = __float_as_uint(f[2] - __uint_as_float(h.z)); l.w = __float_as_uint(f[3] - __uint_as_float(h.w));
          // kind::tf32 ignores the 13 low mantissa bits, so an unscaled tile serves as its own high part
          if (Op::A_SCALE) hi[i] = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
          lo[i] = l;
        }
        // B tile
        uint4* bhi = hi + G::A_BYTES / 16;
        uint4* blo = lo + G::A_BYTES / 16;
#pragma unroll 2
        for (int i = st; i < G::B_BYTES / 16; i += NXF) {
          uint4 v = bhi[i];
          float f[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
          if (Op::B_SCALE) {
            int r, k;
            if (!b_mn) {
              decode_kmajor(i, r, k);
#pragma unroll
              for (int e = 0; e < 4; ++e) { const float sc = op.b_scale(sg, n0 + r, kbase + k + e); f[e] = sc == 0.0f ? 0.0f : f[e] * sc; }
            } else {
              decode_mnmajor(i, r, k);
#pragma unroll
              for (int e = 0; e < 4; ++e) { const float sc = op.b_scale(sg, n0 + r + e, kbase + k); f[e] = sc == 0.0f ? 0.0f : f[e] * sc; }
            }
          }
          uint4 h, l;
          h.x = __float_as_uint(f[0]) & 0xFFFFE000u; h.y = __float_as_uint(f[1]) & 0xFFFFE000u;
          h.z = __float_as_uint(f[2]) & 0xFFFFE000u; h.w = __float_as_uint(f[3]) & 0xFFFFE000u;
          l.x = __float_as_uint(f[0] - __uint_as_float(h.x)); l.y = __float_as_uint(f[1] - __uint_as_float(h.y));
          l.z = __float_as_uint(f[2] - __uint_as_float(h.z)); l.w = __float_as_uint(f[3] - __uint_as_float(h.w));
          if (Op::B_SCALE) bhi[i] = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
          blo[i] = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(split_bar(s));
      }
      // while the tensor core works on segment sg, fold segment sg-1
      if (Op::SEG_EPI && ok && sg >= 1) ok = seg_epilogue(sg - 1);
    }
    if (Op::SEG_EPI && ok && nseg >= 1) ok = seg_epilogue(nseg - 1);
    const bool acc_ok = __all_sync(0xffffffffu, mbar_wait(accum_bar, 0));
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

template <class Op>
// heavy_m: +1 = the last m tile of a batch entry has the most k-steps, -1 = the first one, 0 = all alike
static pmb_status launch(cudaStream_t st, const MapSet& maps, const Op& op, int batches, unsigned int* status, int heavy_m = 0) {
  using G = Geometry<Op::BN>;
  PMB_SMEM_OPT_IN(G::SMEM_BASE + Op::AUX_FLOATS * 4, tc_bgemm_kernel<Op>);
  const unsigned mtiles = (unsigned)cdiv(op.Mdim, BM);
  const int mode = (heavy_m == 0 || batches > 65535 || mtiles < 2) ? 0 : (heavy_m > 0 ? 2 : 1);
  dim3 grid((unsigned)cdiv(op.Ndim, Op::BN), mode ? (unsigned)batches : mtiles, mode ? mtiles : (unsigned)batches);
  tc_bgemm_kernel<Op><<<grid, NTHREADS, G::SMEM_BASE + Op::AUX_FLOATS * 4, st>>>(maps, op, status, mode);
  PMB_LAUNCHED();
  return PMB_OK;
}

}  // namespace tcb
}  // namespace pmb
