// bf16 GEMM on tcgen05 (kind::f16, fp32 accumulation in TMEM) for the bf16-storage configurations:
// C = op(A) op(B) (+ R), A and B bf16 in HBM, C (and R) fp32 or bf16.
//
// CTA = one 128x128 output tile; warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = epilogue.
// bf16 operands need no in-smem processing, so a stage is just the two landed tiles (128 x 64 bf16 each,
// 32 KiB per stage) and the ring is 6 deep.  K-major tiles: 128-byte rows, 128-byte swizzle.  MN-major
// tiles: blocks of 64 elements along M/N, 64 k-rows of 128 bytes per block, same swizzle.
// Every mbarrier wait is bounded; on expiry the kernel raises the device status word and drains.
#include <climits>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>
#include "tc_common.cuh"
#include "kernels.h"

namespace pmb {

static __device__ unsigned int g_bf16_status = 0;

namespace hb { static void sched_reset_current_device(); }

pmb_status read_clear_device_status_bf16(unsigned int* word) {
  unsigned int zero = 0;
  PMB_CUDA(cudaMemcpyFromSymbol(word, g_bf16_status, sizeof(unsigned int)));
  if (*word) {
    PMB_CUDA(cudaMemcpyToSymbol(g_bf16_status, &zero, sizeof(unsigned int)));
    hb::sched_reset_current_device();      // a kernel that gave up may have left its tile-ticket counter out of step
  }
  return PMB_OK;
}

namespace hb {

using namespace tcx;

constexpr int TBM = 128, TBN = 128, TBK = 64;
constexpr int TILE_BYTES = TBM * TBK * 2;   // 16 KiB
// SPLIT = false: plain bf16 operands, a stage holds A and B (32 KiB), 6 stages.
// SPLIT = true : every operand is a pair (hi, lo) of bf16 arrays with hi + lo ~= an fp32 value (16 mantissa bits);
//                a stage holds A_hi, B_hi, A_lo, B_lo (64 KiB), 3 stages, and each k-step issues hi*hi + lo*hi + hi*lo.
template <bool SPLIT> struct Cfg {
  static constexpr int STAGES = SPLIT ? 3 : 6;
  static constexpr int STAGE_BYTES = (SPLIT ? 4 : 2) * TILE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * 2 * 4096 + 1024 + 512;   // + the epilogue's staging slots, barriers and the tile queue
};
constexpr int NTHREADS = 192;
constexpr int TMEM_COLS = 256;               // two 128-column accumulators
constexpr int EPI_SLOT_BYTES = 32 * 32 * 4;  // 32 rows x 32 fp32 columns
constexpr int EPI_BYTES = 4 * 2 * EPI_SLOT_BYTES;
constexpr int NQ = 4;                       // depth of the tile-id queue inside a CTA

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct Params {
  int M, N, K;
  int a_mn_major, b_mn_major;
  void* C; int64_t ldc; const void* R; int out_bf16;
  int tma_out;     // fp32 result (and residual) meet the TMA rules: the epilogue stores through shared memory
  uint16_t* e_hi; uint16_t* e_lo; int64_t lde;   // optional second output: the result as a bf16 pair (TMA-store epilogue only)
};

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {   // round to nearest even
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// Epilogue of one 32-column piece of an output row: adds R when given and stores fp32 or bf16, 16-byte vectors
// when the row is aligned and the piece lies inside the matrix, element by element otherwise.
__device__ __forceinline__ void store_row_piece(const Params& p, int m, int nb, const uint32_t (&r)[32]) {
  if (p.out_bf16) {
    uint16_t* crow = static_cast<uint16_t*>(p.C) + (int64_t)m * p.ldc + nb;
    const uint16_t* rrow = p.R ? static_cast<const uint16_t*>(p.R) + (int64_t)m * p.ldc + nb : nullptr;
    const bool vec = (nb + 32 <= p.N) && ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                     (!p.R || (reinterpret_cast<uintptr_t>(p.R) & 15) == 0);
    if (vec) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
        if (rrow) {
          uint4 q = *reinterpret_cast<const uint4*>(rrow + j);
          const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { v[2 * e] += __uint_as_float(qq[e] << 16); v[2 * e + 1] += __uint_as_float(qq[e] & 0xffff0000u); }
        }
        uint4 o;
        o.x = (uint32_t)float_to_bf16_bits(v[0]) | ((uint32_t)float_to_bf16_bits(v[1]) << 16);
        o.y = (uint32_t)float_to_bf16_bits(v[2]) | ((uint32_t)float_to_bf16_bits(v[3]) << 16);
        o.z = (uint32_t)float_to_bf16_bits(v[4]) | ((uint32_t)float_to_bf16_bits(v[5]) << 16);
        o.w = (uint32_t)float_to_bf16_bits(v[6]) | ((uint32_t)float_to_bf16_bits(v[7]) << 16);
        *reinterpret_cast<uint4*>(crow + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) crow[j] = float_to_bf16_bits(__uint_as_float(r[j]) + (rrow ? bf16_bits_to_float(rrow[j]) : 0.0f));
    }
  } else {
    float* crow = static_cast<float*>(p.C) + (int64_t)m * p.ldc + nb;
    const float* rrow = p.R ? static_cast<const float*>(p.R) + (int64_t)m * p.ldc + nb : nullptr;
    const bool vec = (nb + 32 <= p.N) && ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                     (!p.R || (reinterpret_cast<uintptr_t>(p.R) & 15) == 0);
    if (vec) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        if (rrow) {
          float4 q = *reinterpret_cast<const float4*>(rrow + j);
          v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
        }
        *reinterpret_cast<float4*>(crow + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) crow[j] = __uint_as_float(r[j]) + (rrow ? rrow[j] : 0.0f);
    }
  }
}

// One launch carries up to MAX_GROUP independent products: CTAs [0, pr[0].tiles) work on the first, the next
// pr[1].tiles on the second, and so on (unused entries have tiles == 0).
// Two products whose tile counts each fill the 148 SMs badly (weight-gradient and data-gradient of one projection)
// then share the machine instead of running as two ragged waves.
struct Problem { CUtensorMap mA, mB, mAlo, mBlo, mC, mR; Params p; int tiles_n; int tiles; };
constexpr int MAX_GROUP = 4;
struct Group { Problem pr[MAX_GROUP]; };
__device__ __forceinline__ int pick_problem(const Group& g, int id, int* local) {
  int which = 0, base = 0;
#pragma unroll
  for (int i = 0; i + 1 < MAX_GROUP; ++i) if (id >= base + g.pr[i].tiles && which == i) { base += g.pr[i].tiles; which = i + 1; }
  *local = id - base;
  return which;
}

// TMA store of one 32 x 32 fp32 block (128-byte rows, 128-byte swizzle) and its bookkeeping
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Epilogue of one tile for one epilogue warp: its 32 rows (row0 ..) x `ncols` columns (n0 ..) of the accumulator at
// `tmem_acc` (lane offset included).  fp32 results that meet the TMA rules leave through the warp's two swizzled
// staging slots (slot0) and TMA stores, the residual block TMA-loaded into the slot first (barriers rbar0 / rbar1);
// everything else is stored row by row.  `st` carries the slot parity and the residual barriers' phases across tiles.
struct EpiState { uint32_t pc = 0, rph0 = 0, rph1 = 0; };
__device__ __forceinline__ void epilogue_rows(const Problem& q, const Params& p, uint32_t tmem_acc, int row0, int n0, int ncols, uint32_t slot0,
                                              uint32_t rbar0, uint32_t rbar1, EpiState& st, int lane, volatile uint32_t* abort_flag) {
  if (p.tma_out) {
    if (row0 < p.M) {
      const bool res = p.R != nullptr;
      if (res && lane == 0) {
        const uint32_t slot = st.pc & 1u;
        mbar_expect_tx((slot ? rbar1 : rbar0), EPI_SLOT_BYTES);
        tma_load_2d(slot0 + slot * EPI_SLOT_BYTES, &q.mR, n0, row0, (slot ? rbar1 : rbar0));
      }
#pragma unroll 1
      for (int c0 = 0; c0 < ncols && n0 + c0 < p.N; c0 += 32) {
        const uint32_t slot = st.pc & 1u;
        const uint32_t sbase = slot0 + slot * EPI_SLOT_BYTES + (uint32_t)lane * 128u;
        uint32_t r[32];
        tmem_ld32(tmem_acc + (uint32_t)c0, r);
        if (res) {
          const uint32_t rp = slot ? st.rph1 : st.rph0;
          const bool landed = __all_sync(0xffffffffu, mbar_wait((slot ? rbar1 : rbar0), rp));
          if (slot) st.rph1 ^= 1u; else st.rph0 ^= 1u;
          if (!landed) { if (lane == 0) { atomicOr(&g_bf16_status, 16u); *abort_flag = 1; } }
          else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 v;
              asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                           : "r"(sbase + (uint32_t)((j ^ (lane & 7)) * 16)));
              r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
              r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
              r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
              r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
            }
          }
        }
        if (p.e_hi) {
          // the same values as a (hi, lo) bf16 pair, straight from registers: 64 contiguous bytes per row and array
          const int m = row0 + lane;
          if (m < p.M) {
            uint16_t* eh = p.e_hi + (int64_t)m * p.lde + n0 + c0;
            uint16_t* el = p.e_lo + (int64_t)m * p.lde + n0 + c0;
            if (n0 + c0 + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint32_t h[8], l[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) split_bf16_pair(__uint_as_float(r[j + e]), h[e], l[e]);
                *reinterpret_cast<uint4*>(eh + j) = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
                *reinterpret_cast<uint4*>(el + j) = make_uint4(l[0] | (l[1] << 16), l[2] | (l[3] << 16), l[4] | (l[5] << 16), l[6] | (l[7] << 16));
              }
            } else {
              for (int j = 0; j < 32 && n0 + c0 + j < p.N; ++j) {
                uint32_t h, l;
                split_bf16_pair(__uint_as_float(r[j]), h, l);
                eh[j] = (uint16_t)h; el[j] = (uint16_t)l;
              }
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sbase + (uint32_t)((j ^ (lane & 7)) * 16)),
                       "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        ++st.pc;
        if (lane == 0) {
          tma_store_2d(&q.mC, slot0 + slot * EPI_SLOT_BYTES, n0 + c0, row0);
          bulk_commit();
          bulk_wait_read<1>();               // the other slot's store has read its data: the slot is free again
          if (res && c0 + 32 < ncols && n0 + c0 + 32 < p.N) {
            const uint32_t nslot = st.pc & 1u;
            mbar_expect_tx((nslot ? rbar1 : rbar0), EPI_SLOT_BYTES);
            tma_load_2d(slot0 + nslot * EPI_SLOT_BYTES, &q.mR, n0 + c0 + 32, row0, (nslot ? rbar1 : rbar0));
          }
        }
        __syncwarp();
      }
    }
  } else {
    const int m = row0 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < ncols; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_acc + (uint32_t)c0, r);
      if (m < p.M) store_row_piece(p, m, n0 + c0, r);
    }
  }
}

// Persistent: CTA b works on tiles b, b + gridDim.x, ... of the group.  The operand ring and its phases run on
// across tiles, so the producer is already loading the next tile while the last k-tiles of this one are
// multiplied; the accumulator alternates between two 128-column TMEM buffers, so the epilogue warps drain tile i
// while the tensor core fills tile i + 1.
//   full[s] / empty[s]        operand stage s landed / consumed
//   acc_full[b] / acc_empty[b] accumulator b complete / drained by all four epilogue warps
//   rbar[w][slot]             residual block landed in epilogue warp w's staging slot
// fp32 results leave through shared memory: each epilogue warp writes its 32 rows x 32 columns into a swizzled
// 4 KiB slot (conflict-free 16-byte stores) and one lane hands the slot to a TMA store, which writes whole
// 128-byte row segments and clips at the matrix edge; two slots per warp, so a store is in flight while the next
// block is formed.  The residual block, when there is one, is loaded into the slot first and added in place.
template <bool SPLIT>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_bf16_kernel(const __grid_constant__ Group g, const int total_tiles, unsigned long long* __restrict__ sched, const unsigned long long ticket0) {
  constexpr int STAGES = Cfg<SPLIT>::STAGES;
  constexpr int STAGE_BYTES = Cfg<SPLIT>::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles - raw);
  const uint32_t epi = tiles + STAGES * STAGE_BYTES;                 // 4 warps x 2 slots x 4 KiB
  const uint32_t bars = epi + EPI_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  auto r_bar = [&](int w, int slot) { return bars + 8u * (2 * STAGES + 4 + 2 * w + slot); };
  auto tq_full = [&](int i) { return bars + 8u * (2 * STAGES + 12 + i); };
  auto tq_empty = [&](int i) { return bars + 8u * (2 * STAGES + 12 + NQ + i); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tiles_ptr + STAGES * STAGE_BYTES + EPI_BYTES + 8 * (2 * STAGES + 12 + 2 * NQ));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* tile_q = reinterpret_cast<volatile int*>(tmem_slot + 2);      // NQ tile ids handed from the producer to the other roles
  // CTA b starts with tile b; every further tile is handed out by a device-wide ticket counter (*sched), so a CTA
  // that starts late (its SM was busy with another stream's kernel) finds the rest of the work already taken instead
  // of holding its share back.  A launch draws exactly total_tiles tickets (one per processed tile), so the counter
  // is never reset: ticket t stands for tile gridDim.x + (t - ticket0) % total_tiles, where ticket0 is the counter's
  // value before the launch (launches outside stream capture) or 0 (a captured launch, which owns its counter and
  // advances it by total_tiles per replay).  sched == NULL: CTA b takes tiles b, b + gridDim.x, ...
  auto ticket_tile = [&](unsigned long long t) { return (int)gridDim.x + (int)((t - ticket0) % (unsigned long long)total_tiles); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 4); }
    for (int w = 0; w < 4; ++w) { mbar_init(r_bar(w, 0), 1); mbar_init(r_bar(w, 1), 1); }
    for (int i = 0; i < NQ; ++i) { mbar_init(tq_full(i), 1); mbar_init(tq_empty(i), 5); }    // readers: the MMA thread + four epilogue warps
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // The producer needs the barriers (its own thread initialised them) but not the TMEM address: warp 0 only arrives at
  // the set-up barrier and starts loading while warp 1's TMEM allocation is still under way; the other warps wait.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if (warp == 0) { __syncwarp(); asm volatile("bar.arrive 1, %0;" ::"n"(NTHREADS) : "memory"); }
  else asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = warp == 0 ? 0u : *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      int in_flight = 0;                       // stages armed and possibly not yet landed (for the abort drain)
      bool stop = false;
      int tid = (int)blockIdx.x;
      for (int it = 0; !stop; ++it) {
        // publish this tile (or the end mark) to the MMA and epilogue roles
        const int qs = it % NQ;
        if (!mbar_wait(tq_empty(qs), (((uint32_t)(it / NQ)) & 1u) ^ 1u)) { atomicOr(&g_bf16_status, 32u); *abort_flag = 1; break; }
        tile_q[qs] = tid < total_tiles ? tid : -1;
        mbar_arrive(tq_full(qs));
        if (tid >= total_tiles) break;
        // the next ticket is requested now and used after this tile's loads
        unsigned long long next_ticket = 0;
        if (sched) next_ticket = atomicAdd(sched, 1ull);
        int tile;
        const Problem& q = g.pr[pick_problem(g, tid, &tile)];
        const Params& p = q.p;
        const int m0 = (tile / q.tiles_n) * TBM, n0 = (tile % q.tiles_n) * TBN;
        const int num_kt = (p.K + TBK - 1) / TBK;
        for (int kt = 0; kt < num_kt; ++kt) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) { atomicOr(&g_bf16_status, 1u); *abort_flag = 1; stop = true; break; }
          if (*abort_flag) { stop = true; break; }
          const uint32_t a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + TILE_BYTES;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const int k0 = kt * TBK;
          if (!p.a_mn_major) {
            tma_load_2d(a_dst, &q.mA, k0, m0, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < TBM / 64; ++j) tma_load_2d(a_dst + j * (TBK * 128), &q.mA, m0 + 64 * j, k0, full_bar(s));
          }
          if (!p.b_mn_major) {
            tma_load_2d(b_dst, &q.mB, k0, n0, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < TBN / 64; ++j) tma_load_2d(b_dst + j * (TBK * 128), &q.mB, n0 + 64 * j, k0, full_bar(s));
          }
          if (SPLIT) {
            const uint32_t al_dst = a_dst + 2 * TILE_BYTES, bl_dst = al_dst + TILE_BYTES;
            if (!p.a_mn_major) {
              tma_load_2d(al_dst, &q.mAlo, k0, m0, full_bar(s));
            } else {
#pragma unroll
              for (int j = 0; j < TBM / 64; ++j) tma_load_2d(al_dst + j * (TBK * 128), &q.mAlo, m0 + 64 * j, k0, full_bar(s));
            }
            if (!p.b_mn_major) {
              tma_load_2d(bl_dst, &q.mBlo, k0, n0, full_bar(s));
            } else {
#pragma unroll
              for (int j = 0; j < TBN / 64; ++j) tma_load_2d(bl_dst + j * (TBK * 128), &q.mBlo, n0 + 64 * j, k0, full_bar(s));
            }
          }
          if (in_flight < STAGES) ++in_flight;
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        tid = sched ? ticket_tile(next_ticket) : tid + (int)gridDim.x;
      }
      if (*abort_flag) {
        // the copies already issued still land in this CTA's shared memory: wait (bounded) for each before leaving
        for (int i = 0; i < in_flight; ++i) {
          if (--s < 0) { s = STAGES - 1; ph ^= 1u; }
          mbar_wait(full_bar(s), ph);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t d_hi = desc_hi(1024, 2);
      constexpr uint32_t LO_OFF = (2 * TILE_BYTES) >> 4;        // from the hi tiles of a stage to its lo tiles
      int s = 0; uint32_t ph = 0;
      bool stop = false;
      for (int it = 0; !stop; ++it) {
        const int qs = it % NQ;
        if (!mbar_wait(tq_full(qs), ((uint32_t)(it / NQ)) & 1u)) { atomicOr(&g_bf16_status, 64u); *abort_flag = 1; break; }
        const int tid = tile_q[qs];
        mbar_arrive(tq_empty(qs));
        if (tid < 0) break;
        int tile;
        const Problem& q = g.pr[pick_problem(g, tid, &tile)];
        const Params& p = q.p;
        const int num_kt = (p.K + TBK - 1) / TBK;
        // kind::f16 descriptor: fp32 accumulate (bit 4), A/B format bf16 (=1) at bits 7 and 10, majorness, N, M
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                               ((uint32_t)(TBN >> 3) << 17) | ((uint32_t)(TBM >> 4) << 24);
        // K-major: 8-row groups 1024 B apart, one MMA (K=16) advances 32 B inside the 128-byte row.
        // MN-major: blocks of 64 elements TBK*128 B apart (LBO), 8-k-row groups 1024 B apart (SBO); K=16 spans two groups.
        const uint32_t a_lbo = p.a_mn_major ? TBK * 128 : 16, b_lbo = p.b_mn_major ? TBK * 128 : 16;
        const uint32_t a_step = (p.a_mn_major ? 2048u : 32u) >> 4, b_step = (p.b_mn_major ? 2048u : 32u) >> 4;
        const int b = it & 1;
        if (!mbar_wait(acc_empty(b), (((uint32_t)it >> 1) & 1u) ^ 1u)) { atomicOr(&g_bf16_status, 4u); *abort_flag = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + (uint32_t)(b * TBN);
        for (int kt = 0; kt < num_kt; ++kt) {
          if (!mbar_wait(full_bar(s), ph)) { atomicOr(&g_bf16_status, 2u); *abort_flag = 1; stop = true; break; }
          if (*abort_flag) { stop = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_s = tiles + s * STAGE_BYTES;
          uint32_t al = desc_lo(a_s, a_lbo), bl = desc_lo(a_s + TILE_BYTES, b_lbo);
#pragma unroll
          for (int k = 0; k < TBK / 16; ++k) {
            const uint32_t acc = (kt > 0 || k > 0) ? 1u : 0u;
            if (SPLIT) {
              mma_f16_h(tmem_acc, al + LO_OFF, d_hi, bl, d_hi, idesc, acc);
              mma_f16_h(tmem_acc, al, d_hi, bl + LO_OFF, d_hi, idesc, 1u);
              mma_f16_h(tmem_acc, al, d_hi, bl, d_hi, idesc, 1u);
            } else {
              mma_f16_h(tmem_acc, al, d_hi, bl, d_hi, idesc, acc);
            }
            al += a_step; bl += b_step;
          }
          umma_commit(empty_bar(s));
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!stop) umma_commit(acc_full(b));
      }
    }
  } else {
    const int ew = warp - 2;                       // staging slots and residual barriers of this warp
    const int quarter = warp & 3;                  // the TMEM lanes this warp may read
    const uint32_t slot0 = epi + (uint32_t)ew * (2 * EPI_SLOT_BYTES);
    EpiState est;                                  // slot parity and residual-barrier phases, carried across tiles
    for (int it = 0;; ++it) {
      const int qs = it % NQ;
      const bool have = __all_sync(0xffffffffu, mbar_wait_idle(tq_full(qs), ((uint32_t)(it / NQ)) & 1u));
      if (!have) { if (lane == 0) { atomicOr(&g_bf16_status, 128u); *abort_flag = 1; } break; }
      const int tid = tile_q[qs];
      __syncwarp();
      if (lane == 0) mbar_arrive(tq_empty(qs));
      if (tid < 0) break;
      int tile;
      const Problem& q = g.pr[pick_problem(g, tid, &tile)];
      const Params& p = q.p;
      const int m0 = (tile / q.tiles_n) * TBM, n0 = (tile % q.tiles_n) * TBN;
      const int b = it & 1;
      const bool acc_ok = __all_sync(0xffffffffu, mbar_wait_idle(acc_full(b), ((uint32_t)it >> 1) & 1u));
      if (!acc_ok && lane == 0) { atomicOr(&g_bf16_status, 8u); *abort_flag = 1; }
      if (!acc_ok || __any_sync(0xffffffffu, *abort_flag != 0)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + (uint32_t)(b * TBN) + ((uint32_t)(quarter * 32) << 16);
      const int row0 = m0 + quarter * 32;
      epilogue_rows(q, p, tmem_acc, row0, n0, TBN, slot0, r_bar(ew, 0), r_bar(ew, 1), est, lane, abort_flag);
      // every TMEM read of this warp has completed (tcgen05.wait::ld): hand the accumulator back
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(b));
    }
    if (lane == 0) bulk_wait_all();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- CTA-pair variant ------------------------------------------------------------------------------------
// Two CTAs of a cluster (a CTA pair) own one 256x256 output tile.  Each loads its 128 rows of A and its 128
// columns of B (64 KiB per k-tile with pairs, 32 KiB without, exactly what a 128x128 single-CTA tile loads) and
// the leader issues tcgen05.mma.cta_group::2 with M = 256, N = 256: each SM multiplies its A rows by the B
// columns of both, so a byte fetched from L2 feeds twice the tensor work.  The 128x128 kernel above is bound by
// L2 -> shared-memory traffic at these shapes; this one halves that traffic per flop.
//   full_bar[s]  (leader's copy): both CTAs' loads complete their bytes on it
//   empty_bar[s] (one per CTA):   the leader commits the k-tile's MMAs to both, freeing the stage in both CTAs
//   accum_bar    (one per CTA):   the leader commits the last MMAs to both; each CTA drains its own 128 TMEM lanes
// Every wait is bounded; a CTA that gives up records it, stops issuing work and still joins the closing
// cluster barrier, so its peer never waits for it unboundedly.
// stage = A tile (128 x 64) + B tile (BN2/2 x 64), twice that with pairs; as many stages as fit in 192 KiB
template <bool SPLIT, int BN2> struct PairCfg {
  static constexpr int STAGE_BYTES = (SPLIT ? 2 : 1) * (TILE_BYTES + (BN2 / 2) * TBK * 2);
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES > 8 ? 8 : (192 * 1024) / STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tile load issued by either CTA of the pair, completing bytes on a barrier given as a cluster address
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// BN2 = width of the pair's tile (256 or 128); each CTA loads BN2/2 columns of B.
template <bool SPLIT, int BN2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ Group g) {
  const uint32_t rank = cluster_rank();
  const int cluster_id = (int)(blockIdx.x >> 1);
  int tile;
  const int which = pick_problem(g, cluster_id, &tile);
  const Problem& q = g.pr[which];
  const Params& p = q.p;
  constexpr int BNH = BN2 / 2;                       // B columns (rows of the K-major tile) per CTA
  constexpr int TILE_B = BNH * TBK * 2;
  constexpr int HALF_BYTES = TILE_BYTES + TILE_B;    // one A tile + one B tile
  constexpr int STAGE_BYTES = PairCfg<SPLIT, BN2>::STAGE_BYTES;
  constexpr int STAGES = PairCfg<SPLIT, BN2>::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles - raw);
  const uint32_t bars = tiles + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t accum_bar = bars + 8u * (2 * STAGES);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tiles_ptr + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 1));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = (tile / q.tiles_n) * 256 + (int)rank * TBM;     // this CTA's rows of A and of the output
  const int n0 = (tile % q.tiles_n) * BN2;                      // the pair's columns; this CTA loads B columns n0 + rank*128 ..
  const int nb0 = n0 + (int)rank * BNH;
  const int num_kt = (p.K + TBK - 1) / TBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(BN2) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();     // both CTAs' barriers are initialised before either signals the other's
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int armed = 0;
      for (int kt = 0; kt < num_kt; ++kt) {
        const int s = kt % STAGES;
        const uint32_t ph = (kt / STAGES) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1u)) { atomicOr(&g_bf16_status, 1u); *abort_flag = 1; break; }
        if (*abort_flag) break;
        const uint32_t a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + TILE_BYTES;
        const uint32_t fb = map_to_cta(full_bar(s), 0);            // the leader's barrier collects both CTAs' bytes
        if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
        const int k0 = kt * TBK;
        if (!p.a_mn_major) {
          tma_load_2d_pair(a_dst, &q.mA, k0, m0, fb);
        } else {
#pragma unroll
          for (int j = 0; j < TBM / 64; ++j) tma_load_2d_pair(a_dst + j * (TBK * 128), &q.mA, m0 + 64 * j, k0, fb);
        }
        if (!p.b_mn_major) {
          tma_load_2d_pair(b_dst, &q.mB, k0, nb0, fb);
        } else {
#pragma unroll
          for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(b_dst + j * (TBK * 128), &q.mB, nb0 + 64 * j, k0, fb);
        }
        if (SPLIT) {
          const uint32_t al_dst = a_dst + HALF_BYTES, bl_dst = al_dst + TILE_BYTES;
          if (!p.a_mn_major) {
            tma_load_2d_pair(al_dst, &q.mAlo, k0, m0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < TBM / 64; ++j) tma_load_2d_pair(al_dst + j * (TBK * 128), &q.mAlo, m0 + 64 * j, k0, fb);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(bl_dst, &q.mBlo, k0, nb0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(bl_dst + j * (TBK * 128), &q.mBlo, nb0 + 64 * j, k0, fb);
          }
        }
        armed = kt + 1;
      }
      // after giving up, the leader still waits (bounded) for the loads both CTAs have in flight
      if (*abort_flag && rank == 0)
        for (int kt = max(0, armed - STAGES); kt < armed; ++kt) mbar_wait(full_bar(kt % STAGES), (kt / STAGES) & 1);
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // M = 256 (two CTAs x 128 rows), N = 256
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                             ((uint32_t)(BN2 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      const uint32_t a_lbo = p.a_mn_major ? TBK * 128 : 16, b_lbo = p.b_mn_major ? TBK * 128 : 16;
      const uint32_t d_hi = desc_hi(1024, 2);
      const uint32_t a_step = (p.a_mn_major ? 2048u : 32u) >> 4, b_step = (p.b_mn_major ? 2048u : 32u) >> 4;
      constexpr uint32_t LO_OFF = HALF_BYTES >> 4;
      // the barriers of both CTAs as cluster addresses, once
      uint32_t eb0[STAGES], eb1[STAGES];
#pragma unroll
      for (int i = 0; i < STAGES; ++i) { eb0[i] = map_to_cta(empty_bar(i), 0); eb1[i] = map_to_cta(empty_bar(i), 1); }
      int s = 0; uint32_t ph = 0;
      for (int kt = 0; kt < num_kt; ++kt) {
        if (!mbar_wait(full_bar(s), ph)) { atomicOr(&g_bf16_status, 2u); *abort_flag = 1; break; }
        if (*abort_flag) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_s = tiles + s * STAGE_BYTES;
        uint32_t al = desc_lo(a_s, a_lbo), bl = desc_lo(a_s + TILE_BYTES, b_lbo);
#pragma unroll
        for (int k = 0; k < TBK / 16; ++k) {
          const uint32_t acc = (kt > 0 || k > 0) ? 1u : 0u;
          if (SPLIT) {
            mma_f16_pair_h(tmem_acc, al + LO_OFF, d_hi, bl, d_hi, idesc, acc);
            mma_f16_pair_h(tmem_acc, al, d_hi, bl + LO_OFF, d_hi, idesc, 1u);
            mma_f16_pair_h(tmem_acc, al, d_hi, bl, d_hi, idesc, 1u);
          } else {
            mma_f16_pair_h(tmem_acc, al, d_hi, bl, d_hi, idesc, acc);
          }
          al += a_step; bl += b_step;
        }
        // the commits go through a switch on the stage so that the cluster addresses stay in registers
#pragma unroll
        for (int i = 0; i < STAGES; ++i)
          if (i == s) { umma_commit_pair(eb0[i]); umma_commit_pair(eb1[i]); }
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      umma_commit_pair(map_to_cta(accum_bar, 0));
      umma_commit_pair(map_to_cta(accum_bar, 1));
    }
  } else {
    const bool acc_ok = __all_sync(0xffffffffu, mbar_wait_idle(accum_bar, 0));
    if (!acc_ok && lane == 0) { atomicOr(&g_bf16_status, 8u); *abort_flag = 1; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool aborted = __any_sync(0xffffffffu, *abort_flag != 0);
    if (acc_ok && !aborted) {
      const int lane_base = (warp & 3) * 32;
      const int m = m0 + lane_base + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN2; c0 += 32) {
        if (n0 + c0 >= p.N) break;      // uniform
        uint32_t r[32];
        tmem_ld32(tmem_acc + ((uint32_t)lane_base << 16) + (uint32_t)c0, r);
        if (m < p.M) store_row_piece(p, m, n0 + c0, r);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();     // neither CTA leaves (or frees TMEM) while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(BN2) : "memory");
  }
}

// ---- persistent CTA-pair variant ----------------------------------------------------------------------------
// The CTA-pair kernel above as a tile loop: cluster c works on tiles c, c + clusters, ...; the operand ring keeps
// running across tiles; the accumulator alternates between two TMEM buffers of BN2 columns, so each CTA drains its
// 128 rows of tile i (through the same TMA-store epilogue as the single-CTA kernel) while the leader issues tile
// i + 1.  The epilogue warps of BOTH CTAs hand a buffer back by arriving on the leader's acc_empty barrier (count 8).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
template <bool SPLIT, int BN2> struct PairPCfg {
  static constexpr int STAGE_BYTES = PairCfg<SPLIT, BN2>::STAGE_BYTES;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES > 8 ? 8 : (192 * 1024) / STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 512;
  static constexpr int TMEM = 2 * BN2;
};

template <bool SPLIT, int BN2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1)
gemm_bf16_pairp_kernel(const __grid_constant__ Group g, const int total_tiles) {
  const uint32_t rank = cluster_rank();
  const int cluster_id = (int)(blockIdx.x >> 1), nclusters = (int)(gridDim.x >> 1);
  constexpr int BNH = BN2 / 2;
  constexpr int TILE_B = BNH * TBK * 2;
  constexpr int HALF_BYTES = TILE_BYTES + TILE_B;
  constexpr int STAGE_BYTES = PairPCfg<SPLIT, BN2>::STAGE_BYTES;
  constexpr int STAGES = PairPCfg<SPLIT, BN2>::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles - raw);
  const uint32_t epi = tiles + STAGES * STAGE_BYTES;
  const uint32_t bars = epi + EPI_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  auto r_bar = [&](int w, int slot) { return bars + 8u * (2 * STAGES + 4 + 2 * w + slot); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tiles_ptr + STAGES * STAGE_BYTES + EPI_BYTES + 8 * (2 * STAGES + 12));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 8); }
    for (int w = 0; w < 4; ++w) { mbar_init(r_bar(w, 0), 1); mbar_init(r_bar(w, 1), 1); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "n"(PairPCfg<SPLIT, BN2>::TMEM) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();     // both CTAs' barriers are initialised before either signals the other's
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      int in_flight = 0;
      bool stop = false;
      for (int tid = cluster_id; tid < total_tiles && !stop; tid += nclusters) {
        int tile;
        const Problem& q = g.pr[pick_problem(g, tid, &tile)];
        const Params& p = q.p;
        const int m0 = (tile / q.tiles_n) * 256 + (int)rank * TBM;
        const int nb0 = (tile % q.tiles_n) * BN2 + (int)rank * BNH;
        const int num_kt = (p.K + TBK - 1) / TBK;
        for (int kt = 0; kt < num_kt; ++kt) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) { atomicOr(&g_bf16_status, 1u); *abort_flag = 1; stop = true; break; }
          if (*abort_flag) { stop = true; break; }
          const uint32_t a_dst = tiles + s * STAGE_BYTES, b_dst = a_dst + TILE_BYTES;
          const uint32_t fb = map_to_cta(full_bar(s), 0);            // the leader's barrier collects both CTAs' bytes
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
          const int k0 = kt * TBK;
          if (!p.a_mn_major) {
            tma_load_2d_pair(a_dst, &q.mA, k0, m0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < TBM / 64; ++j) tma_load_2d_pair(a_dst + j * (TBK * 128), &q.mA, m0 + 64 * j, k0, fb);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(b_dst, &q.mB, k0, nb0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(b_dst + j * (TBK * 128), &q.mB, nb0 + 64 * j, k0, fb);
          }
          if (SPLIT) {
            const uint32_t al_dst = a_dst + HALF_BYTES, bl_dst = al_dst + TILE_BYTES;
            if (!p.a_mn_major) {
              tma_load_2d_pair(al_dst, &q.mAlo, k0, m0, fb);
            } else {
#pragma unroll
              for (int j = 0; j < TBM / 64; ++j) tma_load_2d_pair(al_dst + j * (TBK * 128), &q.mAlo, m0 + 64 * j, k0, fb);
            }
            if (!p.b_mn_major) {
              tma_load_2d_pair(bl_dst, &q.mBlo, k0, nb0, fb);
            } else {
#pragma unroll
              for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(bl_dst + j * (TBK * 128), &q.mBlo, nb0 + 64 * j, k0, fb);
            }
          }
          if (in_flight < STAGES) ++in_flight;
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      // after giving up, the leader still waits (bounded) for the loads both CTAs have in flight
      if (*abort_flag && rank == 0) {
        for (int i = 0; i < in_flight; ++i) {
          if (--s < 0) { s = STAGES - 1; ph ^= 1u; }
          mbar_wait(full_bar(s), ph);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t d_hi = desc_hi(1024, 2);
      constexpr uint32_t LO_OFF = HALF_BYTES >> 4;
      uint32_t eb0[STAGES], eb1[STAGES];
#pragma unroll
      for (int i = 0; i < STAGES; ++i) { eb0[i] = map_to_cta(empty_bar(i), 0); eb1[i] = map_to_cta(empty_bar(i), 1); }
      const uint32_t af0[2] = {map_to_cta(acc_full(0), 0), map_to_cta(acc_full(1), 0)};
      const uint32_t af1[2] = {map_to_cta(acc_full(0), 1), map_to_cta(acc_full(1), 1)};
      int s = 0; uint32_t ph = 0;
      int it = 0;
      bool stop = false;
      for (int tid = cluster_id; tid < total_tiles && !stop; tid += nclusters, ++it) {
        int tile;
        const Problem& q = g.pr[pick_problem(g, tid, &tile)];
        const Params& p = q.p;
        const int num_kt = (p.K + TBK - 1) / TBK;
        // M = 256 (two CTAs x 128 rows), N = BN2
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                               ((uint32_t)(BN2 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
        const uint32_t a_lbo = p.a_mn_major ? TBK * 128 : 16, b_lbo = p.b_mn_major ? TBK * 128 : 16;
        const uint32_t a_step = (p.a_mn_major ? 2048u : 32u) >> 4, b_step = (p.b_mn_major ? 2048u : 32u) >> 4;
        const int b = it & 1;
        if (!mbar_wait(acc_empty(b), (((uint32_t)it >> 1) & 1u) ^ 1u)) { atomicOr(&g_bf16_status, 4u); *abort_flag = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + (uint32_t)(b * BN2);
        for (int kt = 0; kt < num_kt; ++kt) {
          if (!mbar_wait(full_bar(s), ph)) { atomicOr(&g_bf16_status, 2u); *abort_flag = 1; stop = true; break; }
          if (*abort_flag) { stop = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_s = tiles + s * STAGE_BYTES;
          uint32_t al = desc_lo(a_s, a_lbo), bl = desc_lo(a_s + TILE_BYTES, b_lbo);
#pragma unroll
          for (int k = 0; k < TBK / 16; ++k) {
            const uint32_t acc = (kt > 0 || k > 0) ? 1u : 0u;
            if (SPLIT) {
              mma_f16_pair_h(tmem_acc, al + LO_OFF, d_hi, bl, d_hi, idesc, acc);
              mma_f16_pair_h(tmem_acc, al, d_hi, bl + LO_OFF, d_hi, idesc, 1u);
              mma_f16_pair_h(tmem_acc, al, d_hi, bl, d_hi, idesc, 1u);
            } else {
              mma_f16_pair_h(tmem_acc, al, d_hi, bl, d_hi, idesc, acc);
            }
            al += a_step; bl += b_step;
          }
#pragma unroll
          for (int i = 0; i < STAGES; ++i)
            if (i == s) { umma_commit_pair(eb0[i]); umma_commit_pair(eb1[i]); }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!stop) { umma_commit_pair(af0[b]); umma_commit_pair(af1[b]); }
      }
    }
  } else {
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const uint32_t slot0 = epi + (uint32_t)ew * (2 * EPI_SLOT_BYTES);
    EpiState est;
    const uint32_t ae[2] = {map_to_cta(acc_empty(0), 0), map_to_cta(acc_empty(1), 0)};      // the leader's barriers
    int it = 0;
    for (int tid = cluster_id; tid < total_tiles; tid += nclusters, ++it) {
      int tile;
      const Problem& q = g.pr[pick_problem(g, tid, &tile)];
      const Params& p = q.p;
      const int m0 = (tile / q.tiles_n) * 256 + (int)rank * TBM, n0 = (tile % q.tiles_n) * BN2;
      const int b = it & 1;
      const bool acc_ok = __all_sync(0xffffffffu, mbar_wait_idle(acc_full(b), ((uint32_t)it >> 1) & 1u));
      if (!acc_ok && lane == 0) { atomicOr(&g_bf16_status, 8u); *abort_flag = 1; }
      if (!acc_ok || __any_sync(0xffffffffu, *abort_flag != 0)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + (uint32_t)(b * BN2) + ((uint32_t)(quarter * 32) << 16);
      const int row0 = m0 + quarter * 32;
      epilogue_rows(q, p, tmem_acc, row0, n0, BN2, slot0, r_bar(ew, 0), r_bar(ew, 1), est, lane, abort_flag);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(ae[b]);
    }
    if (lane == 0) bulk_wait_all();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();     // neither CTA leaves (or frees TMEM) while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(PairPCfg<SPLIT, BN2>::TMEM) : "memory");
  }
}

struct MapKey {
  const void* base; int64_t inner, outer, ld; int bi, bo, f32;
  bool operator<(const MapKey& o) const {
    return std::tie(base, inner, outer, ld, bi, bo, f32) < std::tie(o.base, o.inner, o.outer, o.ld, o.bi, o.bo, o.f32);
  }
};
static std::map<MapKey, CUtensorMap> g_cache;   // shared by every device and host thread: guarded by g_cache_mu
static std::mutex g_cache_mu;

static pmb_status make_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_inner, int box_outer,
                           bool f32 = false) {
  MapKey key{base, inner, outer, ld, box_inner, box_outer, f32 ? 1 : 0};
  std::lock_guard<std::mutex> lock(g_cache_mu);
  auto it = g_cache.find(key);
  if (it == g_cache.end()) {
    if (g_cache.size() > 8192) g_cache.clear();
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(PMB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (f32 ? 4 : 2)};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = enc(&m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(PMB_ERR_CUDA, "cuTensorMapEncodeTiled (%s) failed with code %d", f32 ? "fp32" : "bf16", (int)r);
    it = g_cache.emplace(key, m).first;
  }
  *map = it->second;
  return PMB_OK;
}

// Maps for the epilogue of the single-CTA kernel: 32 x 32 fp32 blocks of C (and of R, which shares C's pitch).
// Leaves tma_out = 0 when the result is bf16 or breaks a TMA rule; the kernel then stores row by row.
static pmb_status make_out_maps(Problem* q) {
  Params& p = q->p;
  p.tma_out = 0;
  if (p.out_bf16 || (p.ldc & 3) || (reinterpret_cast<uintptr_t>(p.C) & 15) || (p.R && (reinterpret_cast<uintptr_t>(p.R) & 15))) return PMB_OK;
  PMB_TRY(make_map(&q->mC, p.C, p.N, p.M, p.ldc, 32, 32, true));
  if (p.R) PMB_TRY(make_map(&q->mR, p.R, p.N, p.M, p.ldc, 32, 32, true));
  p.tma_out = 1;
  return PMB_OK;
}

// Ticket counters of the persistent kernel (64-bit, never reset; see the kernel).  Launches outside stream capture
// share EAGER_SLOTS counters round-robin and are told the counter's value before the launch, which the host tracks
// (a launch draws exactly `tiles` tickets); a captured launch keeps a counter of its own for the life of the graph,
// from a range that is never recycled.  Returns NULL (static tile order) when that range is used up, the counters
// cannot be allocated, or PMB_GEMM_SCHED=0.
constexpr unsigned EAGER_SLOTS = 4096, GRAPH_SLOTS = 61440;
static unsigned long long* g_sched_base[PMB_MAX_DEVICES] = {};
static std::vector<unsigned long long> g_sched_shadow[PMB_MAX_DEVICES];
static std::mutex g_sched_mu;

// After a kernel gave up on a bounded wait it may have drawn fewer tickets than its launch was accounted for: put
// every counter of the current device (and the host's record of them) back to zero, so that later launches start
// from a consistent state.  Called when the status word is read and found raised.
static void sched_reset_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PMB_MAX_DEVICES) return;
  std::lock_guard<std::mutex> lock(g_sched_mu);
  if (!g_sched_base[dev]) return;
  cudaMemset(g_sched_base[dev], 0, (size_t)(EAGER_SLOTS + GRAPH_SLOTS) * sizeof(unsigned long long));
  g_sched_shadow[dev].assign(EAGER_SLOTS, 0ull);
}

static unsigned long long* sched_counter(cudaStream_t st, int64_t tiles, unsigned long long* ticket0) {
  unsigned long long** base = g_sched_base;
  std::vector<unsigned long long>* shadow = g_sched_shadow;
  std::mutex& mu = g_sched_mu;
  static bool failed[PMB_MAX_DEVICES] = {};
  static unsigned eager_next[PMB_MAX_DEVICES] = {}, graph_next[PMB_MAX_DEVICES] = {};
  static const int on = [] { const char* e = getenv("PMB_GEMM_SCHED"); return (e && e[0] == '0') ? 0 : 1; }();   // 0: static tile order
  *ticket0 = 0;
  if (!on) return nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PMB_MAX_DEVICES) return nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    if (failed[dev] || cap != cudaStreamCaptureStatusNone) return nullptr;      // (first use must be outside capture)
    const size_t bytes = (size_t)(EAGER_SLOTS + GRAPH_SLOTS) * sizeof(unsigned long long);
    if (cudaMalloc(&base[dev], bytes) != cudaSuccess || cudaMemset(base[dev], 0, bytes) != cudaSuccess) {
      cudaGetLastError(); failed[dev] = true; base[dev] = nullptr; return nullptr;
    }
    shadow[dev].assign(EAGER_SLOTS, 0ull);
  }
  if (cap == cudaStreamCaptureStatusNone) {
    const unsigned slot = eager_next[dev]++ % EAGER_SLOTS;
    *ticket0 = shadow[dev][slot];
    shadow[dev][slot] += (unsigned long long)tiles;
    return base[dev] + slot;
  }
  if (graph_next[dev] >= GRAPH_SLOTS) return nullptr;
  return base[dev] + EAGER_SLOTS + graph_next[dev]++;
}

// One persistent CTA per SM, fewer when there are fewer tiles.
static unsigned persistent_grid(int64_t tiles) {
  static int sms[PMB_MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int n = 148;
  if (dev >= 0 && dev < PMB_MAX_DEVICES) {
    if (!sms[dev]) { int v = 0; if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms[dev] = v; else sms[dev] = 148; }
    n = sms[dev];
  }
  return (unsigned)(tiles < n ? tiles : n);
}

}  // namespace hb

// Row pitches must be multiples of 8 elements (16 bytes) and the bases 16-byte aligned (TMA rules).
pmb_status gemm_bf16(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                     const void* B, int64_t ldb, void* C, int64_t ldc, const void* R, int out_bf16) {
  using namespace hb;
  if (M <= 0 || N <= 0 || K <= 0) return fail(PMB_ERR_SHAPE, "gemm_bf16: non-positive dimension");
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return fail(PMB_ERR_SHAPE, "gemm_bf16: operands need 16-byte aligned bases and row pitches that are multiples of 8 elements");
  if (cdiv(M, TBM) * cdiv(N, TBN) > 0x7fffffff) return fail(PMB_ERR_SHAPE, "gemm_bf16: too many tiles");
  PMB_SMEM_OPT_IN(Cfg<false>::SMEM_BYTES, gemm_bf16_kernel<false>);
  Group g{};
  Problem& q = g.pr[0];
  if (!ta) PMB_TRY(make_map(&q.mA, A, K, M, lda, TBK, TBM)); else PMB_TRY(make_map(&q.mA, A, M, K, lda, 64, TBK));
  if (tb) PMB_TRY(make_map(&q.mB, B, K, N, ldb, TBK, TBN)); else PMB_TRY(make_map(&q.mB, B, N, K, ldb, 64, TBK));
  Params& p = q.p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.a_mn_major = ta ? 1 : 0; p.b_mn_major = tb ? 0 : 1;
  p.C = C; p.ldc = ldc; p.R = R; p.out_bf16 = out_bf16;
  q.tiles_n = (int)cdiv(N, TBN); q.tiles = (int)(cdiv(M, TBM) * cdiv(N, TBN));
  PMB_TRY(make_out_maps(&q));
  for (int i = 1; i < MAX_GROUP; ++i) { g.pr[i].tiles_n = 1; g.pr[i].tiles = 0; }
  {
    static const int env = [] { const char* e = getenv("PMB_GEMM_PAIR"); return e ? atoi(e) : -1; }();
    static const int min_clusters = [] { const char* e = getenv("PMB_GEMM_PAIR_MIN"); return e ? atoi(e) : 18; }();
    const int64_t clusters = cdiv(M, 256) * cdiv(N, 256);
    const bool pair = env >= 0 ? env != 0 : (M > 128 && clusters >= min_clusters);
    if (pair) {
      // 256x256 tiles on the persistent CTA-pair kernel (see pick_pair_mode)
      PMB_SMEM_OPT_IN((PairPCfg<false, 256>::SMEM_BYTES), gemm_bf16_pairp_kernel<false, 256>);
      q.tiles_n = (int)cdiv(N, 256); q.tiles = (int)clusters;
      ProfScope prof(st, "gemm_bf16", 2.0 * M * N * K, 2.0 * ((double)M * K + (double)K * N) + (out_bf16 ? 2.0 : 4.0) * M * N * (R ? 2 : 1));
      const int64_t slots = persistent_grid(148) / 2;
      const unsigned grid = 2u * (unsigned)(clusters < slots ? clusters : slots);
      gemm_bf16_pairp_kernel<false, 256><<<grid, NTHREADS, PairPCfg<false, 256>::SMEM_BYTES, st>>>(g, (int)clusters);
      PMB_LAUNCHED();
      return PMB_OK;
    }
  }
  ProfScope prof(st, "gemm_bf16", 2.0 * M * N * K, 2.0 * ((double)M * K + (double)K * N) + (out_bf16 ? 2.0 : 4.0) * M * N * (R ? 2 : 1));
  {
    unsigned long long t0 = 0;
    unsigned long long* sc = sched_counter(st, q.tiles, &t0);
    gemm_bf16_kernel<false><<<persistent_grid(q.tiles), NTHREADS, Cfg<false>::SMEM_BYTES, st>>>(g, q.tiles, sc, t0);
  }
  PMB_LAUNCHED();
  return PMB_OK;
}

// ---- fp32 GEMM through bf16 pairs ------------------------------------------------------------------
// a = hi + lo with hi = bf16(a), lo = bf16(a - hi): 16 mantissa bits, relative representation error <= 2^-17.
// One thread = 4 consecutive columns of the pair; columns in [cols, ld16) are written as zero.
__global__ void split_pair16_kernel(const float* __restrict__ src, int64_t rows, int64_t cols, int64_t ld,
                                    uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, int64_t ld16, int vec) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t c4 = ld16 / 4;
  if (i >= rows * c4) return;
  int64_t r = i / c4, c = (i % c4) * 4;
  float f[4];
  if (vec && c + 4 <= cols) {
    float4 v = *reinterpret_cast<const float4*>(src + r * ld + c);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = (c + e < cols) ? src[r * ld + c + e] : 0.0f;
  }
  uint32_t h[4], l[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    h[e] = hb::float_to_bf16_bits(f[e]);
    l[e] = hb::float_to_bf16_bits(f[e] - hb::bf16_bits_to_float((uint16_t)h[e]));
  }
  *reinterpret_cast<uint2*>(hi + r * ld16 + c) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
  *reinterpret_cast<uint2*>(lo + r * ld16 + c) = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
}

pmb_status split_pair16(cudaStream_t st, const float* src, int64_t rows, int64_t cols, int64_t ld, uint16_t* hi, uint16_t* lo,
                        int64_t ld16) {
  if ((ld16 & 7) || ld16 < cols || ((reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 15))
    return fail(PMB_ERR_ARG, "split_pair16: the pair needs 16-byte aligned bases and a row pitch that is a multiple of 8");
  const int vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (ld & 3) == 0) ? 1 : 0;
  ProfScope prof(st, "split_f32_bf16x2", 0.0, 8.0 * rows * cols);
  split_pair16_kernel<<<(unsigned)cdiv(rows * (ld16 / 4), 256), 256, 0, st>>>(src, rows, cols, ld, hi, lo, ld16, vec);
  PMB_LAUNCHED();
  return PMB_OK;
}

// Columns [0, cols) of each row only (cols a multiple of 4); the rest of the destination pitch is left alone, so two
// sources can share one pair buffer side by side.
__global__ void split_pair16_cols_kernel(const float* __restrict__ src, int64_t rows, int64_t cols, int64_t ld,
                                         uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, int64_t ld16) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t c4 = cols / 4;
  if (i >= rows * c4) return;
  const int64_t r = i / c4, c = (i % c4) * 4;
  const float* s = src + r * ld + c;
  store_pair4(hi + r * ld16 + c, lo ? lo + r * ld16 + c : nullptr, s[0], s[1], s[2], s[3]);
}

pmb_status split_pair16_strided(cudaStream_t st, const float* src, int64_t rows, int64_t cols, int64_t ld, uint16_t* hi, uint16_t* lo,
                                int64_t ld16) {
  if ((cols & 3) || (ld16 & 3) || ld16 < cols || ((reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 7))
    return fail(PMB_ERR_ARG, "split_pair16_strided: column count and pitch must be multiples of 4, destinations 8-byte aligned");
  split_pair16_cols_kernel<<<(unsigned)cdiv(rows * (cols / 4), 256), 256, 0, st>>>(src, rows, cols, ld, hi, lo, ld16);
  PMB_LAUNCHED();
  return PMB_OK;
}

bool gemm_pairs_enabled() {
  static const int on = [] { const char* e = getenv("PMB_GEMM_ENGINE"); return (e && (strcmp(e, "tf32") == 0 || strcmp(e, "simt") == 0)) ? 0 : 1; }();
  return on != 0;
}

// Tile shape of the pair GEMM: 0 = 128x128 single-CTA tiles, 1 = 256x128 CTA-pair tiles, 2 = 256x256 CTA-pair tiles.
// `tile_mode` >= 0 (engines 4 / 5 / 6 of the public GEMM entry) or PMB_GEMM_PAIR=0/1/2 force it.
static int pick_pair_mode(const PairGemm* gs, int n, int tile_mode) {
  static const int env = [] { const char* e = getenv("PMB_GEMM_PAIR"); return e ? atoi(e) : -1; }();
  const int forced = tile_mode >= 0 ? tile_mode : env;
  if (forced >= 0 && forced <= 4) return forced;          // 3 / 4: the persistent CTA-pair kernel with 256x128 / 256x256 tiles
  // 256x256 CTA-pair tiles on the persistent pair kernel fetch half the operand bytes per flop and read half as
  // much shared memory per MMA.  Alone, at 2048 tokens, they win where there is at least half a wave of the 74
  // cluster slots (in_proj forward 36.8 against 39.6 us, dnormed 23.1 against 28.2, dW_in 41.4 against 55.7) and lose
  // below (out_proj forward 33.3 against 27.0 us at 24 clusters); inside the training step, where other streams'
  // kernels fill the SMs a short launch leaves idle, the threshold that measured best is 18 clusters per product
  // (step 13.35 ms with the single-CTA kernel everywhere, 13.05 at 37, 12.86 at 18, 12.95 at 12).
  // 256x128 pair tiles measured no faster than single-CTA tiles.  PMB_GEMM_PAIR_MIN overrides the threshold.
  static const int half_wave = [] { const char* e = getenv("PMB_GEMM_PAIR_MIN"); return e ? atoi(e) : 18; }();
  for (int i = 0; i < n; ++i) {
    if (gs[i].M <= 128) return 0;        // a pair tile would be half empty
    if (cdiv(gs[i].M, 256) * cdiv(gs[i].N, 256) < half_wave) return 0;
  }
  return 4;
}

// C (fp32) = op(A) op(B) (+ R) with both operands given as bf16 pairs: three kind::f16 MMAs per k-step.
// Relative accuracy ~1e-5 of the result's scale; twice the tensor-core rate and less than half the shared-memory
// traffic of the 3xTF32 kernel.  Up to two independent products go out as one launch; the tiles of g[0] are
// scheduled first, so put the product with the longer K there.
pmb_status gemm_pairs_group(cudaStream_t st, const PairGemm* gs, int n, int tile_mode) {
  using namespace hb;
  if (n < 1 || n > MAX_GROUP) return fail(PMB_ERR_ARG, "gemm_pairs_group: 1 to %d products per launch", MAX_GROUP);
  PMB_SMEM_OPT_IN(Cfg<true>::SMEM_BYTES, gemm_bf16_kernel<true>);
  Group g{};
  for (int i = 1; i < MAX_GROUP; ++i) { g.pr[i].tiles_n = 1; g.pr[i].tiles = 0; }
  double flops = 0.0, bytes = 0.0;
  int64_t total = 0;
  for (int i = 0; i < n; ++i) {
    const PairGemm& e = gs[i];
    const int64_t M = e.M, N = e.N, K = e.K;
    if (M <= 0 || N <= 0 || K <= 0) return fail(PMB_ERR_SHAPE, "gemm_pairs: M, N, K must be positive");
    if ((e.A.ld & 7) || (e.B.ld & 7) ||
        ((reinterpret_cast<uintptr_t>(e.A.hi) | reinterpret_cast<uintptr_t>(e.A.lo) | reinterpret_cast<uintptr_t>(e.B.hi) | reinterpret_cast<uintptr_t>(e.B.lo)) & 15))
      return fail(PMB_ERR_UNSUPPORTED, "gemm_pairs: operands need 16-byte aligned bases and row pitches that are multiples of 8");
    Problem& q = g.pr[i];
    if (!e.ta) { PMB_TRY(make_map(&q.mA, e.A.hi, K, M, e.A.ld, TBK, TBM)); PMB_TRY(make_map(&q.mAlo, e.A.lo, K, M, e.A.ld, TBK, TBM)); }
    else { PMB_TRY(make_map(&q.mA, e.A.hi, M, K, e.A.ld, 64, TBK)); PMB_TRY(make_map(&q.mAlo, e.A.lo, M, K, e.A.ld, 64, TBK)); }
    if (e.tb) { PMB_TRY(make_map(&q.mB, e.B.hi, K, N, e.B.ld, TBK, TBN)); PMB_TRY(make_map(&q.mBlo, e.B.lo, K, N, e.B.ld, TBK, TBN)); }
    else { PMB_TRY(make_map(&q.mB, e.B.hi, N, K, e.B.ld, 64, TBK)); PMB_TRY(make_map(&q.mBlo, e.B.lo, N, K, e.B.ld, 64, TBK)); }
    Params& p = q.p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.a_mn_major = e.ta ? 1 : 0; p.b_mn_major = e.tb ? 0 : 1;
    p.C = e.C; p.ldc = e.ldc; p.R = e.R; p.out_bf16 = 0;
    PMB_TRY(make_out_maps(&q));
    p.e_hi = const_cast<uint16_t*>(e.emit.hi); p.e_lo = const_cast<uint16_t*>(e.emit.lo); p.lde = e.emit.ld;   // (Pair16 is declared for reading; this one is written)
    if (p.e_hi && (!p.tma_out || !p.e_lo || (p.lde & 7) || ((reinterpret_cast<uintptr_t>(p.e_hi) | reinterpret_cast<uintptr_t>(p.e_lo)) & 15)))
      return fail(PMB_ERR_UNSUPPORTED, "gemm_pairs: the pair output needs the TMA-store epilogue, 16-byte aligned arrays and a pitch that is a multiple of 8");
    q.tiles_n = (int)cdiv(N, TBN);
    const int64_t t = cdiv(M, TBM) * cdiv(N, TBN);
    total += t;
    if (total > 0x7fffffff) return fail(PMB_ERR_UNSUPPORTED, "gemm_pairs: too many tiles");
    q.tiles = (int)t;
    flops += 2.0 * M * N * K;
    bytes += 4.0 * ((double)M * K + (double)K * N + (double)M * N * (e.R ? 2 : 1));
  }
  int pair_mode = pick_pair_mode(gs, n, tile_mode);
  for (int i = 0; i < n; ++i) if (gs[i].emit.hi && pair_mode <= 2) pair_mode = 0;      // (the one-tile-per-cluster kernels do not write the pair output)
  if (pair_mode) {
    const int bn2 = (pair_mode == 2 || pair_mode == 4) ? 256 : 128;
    PMB_SMEM_OPT_IN((PairCfg<true, 256>::SMEM_BYTES), gemm_bf16_pair_kernel<true, 256>);
    PMB_SMEM_OPT_IN((PairCfg<true, 128>::SMEM_BYTES), gemm_bf16_pair_kernel<true, 128>);
    int64_t clusters = 0;
    for (int i = 0; i < n; ++i) {
      const PairGemm& e = gs[i];
      Problem& q = g.pr[i];
      // B boxes of the pair kernel are BN2/2 rows tall (K-major tiles); MN-major boxes stay 64 columns wide
      if (e.tb) { PMB_TRY(make_map(&q.mB, e.B.hi, e.K, e.N, e.B.ld, TBK, bn2 / 2)); PMB_TRY(make_map(&q.mBlo, e.B.lo, e.K, e.N, e.B.ld, TBK, bn2 / 2)); }
      q.tiles_n = (int)cdiv(e.N, bn2);
      q.tiles = (int)(cdiv(e.M, 256) * cdiv(e.N, bn2));
      clusters += q.tiles;
    }
    if (pair_mode >= 3) {
      ProfScope prof(st, "gemm_bf16x2", flops, bytes);
      const int64_t slots = persistent_grid(148) / 2;
      const unsigned grid = 2u * (unsigned)(clusters < slots ? clusters : slots);
      if (pair_mode == 4) {
        PMB_SMEM_OPT_IN((PairPCfg<true, 256>::SMEM_BYTES), gemm_bf16_pairp_kernel<true, 256>);
        gemm_bf16_pairp_kernel<true, 256><<<grid, NTHREADS, PairPCfg<true, 256>::SMEM_BYTES, st>>>(g, (int)clusters);
      } else {
        PMB_SMEM_OPT_IN((PairPCfg<true, 128>::SMEM_BYTES), gemm_bf16_pairp_kernel<true, 128>);
        gemm_bf16_pairp_kernel<true, 128><<<grid, NTHREADS, PairPCfg<true, 128>::SMEM_BYTES, st>>>(g, (int)clusters);
      }
      PMB_LAUNCHED();
      return PMB_OK;
    }
    ProfScope prof(st, pair_mode == 2 ? "gemm_bf16x2_pair256" : "gemm_bf16x2_pair128", flops, bytes);
    if (pair_mode == 2) gemm_bf16_pair_kernel<true, 256><<<(unsigned)(2 * clusters), NTHREADS, PairCfg<true, 256>::SMEM_BYTES, st>>>(g);
    else gemm_bf16_pair_kernel<true, 128><<<(unsigned)(2 * clusters), NTHREADS, PairCfg<true, 128>::SMEM_BYTES, st>>>(g);
    PMB_LAUNCHED();
    return PMB_OK;
  }
  ProfScope prof(st, "gemm_bf16x2", flops, bytes);
  {
    unsigned long long t0 = 0;
    unsigned long long* sc = sched_counter(st, total, &t0);
    gemm_bf16_kernel<true><<<persistent_grid(total), NTHREADS, Cfg<true>::SMEM_BYTES, st>>>(g, (int)total, sc, t0);
  }
  PMB_LAUNCHED();
  return PMB_OK;
}

pmb_status gemm_pairs(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const Pair16& A, const Pair16& B,
                      float* C, int64_t ldc, const float* R, int tile_mode) {
  PairGemm e{ta, tb, M, N, K, A, B, C, ldc, R};
  return gemm_pairs_group(st, &e, 1, tile_mode);
}

// Library-owned scratch for the pairs of callers that hand in fp32 operands (one per device).
// pmb_gemm_reserve_scratch() sizes it up front for callers that must not allocate later.
// A block that has been handed out is never freed or moved: kernels already enqueued, and CUDA graphs that
// captured a call, keep using its address.  When a larger product arrives a new, larger block is allocated
// beside the old ones (the old ones stay until the process ends); there is no device-wide synchronisation.
static void* g_scratch[PMB_MAX_DEVICES] = {nullptr};
static size_t g_scratch_bytes[PMB_MAX_DEVICES] = {0};
static std::mutex g_scratch_mu;

pmb_status gemm_scratch(size_t bytes, void** out, cudaStream_t user_stream, bool check_capture) {
  int dev = 0;
  PMB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= PMB_MAX_DEVICES) return fail(PMB_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_bytes[dev] < bytes) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (check_capture && cudaStreamIsCapturing(user_stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
      return fail(PMB_ERR_WORKSPACE, "gemm: the pair scratch would have to grow during stream capture; call pmb_gemm_reserve_scratch(%zu) first", bytes);
    size_t want = align_up(bytes + bytes / 4, (size_t)1 << 20);
    void* fresh = nullptr;
    PMB_CUDA(cudaMalloc(&fresh, want));
    g_scratch[dev] = fresh;          // the previous block is deliberately kept alive
    g_scratch_bytes[dev] = want;
  }
  *out = g_scratch[dev];
  return PMB_OK;
}

// fp32 operands: one elementwise pass each into the scratch (rows compacted to a pitch that is a multiple of 8),
// then gemm_pairs.
pmb_status gemm_f32_via_bf16x2(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                               const float* B, int64_t ldb, float* C, int64_t ldc, const float* R, int tile_mode) {
  const int64_t a_rows = ta ? K : M, a_cols = ta ? M : K, b_rows = tb ? N : K, b_cols = tb ? K : N;
  const int64_t a_ld = (int64_t)align_up((size_t)a_cols, 8), b_ld = (int64_t)align_up((size_t)b_cols, 8);
  const size_t a_el = align_up((size_t)a_rows * a_ld, 64), b_el = align_up((size_t)b_rows * b_ld, 64);
  void* scratch = nullptr;
  PMB_TRY(gemm_scratch((2 * a_el + 2 * b_el) * 2 + 1024, &scratch, st, true));
  uint16_t* a_hi = static_cast<uint16_t*>(scratch);
  uint16_t* a_lo = a_hi + a_el;
  uint16_t* b_hi = a_lo + a_el;
  uint16_t* b_lo = b_hi + b_el;
  PMB_TRY(split_pair16(st, A, a_rows, a_cols, lda, a_hi, a_lo, a_ld));
  PMB_TRY(split_pair16(st, B, b_rows, b_cols, ldb, b_hi, b_lo, b_ld));
  return gemm_pairs(st, ta, tb, M, N, K, Pair16{a_hi, a_lo, a_ld}, Pair16{b_hi, b_lo, b_ld}, C, ldc, R, tile_mode);
}

}  // namespace pmb

extern "C" pmb_status pmb_gemm_reserve_scratch(size_t bytes) {
  void* p = nullptr;
  return pmb::gemm_scratch(bytes, &p, nullptr, false);
}

extern "C" pmb_status pmb_gemm_bf16(void* stream, int32_t trans_a, int32_t trans_b, int64_t M, int64_t N, int64_t K,
                                    const uint16_t* d_A, int64_t lda, const uint16_t* d_B, int64_t ldb,
                                    void* d_C, int64_t ldc, const void* d_R, int32_t out_bf16) {
  using namespace pmb;
  if (!d_A || !d_B || !d_C) return fail(PMB_ERR_ARG, "gemm_bf16: NULL operand");
  if (lda < (trans_a ? M : K) || ldb < (trans_b ? K : N) || ldc < N) return fail(PMB_ERR_SHAPE, "gemm_bf16: leading dimension smaller than the row length");
  return gemm_bf16(static_cast<cudaStream_t>(stream), trans_a != 0, trans_b != 0, M, N, K, d_A, lda, d_B, ldb, d_C, ldc, d_R, out_bf16 != 0);
}
