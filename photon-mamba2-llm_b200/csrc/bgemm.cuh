// 64x64-tile fp32 FMA contraction kernel, specialised by operand/epilogue functors.
#pragma once
#include "common.cuh"

namespace pmb {

constexpr int BM = 64, BN = 64, BK = 16, NTHR = 256;

// ---------------------------------------------------------------------------------------------
// Generic tile kernel.  Op interface (all __device__):
//   int Mdim, Ndim;  bool init(int batch, int m0, int n0)  -> false = tile not needed
//   int nseg();  void krange(int seg, int m0, int n0, int& k0, int& k1)  (k0 multiple of BK)
//   bool a_kcontig(int seg), b_kcontig(int seg)   memory contiguity of the operands (for coalescing)
//   float a(int seg, int m, int k), b(int seg, int k, int n)   (called only in range)
//   float seg_scale(int seg, int m, int n)   (only when Op::SEG_SCALE)
//   bool seg_active(int seg)                 (false = segment belongs to another split of the same tile)
//   void store(int m, int n, float v)
// ---------------------------------------------------------------------------------------------
template <class Op>
__global__ void __launch_bounds__(NTHR) bgemm_kernel(Op op) {
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (!op.init(blockIdx.z, m0, n0)) return;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  float total[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) total[i][j] = 0.0f;
  const int nseg = op.nseg();
  for (int seg = 0; seg < nseg; ++seg) {
    if (!op.seg_active(seg)) continue;  // split-K: this CTA owns a subset of the segments
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    int kb, ke;
    op.krange(seg, m0, n0, kb, ke);
    const bool akc = op.a_kcontig(seg), bkc = op.b_kcontig(seg);
    for (int k0 = kb; k0 < ke; k0 += BK) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int m, k;
        if (akc) { k = tid & 15; m = (tid >> 4) + 16 * j; } else { m = tid & 63; k = (tid >> 6) + 4 * j; }
        float v = 0.0f;
        if (m0 + m < op.Mdim && k0 + k < ke) v = op.a(seg, m0 + m, k0 + k);
        As[k][m] = v;
        int n, k2;
        if (bkc) { k2 = tid & 15; n = (tid >> 4) + 16 * j; } else { n = tid & 63; k2 = (tid >> 6) + 4 * j; }
        float w = 0.0f;
        if (n0 + n < op.Ndim && k0 + k2 < ke) w = op.b(seg, k0 + k2, n0 + n);
        Bs[k2][n] = w;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < BK; ++k) {
        float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
        float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
        float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (Op::SEG_SCALE) {
          int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
          float s = (m < op.Mdim && n < op.Ndim) ? op.seg_scale(seg, m, n) : 0.0f;
          total[i][j] = fmaf(acc[i][j], s, total[i][j]);
        } else {
          total[i][j] += acc[i][j];
        }
      }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < op.Mdim && n < op.Ndim) op.store(m, n, total[i][j]);
    }
}

template <class Op>
static pmb_status launch_bgemm(cudaStream_t st, const Op& op, int batches) {
  dim3 grid((unsigned)cdiv(op.Ndim, BN), (unsigned)cdiv(op.Mdim, BM), (unsigned)batches);
  bgemm_kernel<Op><<<grid, NTHR, 0, st>>>(op);
  PMB_LAUNCHED();
  return PMB_OK;
}

}  // namespace pmb
