// 3xTF32 GEMM variant for problems with few output tiles: 128x64 tiles, 2-stage ring, two CTAs resident per SM
// (tc_bgemm_kernel with a pass-through Op).  Small GEMMs are bound by per-tile latency (pipeline fill, TMEM
// allocation, epilogue), which a second resident CTA overlaps; large GEMMs keep the 128x128 kernel of gemm_tc.cu,
// whose shared-memory traffic per FLOP is lower.
#include <map>
#include <tuple>
#include "common.cuh"
#include "kernels.h"
#include "tc_bgemm.cuh"

namespace pmb {

static __device__ unsigned int g_small_status = 0;

pmb_status read_clear_device_status_small(unsigned int* word) {
  unsigned int zero = 0;
  PMB_CUDA(cudaMemcpyFromSymbol(word, g_small_status, sizeof(unsigned int)));
  if (*word) PMB_CUDA(cudaMemcpyToSymbol(g_small_status, &zero, sizeof(unsigned int)));
  return PMB_OK;
}

namespace {

struct OpGemm64 {
  static constexpr int BN = 64;
  static constexpr bool A_SCALE = false, B_SCALE = false, SEG_EPI = false;
  static constexpr int AUX_FLOATS = 0;
  float* aux;
  __device__ void stage(int, int) {}
  int Mdim, Ndim, K, a_mn, b_mn;
  float* C; int64_t ldc; const float* R;
  __device__ bool init(int, int, int) { return true; }
  __device__ int nseg() const { return 1; }
  __device__ void seg(int, int, int, int& kt0, int& kt1, int& am, int& bm, int& amn, int& bmn) const {
    kt0 = 0; kt1 = (K + 31) / 32; am = 0; bm = 1; amn = a_mn; bmn = b_mn;
  }
  __device__ void a_coord(int, int kt, int m0, int& c0, int& c1, int& c2) const {
    if (!a_mn) { c0 = kt * 32; c1 = m0; } else { c0 = m0; c1 = kt * 32; }
    c2 = 0;
  }
  __device__ void b_coord(int, int kt, int n0, int& c0, int& c1, int& c2) const {
    if (!b_mn) { c0 = kt * 32; c1 = n0; } else { c0 = n0; c1 = kt * 32; }
    c2 = 0;
  }
  __device__ void a_scale4(int, int, int, int, float (&)[4]) const {}
  __device__ float b_scale(int, int, int) const { return 1.0f; }
  __device__ void seg_accumulate(int, int, int, const float (&)[32], float (&)[32]) const {}
  __device__ void stage_seg(int, int, int) {}
  __device__ void store(int m, int nb, const float (&v)[32]) const {
    float* crow = C + (int64_t)m * ldc + nb;
    const float* rrow = R ? R + (int64_t)m * ldc + nb : nullptr;
    const bool vec = (nb + 32 <= Ndim) && ((ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) &&
                     (!R || (reinterpret_cast<uintptr_t>(R) & 15) == 0);
    if (vec) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (rrow) { float4 q = *reinterpret_cast<const float4*>(rrow + j); o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w; }
        *reinterpret_cast<float4*>(crow + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (nb + j < Ndim) crow[j] = v[j] + (rrow ? rrow[j] : 0.0f);
    }
  }
};

struct Key {
  const void* base; int64_t d0, d1, ld; int b0, b1; bool mn;
  bool operator<(const Key& o) const { return std::tie(base, d0, d1, ld, b0, b1, mn) < std::tie(o.base, o.d0, o.d1, o.ld, o.b0, o.b1, o.mn); }
};
std::map<Key, CUtensorMap> g_cache;

pmb_status get_map(CUtensorMap* out, const float* base, int64_t d0, int64_t d1, int64_t ld, int b0, int b1, bool mn) {
  Key key{base, d0, d1, ld, b0, b1, mn};
  auto it = g_cache.find(key);
  if (it == g_cache.end()) {
    if (g_cache.size() > 8192) g_cache.clear();
    CUtensorMap m;
    int64_t dims[3] = {d0, d1, 1}, strides[2] = {ld, ld * d1};
    int box[3] = {b0, b1, 1};
    PMB_TRY(tcx::make_map(&m, base, 3, dims, strides, box, mn));
    it = g_cache.emplace(key, m).first;
  }
  *out = it->second;
  return PMB_OK;
}

unsigned int* status_ptr() {
  static unsigned int* ptr[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!ptr[dev]) cudaGetSymbolAddress((void**)&ptr[dev], g_small_status);
  return ptr[dev];
}

}  // namespace

pmb_status gemm_tc_small(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                         const float* B, int64_t ldb, float* C, int64_t ldc, const float* R) {
  tcb::MapSet ms{};
  // A: ta=0 stored (M,K) K-major; ta=1 stored (K,M) M-contiguous.  B: tb=1 stored (N,K) K-major; tb=0 stored (K,N).
  if (!ta) PMB_TRY(get_map(&ms.m[0], A, K, M, lda, 32, 128, false)); else PMB_TRY(get_map(&ms.m[0], A, M, K, lda, 32, 32, true));
  if (tb) PMB_TRY(get_map(&ms.m[1], B, K, N, ldb, 32, 64, false)); else PMB_TRY(get_map(&ms.m[1], B, N, K, ldb, 32, 32, true));
  ms.m[2] = ms.m[0]; ms.m[3] = ms.m[0];
  OpGemm64 op{};
  op.Mdim = (int)M; op.Ndim = (int)N; op.K = (int)K; op.a_mn = ta ? 1 : 0; op.b_mn = tb ? 0 : 1;
  op.C = C; op.ldc = ldc; op.R = R;
  ProfScope prof(st, "gemm_3xtf32_small", 2.0 * M * N * K, 4.0 * ((double)M * K + (double)K * N + (double)M * N * (R ? 2 : 1)));
  return tcb::launch(st, ms, op, 1, status_ptr());
}

}  // namespace pmb
