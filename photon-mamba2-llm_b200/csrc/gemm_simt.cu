// fp32 FMA GEMM for shapes the tensor-core path does not take (unaligned leading dimensions, tiny
// problems) and as an independent device-side cross-check of it.  Runs on the GPU; there is no CPU path.
#include "common.cuh"
#include "kernels.h"
#include "bgemm.cuh"

namespace pmb {

struct OpGemm {
  static constexpr bool SEG_SCALE = false;
  int Mdim, Ndim, K, ta, tb;
  const float* A; int64_t lda; const float* B; int64_t ldb; float* C; int64_t ldc; const float* R;
  __device__ bool init(int, int, int) { return true; }
  __device__ int nseg() const { return 1; }
  __device__ void krange(int, int, int, int& k0, int& k1) const { k0 = 0; k1 = K; }
  __device__ bool a_kcontig(int) const { return ta == 0; }
  __device__ bool b_kcontig(int) const { return tb != 0; }
  __device__ float a(int, int m, int k) const { return ta ? A[(int64_t)k * lda + m] : A[(int64_t)m * lda + k]; }
  __device__ float b(int, int k, int n) const { return tb ? B[(int64_t)n * ldb + k] : B[(int64_t)k * ldb + n]; }
  __device__ float seg_scale(int, int, int) const { return 1.0f; }
  __device__ bool seg_active(int) const { return true; }
  __device__ void store(int m, int n, float v) const {
    int64_t i = (int64_t)m * ldc + n;
    C[i] = R ? v + R[i] : v;
  }
};

pmb_status gemm_simt(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                     const float* B, int64_t ldb, float* C, int64_t ldc, const float* R) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(PMB_ERR_SHAPE, "gemm: non-positive dimension");
  if (M > 64 * 65535LL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(PMB_ERR_SHAPE, "gemm: dimension too large");
  OpGemm op{};
  op.Mdim = (int)M; op.Ndim = (int)N; op.K = (int)K; op.ta = ta; op.tb = tb;
  op.A = A; op.lda = lda; op.B = B; op.ldb = ldb; op.C = C; op.ldc = ldc; op.R = R;
  ProfScope prof(st, "gemm_simt", 2.0 * M * N * K, 4.0 * ((double)M * K + (double)K * N + (double)M * N * (R ? 2 : 1)));
  return launch_bgemm(st, op, 1);
}

}  // namespace pmb
