// Flat Mamba2 language model training step (forward + backward, no optimizer): tied embedding ->
// checkpointed residual stack -> tied head -> mean cross-entropy.  Mirrors
// FlatMamba::forward_checkpointed_hidden + fused cross-entropy + checkpoint_backward
// (crates/pm-core/src/flat.rs:122-161, crates/pm-train/src/loss.rs:121-138, crates/pm-core/src/checkpoint.rs:110-135).
// The logits are produced in row tiles of at most LM_TILE_ROWS tokens and turned into their gradient in
// place, so the (tokens, vocab) matrix never exists as a whole (the reference tiles for the same reason,
// crates/pm-core/src/loss.rs:73-209).
#include <vector>
#include <cstdlib>
#include <initializer_list>
#include <vector>
#include "common.cuh"
#include "kernels.h"

namespace pmb {

// Row tile of the tied head: (rows, vocab) fp32 logits exist for one tile at a time.  1024 rows (206 MB at a 50k
// vocabulary) cost 1.7 % of the headline step against 2048 (412 MB); PMB_LM_TILE_ROWS overrides it (>= 128).
constexpr int LM_TILE_ROWS = 1024;
constexpr int HEAD_SPLITK = 3;

__global__ void embedding_fwd_kernel(const float* __restrict__ table, const int64_t* __restrict__ ids, float* __restrict__ out,
                                     int64_t rows, int D, int V, unsigned int* __restrict__ bad) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t n = rows * (D / 4);
  if (i >= n) return;
  int64_t r = i / (D / 4);
  int c = (int)(i % (D / 4)) * 4;
  int64_t id = ids[r];
  if (id < 0 || id >= V) { if (c == 0) atomicOr(bad, 1u); id = 0; }   // flagged; row 0 stands in so that nothing reads out of bounds
  *reinterpret_cast<float4*>(out + r * D + c) = *reinterpret_cast<const float4*>(table + id * D + c);
}

// bf16-storage variants: rows are gathered from / scattered out of bf16 activations
__global__ void embedding_fwd_bf16_kernel(const uint16_t* __restrict__ table16, const int64_t* __restrict__ ids, uint16_t* __restrict__ out,
                                          int64_t rows, int D, int V, unsigned int* __restrict__ bad) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t n = rows * (D / 8);
  if (i >= n) return;
  int64_t r = i / (D / 8);
  int c = (int)(i % (D / 8)) * 8;
  int64_t id = ids[r];
  if (id < 0 || id >= V) { if (c == 0) atomicOr(bad, 1u); id = 0; }
  *reinterpret_cast<uint4*>(out + r * D + c) = *reinterpret_cast<const uint4*>(table16 + id * D + c);
}

__global__ void embedding_bwd_bf16_kernel(float* __restrict__ dtable, const int64_t* __restrict__ ids, const uint16_t* __restrict__ dh,
                                          int64_t rows, int D, int V) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D) return;
  int64_t r = i / D;
  int c = (int)(i % D);
  int64_t id = ids[r];
  if (id < 0 || id >= V) return;
  atomicAdd(dtable + id * D + c, __uint_as_float((uint32_t)dh[i] << 16));
}

__global__ void embedding_bwd_kernel(float* __restrict__ dtable, const int64_t* __restrict__ ids, const float* __restrict__ dh,
                                     int64_t rows, int D, int V, float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D) return;
  int64_t r = i / D;
  int c = (int)(i % D);
  int64_t id = ids[r];
  if (id < 0 || id >= V) return;
  atomicAdd(dtable + id * D + c, dh[i] * scale);
}

// One block per row.  Pass 1: online max / sum-exp; pass 2: logits <- (softmax - onehot) * inv_rows.
// row_loss[r] = logsumexp - logit[target].
__global__ void __launch_bounds__(256) cross_entropy_kernel(float* __restrict__ logits, int64_t ld, int V,
                                                            const int64_t* __restrict__ targets, float* __restrict__ row_loss,
                                                            float inv_rows, uint16_t* __restrict__ d_hi, uint16_t* __restrict__ d_lo,
                                                            unsigned int* __restrict__ bad) {
  __shared__ float red[32];
  __shared__ float sh_max;
  int64_t r = blockIdx.x;
  float* row = logits + r * ld;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, row[i]);
  // block max
  {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[w] = m;
    __syncthreads();
    if (w == 0) {
      float v = lane < (int)(blockDim.x >> 5) ? red[lane] : -INFINITY;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) sh_max = v;
    }
    __syncthreads();
    m = sh_max;
  }
  float s = 0.0f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(row[i] - m);
  float tot = block_sum(s, red);
  float lse = m + logf(tot);
  int64_t tg = targets[r];
  if (threadIdx.x == 0) {
    row_loss[r] = (tg >= 0 && tg < V) ? lse - row[tg] : 0.0f;
    if (tg < 0 || tg >= V) atomicOr(bad, 2u);     // the reference's gather fails on such a target; here the row is flagged
  }
  __syncthreads();
  float inv = 1.0f / tot;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float pr = expf(row[i] - m) * inv;
    float gl = (pr - (i == tg ? 1.0f : 0.0f)) * inv_rows;
    if (d_hi) {   // the gradient is only ever a GEMM operand: emit it as a (hi, lo) bf16 pair, same pitch as the logits
      uint32_t u = __float_as_uint(gl);
      uint32_t h = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
      uint32_t ul = __float_as_uint(gl - __uint_as_float(h << 16));
      d_hi[r * ld + i] = (uint16_t)h;
      d_lo[r * ld + i] = (uint16_t)((ul + 0x7fffu + ((ul >> 16) & 1u)) >> 16);
    } else {
      row[i] = gl;
    }
  }
}

// Same loss, with the row staged in shared memory (one read of the logits) and the gradient written back over
// the row as a (hi, lo) bf16 pair: hi[i] at uint16 index i of the row, lo[i] at uint16 index ld + i, i.e. the pair
// matrices have a pitch of 2*ld uint16 and share the logits buffer.  Needs V floats of dynamic shared memory.
// write_lo == 0 (bf16 storage): only the bf16-rounded gradient is written (same place, same pitch).
constexpr int CE_THREADS = 1024;
// The kernel's dynamic shared-memory limit is raised to this fixed maximum (once per device, at the first launch)
// whatever the model's vocabulary, so that handles with different vocabularies can coexist in one process.
constexpr int CE_MAX_SMEM = 200 * 1024;
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_pair_inplace_kernel(float* __restrict__ logits, int64_t ld, int V,
                                                                                const int64_t* __restrict__ targets,
                                                                                float* __restrict__ row_loss, float inv_rows, int write_lo,
                                                                                unsigned int* __restrict__ bad) {
  extern __shared__ float srow[];
  __shared__ float red[32];
  const int64_t r = blockIdx.x;
  float* row = logits + r * ld;
  const int V4 = V >> 2;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V4; i += CE_THREADS) {
    float4 v = reinterpret_cast<const float4*>(row)[i];
    reinterpret_cast<float4*>(srow)[i] = v;
    m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
  }
  for (int i = 4 * V4 + threadIdx.x; i < V; i += CE_THREADS) { float v = row[i]; srow[i] = v; m = fmaxf(m, v); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[threadIdx.x & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const int64_t tg = targets[r];
  const float tlogit = (tg >= 0 && tg < V) ? srow[tg] : 0.0f;
  __syncthreads();                         // every thread has read srow[tg] before the loop below overwrites the row
  float s = 0.0f;
  for (int i = threadIdx.x; i < V; i += CE_THREADS) { float e = expf(srow[i] - m); srow[i] = e; s += e; }
  const float tot = block_sum(s, red);
  if (threadIdx.x == 0) {
    row_loss[r] = (tg >= 0 && tg < V) ? m + logf(tot) - tlogit : 0.0f;
    if (tg < 0 || tg >= V) atomicOr(bad, 2u);
  }
  const float inv = 1.0f / tot;
  uint16_t* hi = reinterpret_cast<uint16_t*>(row);
  uint16_t* lo = hi + ld;
  auto split = [](float v, uint32_t& h, uint32_t& l) {
    uint32_t u = __float_as_uint(v);
    h = (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
    uint32_t ul = __float_as_uint(v - __uint_as_float(h << 16));
    l = (ul + 0x7fffu + ((ul >> 16) & 1u)) >> 16;
  };
  for (int i = threadIdx.x; i < V4; i += CE_THREADS) {
    float4 e = reinterpret_cast<const float4*>(srow)[i];
    const int c = 4 * i;
    float g[4] = {e.x * inv, e.y * inv, e.z * inv, e.w * inv};
    uint32_t h[4], l4[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { if (c + k == tg) g[k] -= 1.0f; split(g[k] * inv_rows, h[k], l4[k]); }
    *reinterpret_cast<uint2*>(hi + c) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
    if (write_lo) *reinterpret_cast<uint2*>(lo + c) = make_uint2(l4[0] | (l4[1] << 16), l4[2] | (l4[3] << 16));
  }
  for (int i = 4 * V4 + threadIdx.x; i < V; i += CE_THREADS) {
    uint32_t h, l1;
    split((srow[i] * inv - (i == tg ? 1.0f : 0.0f)) * inv_rows, h, l1);
    hi[i] = (uint16_t)h; if (write_lo) lo[i] = (uint16_t)l1;
  }
}

// ---- two-level wiring: mean-pool groups of GROUP tokens down, repeat up with a one-group causal shift.
// Storage type T is float or bf16 bits (uint16_t); arithmetic in fp32.
template <class T> __device__ __forceinline__ float ld_act(const T* p);
template <> __device__ __forceinline__ float ld_act<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_act<uint16_t>(const uint16_t* p) { return __uint_as_float((uint32_t)(*p) << 16); }
template <class T> __device__ __forceinline__ void st_act(T* p, float v);
template <> __device__ __forceinline__ void st_act<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_act<uint16_t>(uint16_t* p, float v) {
  uint32_t u = __float_as_uint(v);
  u += 0x7fffu + ((u >> 16) & 1u);
  *p = (uint16_t)(u >> 16);
}

// mode 0: out[b,g,:] = mean_j in[b,GROUP*g+j,:]                      (pool, out has T/GROUP rows per sequence)
// mode 1: out[b,t,:] = a[b,t,:] + (t/GROUP >= 1 ? in[b,t/GROUP-1,:] : 0)   (shifted repeat, added to a)
// mode 2: out[b,g,:] = (g+1 < T/GROUP) ? sum_j in[b,GROUP*(g+1)+j,:] : 0   (adjoint of mode 1 w.r.t. `in`)
// mode 3: out[b,t,:] = a[b,t,:] + in[b,t/GROUP,:] / GROUP                   (adjoint of mode 0, accumulated onto a)
template <class T>
__global__ void hier_kernel(const T* __restrict__ in, const T* __restrict__ a, T* __restrict__ out, int B, int Tfull, int D, int GROUP, int mode) {
  const int Tg = Tfull / GROUP;
  const bool coarse_out = (mode == 0 || mode == 2);
  const int64_t rows = (int64_t)B * (coarse_out ? Tg : Tfull);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D) return;
  const int c = (int)(i % D); const int64_t r = i / D;
  const int per = coarse_out ? Tg : Tfull;
  const int b = (int)(r / per), t = (int)(r % per);
  float v = 0.0f;
  if (mode == 0) {
    for (int j = 0; j < GROUP; ++j) v += ld_act(in + ((int64_t)b * Tfull + (int64_t)t * GROUP + j) * D + c);
    v /= (float)GROUP;
  } else if (mode == 1) {
    v = ld_act(a + i);
    const int g = t / GROUP;
    if (g >= 1) v += ld_act(in + ((int64_t)b * Tg + g - 1) * D + c);
  } else if (mode == 2) {
    if (t + 1 < Tg)
      for (int j = 0; j < GROUP; ++j) v += ld_act(in + ((int64_t)b * Tfull + (int64_t)(t + 1) * GROUP + j) * D + c);
  } else {
    v = ld_act(a + i) + ld_act(in + ((int64_t)b * Tg + t / GROUP) * D + c) / (float)GROUP;
  }
  st_act(out + i, v);
}

// out = sum of n slabs of `elems` floats (split-K partial products), float4 lanes
__global__ void sum_slabs_kernel(const float* __restrict__ part, int n, int64_t elems, float* __restrict__ out) {
  int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= elems) return;
  float4 a = *reinterpret_cast<const float4*>(part + i);
  for (int s = 1; s < n; ++s) {
    const float4 b = *reinterpret_cast<const float4*>(part + (int64_t)s * elems + i);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  }
  *reinterpret_cast<float4*>(out + i) = a;
}

__global__ void __launch_bounds__(256) mean_kernel(const float* __restrict__ v, int64_t n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.0f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s += v[i];
  float tot = block_sum(s, red);
  if (threadIdx.x == 0) *out = tot / (float)n;
}

}  // namespace pmb

using namespace pmb;

struct pmb_lm {
  pmb_mamba2_config cfg;
  Dims d;
  int L, V, Vp, tile_rows;
  int64_t n_params;
  std::vector<int64_t> off;  // [0] embedding, then 8 per layer
  float* params = nullptr;
  float* grads = nullptr;
  float* saved = nullptr;     // (L+1) x (M, D)
  float* dhidden = nullptr;   // (M, D)
  float* logits = nullptr;    // (tile_rows, Vp)
  float* row_loss = nullptr;  // (M)
  float* loss = nullptr;      // scalar
  unsigned int* bad = nullptr;
  int64_t* ids = nullptr;
  int64_t* targets = nullptr;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  int bf16 = 0;               // storage dtype of activations / GEMM operands
  uint16_t* params16 = nullptr;   // bf16 copy of the flat parameter buffer, refreshed every step
  uint16_t* dlogits16 = nullptr;  // (tile_rows, Vp)
  // fp32 storage with pair GEMMs: (hi, lo) bf16 pairs of the flat parameters (refreshed every step), of the
  // logits gradient tile and of the final hidden rows
  int pairs = 0;
  int ce_inplace = 0;         // the logits row fits in shared memory: the gradient pair overwrites the logits tile
  uint16_t *params_hi = nullptr, *params_lo = nullptr, *dlog_hi = nullptr, *dlog_lo = nullptr, *hid_hi = nullptr, *hid_lo = nullptr;
  float* dh_part = nullptr;   // HEAD_SPLITK partial products of dhidden = dlogits E (few tiles, very long K)
  uint16_t* l1_pair = nullptr; // two-level fp32 model: (hi, lo) pairs of `pooled` and `dh1`, 4 x (M/group, D) bf16
  std::vector<Weights16> lw16;
  // hierarchical variant (L1 > 0): level 0 = layers [0,L0) at token rate, level 1 = layers [L0,L0+L1) at 1/group rate
  int L0 = 0, L1 = 0, group = 1;
  Dims d1;                    // level-1 dims (seqlen / group)
  int64_t off_proj = -1;      // (D,D) projection into level 1
  void* saved1 = nullptr;     // (L1+1) x (M/group, D)
  void* pooled = nullptr;     // (M/group, D)  mean-pooled level-0 output
  void* dpool = nullptr;      // (M/group, D)  gradient w.r.t. pooled
  void* dh1 = nullptr;        // (M/group, D)
  void* hsum = nullptr;       // (M, D)  h0 + shifted repeat of h1
  int64_t act_bytes = 0;
  std::vector<pmb_block_params> lp;
  std::vector<pmb_block_grads> lg;
  // data-parallel step (fp32 storage): the token-lookup share of the embedding gradient is exchanged as rows, see
  // pmb_lm_step_device_dp.  split_table != 0 while such a step is being enqueued.
  int split_table = 0;
  void* table_stream = nullptr;   // the stream on which the head's share of the table gradient completes
  char* gather = nullptr;         // world_size x [(M, D) rows | (M) ids]
  size_t gather_bytes = 0;
};

static int64_t tensor_elems(const Dims& d, int which) {
  switch (which) {
    case 0: return (int64_t)d.D * d.J;
    case 1: return (int64_t)d.X * d.K;
    case 2: return d.X;
    case 3: case 4: case 5: return d.H;
    case 6: return d.I;
    case 7: return (int64_t)d.I * d.D;
  }
  return 0;
}

static pmb_status lm_create_impl(const pmb_mamba2_config* cfg, int L0, int L1, int group, int vocab, int batch, int seqlen,
                                 int bf16_storage, pmb_lm** out) {
  if (!out) return fail(PMB_ERR_ARG, "lm_create: out is NULL");
  *out = nullptr;
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  if (bf16_storage && ((d.D % 8) || (d.J % 8) || (d.I % 8)))
    return fail(PMB_ERR_SHAPE, "lm_create: bf16 storage needs d_model, d_inner and in_proj_dim to be multiples of 8");
  if (L0 <= 0 || L1 < 0 || vocab <= 0) return fail(PMB_ERR_SHAPE, "lm_create: layer counts and vocab must be positive");
  if (d.D % 4 != 0) return fail(PMB_ERR_SHAPE, "lm_create: d_model must be a multiple of 4");
  if (L1 > 0 && (group < 2 || seqlen % group != 0)) return fail(PMB_ERR_SHAPE, "lm_create: seqlen %d is not a multiple of the pooling group %d", seqlen, group);
  const int n_layers = L0 + L1;
  pmb_lm* lm = new pmb_lm();
  lm->cfg = *cfg; lm->d = d; lm->L = n_layers; lm->L0 = L0; lm->L1 = L1; lm->group = L1 > 0 ? group : 1;
  lm->V = vocab; lm->bf16 = bf16_storage ? 1 : 0;
  if (L1 > 0) {
    pmb_status s1 = make_dims(cfg, batch, seqlen / group, &lm->d1);
    if (s1 != PMB_OK) { delete lm; return s1; }
  }
  lm->Vp = (int)align_up((size_t)vocab, 64);
  int tile_cap = LM_TILE_ROWS;
  if (const char* e = getenv("PMB_LM_TILE_ROWS")) { int v = atoi(e); if (v >= 128) tile_cap = v; }
  lm->tile_rows = (int)(d.M < tile_cap ? d.M : tile_cap);
  int64_t o = 0;
  auto place = [&](int64_t n) { int64_t at = o; o += (int64_t)align_up((size_t)n, 64); return at; };
  lm->off.push_back(place((int64_t)vocab * d.D));
  for (int l = 0; l < n_layers; ++l) {
    if (L1 > 0 && l == L0) lm->off_proj = place((int64_t)d.D * d.D);
    for (int w = 0; w < 8; ++w) lm->off.push_back(place(tensor_elems(d, w)));
  }
  lm->n_params = o;
  lm->ws_bytes = stack_ws_bytes(d, lm->bf16 != 0, !bf16_storage && block_uses_pairs(d));   // two forward slots: the backward recomputes one block ahead
  const size_t esz = lm->bf16 ? 2 : 4;
  size_t slot = (size_t)d.M * d.D * esz;
  size_t slot1 = L1 > 0 ? (size_t)lm->d1.M * d.D * esz : 0;
  auto alloc = [&](void** p, size_t bytes) -> bool { return cudaMalloc(p, bytes) == cudaSuccess; };
  bool ok = true;
  ok = ok && alloc((void**)&lm->params, (size_t)o * 4);
  ok = ok && alloc((void**)&lm->grads, (size_t)o * 4);
  ok = ok && alloc((void**)&lm->saved, slot * (L0 + 1));
  ok = ok && alloc((void**)&lm->dhidden, slot);
  ok = ok && alloc((void**)&lm->logits, (size_t)lm->tile_rows * lm->Vp * 4);
  ok = ok && alloc((void**)&lm->row_loss, (size_t)d.M * 4);
  ok = ok && alloc((void**)&lm->loss, 256);
  ok = ok && alloc((void**)&lm->bad, 256);
  ok = ok && alloc((void**)&lm->ids, (size_t)d.M * 8);
  ok = ok && alloc((void**)&lm->targets, (size_t)d.M * 8);
  ok = ok && alloc(&lm->ws, lm->ws_bytes);
  lm->pairs = (!lm->bf16 && block_uses_pairs(d)) ? 1 : 0;
  size_t pair_bytes = 0;
  if (lm->pairs) {
    const size_t tv = (size_t)lm->tile_rows * lm->Vp * 2, td = (size_t)lm->tile_rows * d.D * 2;
    ok = ok && alloc((void**)&lm->params_hi, (size_t)o * 2) && alloc((void**)&lm->params_lo, (size_t)o * 2);
    lm->ce_inplace = ((size_t)vocab * 4 <= (size_t)CE_MAX_SMEM) ? 1 : 0;
    if (!lm->ce_inplace) ok = ok && alloc((void**)&lm->dlog_hi, tv) && alloc((void**)&lm->dlog_lo, tv);
    ok = ok && alloc((void**)&lm->hid_hi, td) && alloc((void**)&lm->hid_lo, td);
    ok = ok && alloc((void**)&lm->dh_part, (size_t)HEAD_SPLITK * lm->tile_rows * d.D * 4);
    pair_bytes = (lm->ce_inplace ? 0 : 2 * tv) + 2 * td + (size_t)HEAD_SPLITK * lm->tile_rows * d.D * 4;
  }
  if (lm->bf16) {
    ok = ok && alloc((void**)&lm->params16, (size_t)o * 2);
    lm->ce_inplace = ((size_t)vocab * 4 <= (size_t)CE_MAX_SMEM) ? 1 : 0;
    if (!lm->ce_inplace) ok = ok && alloc((void**)&lm->dlogits16, (size_t)lm->tile_rows * lm->Vp * 2);
  }
  if (L1 > 0) {
    ok = ok && alloc(&lm->saved1, slot1 * (L1 + 1));
    ok = ok && alloc(&lm->pooled, slot1);
    ok = ok && alloc(&lm->dpool, slot1);
    ok = ok && alloc(&lm->dh1, slot1);
    ok = ok && alloc(&lm->hsum, slot);
    if (lm->pairs) ok = ok && alloc((void**)&lm->l1_pair, (size_t)4 * lm->d1.M * d.D * 2);
  }
  if (!ok) {
    pmb_status s = fail(PMB_ERR_CUDA, "lm_create: cudaMalloc failed: %s", cudaGetErrorString(cudaGetLastError()));
    pmb_lm_destroy(lm);
    return s;
  }
  cudaMemset(lm->params, 0, (size_t)o * 4);
  cudaMemset(lm->grads, 0, (size_t)o * 4);
  cudaMemset(lm->bad, 0, 256);
  lm->act_bytes = (int64_t)(slot * (L0 + 1) + slot1 * (L1 + 1) + slot + 3 * slot1 + (L1 > 0 ? slot : 0) +
                            (size_t)lm->tile_rows * lm->Vp * ((lm->bf16 && !lm->ce_inplace) ? 6 : 4) + pair_bytes + (size_t)d.M * 4 + lm->ws_bytes);
  lm->lp.resize(n_layers); lm->lg.resize(n_layers); lm->lw16.resize(n_layers);
  for (int l = 0; l < n_layers; ++l) {
    const int64_t* f = &lm->off[1 + 8 * l];
    float* P = lm->params; float* G = lm->grads;
    lm->lp[l] = pmb_block_params{P + f[0], P + f[1], P + f[2], P + f[3], P + f[4], P + f[5], P + f[6], P + f[7]};
    lm->lg[l] = pmb_block_grads{G + f[0], G + f[1], G + f[2], G + f[3], G + f[4], G + f[5], G + f[6], G + f[7]};
    lm->lw16[l] = Weights16{lm->params16 ? lm->params16 + f[0] : nullptr, lm->params16 ? lm->params16 + f[7] : nullptr};
    if (lm->pairs) lm->lw16[l] = Weights16{lm->params_hi + f[0], lm->params_hi + f[7], lm->params_lo + f[0], lm->params_lo + f[7], true};
  }
  *out = lm;
  return PMB_OK;
}

extern "C" pmb_status pmb_lm_create(const pmb_mamba2_config* cfg, int32_t n_layers, int32_t vocab, int32_t batch,
                                    int32_t seqlen, pmb_lm** out) {
  return lm_create_impl(cfg, n_layers, 0, 1, vocab, batch, seqlen, 0, out);
}

extern "C" pmb_status pmb_lm_create_dtype(const pmb_mamba2_config* cfg, int32_t n_layers, int32_t vocab, int32_t batch,
                                          int32_t seqlen, int32_t bf16_storage, pmb_lm** out) {
  return lm_create_impl(cfg, n_layers, 0, 1, vocab, batch, seqlen, bf16_storage, out);
}

extern "C" pmb_status pmb_lm_create_hier(const pmb_mamba2_config* cfg, int32_t n_layers_level0, int32_t n_layers_level1,
                                         int32_t group, int32_t vocab, int32_t batch, int32_t seqlen, int32_t bf16_storage,
                                         pmb_lm** out) {
  if (n_layers_level1 <= 0) return fail(PMB_ERR_SHAPE, "lm_create_hier: level 1 needs at least one layer");
  return lm_create_impl(cfg, n_layers_level0, n_layers_level1, group, vocab, batch, seqlen, bf16_storage, out);
}

extern "C" void pmb_lm_destroy(pmb_lm* lm) {
  if (!lm) return;
  cudaFree(lm->params); cudaFree(lm->grads); cudaFree(lm->saved); cudaFree(lm->dhidden); cudaFree(lm->logits);
  cudaFree(lm->row_loss); cudaFree(lm->loss); cudaFree(lm->bad); cudaFree(lm->ids); cudaFree(lm->targets); cudaFree(lm->ws); cudaFree(lm->params16); cudaFree(lm->dlogits16);
  cudaFree(lm->params_hi); cudaFree(lm->params_lo); cudaFree(lm->dlog_hi); cudaFree(lm->dlog_lo); cudaFree(lm->hid_hi); cudaFree(lm->hid_lo); cudaFree(lm->dh_part);
  cudaFree(lm->gather); cudaFree(lm->l1_pair); cudaFree(lm->saved1); cudaFree(lm->pooled); cudaFree(lm->dpool); cudaFree(lm->dh1); cudaFree(lm->hsum);
  delete lm;
}

extern "C" int64_t pmb_lm_param_count(const pmb_lm* lm) { return lm ? lm->n_params : 0; }
extern "C" int64_t pmb_lm_param_offset(const pmb_lm* lm, int32_t layer, int32_t which) {
  if (!lm) return -1;
  if (layer == -2) return lm->off_proj;   // (D,D) projection into level 1 (hierarchical variant), else -1
  if (layer < 0) return lm->off[0];
  if (layer >= lm->L || which < 0 || which > 7) return -1;
  return lm->off[1 + 8 * layer + which];
}
extern "C" float* pmb_lm_params(pmb_lm* lm) { return lm ? lm->params : nullptr; }
extern "C" float* pmb_lm_grads(pmb_lm* lm) { return lm ? lm->grads : nullptr; }
extern "C" int64_t pmb_lm_activation_bytes(const pmb_lm* lm) { return lm ? lm->act_bytes : 0; }
extern "C" void pmb_lm_activation_detail(const pmb_lm* lm, int64_t* h_out3) {
  if (!lm || !h_out3) return;
  const size_t esz = lm->bf16 ? 2 : 4;
  h_out3[0] = (int64_t)((size_t)lm->d.M * lm->d.D * esz * (lm->L0 + 1) + (lm->L1 > 0 ? (size_t)lm->d1.M * lm->d.D * esz * (lm->L1 + 1) : 0));                          // stored for backward: block inputs
  h_out3[1] = (int64_t)lm->ws_bytes;                                                              // transient: one block's workspace
  h_out3[2] = (int64_t)((size_t)lm->tile_rows * lm->Vp * (lm->ce_inplace ? 4 : (lm->bf16 ? 6 : (lm->pairs ? 8 : 4))) + (size_t)lm->d.M * lm->d.D * esz +
                        (lm->pairs ? (size_t)lm->tile_rows * lm->d.D * 4 : 0));  // transient: logits tile (+ its gradient's pair), d(hidden)
}
extern "C" const float* pmb_lm_loss_device(const pmb_lm* lm) { return lm ? lm->loss : nullptr; }

extern "C" pmb_status pmb_lm_bad_tokens(pmb_lm* lm, void* stream, int32_t* h_flags_out) {
  if (!lm || !h_flags_out) return fail(PMB_ERR_ARG, "lm_bad_tokens: NULL argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned int bad = 0;
  PMB_CUDA(cudaMemcpyAsync(&bad, lm->bad, sizeof(bad), cudaMemcpyDeviceToHost, st));
  PMB_CUDA(cudaStreamSynchronize(st));
  if (bad) PMB_CUDA(cudaMemsetAsync(lm->bad, 0, sizeof(bad), st));
  *h_flags_out = (int32_t)bad;
  return PMB_OK;
}

// hier_kernel launcher on the model's storage dtype
static pmb_status hier_op(pmb_lm* lm, cudaStream_t st, const void* in, const void* a, void* out, int mode) {
  const Dims& d = lm->d;
  const bool coarse = (mode == 0 || mode == 2);
  int64_t n = (coarse ? lm->d1.M : d.M) * (int64_t)d.D;
  ProfScope prof(st, "hier_pool_repeat", 0.0, (lm->bf16 ? 2.0 : 4.0) * 3.0 * d.M * d.D / (coarse ? lm->group : 1));
  if (lm->bf16) hier_kernel<uint16_t><<<(unsigned)cdiv(n, 256), 256, 0, st>>>((const uint16_t*)in, (const uint16_t*)a, (uint16_t*)out, d.B, d.T, d.D, lm->group, mode);
  else hier_kernel<float><<<(unsigned)cdiv(n, 256), 256, 0, st>>>((const float*)in, (const float*)a, (float*)out, d.B, d.T, d.D, lm->group, mode);
  PMB_LAUNCHED();
  return PMB_OK;
}

// storage-dtype GEMM: C = op(A) op(B) with A, B, C in the model's activation dtype except where noted
static pmb_status lm_gemm(pmb_lm* lm, cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda,
                          const void* B16_or_f32, int64_t ldb, void* C, int64_t ldc, int out_storage) {
  if (lm->bf16) return gemm_bf16(st, ta, tb, M, N, K, A, lda, B16_or_f32, ldb, C, ldc, nullptr, out_storage);
  return gemm(st, ta, tb, M, N, K, (const float*)A, lda, (const float*)B16_or_f32, ldb, (float*)C, ldc, nullptr, 0);
}

// (hi, lo) pair of a level-1 activation (M/group, D) in the handle's own buffer (slot 0: pooled, slot 1: dh1), so that
// the two-level fp32 model never touches the library-wide GEMM scratch: a captured step keeps valid addresses
// whatever other GEMM calls the process makes later.
static pmb_status l1_split(pmb_lm* lm, cudaStream_t st, const void* src, int slot, Pair16* out) {
  const int64_t M1 = lm->d1.M; const int D = lm->d.D;
  uint16_t* hi = lm->l1_pair + (size_t)(2 * slot) * M1 * D;
  uint16_t* lo = hi + (size_t)M1 * D;
  PMB_TRY(split_pair16(st, static_cast<const float*>(src), M1, D, D, hi, lo, D));
  *out = Pair16{hi, lo, D};
  return PMB_OK;
}

extern "C" pmb_status pmb_lm_step_device(pmb_lm* lm, void* stream, const int64_t* d_ids, const int64_t* d_targets,
                                         pmb_layer_callback on_layer_done, void* user) {
  if (!lm || !d_ids || !d_targets) return fail(PMB_ERR_ARG, "lm_step: NULL argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Dims& d = lm->d;
  const int64_t M = d.M;
  const int D = d.D, V = lm->V, Vp = lm->Vp;
  float* table = lm->params + lm->off[0];
  float* dtable = lm->grads + lm->off[0];
  size_t slot = (size_t)M * D;
  const bool h16 = lm->bf16 != 0;
  const size_t esz = h16 ? 2 : 4;
  const bool hier = lm->L1 > 0;
  const int L0 = lm->L0, L1 = lm->L1;
  const uint16_t* table16 = h16 ? lm->params16 + lm->off[0] : nullptr;
  const bool prs = lm->pairs != 0;
  const Weights16* w16 = (h16 || prs) ? lm->lw16.data() : nullptr;
  // the fp32 masters may have been updated by the optimizer since the last step: refresh their pairs
  if (prs) PMB_TRY(split_pair16(st, lm->params, 1, lm->n_params, lm->n_params, lm->params_hi, lm->params_lo, lm->n_params));
  const Pair16 table_p{prs ? lm->params_hi + lm->off[0] : nullptr, prs ? lm->params_lo + lm->off[0] : nullptr, D};
  if (h16) {
    // the fp32 masters may have been updated by the optimizer since the last step
    PMB_TRY(cast_f32_bf16(st, lm->params, lm->params16, lm->n_params));
    embedding_fwd_bf16_kernel<<<(unsigned)cdiv(M * (D / 8), 256), 256, 0, st>>>(table16, d_ids, static_cast<uint16_t*>((void*)lm->saved), M, D, V, lm->bad);
  } else {
    embedding_fwd_kernel<<<(unsigned)cdiv(M * (D / 4), 256), 256, 0, st>>>(table, d_ids, lm->saved, M, D, V, lm->bad);
  }
  PMB_LAUNCHED();
  PMB_TRY(stack_fwd(st, d, L0, lm->lp.data(), w16, lm->saved, lm->ws, lm->ws_bytes));
  const char* hidden = reinterpret_cast<const char*>(lm->saved) + (size_t)L0 * slot * esz;
  const void* wproj = nullptr;
  if (hier) {
    // level 1: mean-pool groups of tokens, project, run the second stack at 1/group rate, add its output back
    // shifted by one group so that no token sees its own group's future (the two-level benchmark model's wiring)
    const int64_t M1 = lm->d1.M;
    wproj = h16 ? (const void*)(lm->params16 + lm->off_proj) : (const void*)(lm->params + lm->off_proj);
    PMB_TRY(hier_op(lm, st, hidden, nullptr, lm->pooled, 0));
    if (prs) {
      Pair16 pooled_p;
      PMB_TRY(l1_split(lm, st, lm->pooled, 0, &pooled_p));
      PMB_TRY(gemm_pairs(st, 0, 0, M1, D, D, pooled_p, Pair16{lm->params_hi + lm->off_proj, lm->params_lo + lm->off_proj, D},
                         static_cast<float*>(lm->saved1), D, nullptr));
    } else {
      PMB_TRY(lm_gemm(lm, st, 0, 0, M1, D, D, lm->pooled, D, wproj, D, lm->saved1, D, 1));
    }
    PMB_TRY(stack_fwd(st, lm->d1, L1, lm->lp.data() + L0, w16 ? w16 + L0 : nullptr, lm->saved1, lm->ws, lm->ws_bytes));
    const char* h1 = reinterpret_cast<const char*>(lm->saved1) + (size_t)L1 * M1 * D * esz;
    PMB_TRY(hier_op(lm, st, h1, hidden, lm->hsum, 1));
    hidden = reinterpret_cast<const char*>(lm->hsum);
  }
  char* dhid = reinterpret_cast<char*>(lm->dhidden);
  SideLane* table_lane = nullptr;
  if (prs) {
    static const int on = [] { const char* e = getenv("PMB_HEAD_CONCURRENT"); return (e && e[0] == '0') ? 0 : 1; }();
    if (on) PMB_TRY(get_side_lane(4, &table_lane));
  }
  for (int64_t r0 = 0; r0 < M; r0 += lm->tile_rows) {
    int64_t rows = M - r0 < lm->tile_rows ? M - r0 : lm->tile_rows;
    const void* hrows = hidden + (size_t)r0 * D * esz;
    // logits = hidden E^T   (photon/embedding.rs:54-60), kept in fp32 for the softmax
    const Pair16 hid_p{lm->hid_hi, lm->hid_lo, D};
    const Pair16 dlog_p = lm->ce_inplace ? Pair16{reinterpret_cast<uint16_t*>(lm->logits), reinterpret_cast<uint16_t*>(lm->logits) + Vp, 2 * (int64_t)Vp}
                                         : Pair16{lm->dlog_hi, lm->dlog_lo, Vp};
    if (h16) PMB_TRY(gemm_bf16(st, 0, 1, rows, V, D, hrows, D, table16, D, lm->logits, Vp, nullptr, 0));
    else if (prs) {
      PMB_TRY(split_pair16(st, static_cast<const float*>(hrows), rows, D, D, lm->hid_hi, lm->hid_lo, D));
      PMB_TRY(gemm_pairs(st, 0, 1, rows, V, D, hid_p, table_p, lm->logits, Vp, nullptr));
    }
    else PMB_TRY(gemm(st, 0, 1, rows, V, D, static_cast<const float*>(hrows), D, table, D, lm->logits, Vp, nullptr, 0));
    { ProfScope prof(st, "cross_entropy", 0.0, 4.0 * rows * 3.0 * V);
    if ((prs || h16) && lm->ce_inplace) {
      PMB_SMEM_OPT_IN(CE_MAX_SMEM, cross_entropy_pair_inplace_kernel);
      cross_entropy_pair_inplace_kernel<<<(unsigned)rows, CE_THREADS, (size_t)V * 4, st>>>(lm->logits, Vp, V, d_targets + r0, lm->row_loss + r0, 1.0f / (float)M, prs ? 1 : 0, lm->bad);
    } else
      cross_entropy_kernel<<<(unsigned)rows, 256, 0, st>>>(lm->logits, Vp, V, d_targets + r0, lm->row_loss + r0, 1.0f / (float)M,
                                                           prs ? lm->dlog_hi : nullptr, prs ? lm->dlog_lo : nullptr, lm->bad);
    PMB_LAUNCHED(); }
    // dhidden = dlogits E ;  dE (+)= dlogits^T hidden
    if (h16) {
      // in place: the bf16 gradient sits at the start of each logits row (pitch 2*Vp bf16 elements)
      const uint16_t* dl16 = lm->ce_inplace ? reinterpret_cast<const uint16_t*>(lm->logits) : lm->dlogits16;
      const int64_t ldl = lm->ce_inplace ? 2 * (int64_t)Vp : Vp;
      if (!lm->ce_inplace) PMB_TRY(cast_f32_bf16(st, lm->logits, lm->dlogits16, rows * Vp));
      PMB_TRY(gemm_bf16(st, 0, 0, rows, D, V, dl16, ldl, table16, D, dhid + (size_t)r0 * D * 2, D, nullptr, 1));
      PMB_TRY(gemm_bf16(st, 1, 0, V, D, rows, dl16, ldl, hrows, D, dtable, D, r0 == 0 ? nullptr : dtable, 0));
    } else if (prs && table_lane) {
      // only dhidden is needed now; the embedding-table gradient runs on its own stream (next to the first blocks of
      // the stack backward for the last row tile) and is joined before the embedding scatter.  With several row tiles
      // the next tile's logits overwrite the buffer this tile's dE still reads, so the caller's stream waits for the
      // lane before each further tile (below).
      // dhidden has 16 x 6 tiles and K = vocab: split K three ways (one launch, three products into three slabs)
      // so that the product the whole backward waits for uses the machine, then add the slabs
      {
        PairGemm parts[HEAD_SPLITK];
        const int64_t kstep = (int64_t)align_up((size_t)cdiv(V, HEAD_SPLITK), 64);
        int np = 0;
        for (int64_t k0 = 0; k0 < V && np < HEAD_SPLITK; k0 += kstep, ++np) {
          const int64_t kk = V - k0 < kstep ? V - k0 : kstep;
          parts[np] = PairGemm{0, 0, rows, D, kk, Pair16{dlog_p.hi + k0, dlog_p.lo + k0, dlog_p.ld},
                               Pair16{table_p.hi + k0 * D, table_p.lo + k0 * D, table_p.ld}, lm->dh_part + (size_t)np * rows * D, D, nullptr};
        }
        PMB_TRY(gemm_pairs_group(st, parts, np));
        ProfScope prof(st, "head_splitk_sum", 0.0, 4.0 * (np + 1) * rows * D);
        sum_slabs_kernel<<<(unsigned)cdiv(rows * D / 4, 256), 256, 0, st>>>(lm->dh_part, np, rows * D, lm->dhidden + r0 * D);
        PMB_LAUNCHED();
      }
      PMB_TRY(order_after(st, table_lane->ev[0], table_lane->s));
      PMB_TRY(gemm_pairs(table_lane->s, 1, 0, V, D, rows, dlog_p, hid_p, dtable, D, r0 == 0 ? nullptr : dtable));
      if (r0 + rows < M) PMB_TRY(order_after(table_lane->s, table_lane->ev[2], st));   // the tile buffers are reused next
    } else if (prs) {
      // one launch: the few long-K tiles of dhidden first, the many short tiles of dE fill the other SMs
      const PairGemm both[2] = {{0, 0, rows, D, V, dlog_p, table_p, lm->dhidden + r0 * D, D, nullptr},
                                {1, 0, V, D, rows, dlog_p, hid_p, dtable, D, r0 == 0 ? nullptr : dtable}};
      PMB_TRY(gemm_pairs_group(st, both, 2));
    } else {
      PMB_TRY(gemm(st, 0, 0, rows, D, V, lm->logits, Vp, table, D, lm->dhidden + r0 * D, D, nullptr, 0));
      PMB_TRY(gemm(st, 1, 0, V, D, rows, lm->logits, Vp, static_cast<const float*>(hrows), D, dtable, D, r0 == 0 ? nullptr : dtable, 0));
    }
  }
  mean_kernel<<<1, 256, 0, st>>>(lm->row_loss, M, lm->loss);
  PMB_LAUNCHED();
  if (hier) {
    const int64_t M1 = lm->d1.M;
    // adjoint of the shifted repeat, level-1 backward, projection gradients, adjoint of the pooling
    PMB_TRY(hier_op(lm, st, lm->dhidden, nullptr, lm->dh1, 2));
    struct Shift { pmb_layer_callback cb; void* user; int base; } sh{on_layer_done, user, L0};
    auto shifted = [](int32_t layer, void* u) { Shift* s = static_cast<Shift*>(u); if (s->cb) s->cb(layer + s->base, s->user); };
    PMB_TRY(stack_bwd(st, lm->d1, L1, lm->lp.data() + L0, w16 ? w16 + L0 : nullptr, lm->lg.data() + L0, lm->saved1, lm->dh1, lm->ws,
                      lm->ws_bytes, on_layer_done ? +shifted : nullptr, &sh));
    float* dproj = lm->grads + lm->off_proj;
    // dW_proj = pooled^T du (fp32) ;  dpool = du W_proj^T
    if (h16) {
      PMB_TRY(gemm_bf16(st, 1, 0, D, D, M1, lm->pooled, D, lm->dh1, D, dproj, D, nullptr, 0));
      PMB_TRY(gemm_bf16(st, 0, 1, M1, D, D, lm->dh1, D, wproj, D, lm->dpool, D, nullptr, 1));
    } else if (prs) {
      Pair16 pooled_p, dh1_p;
      PMB_TRY(l1_split(lm, st, lm->pooled, 0, &pooled_p));
      PMB_TRY(l1_split(lm, st, lm->dh1, 1, &dh1_p));
      PMB_TRY(gemm_pairs(st, 1, 0, D, D, M1, pooled_p, dh1_p, dproj, D, nullptr));
      PMB_TRY(gemm_pairs(st, 0, 1, M1, D, D, dh1_p, Pair16{lm->params_hi + lm->off_proj, lm->params_lo + lm->off_proj, D},
                         static_cast<float*>(lm->dpool), D, nullptr));
    } else {
      PMB_TRY(gemm(st, 1, 0, D, D, M1, (const float*)lm->pooled, D, (const float*)lm->dh1, D, dproj, D, nullptr, 0));
      PMB_TRY(gemm(st, 0, 1, M1, D, D, (const float*)lm->dh1, D, (const float*)wproj, D, (float*)lm->dpool, D, nullptr, 0));
    }
    PMB_TRY(hier_op(lm, st, lm->dpool, lm->dhidden, lm->dhidden, 3));
  }
  // the head's share of the table gradient is complete (on the lane that formed it): a data-parallel step starts its
  // all-reduce now, next to the whole stack backward
  if (lm->split_table && on_layer_done) { lm->table_stream = table_lane ? table_lane->s : st; on_layer_done(-2, user); }
  PMB_TRY(stack_bwd(st, d, L0, lm->lp.data(), w16, lm->lg.data(), lm->saved, lm->dhidden, lm->ws, lm->ws_bytes, on_layer_done, user));
  if (table_lane) PMB_TRY(order_after(table_lane->s, table_lane->ev[1], st));
  if (!lm->split_table) {      // (otherwise the callback below scatter-adds the rows of every rank)
    if (h16) embedding_bwd_bf16_kernel<<<(unsigned)cdiv(M * D, 256), 256, 0, st>>>(dtable, d_ids, reinterpret_cast<const uint16_t*>(lm->dhidden), M, D, V);
    else embedding_bwd_kernel<<<(unsigned)cdiv(M * D, 256), 256, 0, st>>>(dtable, d_ids, lm->dhidden, M, D, V, 1.0f);
    PMB_LAUNCHED();
  }
  if (on_layer_done) on_layer_done(-1, user);
  return PMB_OK;
}

// ---- data-parallel step: the same step with each layer's gradient bucket all-reduced (averaged) over the
// communicator as soon as that layer's gradient kernels are enqueued, the embedding (and projection) bucket last.
struct DpStep { pmb_lm* lm; pmb_dp* dp; void* stream; pmb_status status; const int64_t* ids; };

static void dp_layer_done(int32_t layer, void* user) {
  DpStep* c = static_cast<DpStep*>(user);
  if (c->status != PMB_OK) return;
  pmb_lm* lm = c->lm;
  auto reduce = [&](int64_t a, int64_t b) { if (b > a && c->status == PMB_OK) c->status = pmb_dp_allreduce_async(c->dp, c->stream, lm->grads + a, b - a); };
  if (layer >= 0) {
    // the layer's 8 tensors are contiguous; the bucket ends where the next item of the flat buffer starts
    const int64_t a = lm->off[1 + 8 * layer];
    int64_t b = lm->n_params;
    if (layer + 1 < lm->L) b = lm->off[1 + 8 * (layer + 1)];
    if (lm->off_proj >= a && lm->off_proj < b) b = lm->off_proj;    // the projection sits between the two stacks
    reduce(a, b);
  } else if (layer == -2) {
    // the tied head's share of the embedding gradient, ordered after the stream that formed it
    if (c->status == PMB_OK) c->status = pmb_dp_allreduce_async(c->dp, lm->table_stream, lm->grads + lm->off[0], lm->off[1] - lm->off[0]);
  } else {
    if (lm->off_proj >= 0) reduce(lm->off_proj, lm->off_proj + (int64_t)align_up((size_t)lm->d.D * lm->d.D, 64));
    if (!lm->split_table) { reduce(lm->off[0], lm->off[1]); return; }
    // token-lookup share: every rank's (M, D) rows of dhidden and its M ids, gathered, then added by every rank
    // with weight 1 / world_size onto the averaged head share
    if (c->status != PMB_OK) return;
    cudaStream_t st = static_cast<cudaStream_t>(c->stream);
    const int64_t M = lm->d.M; const int D = lm->d.D;
    const int n = pmb_dp_world_size(c->dp);
    const size_t row_bytes = (size_t)M * D * sizeof(float), id_bytes = (size_t)M * sizeof(int64_t);
    char* rows_all = lm->gather; char* ids_all = lm->gather + (size_t)n * row_bytes;
    c->status = pmb_dp_allgather_async(c->dp, st, lm->dhidden, rows_all, (int64_t)row_bytes);
    if (c->status == PMB_OK) c->status = pmb_dp_allgather_async(c->dp, st, c->ids, ids_all, (int64_t)id_bytes);
    if (c->status == PMB_OK) c->status = pmb_dp_sync(c->dp, st);     // (also: the head share's all-reduce has finished)
    if (c->status != PMB_OK) return;
    embedding_bwd_kernel<<<(unsigned)cdiv((int64_t)n * M * D, 256), 256, 0, st>>>(lm->grads + lm->off[0], reinterpret_cast<const int64_t*>(ids_all),
                                                                                 reinterpret_cast<const float*>(rows_all), (int64_t)n * M, D, lm->V, 1.0f / (float)n);
    if (cudaGetLastError() != cudaSuccess) c->status = fail(PMB_ERR_CUDA, "embedding scatter launch failed");
  }
}

extern "C" pmb_status pmb_lm_step_device_dp(pmb_lm* lm, void* stream, const int64_t* d_ids, const int64_t* d_targets, pmb_dp* dp) {
  if (!dp) return fail(PMB_ERR_ARG, "lm_step_device_dp: NULL communicator");
  if (!lm) return fail(PMB_ERR_ARG, "lm_step_device_dp: NULL handle");
  DpStep c{lm, dp, stream, PMB_OK, d_ids};
  const int n = pmb_dp_world_size(dp);
  // the row exchange of the embedding gradient: fp32 storage, more than one rank
  lm->split_table = (n > 1 && !lm->bf16) ? 1 : 0;
  if (lm->split_table) {
    const size_t need = (size_t)n * ((size_t)lm->d.M * lm->d.D * sizeof(float) + (size_t)lm->d.M * sizeof(int64_t));
    if (lm->gather_bytes < need) {     // first data-parallel step (make it outside stream capture)
      cudaFree(lm->gather); lm->gather = nullptr; lm->gather_bytes = 0;
      if (cudaMalloc(&lm->gather, need) != cudaSuccess) { lm->split_table = 0; return fail(PMB_ERR_CUDA, "lm_step_device_dp: cannot allocate the gather buffer"); }
      lm->gather_bytes = need;
    }
  }
  pmb_status s = pmb_lm_step_device(lm, stream, d_ids, d_targets, dp_layer_done, &c);
  lm->split_table = 0;
  PMB_TRY(s);
  PMB_TRY(c.status);
  return pmb_dp_sync(dp, stream);
}

// ---- weights checkpoint I/O (crates/pm-train/src/checkpoint.rs:25-97): parameters by position, "p_0000"...
namespace pmb {
pmb_status safetensors_save_f32(const char* path, int n, const int64_t* shapes, const int32_t* ranks, const float* const* data);
pmb_status safetensors_load_f32(const char* path, int n, const int64_t* shapes, const int32_t* ranks, float* const* data);
}

// tensors of the handle in `append_params` order: offsets into the flat buffer, shapes, ranks
static void lm_tensor_table(const pmb_lm* lm, std::vector<int64_t>* offs, std::vector<int64_t>* shapes, std::vector<int32_t>* ranks) {
  const Dims& d = lm->d;
  auto add = [&](int64_t off, std::initializer_list<int64_t> sh) {
    offs->push_back(off); ranks->push_back((int32_t)sh.size());
    for (int64_t x : sh) shapes->push_back(x);
  };
  add(lm->off[0], {lm->V, d.D});
  for (int l = 0; l < lm->L; ++l) {
    if (lm->L1 > 0 && l == lm->L0) add(lm->off_proj, {d.D, d.D});
    const int64_t* f = &lm->off[1 + 8 * l];
    add(f[0], {d.D, d.J}); add(f[1], {d.X, 1, d.K}); add(f[2], {d.X}); add(f[3], {d.H}); add(f[4], {d.H}); add(f[5], {d.H});
    add(f[6], {d.I}); add(f[7], {d.I, d.D});
  }
}

extern "C" pmb_status pmb_lm_save_safetensors(pmb_lm* lm, void* stream, const char* path) {
  if (!lm || !path) return fail(PMB_ERR_ARG, "lm_save: NULL argument");
  std::vector<int64_t> offs, shapes; std::vector<int32_t> ranks;
  lm_tensor_table(lm, &offs, &shapes, &ranks);
  std::vector<float> host((size_t)lm->n_params);
  PMB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  PMB_CUDA(cudaMemcpy(host.data(), lm->params, host.size() * 4, cudaMemcpyDeviceToHost));
  std::vector<const float*> ptrs;
  for (int64_t o : offs) ptrs.push_back(host.data() + o);
  return safetensors_save_f32(path, (int)offs.size(), shapes.data(), ranks.data(), ptrs.data());
}

extern "C" pmb_status pmb_lm_load_safetensors(pmb_lm* lm, void* stream, const char* path) {
  if (!lm || !path) return fail(PMB_ERR_ARG, "lm_load: NULL argument");
  std::vector<int64_t> offs, shapes; std::vector<int32_t> ranks;
  lm_tensor_table(lm, &offs, &shapes, &ranks);
  std::vector<float> host((size_t)lm->n_params, 0.0f);
  std::vector<float*> ptrs;
  for (int64_t o : offs) ptrs.push_back(host.data() + o);
  PMB_TRY(safetensors_load_f32(path, (int)offs.size(), shapes.data(), ranks.data(), ptrs.data()));   // nothing is touched on error
  PMB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  PMB_CUDA(cudaMemcpy(lm->params, host.data(), host.size() * 4, cudaMemcpyHostToDevice));
  return PMB_OK;
}

extern "C" pmb_status pmb_lm_step_host(pmb_lm* lm, void* stream, const int64_t* h_ids, const int64_t* h_targets,
                                       float* h_loss, pmb_layer_callback on_layer_done, void* user) {
  if (!lm || !h_ids || !h_targets || !h_loss) return fail(PMB_ERR_ARG, "lm_step_host: NULL argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  size_t bytes = (size_t)lm->d.M * sizeof(int64_t);
  PMB_CUDA(cudaMemcpyAsync(lm->ids, h_ids, bytes, cudaMemcpyHostToDevice, st));
  PMB_CUDA(cudaMemcpyAsync(lm->targets, h_targets, bytes, cudaMemcpyHostToDevice, st));
  PMB_TRY(pmb_lm_step_device(lm, stream, lm->ids, lm->targets, on_layer_done, user));
  PMB_CUDA(cudaMemcpyAsync(h_loss, lm->loss, sizeof(float), cudaMemcpyDeviceToHost, st));
  PMB_CUDA(cudaStreamSynchronize(st));
  unsigned int bad = 0;
  PMB_CUDA(cudaMemcpy(&bad, lm->bad, sizeof(bad), cudaMemcpyDeviceToHost));
  if (bad) {
    cudaMemset(lm->bad, 0, sizeof(bad));
    return fail(PMB_ERR_ARG, "lm_step_host: %s outside [0, vocab)", (bad & 1u) ? ((bad & 2u) ? "token ids and targets were" : "a token id was") : "a target was");
  }
  return PMB_OK;
}
