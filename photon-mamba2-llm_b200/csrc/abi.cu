// C ABI entry points for the individual kernels, library-wide state, and the GEMM engine dispatch.
#include <cstdio>
#include <cstdlib>
#include <initializer_list>
#include "common.cuh"
#include "kernels.h"
#include "ssd_tc.h"
#include "ssd_fused.h"

namespace pmb {

thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};
bool g_prof_on = false;
std::vector<ProfRec> g_prof;

pmb_status gemm(cudaStream_t st, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda,
                const float* B, int64_t ldb, float* C, int64_t ldc, const float* R, int engine) {
  if (!A || !B || !C) return fail(PMB_ERR_ARG, "gemm: NULL operand");
  // PMB_GEMM_ENGINE=simt routes engine-0 ("auto") calls to the fp32 FMA kernel: a debugging aid for
  // telling a tensor-core problem from a problem elsewhere.  Explicit engine requests are honoured as given.
  static const int forced = [] { const char* e = getenv("PMB_GEMM_ENGINE"); return (e && strcmp(e, "simt") == 0) ? 1 : 0; }();
  if (engine == 0 && forced) engine = 1;
  if (engine == 1) return gemm_simt(st, ta, tb, M, N, K, A, lda, B, ldb, C, ldc, R);
  // engine 4, and "auto" unless PMB_GEMM_ENGINE=tf32: split both operands into bf16 pairs and use the kind::f16 kernel
  static const int no_x2 = [] { const char* e = getenv("PMB_GEMM_ENGINE"); return (e && strcmp(e, "tf32") == 0) ? 1 : 0; }();
  if (engine == 4 || engine == 5 || engine == 6 || (engine == 0 && !no_x2)) {
    // (the split pass compacts rows to a pitch that meets TMA's 16-byte rules, so every fp32 operand qualifies)
    return gemm_f32_via_bf16x2(st, ta, tb, M, N, K, A, lda, B, ldb, C, ldc, R, engine == 4 ? 0 : engine == 5 ? 2 : engine == 6 ? 1 : -1);
  }
  bool ok = gemm_tc_supported(ta, tb, M, N, K, A, lda, B, ldb, C, ldc);
  if ((engine == 2 || engine == 3) && !ok) return fail(PMB_ERR_UNSUPPORTED, "gemm: tcgen05 engine needs 16-byte aligned operands and leading dimensions");
  if (ok) {
    // The 128x64 / two-CTAs-per-SM variant (engine 3, or problems with fewer 128x128 tiles than PMB_GEMM_SMALL_TILES)
    // measured slower than the 128x128 kernel on every GEMM of the LM step (the loop is bound by shared-memory
    // traffic, not by per-tile latency), so it is off by default.
    static const int small_env = [] { const char* e = getenv("PMB_GEMM_SMALL_TILES"); return e ? atoi(e) : 0; }();
    const int64_t tiles = cdiv(M, 128) * cdiv(N, 128);
    if (engine == 3 || (engine == 0 && tiles < small_env)) return gemm_tc_small(st, ta, tb, M, N, K, A, lda, B, ldb, C, ldc, R);
    return gemm_tc(st, ta, tb, M, N, K, A, lda, B, ldb, C, ldc, R);
  }
  return gemm_simt(st, ta, tb, M, N, K, A, lda, B, ldb, C, ldc, R);
}

static SideLane g_lanes[64][7];
static int g_lanes_enabled = 1;   // pmb_set_concurrency(0): every caller gets no lane and runs its chains on the one stream

pmb_status get_side_lane(int idx, SideLane** out) {
  *out = nullptr;
  if (!g_lanes_enabled) return PMB_OK;
  int dev = 0;
  PMB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || idx < 0 || idx >= 7) return PMB_OK;
  SideLane& l = g_lanes[dev][idx];
  if (!l.s) {
    // lanes that carry the critical chain of the stack backward (6: gradient kernels of the current block, 0: the
    // scan backward's second chain, 5: its dB branch) get the highest stream priority, so that their CTAs are placed ahead of the
    // recompute-ahead and the deferred GEMMs whenever an SM frees up
    int least = 0, greatest = 0;
    PMB_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    PMB_CUDA(cudaStreamCreateWithPriority(&l.s, cudaStreamNonBlocking, (idx == 0 || idx == 5 || idx == 6) ? greatest : least));
    for (int i = 0; i < 6; ++i) PMB_CUDA(cudaEventCreateWithFlags(&l.ev[i], cudaEventDisableTiming));
  }
  *out = &l;
  return PMB_OK;
}

void set_lanes_enabled(int on) { g_lanes_enabled = on ? 1 : 0; }

pmb_status order_after(cudaStream_t from, cudaEvent_t ev, cudaStream_t to) {
  PMB_CUDA(cudaEventRecord(ev, from));
  PMB_CUDA(cudaStreamWaitEvent(to, ev, 0));
  return PMB_OK;
}

}  // namespace pmb

using namespace pmb;

extern "C" const char* pmb_last_error(void) { return g_err; }
extern "C" const char* pmb_version(void) { return "pm_b200 0.1 sm_100a"; }
extern "C" int64_t pmb_launch_count(void) { return (int64_t)g_launches.load(); }

extern "C" void pmb_profile_start(void) {
  for (auto& r : g_prof) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
  g_prof.clear();
  g_prof_on = true;
}

// Writes a JSON array [{"name":..,"launches":..,"ms":..,"flops":..,"bytes":..},...] (totals per scope name).
extern "C" pmb_status pmb_profile_stop(char* h_json, size_t capacity) {
  g_prof_on = false;
  PMB_CUDA(cudaDeviceSynchronize());
  struct Agg { const char* name; long n; double ms, flops, bytes; };
  std::vector<Agg> agg;
  // PMB_PROFILE_TIMELINE=<file>: also write "name,start_ms,end_ms" per scope, relative to the first scope's start,
  // so that overlap between the internal streams can be read off
  if (const char* tl = getenv("PMB_PROFILE_TIMELINE")) {
    if (FILE* f = g_prof.empty() ? nullptr : fopen(tl, "w")) {
      for (auto& r : g_prof) {
        float t0 = 0.0f, t1 = 0.0f;
        cudaEventElapsedTime(&t0, g_prof[0].e0, r.e0);
        cudaEventElapsedTime(&t1, g_prof[0].e0, r.e1);
        fprintf(f, "%s,%.4f,%.4f\n", r.name, t0, t1);
      }
      fclose(f);
    }
  }
  for (auto& r : g_prof) {
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, r.e0, r.e1);
    cudaEventDestroy(r.e0); cudaEventDestroy(r.e1);
    size_t i = 0;
    for (; i < agg.size(); ++i) if (strcmp(agg[i].name, r.name) == 0) break;
    if (i == agg.size()) agg.push_back(Agg{r.name, 0, 0, 0, 0});
    agg[i].n += 1; agg[i].ms += ms; agg[i].flops += r.flops; agg[i].bytes += r.bytes;
  }
  g_prof.clear();
  if (!h_json || capacity < 3) return fail(PMB_ERR_ARG, "profile_stop: buffer too small");
  size_t off = 0;
  off += snprintf(h_json + off, capacity - off, "[");
  for (size_t i = 0; i < agg.size() && off + 256 < capacity; ++i)
    off += snprintf(h_json + off, capacity - off, "%s{\"name\":\"%s\",\"launches\":%ld,\"ms\":%.6f,\"flops\":%.6e,\"bytes\":%.6e}",
                    i ? "," : "", agg[i].name, agg[i].n, agg[i].ms, agg[i].flops, agg[i].bytes);
  snprintf(h_json + off, capacity - off, "]");
  return PMB_OK;
}

extern "C" void pmb_set_concurrency(int32_t on) { pmb::set_lanes_enabled(on); }

extern "C" pmb_status pmb_device_status(int32_t* h_word_out) {
  unsigned int w = 0, w2 = 0;
  PMB_TRY(read_clear_device_status(&w));
  PMB_TRY(read_clear_device_status_ssd(&w2));
  w |= w2 << 8;
  PMB_TRY(read_clear_device_status_bf16(&w2));
  w |= w2 << 16;
  PMB_TRY(read_clear_device_status_small(&w2));
  w |= w2 << 24;
  PMB_TRY(read_clear_device_status_fused(&w2));   // shares the scan kernels' byte
  w |= (w2 & 0x7fu) << 8;
  PMB_TRY(read_clear_device_status_pairs(&w2));
  w |= (w2 & 0x7fu) << 8;
  if (h_word_out) *h_word_out = (int32_t)w;
  return PMB_OK;
}

namespace pmb { pmb_status bounded_wait_selftest(cudaStream_t st, uint32_t polls); }

extern "C" pmb_status pmb_selftest_bounded_wait(void* stream, uint32_t polls) {
  if (polls == 0 || polls > (1u << 20)) return fail(PMB_ERR_ARG, "selftest_bounded_wait: polls must be in 1..2^20");
  return bounded_wait_selftest(static_cast<cudaStream_t>(stream), polls);
}

extern "C" int32_t pmb_selftest_device_once(void) {
  DeviceOnce f;
  int bad = 0;
  for (int d : {0, 1, PMB_MAX_DEVICES - 1}) {
    if (!f.pending(d)) ++bad;          // every ordinal starts pending
    f.mark(d);
    if (f.pending(d)) ++bad;           // and is done after its own mark
  }
  if (!f.pending(2)) ++bad;            // marking one ordinal leaves the others pending
  if (!f.pending(-1) || !f.pending(PMB_MAX_DEVICES)) ++bad;   // ordinals outside the table are never skipped
  f.mark(PMB_MAX_DEVICES);             // ... and marking them is a no-op, not an out-of-bounds write
  if (!f.pending(PMB_MAX_DEVICES)) ++bad;
  return bad;
}

extern "C" pmb_status pmb_gemm_f32(void* stream, int32_t trans_a, int32_t trans_b, int64_t M, int64_t N, int64_t K,
                                   const float* d_A, int64_t lda, const float* d_B, int64_t ldb,
                                   float* d_C, int64_t ldc, const float* d_R, int32_t engine) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(PMB_ERR_SHAPE, "gemm: M, N, K must be positive (got %lld, %lld, %lld)", (long long)M, (long long)N, (long long)K);
  if (lda < (trans_a ? M : K) || ldb < (trans_b ? K : N) || ldc < N) return fail(PMB_ERR_SHAPE, "gemm: leading dimension smaller than the row length");
  if (engine < 0 || engine > 6) return fail(PMB_ERR_ARG, "gemm: engine must be 0..6");
  return gemm(static_cast<cudaStream_t>(stream), trans_a != 0, trans_b != 0, M, N, K, d_A, lda, d_B, ldb, d_C, ldc, d_R, engine);
}

extern "C" pmb_status pmb_conv_silu_dt_fwd(void* stream, const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen,
                                           const float* d_xzd, const float* d_conv_w, const float* d_conv_b,
                                           const float* d_dt_bias, float* d_act, float* d_dt) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  if (!d_xzd || !d_conv_w || !d_act || (d_dt && !d_dt_bias)) return fail(PMB_ERR_ARG, "conv_silu_dt_fwd: NULL argument");
  return conv_silu_dt_fwd(static_cast<cudaStream_t>(stream), d, d_xzd, d_conv_w, d_conv_b, d_dt_bias, d_act, d_dt);
}

extern "C" size_t pmb_conv_bwd_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen) {
  Dims d;
  if (make_dims(cfg, batch, seqlen, &d) != PMB_OK) return 0;
  return conv_bwd_ws_bytes(d);
}

extern "C" pmb_status pmb_conv_silu_bwd(void* stream, const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen,
                                        const float* d_xzd, const float* d_conv_w, const float* d_conv_b,
                                        const float* d_dact, float* d_dxzd, float* d_dconv_w, float* d_dconv_b,
                                        void* d_ws, size_t ws_bytes) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  if (!d_xzd || !d_conv_w || !d_dact || !d_dxzd || !d_dconv_w || !d_dconv_b || !d_ws) return fail(PMB_ERR_ARG, "conv_silu_bwd: NULL argument");
  return conv_silu_bwd(static_cast<cudaStream_t>(stream), d, d_xzd, d_conv_w, d_conv_b, d_dact, d_dxzd, d_dconv_w, d_dconv_b, d_ws, ws_bytes);
}

static pmb_status ssd_check(int32_t batch, int32_t seqlen, int32_t H, int32_t P, int32_t N, int32_t G, int32_t Q) {
  if (batch <= 0 || seqlen <= 0 || H <= 0 || P <= 0 || N <= 0) return fail(PMB_ERR_SHAPE, "ssd: non-positive dimension");
  if (!(G == 1 || G == H)) return fail(PMB_ERR_SHAPE, "ssd: n_groups must be 1 or n_heads");
  if (Q <= 0 || seqlen % Q != 0) return fail(PMB_ERR_SHAPE, "ssd: seqlen %d is not a multiple of block_len %d", seqlen, Q);
  return PMB_OK;
}

extern "C" size_t pmb_ssd_workspace_bytes(int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                          int32_t d_state, int32_t n_groups, int32_t block_len) {
  if (ssd_check(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len) != PMB_OK) return 0;
  return ssd_ws_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, nullptr, 0, nullptr);
}

extern "C" pmb_status pmb_ssd_scan_fwd(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                       int32_t d_state, int32_t n_groups, int32_t block_len,
                                       const float* d_x, int64_t ldx, const float* d_a,
                                       const float* d_b, const float* d_c, int64_t ldbc,
                                       const float* d_init_state, float* d_y, int64_t ldy, float* d_final_state,
                                       void* d_ws, size_t ws_bytes) {
  PMB_TRY(ssd_check(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len));
  if (!d_x || !d_a || !d_b || !d_c || !d_y || !d_ws) return fail(PMB_ERR_ARG, "ssd_scan_fwd: NULL argument");
  if (ldx < (int64_t)n_heads * d_head || ldy < (int64_t)n_heads * d_head || ldbc < (int64_t)n_groups * d_state)
    return fail(PMB_ERR_SHAPE, "ssd_scan_fwd: token stride smaller than the row length");
  SsdWs ws;
  if (ssd_ws_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_ws, ws_bytes, &ws) == 0)
    return fail(PMB_ERR_WORKSPACE, "ssd workspace too small");
  SsdIn in{};
  in.B = batch; in.T = seqlen; in.H = n_heads; in.P = d_head; in.N = d_state; in.G = n_groups; in.Q = block_len;
  in.x = d_x; in.ldx = ldx; in.a = d_a; in.b = d_b; in.c = d_c; in.ldbc = ldbc;
  return ssd_fwd(static_cast<cudaStream_t>(stream), in, d_init_state, d_y, ldy, d_final_state, ws);
}

extern "C" pmb_status pmb_ssd_scan_bwd(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                       int32_t d_state, int32_t n_groups, int32_t block_len,
                                       const float* d_x, int64_t ldx, const float* d_a,
                                       const float* d_b, const float* d_c, int64_t ldbc,
                                       const float* d_y, int64_t ldy, const float* d_dy, int64_t lddy,
                                       float* d_dx, int64_t lddx, float* d_da, float* d_db, float* d_dc, int64_t lddbc,
                                       void* d_ws, size_t ws_bytes) {
  PMB_TRY(ssd_check(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len));
  if (!d_x || !d_a || !d_b || !d_c || !d_y || !d_dy || !d_dx || !d_da || !d_db || !d_dc || !d_ws)
    return fail(PMB_ERR_ARG, "ssd_scan_bwd: NULL argument");
  SsdWs ws;
  if (ssd_ws_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_ws, ws_bytes, &ws) == 0)
    return fail(PMB_ERR_WORKSPACE, "ssd workspace too small");
  SsdIn in{};
  in.B = batch; in.T = seqlen; in.H = n_heads; in.P = d_head; in.N = d_state; in.G = n_groups; in.Q = block_len;
  in.x = d_x; in.ldx = ldx; in.a = d_a; in.b = d_b; in.c = d_c; in.ldbc = ldbc;
  SsdGrads g{};
  g.dx = d_dx; g.lddx = lddx; g.db = d_db; g.dc = d_dc; g.lddbc = lddbc; g.da = d_da;
  return ssd_bwd(static_cast<cudaStream_t>(stream), in, d_y, ldy, d_dy, lddy, g, ws);
}

extern "C" pmb_status pmb_gated_rmsnorm_fwd(void* stream, int64_t rows, int32_t width, float eps,
                                            const float* d_y, const float* d_z, int64_t ldz, const float* d_w,
                                            float* d_out, float* d_rstd) {
  if (rows <= 0 || width <= 0 || ldz < width) return fail(PMB_ERR_SHAPE, "gated_rmsnorm_fwd: bad shape");
  if (!d_y || !d_z || !d_w || !d_out) return fail(PMB_ERR_ARG, "gated_rmsnorm_fwd: NULL argument");
  return gated_rmsnorm_fwd(static_cast<cudaStream_t>(stream), rows, width, eps, d_y, d_z, ldz, d_w, d_out, d_rstd);
}

extern "C" size_t pmb_gated_rmsnorm_bwd_workspace_bytes(int64_t rows, int32_t width) {
  if (rows <= 0 || width <= 0) return 0;
  return gated_rmsnorm_bwd_ws_bytes(rows, width);
}

extern "C" pmb_status pmb_gated_rmsnorm_bwd(void* stream, int64_t rows, int32_t width,
                                            const float* d_dout, const float* d_y, const float* d_z, int64_t ldz,
                                            const float* d_w, const float* d_rstd,
                                            float* d_dy, float* d_dz, int64_t lddz, float* d_dw,
                                            void* d_ws, size_t ws_bytes) {
  if (rows <= 0 || width <= 0 || ldz < width || lddz < width) return fail(PMB_ERR_SHAPE, "gated_rmsnorm_bwd: bad shape");
  if (!d_dout || !d_y || !d_z || !d_w || !d_rstd || !d_dy || !d_dz || !d_dw || !d_ws) return fail(PMB_ERR_ARG, "gated_rmsnorm_bwd: NULL argument");
  return gated_rmsnorm_bwd(static_cast<cudaStream_t>(stream), rows, width, d_dout, d_y, d_z, ldz, d_w, d_rstd, d_dy, d_dz, lddz, d_dw, d_ws, ws_bytes);
}

// ---- scan with bf16 inputs / fp32 state (x, B, C, y and their gradients bf16; a, da and the states fp32).
// The operands are widened into a staging area at the end of the workspace and the fp32 (3xTF32) path runs on them.
namespace pmb {
__global__ void cast_bf16_f32_kernel(const uint16_t* __restrict__ src, float* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __uint_as_float((uint32_t)src[i] << 16);
}
static pmb_status widen(cudaStream_t st, const uint16_t* src, float* dst, int64_t n) {
  ProfScope prof(st, "cast_bf16_f32", 0.0, 6.0 * n);
  cast_bf16_f32_kernel<<<(unsigned)cdiv(n, 256), 256, 0, st>>>(src, dst, n);
  PMB_LAUNCHED();
  return PMB_OK;
}
struct Bf16Stage { float *x, *b, *c, *y, *dy, *dx, *db, *dc; };
static size_t bf16_stage_layout(int B, int T, int H, int P, int N, int G, int Q, void* base, size_t bytes, SsdWs* ws, Bf16Stage* sg) {
  size_t core = ssd_ws_layout(B, T, H, P, N, G, Q, nullptr, 0, nullptr);
  if (base && ssd_ws_layout(B, T, H, P, N, G, Q, base, bytes, ws) == 0) return 0;
  Arena ar(base ? static_cast<char*>(base) + core : nullptr, base ? (bytes > core ? bytes - core : 0) : 0);
  size_t hp = (size_t)B * T * H * P, gn = (size_t)B * T * G * N;
  Bf16Stage s;
  s.x = ar.take<float>(hp); s.b = ar.take<float>(gn); s.c = ar.take<float>(gn); s.y = ar.take<float>(hp);
  s.dy = ar.take<float>(hp); s.dx = ar.take<float>(hp); s.db = ar.take<float>(gn); s.dc = ar.take<float>(gn);
  if (sg) *sg = s;
  return ar.ok ? core + ar.used() : 0;
}
}  // namespace pmb

extern "C" size_t pmb_ssd_workspace_bytes_bf16(int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                               int32_t d_state, int32_t n_groups, int32_t block_len) {
  if (ssd_check(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len) != PMB_OK) return 0;
  if (ssd16_supported(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len))
    return ssd16_ws_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, nullptr, 0, nullptr, nullptr, nullptr);
  return bf16_stage_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, nullptr, 0, nullptr, nullptr);
}

extern "C" pmb_status pmb_ssd_scan_fwd_bf16(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                            int32_t d_state, int32_t n_groups, int32_t block_len,
                                            const uint16_t* d_x, const float* d_a, const uint16_t* d_b, const uint16_t* d_c,
                                            const float* d_init_state, uint16_t* d_y, float* d_final_state,
                                            void* d_ws, size_t ws_bytes) {
  PMB_TRY(ssd_check(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len));
  if (!d_x || !d_a || !d_b || !d_c || !d_y || !d_ws) return fail(PMB_ERR_ARG, "ssd_scan_fwd_bf16: NULL argument");
  if (ssd16_supported(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len)) {
    // the inputs go to the tensor cores as they are
    if ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_b) | reinterpret_cast<uintptr_t>(d_c) | reinterpret_cast<uintptr_t>(d_y)) & 15)
      return fail(PMB_ERR_SHAPE, "ssd_scan_fwd_bf16: x, b, c and y must be 16-byte aligned");
    SsdWs w16;
    if (ssd16_ws_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_ws, ws_bytes, &w16, nullptr, nullptr) == 0)
      return fail(PMB_ERR_WORKSPACE, "ssd bf16 workspace too small");
    return ssd16_fwd(static_cast<cudaStream_t>(stream), batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_x, d_a, d_b, d_c,
                     d_init_state, d_y, d_final_state, w16);
  }
  SsdWs ws; Bf16Stage sg;
  if (bf16_stage_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_ws, ws_bytes, &ws, &sg) == 0)
    return fail(PMB_ERR_WORKSPACE, "ssd bf16 workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int64_t hp = (int64_t)batch * seqlen * n_heads * d_head, gn = (int64_t)batch * seqlen * n_groups * d_state;
  PMB_TRY(widen(st, d_x, sg.x, hp)); PMB_TRY(widen(st, d_b, sg.b, gn)); PMB_TRY(widen(st, d_c, sg.c, gn));
  SsdIn in{};
  in.B = batch; in.T = seqlen; in.H = n_heads; in.P = d_head; in.N = d_state; in.G = n_groups; in.Q = block_len;
  in.x = sg.x; in.ldx = (int64_t)n_heads * d_head; in.a = d_a; in.b = sg.b; in.c = sg.c; in.ldbc = (int64_t)n_groups * d_state;
  PMB_TRY(ssd_fwd(st, in, d_init_state, sg.y, in.ldx, d_final_state, ws));
  return cast_f32_bf16(st, sg.y, d_y, hp);
}

extern "C" pmb_status pmb_ssd_scan_bwd_bf16(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                            int32_t d_state, int32_t n_groups, int32_t block_len,
                                            const float* d_a, const uint16_t* d_dy,
                                            uint16_t* d_dx, float* d_da, uint16_t* d_db, uint16_t* d_dc,
                                            void* d_ws, size_t ws_bytes) {
  PMB_TRY(ssd_check(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len));
  if (!d_a || !d_dy || !d_dx || !d_da || !d_db || !d_dc || !d_ws) return fail(PMB_ERR_ARG, "ssd_scan_bwd_bf16: NULL argument");
  if (ssd16_supported(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len)) {
    if ((reinterpret_cast<uintptr_t>(d_dy) | reinterpret_cast<uintptr_t>(d_dx) | reinterpret_cast<uintptr_t>(d_db) | reinterpret_cast<uintptr_t>(d_dc)) & 15)
      return fail(PMB_ERR_SHAPE, "ssd_scan_bwd_bf16: dy, dx, db and dc must be 16-byte aligned");
    SsdWs w16; float *db32 = nullptr, *dc32 = nullptr;
    if (ssd16_ws_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_ws, ws_bytes, &w16, &db32, &dc32) == 0)
      return fail(PMB_ERR_WORKSPACE, "ssd bf16 workspace too small");
    return ssd16_bwd(static_cast<cudaStream_t>(stream), batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_a, d_dy,
                     d_dx, d_da, d_db, d_dc, w16, db32, dc32);
  }
  SsdWs ws; Bf16Stage sg;
  if (bf16_stage_layout(batch, seqlen, n_heads, d_head, d_state, n_groups, block_len, d_ws, ws_bytes, &ws, &sg) == 0)
    return fail(PMB_ERR_WORKSPACE, "ssd bf16 workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int64_t hp = (int64_t)batch * seqlen * n_heads * d_head, gn = (int64_t)batch * seqlen * n_groups * d_state;
  PMB_TRY(widen(st, d_dy, sg.dy, hp));
  SsdIn in{};
  in.B = batch; in.T = seqlen; in.H = n_heads; in.P = d_head; in.N = d_state; in.G = n_groups; in.Q = block_len;
  in.x = sg.x; in.ldx = (int64_t)n_heads * d_head; in.a = d_a; in.b = sg.b; in.c = sg.c; in.ldbc = (int64_t)n_groups * d_state;
  SsdGrads g{};
  g.dx = sg.dx; g.lddx = in.ldx; g.db = sg.db; g.dc = sg.dc; g.lddbc = in.ldbc; g.da = d_da;
  PMB_TRY(ssd_bwd(st, in, sg.y, in.ldx, sg.dy, in.ldx, g, ws));
  PMB_TRY(cast_f32_bf16(st, sg.dx, d_dx, hp));
  PMB_TRY(cast_f32_bf16(st, sg.db, d_db, gn));
  return cast_f32_bf16(st, sg.dc, d_dc, gn);
}
