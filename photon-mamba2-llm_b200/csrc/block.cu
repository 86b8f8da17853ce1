// Host orchestration of one Mamba2 block (forward, and backward with in-call recompute) and of the
// residual stack with the re-planned checkpoint policy: across the stack only each block's input is
// kept; everything else (projection outputs, conv activations, chunk states, gate inputs) lives in one
// transient workspace that every layer reuses.
#include "common.cuh"
#include "kernels.h"
#include "ssd_tc.h"

namespace pmb {

// One block per head: ddt_raw = ddt * sigmoid(dt_raw + bias) written into the dt columns of dxzd;
// ddt_bias[h] = sum over tokens; da_log[h] = A[h] * dA[h]  (A = -exp(a_log)).
__global__ void __launch_bounds__(256) dt_bwd_kernel(const float* __restrict__ xzd, float* __restrict__ dxzd, int64_t ld, int col0,
                                                     const float* __restrict__ dt_bias, const float* __restrict__ ddt,
                                                     const float* __restrict__ A, const float* __restrict__ dA,
                                                     float* __restrict__ ddt_bias, float* __restrict__ da_log, int64_t rows, int H,
                                                     uint16_t* __restrict__ pair_hi, uint16_t* __restrict__ pair_lo) {
  __shared__ float red[32];
  int h = blockIdx.x;
  float bias = dt_bias[h], acc = 0.0f;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) {
    float s = sigmoid_acc(xzd[r * ld + col0 + h] + bias);
    float g = ddt[r * H + h] * s;
    if (pair_hi) { uint32_t hh, ll; split_bf16_pair(g, hh, ll); pair_hi[r * ld + col0 + h] = (uint16_t)hh; if (pair_lo) pair_lo[r * ld + col0 + h] = (uint16_t)ll; }
    else dxzd[r * ld + col0 + h] = g;
    acc += g;
  }
  float tot = block_sum(acc, red);
  if (threadIdx.x == 0) {
    ddt_bias[h] = tot;
    da_log[h] = A[h] * dA[h];
  }
}

// fp32 -> bf16 (round to nearest even), 4 elements per thread
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, int64_t n4, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  auto cvt = [](float f) -> uint32_t {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (u >> 16) | 0x40;
    u += 0x7fffu + ((u >> 16) & 1u);
    return u >> 16;
  };
  if (i < n4) {
    float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    o.x = cvt(v.x) | (cvt(v.y) << 16);
    o.y = cvt(v.z) | (cvt(v.w) << 16);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
  if (i == 0) for (int64_t j = n4 * 4; j < n; ++j) dst[j] = (uint16_t)cvt(src[j]);
}

pmb_status cast_f32_bf16(cudaStream_t st, const float* src, uint16_t* dst, int64_t n) {
  int64_t n4 = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) ? 0 : n / 4;
  ProfScope prof(st, "cast_f32_bf16", 0.0, 6.0 * n);
  cast_f32_bf16_kernel<<<(unsigned)cdiv(n4 > 0 ? n4 : 1, 256), 256, 0, st>>>(src, dst, n4, n);
  PMB_LAUNCHED();
  return PMB_OK;
}

struct BlockWs {
  float *xzd, *act, *dt, *y, *rstd, *normed, *Aneg;
  SsdWs ssd;
  float *dnormed, *dxzd, *dact, *ddt, *dA, *scratch, *scratch2;   // scratch: conv partials; scratch2: norm partials
  size_t scratch_bytes, scratch2_bytes;
  uint16_t *normed16, *dxzd16;   // bf16 copies of the two GEMM operands (bf16-storage mode only)
  // fp32 mode with pair GEMMs: (hi, lo) bf16 pairs of every GEMM operand
  uint16_t *x_hi, *x_lo, *dout_hi, *dout_lo, *normed_hi, *normed_lo, *dxzd_hi, *dxzd_lo, *win_hi, *win_lo, *wout_hi, *wout_lo;
};

bool block_uses_pairs(const Dims& d) { return gemm_pairs_enabled() && !(d.D % 8) && !(d.J % 8) && !(d.I % 8); }

// The workspace has a forward part (everything the recompute produces and the gradient kernels read) and a
// backward part.  With nslots == 2 the forward part exists twice, so that the recompute of the next block can run
// (on another stream) while the gradient kernels of the current block still read the other copy; `slot` selects
// the copy this BlockWs points at.
// presplit: the caller brings (hi, lo) pairs of the two projection weights (the LM handle does), so none are kept here
static size_t block_ws_layout(const Dims& d, void* base, size_t bytes, BlockWs* out, bool bf16 = false, int nslots = 1, int slot = 0, bool presplit = false) {
  Arena ar(base, bytes);
  BlockWs w{};
  const bool pairs = !bf16 && block_uses_pairs(d);
  const size_t md = (size_t)d.M * d.D, mi = (size_t)d.M * d.I, mj = (size_t)d.M * d.J, dj = (size_t)d.D * d.J, id = (size_t)d.I * d.D;
  for (int sl = 0; sl < nslots; ++sl) {
    BlockWs f{};
    f.xzd = ar.take<float>(mj);
    f.act = ar.take<float>((size_t)d.M * d.X);
    f.dt = ar.take<float>((size_t)d.M * d.H);
    f.y = ar.take<float>(mi);
    f.rstd = ar.take<float>((size_t)d.M);
    f.normed = ar.take<float>(pairs ? 0 : mi);       // with pair GEMMs the normalised output only exists as a pair
    f.Aneg = ar.take<float>((size_t)d.H);
    ssd_ws_take(ar, d.B, d.T, d.H, d.P, d.N, d.G, d.Q, &f.ssd, 1);     // what the scan's forward leaves for its backward
    f.normed16 = ar.take<uint16_t>(bf16 ? mi : 0);
    if (pairs) {
      f.x_hi = ar.take<uint16_t>(md); f.x_lo = ar.take<uint16_t>(md);
      f.normed_hi = ar.take<uint16_t>(mi); f.normed_lo = ar.take<uint16_t>(mi);
      if (!presplit) { f.win_hi = ar.take<uint16_t>(dj); f.win_lo = ar.take<uint16_t>(dj); }
    }
    if (sl == slot) w = f;
  }
  // the gradient of the normalised gate output may overwrite it: dW_out (which reads `normed`, or its bf16 copy)
  // is enqueued before the GEMM that writes `dnormed`.  With pair GEMMs there is no fp32 `normed` to reuse.
  ssd_ws_take(ar, d.B, d.T, d.H, d.P, d.N, d.G, d.Q, &w.ssd, 2);       // the scan's backward-only buffers: one copy
  w.dnormed = pairs ? ar.take<float>(mi) : w.normed;
  // (with pair GEMMs the three producers of dxzd write the pair directly and the fp32 copy is never formed)
  w.dxzd = pairs ? nullptr : ar.take<float>(mj);
  w.dact = ar.take<float>((size_t)d.M * d.X);
  w.ddt = ar.take<float>((size_t)d.M * d.H);
  w.dA = ar.take<float>((size_t)d.H);
  // separate partial buffers: the reductions over them run on a side stream, next to later kernels of the block
  w.scratch_bytes = conv_bwd_ws_bytes(d);
  w.scratch = reinterpret_cast<float*>(ar.take<char>(w.scratch_bytes));
  w.scratch2_bytes = gated_rmsnorm_bwd_ws_bytes(d.M, d.I);
  w.scratch2 = reinterpret_cast<float*>(ar.take<char>(w.scratch2_bytes));
  w.dxzd16 = ar.take<uint16_t>(bf16 ? mj : 0);
  if (pairs) {
    w.dout_hi = ar.take<uint16_t>(md); w.dout_lo = ar.take<uint16_t>(md);
    w.dxzd_hi = ar.take<uint16_t>(mj); w.dxzd_lo = ar.take<uint16_t>(mj);
    if (!presplit) { w.wout_hi = ar.take<uint16_t>(id); w.wout_lo = ar.take<uint16_t>(id); }
  }
  if (out) *out = w;
  return ar.ok ? ar.used() : 0;
}

size_t block_ws_bytes(const Dims& d, bool bf16) { return block_ws_layout(d, nullptr, 0, nullptr, bf16); }
size_t stack_ws_bytes(const Dims& d, bool bf16, bool presplit) { return block_ws_layout(d, nullptr, 0, nullptr, bf16, 2, 0, presplit); }

static SsdIn ssd_inputs(const Dims& d, const pmb_block_params& p, const BlockWs& w) {
  SsdIn in{};
  in.B = d.B; in.T = d.T; in.H = d.H; in.P = d.P; in.N = d.N; in.G = d.G; in.Q = d.Q;
  in.x = w.act; in.ldx = d.X;
  in.dt = w.dt; in.A = w.Aneg; in.a = nullptr;
  in.b = w.act + d.I; in.c = w.act + d.I + d.G * d.N; in.ldbc = d.X;
  in.D = p.d_skip;
  return in;
}

// Steps 1-8 of Mamba2Block::forward (block.rs:143-222): everything up to the normalised gate output.
// In bf16-storage mode (w16 != NULL) x is bf16, the two projections run as bf16 GEMMs with fp32 accumulation
// against bf16 copies of the weights, and everything between them (the reference's "fp32 islands",
// block.rs:24-42) stays in fp32.
// Pair of a weight matrix: the caller's pre-split copy when there is one, else split here into the workspace.
static pmb_status weight_pair(cudaStream_t st, const Weights16* wx, bool in_proj, const float* src, int64_t rows, int64_t cols,
                              uint16_t* hi, uint16_t* lo, Pair16* out) {
  if (wx && wx->pairs) { *out = in_proj ? Pair16{wx->in_proj, wx->in_lo, cols} : Pair16{wx->out_proj, wx->out_lo, cols}; return PMB_OK; }
  PMB_TRY(split_pair16(st, src, rows, cols, cols, hi, lo, cols));
  *out = Pair16{hi, lo, cols};
  return PMB_OK;
}

// x_pair_ready: the (hi, lo) pair of x is already in the workspace (written by the GEMM that produced x)
static pmb_status block_fwd_core(cudaStream_t st, const Dims& d, const pmb_block_params& p, const void* x, const BlockWs& w,
                                 const Weights16* wx, bool x_pair_ready = false) {
  const Weights16* w16 = storage_is_bf16(wx) ? wx : nullptr;
  const bool pr = !w16 && block_uses_pairs(d);
  if (w16) PMB_TRY(gemm_bf16(st, 0, 0, d.M, d.J, d.D, x, d.D, w16->in_proj, d.J, w.xzd, d.J, nullptr, 0));
  else if (pr) {
    Pair16 win;
    if (!x_pair_ready) PMB_TRY(split_pair16(st, static_cast<const float*>(x), d.M, d.D, d.D, w.x_hi, w.x_lo, d.D));
    PMB_TRY(weight_pair(st, wx, true, p.in_proj_weight, d.D, d.J, w.win_hi, w.win_lo, &win));
    PMB_TRY(gemm_pairs(st, 0, 0, d.M, d.J, d.D, Pair16{w.x_hi, w.x_lo, d.D}, win, w.xzd, d.J, nullptr));
  }
  else PMB_TRY(gemm(st, 0, 0, d.M, d.J, d.D, static_cast<const float*>(x), d.D, p.in_proj_weight, d.J, w.xzd, d.J, nullptr, 0));
  // dt = softplus(dt_raw + bias) and A = -exp(a_log) are formed by the scan's first kernel (the chunk cumsum)
  // the B | C columns leave the conv kernel as a bf16 pair too when the fused scan kernels will read them
  ConvPairOut bc{};
  // (bf16 storage: the scan reads the hi halves alone, so the lo halves are not written)
  if (w.ssd.bc_hi) bc = ConvPairOut{w.ssd.bc_hi, w16 ? nullptr : w.ssd.bc_lo, d.I, 2 * d.G * d.N};
  PMB_TRY(conv_silu_dt_fwd(st, d, w.xzd, p.conv1d_weight, p.conv1d_bias, p.dt_bias, w.act, nullptr, w.ssd.bc_hi ? &bc : nullptr));
  SsdIn sin = ssd_inputs(d, p, w);
  sin.plain16 = w16 != nullptr;
  sin.bc_pair_ready = bc.hi != nullptr;
  sin.dt_raw = w.xzd + d.I + d.X; sin.ld_raw = d.J; sin.dt_bias = p.dt_bias; sin.a_log = p.a_log;
  PMB_TRY(ssd_fwd(st, sin, nullptr, w.y, d.I, nullptr, w.ssd));
  // with pair GEMMs the normalised output is only ever a GEMM operand: write it as a pair, skip the fp32 copy
  // (bf16 storage: the same with a plain bf16 rounding, lo == NULL)
  if (pr) PMB_TRY(gated_rmsnorm_fwd(st, d.M, d.I, d.eps, w.y, w.xzd, d.J, p.norm_weight, nullptr, w.rstd, w.normed_hi, w.normed_lo));
  else if (w16) PMB_TRY(gated_rmsnorm_fwd(st, d.M, d.I, d.eps, w.y, w.xzd, d.J, p.norm_weight, nullptr, w.rstd, w.normed16, nullptr));
  else PMB_TRY(gated_rmsnorm_fwd(st, d.M, d.I, d.eps, w.y, w.xzd, d.J, p.norm_weight, w.normed, w.rstd));
  return PMB_OK;
}

pmb_status block_fwd(cudaStream_t st, const Dims& d, const pmb_block_params& p, const void* x, const void* residual,
                     void* out, void* ws, size_t ws_bytes, const Weights16* wx, bool x_pair_ready, bool emit_out_pair) {
  const Weights16* w16 = storage_is_bf16(wx) ? wx : nullptr;
  const bool pr = !w16 && block_uses_pairs(d);
  BlockWs w;
  if (block_ws_layout(d, ws, ws_bytes, &w, w16 != nullptr, 1, 0, wx && wx->pairs) == 0 || !ws)
    return fail(PMB_ERR_WORKSPACE, "block workspace too small (%zu < %zu)", ws_bytes, block_ws_bytes(d, w16 != nullptr));
  PMB_TRY(block_fwd_core(st, d, p, x, w, wx, x_pair_ready && pr));
  if (w16) PMB_TRY(gemm_bf16(st, 0, 0, d.M, d.D, d.I, w.normed16, d.I, w16->out_proj, d.D, out, d.D, residual, 1));
  else if (pr) {
    Pair16 wout;
    PMB_TRY(weight_pair(st, wx, false, p.out_proj_weight, d.I, d.D, w.wout_hi, w.wout_lo, &wout));
    // the next block reads this output as its in_proj operand: its pair leaves the epilogue (into the x pair of the
    // one forward slot, which this block's own in_proj has long finished reading)
    PairGemm e{0, 0, d.M, d.D, d.I, Pair16{w.normed_hi, w.normed_lo, d.I}, wout, static_cast<float*>(out), d.D, static_cast<const float*>(residual)};
    if (emit_out_pair) e.emit = Pair16{w.x_hi, w.x_lo, d.D};
    PMB_TRY(gemm_pairs_group(st, &e, 1));
  }
  else PMB_TRY(gemm(st, 0, 0, d.M, d.D, d.I, w.normed, d.I, p.out_proj_weight, d.D, static_cast<float*>(out), d.D, static_cast<const float*>(residual), 0));
  return PMB_OK;
}

// Backward of one block = recompute of steps 1-8 into forward slot `slot`, then the gradient kernels reading it.
// block_bwd runs both on one stream; stack_bwd runs the recompute of block l-1 on a second stream while the
// gradient kernels of block l are in flight (two forward slots).
static pmb_status block_recompute(cudaStream_t st, const Dims& d, const pmb_block_params& p, const void* x, void* ws, size_t ws_bytes,
                                  const Weights16* wx, int nslots, int slot) {
  const bool bf = storage_is_bf16(wx);
  BlockWs w;
  if (block_ws_layout(d, ws, ws_bytes, &w, bf, nslots, slot, wx && wx->pairs) == 0 || !ws)
    return fail(PMB_ERR_WORKSPACE, "block workspace too small (%zu < %zu)", ws_bytes, block_ws_layout(d, nullptr, 0, nullptr, bf, nslots, 0));
  return block_fwd_core(st, d, p, x, w, wx);
}

static pmb_status block_grads(cudaStream_t st, const Dims& d, const pmb_block_params& p, const void* x, const void* dout,
                              const void* dx_accum, void* dx, const pmb_block_grads& g, void* ws, size_t ws_bytes, const Weights16* wx,
                              int nslots, int slot, cudaEvent_t recompute_done, bool dout_pair_ready = false, bool emit_dx_pair = false) {
  const Weights16* w16 = storage_is_bf16(wx) ? wx : nullptr;
  const bool pr = !w16 && block_uses_pairs(d);
  BlockWs w;
  if (block_ws_layout(d, ws, ws_bytes, &w, w16 != nullptr, nslots, slot, wx && wx->pairs) == 0 || !ws)
    return fail(PMB_ERR_WORKSPACE, "block workspace too small (%zu < %zu)", ws_bytes, block_ws_layout(d, nullptr, 0, nullptr, w16 != nullptr, nslots, 0));
  // The out_proj gradients do not wait for the recompute (dnormed = dout W_out^T needs neither x nor the recomputed
  // activations) and dW_out is needed only when the block is done: with pair GEMMs both go to a side stream, where
  // their CTAs fill the SMs that the latency-bound recompute and scan kernels leave idle.
  SideLane* gl = nullptr;
  if (pr) {
    static const int on = [] { const char* e = getenv("PMB_BLOCK_CONCURRENT"); return (e && e[0] == '0') ? 0 : 1; }();
    if (on) PMB_TRY(get_side_lane(1, &gl));
  }
  Pair16 wout{}, dop{w.dout_hi, w.dout_lo, d.D};
  if (pr) {
    // (the block above wrote the pair of its dx, which is this block's dout, from its last GEMM's epilogue)
    if (!dout_pair_ready) PMB_TRY(split_pair16(st, static_cast<const float*>(dout), d.M, d.D, d.D, w.dout_hi, w.dout_lo, d.D));
    PMB_TRY(weight_pair(st, wx, false, p.out_proj_weight, d.I, d.D, w.wout_hi, w.wout_lo, &wout));
    // dnormed heads the critical chain of this block: it stays on the caller's stream; only dW_out is deferred
    if (gl) PMB_TRY(gemm_pairs(st, 0, 1, d.M, d.I, d.D, dop, wout, w.dnormed, d.I, nullptr));
  }
  // the recomputed activations (enqueued by the caller, possibly on another stream) are needed from here on
  if (recompute_done) PMB_CUDA(cudaStreamWaitEvent(st, recompute_done, 0));
  // out_proj: dW_out = normed^T dout;  dnormed = dout W_out^T
  if (w16) {
    PMB_TRY(gemm_bf16(st, 1, 0, d.I, d.D, d.M, w.normed16, d.I, dout, d.D, g.out_proj_weight, d.D, nullptr, 0));
    PMB_TRY(gemm_bf16(st, 0, 1, d.M, d.I, d.D, dout, d.D, w16->out_proj, d.D, w.dnormed, d.I, nullptr, 0));
  } else if (pr && gl) {
    PMB_TRY(order_after(st, gl->ev[2], gl->s));                 // the recomputed normed pair is ready
    PMB_TRY(gemm_pairs(gl->s, 1, 0, d.I, d.D, d.M, Pair16{w.normed_hi, w.normed_lo, d.I}, dop, g.out_proj_weight, d.D, nullptr));
    PMB_CUDA(cudaEventRecord(gl->ev[0], gl->s));                // the last reader of the dout pair
  } else if (pr) {
    const PairGemm both[2] = {{1, 0, d.I, d.D, d.M, Pair16{w.normed_hi, w.normed_lo, d.I}, dop, g.out_proj_weight, d.D, nullptr},
                              {0, 1, d.M, d.I, d.D, dop, wout, w.dnormed, d.I, nullptr}};
    PMB_TRY(gemm_pairs_group(st, both, 2));
  } else {
    const float* df = static_cast<const float*>(dout);
    PMB_TRY(gemm(st, 1, 0, d.I, d.D, d.M, w.normed, d.I, df, d.D, g.out_proj_weight, d.D, nullptr, 0));
    PMB_TRY(gemm(st, 0, 1, d.M, d.I, d.D, df, d.D, p.out_proj_weight, d.D, w.dnormed, d.I, nullptr, 0));
  }
  // gate + norm: dy (in place over dnormed), dz -> z columns of dxzd
  // With pair GEMMs the three producers of dxzd (this kernel: dz; the scan's dt path: ddt_raw; the conv backward:
  // dxBC) write the (hi, lo) pair directly and the fp32 dxzd is never formed.  The norm backward also emits
  // dY exp(S) for the scan backward when the tensor-core scan will run.
  uint16_t* ph = pr ? w.dxzd_hi : (w16 ? w.dxzd16 : nullptr);   // bf16 storage: plain bf16 rounding, no low part
  uint16_t* pl = pr ? w.dxzd_lo : nullptr;
  SsdIn sin = ssd_inputs(d, p, w);
  sin.plain16 = w16 != nullptr;
  NormBwdExtra ex{};
  ex.dz_hi = ph; ex.dz_lo = pl;
  if ((pr || w16) && ssd_tc_supported(sin) && (d.P % 4 == 0)) {
    ex.S = w.ssd.S; ex.H = d.H; ex.P = d.P; ex.T = d.T; sin.dys_ready = true;
    if (w.ssd.dy_hi) {   // the scan backward runs on bf16 pairs: dY and dY exp(S) leave the norm backward as pairs
      ex.dy_hi = w.ssd.dy_hi; ex.dy_lo = w16 ? nullptr : w.ssd.dy_lo; sin.dy_pair_ready = true;
      ex.dys_hi = w.ssd.dys_hi; ex.dys_lo = w16 ? nullptr : w.ssd.dys_lo;
    } else {
      ex.dys = w.ssd.dys;
    }
  }
  PMB_TRY(gated_rmsnorm_bwd(st, d.M, d.I, w.dnormed, w.y, w.xzd, d.J, p.norm_weight, w.rstd, w.dnormed, w.dxzd, d.J,
                            g.norm_weight, w.scratch2, w.scratch2_bytes, gl, &ex));
  // scan
  SsdGrads sg{};
  sg.dx = w.dact; sg.lddx = d.X;
  sg.db = w.dact + d.I; sg.dc = w.dact + d.I + d.G * d.N; sg.lddbc = d.X;
  sg.da = nullptr; sg.ddt = w.ddt; sg.dA = w.dA; sg.dD = g.d_skip;
  // the pair path of the scan backward writes the dt columns of the dxzd pair, d_dt_bias and d_a_log itself
  const bool scan_dt = ph && ssd_bwd_takes_pairs(sin, w.dnormed, d.I, sg);
  if (scan_dt) { sg.raw.hi = ph; sg.raw.lo = pl; sg.raw.ld = d.J; sg.raw.col0 = d.I + d.X; sg.raw.d_dt_bias = g.dt_bias; sg.raw.d_a_log = g.a_log; }
  PMB_TRY(ssd_bwd(st, sin, w.y, d.I, w.dnormed, d.I, sg, w.ssd));
  // otherwise the dt columns (one block per head: a latency-bound loop over the tokens) run next to the conv backward
  if (!scan_dt) {
    cudaStream_t sdt = st;
    if (gl) { PMB_TRY(order_after(st, gl->ev[4], gl->s)); sdt = gl->s; }
    {
      ProfScope prof(sdt, "dt_bwd", 0.0, 16.0 * d.M * d.H);
      dt_bwd_kernel<<<(unsigned)d.H, 256, 0, sdt>>>(w.xzd, w.dxzd, d.J, d.I + d.X, p.dt_bias, w.ddt, w.Aneg, w.dA, g.dt_bias, g.a_log, d.M, d.H, ph, pl);
      PMB_LAUNCHED();
    }
    if (gl) PMB_CUDA(cudaEventRecord(gl->ev[5], gl->s));
  }
  // conv + SiLU
  PMB_TRY(conv_silu_bwd(st, d, w.xzd, p.conv1d_weight, p.conv1d_bias, w.dact, w.dxzd, g.conv1d_weight, g.conv1d_bias,
                        w.scratch, w.scratch_bytes, gl, ph, pl));
  // in_proj: dW_in = x^T dxzd;  dx = dxzd W_in^T (+ accumulated residual gradient)
  if (w16) {
    PMB_TRY(gemm_bf16(st, 1, 0, d.D, d.J, d.M, x, d.D, w.dxzd16, d.J, g.in_proj_weight, d.J, nullptr, 0));
    PMB_TRY(gemm_bf16(st, 0, 1, d.M, d.D, d.J, w.dxzd16, d.J, w16->in_proj, d.J, dx, d.D, dx_accum, 1));
  } else if (pr) {
    // x and W_in were split by the recompute above
    const Pair16 win = (wx && wx->pairs) ? Pair16{wx->in_proj, wx->in_lo, d.J} : Pair16{w.win_hi, w.win_lo, d.J};
    const Pair16 dxp{w.dxzd_hi, w.dxzd_lo, d.J};
    // the two gradients of in_proj as one launch, longer K first
    PairGemm gx{0, 1, d.M, d.D, d.J, dxp, win, static_cast<float*>(dx), d.D, static_cast<const float*>(dx_accum)};
    if (emit_dx_pair) {
      // dx is the next block's dout: its pair goes over this block's dout pair, once dW_out has read it
      gx.emit = Pair16{w.dout_hi, w.dout_lo, d.D};
      if (gl) PMB_CUDA(cudaStreamWaitEvent(st, gl->ev[0], 0));
    }
    const PairGemm gw{1, 0, d.D, d.J, d.M, Pair16{w.x_hi, w.x_lo, d.D}, dxp, g.in_proj_weight, d.J, nullptr};
    const PairGemm both[2] = {d.J >= d.M ? gx : gw, d.J >= d.M ? gw : gx};
    if (gl && !scan_dt) PMB_CUDA(cudaStreamWaitEvent(st, gl->ev[5], 0));      // the dt columns of the dxzd pair
    PMB_TRY(gemm_pairs_group(st, both, 2));
    if (gl) PMB_TRY(order_after(gl->s, gl->ev[3], st));           // dW_out and the small reductions are done when this block is
  } else {
    PMB_TRY(gemm(st, 1, 0, d.D, d.J, d.M, static_cast<const float*>(x), d.D, w.dxzd, d.J, g.in_proj_weight, d.J, nullptr, 0));
    PMB_TRY(gemm(st, 0, 1, d.M, d.D, d.J, w.dxzd, d.J, p.in_proj_weight, d.J, static_cast<float*>(dx), d.D, static_cast<const float*>(dx_accum), 0));
  }
  return PMB_OK;
}

pmb_status block_bwd(cudaStream_t st, const Dims& d, const pmb_block_params& p, const void* x, const void* dout,
                     const void* dx_accum, void* dx, const pmb_block_grads& g, void* ws, size_t ws_bytes, const Weights16* wx,
                     bool dout_pair_ready, bool emit_dx_pair) {
  PMB_TRY(block_recompute(st, d, p, x, ws, ws_bytes, wx, 1, 0));
  return block_grads(st, d, p, x, dout, dx_accum, dx, g, ws, ws_bytes, wx, 1, 0, nullptr, dout_pair_ready, emit_dx_pair);
}

}  // namespace pmb

// -----------------------------------------------------------------------------------------------
// C ABI
// -----------------------------------------------------------------------------------------------
using namespace pmb;

extern "C" size_t pmb_mamba2_block_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen) {
  Dims d;
  if (make_dims(cfg, batch, seqlen, &d) != PMB_OK) return 0;
  return block_ws_bytes(d, false);
}

extern "C" pmb_status pmb_mamba2_block_fwd(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                           int32_t batch, int32_t seqlen, const float* d_x, const float* d_residual,
                                           float* d_out, void* d_ws, size_t ws_bytes) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  if (!params || !d_x || !d_out) return fail(PMB_ERR_ARG, "block_fwd: NULL argument");
  return block_fwd(static_cast<cudaStream_t>(stream), d, *params, d_x, d_residual, d_out, d_ws, ws_bytes, nullptr);
}

extern "C" pmb_status pmb_mamba2_block_bwd(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                           int32_t batch, int32_t seqlen, const float* d_x, const float* d_dout,
                                           const float* d_dx_accum, float* d_dx, const pmb_block_grads* grads,
                                           void* d_ws, size_t ws_bytes) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  if (!params || !grads || !d_x || !d_dout || !d_dx) return fail(PMB_ERR_ARG, "block_bwd: NULL argument");
  return block_bwd(static_cast<cudaStream_t>(stream), d, *params, d_x, d_dout, d_dx_accum, d_dx, *grads, d_ws, ws_bytes, nullptr);
}

namespace pmb {

// Residual stack with block-input checkpoints.  `saved` holds n_layers+1 slots of (M,D) in the storage dtype
// (fp32, or bf16 when w16 != NULL); slot l = input of block l.
pmb_status stack_fwd(cudaStream_t st, const Dims& d, int n_layers, const pmb_block_params* layers, const Weights16* w16,
                     void* saved, void* ws, size_t ws_bytes) {
  size_t slot = (size_t)d.M * d.D * (storage_is_bf16(w16) ? 2 : 4);
  char* base = static_cast<char*>(saved);
  for (int l = 0; l < n_layers; ++l) {
    const void* h = base + (size_t)l * slot;
    PMB_TRY(block_fwd(st, d, layers[l], h, h, base + (size_t)(l + 1) * slot, ws, ws_bytes, w16 ? &w16[l] : nullptr, l > 0, l + 1 < n_layers));
  }
  return PMB_OK;
}

// dh_{l-1} = dh_l + dBlock_l/dx  (checkpoint.rs:110-135 reproduces this sum through the residual adds).
// With a workspace of stack_ws_bytes() the recompute of block l-1 is enqueued on a second stream before the
// gradient kernels of block l, into the other forward slot: it needs only the saved block input, and at a few
// thousand tokens both halves are latency-bound chains that leave most SMs idle, so they overlap well.
// PMB_RECOMPUTE_AHEAD=0 turns it off.
pmb_status stack_bwd(cudaStream_t st, const Dims& d, int n_layers, const pmb_block_params* layers, const Weights16* w16,
                     const pmb_block_grads* grads, const void* saved, void* dhidden, void* ws, size_t ws_bytes,
                     pmb_layer_callback on_layer_done, void* user) {
  const bool bf = storage_is_bf16(w16);
  size_t slot = (size_t)d.M * d.D * (bf ? 2 : 4);
  const char* base = static_cast<const char*>(saved);
  static const int ahead_on = [] { const char* e = getenv("PMB_RECOMPUTE_AHEAD"); return (e && e[0] == '0') ? 0 : 1; }();
  SideLane* rl = nullptr;
  // (fp32 blocks whose dimensions rule out pre-split pairs send their GEMMs through the library's one scratch
  // buffer, which two streams must not share: those stay serial)
  if (ahead_on && n_layers > 1 && (bf || block_uses_pairs(d)) && ws_bytes >= stack_ws_bytes(d, bf, w16 && w16->pairs)) PMB_TRY(get_side_lane(3, &rl));
  if (!rl) {
    for (int l = n_layers - 1; l >= 0; --l) {
      PMB_TRY(block_bwd(st, d, layers[l], base + (size_t)l * slot, dhidden, dhidden, dhidden, grads[l], ws, ws_bytes, w16 ? &w16[l] : nullptr,
                        l + 1 < n_layers, l > 0));
      if (on_layer_done) on_layer_done(l, user);
    }
    return PMB_OK;
  }
  // events: ev[0], ev[1] = recompute into slot 0 / 1 finished;  ev[2], ev[3] = gradient kernels reading slot 0 / 1 finished
  cudaStream_t sr = rl->s;
  // The gradient kernels run on a high-priority internal stream (the caller's stream has the lowest priority a
  // stream can have, the same as the recompute's): when an SM frees up, the chain every later block waits for
  // goes first.  `user_st` only waits for that stream before each callback and at the end.
  cudaStream_t user_st = st;
  SideLane* cl = nullptr;
  {
    static const int prio_on = [] { const char* e = getenv("PMB_PRIORITY_LANE"); return (e && e[0] == '0') ? 0 : 1; }();
    if (prio_on) PMB_TRY(get_side_lane(6, &cl));
  }
  if (cl) { PMB_TRY(order_after(user_st, cl->ev[0], cl->s)); st = cl->s; }
  PMB_CUDA(cudaEventRecord(rl->ev[2], st));            // everything before this call (saved inputs, weights) is ready,
  PMB_CUDA(cudaEventRecord(rl->ev[3], st));            // and both slots are free
  auto recompute = [&](int l) -> pmb_status {
    const int sl = l & 1;
    PMB_CUDA(cudaStreamWaitEvent(sr, rl->ev[2 + sl], 0));
    PMB_TRY(block_recompute(sr, d, layers[l], base + (size_t)l * slot, ws, ws_bytes, w16 ? &w16[l] : nullptr, 2, sl));
    PMB_CUDA(cudaEventRecord(rl->ev[sl], sr));
    return PMB_OK;
  };
  PMB_TRY(recompute(n_layers - 1));
  for (int l = n_layers - 1; l >= 0; --l) {
    const int sl = l & 1;
    if (l > 0) PMB_TRY(recompute(l - 1));                // into the other slot, whose last readers were block l+1's kernels
    PMB_TRY(block_grads(st, d, layers[l], base + (size_t)l * slot, dhidden, dhidden, dhidden, grads[l], ws, ws_bytes,
                        w16 ? &w16[l] : nullptr, 2, sl, rl->ev[sl], l + 1 < n_layers, l > 0));
    PMB_CUDA(cudaEventRecord(rl->ev[2 + sl], st));
    if (on_layer_done) {
      if (cl) PMB_TRY(order_after(st, cl->ev[1], user_st));   // the callback orders its work after the caller's stream
      on_layer_done(l, user);
    }
  }
  if (cl) PMB_TRY(order_after(st, cl->ev[1], user_st));
  return PMB_OK;
}

}  // namespace pmb

extern "C" size_t pmb_stack_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen) {
  Dims d;
  if (make_dims(cfg, batch, seqlen, &d) != PMB_OK) return 0;
  return stack_ws_bytes(d, false, false);
}

extern "C" pmb_status pmb_stack_fwd_ckpt(void* stream, const pmb_mamba2_config* cfg, int32_t n_layers,
                                         const pmb_block_params* layers, int32_t batch, int32_t seqlen,
                                         float* d_saved, void* d_ws, size_t ws_bytes) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  if (!layers || !d_saved || n_layers <= 0) return fail(PMB_ERR_ARG, "stack_fwd: bad argument");
  return stack_fwd(static_cast<cudaStream_t>(stream), d, n_layers, layers, nullptr, d_saved, d_ws, ws_bytes);
}

extern "C" pmb_status pmb_stack_bwd(void* stream, const pmb_mamba2_config* cfg, int32_t n_layers,
                                    const pmb_block_params* layers, const pmb_block_grads* grads,
                                    int32_t batch, int32_t seqlen, const float* d_saved, float* d_dhidden,
                                    void* d_ws, size_t ws_bytes, pmb_layer_callback on_layer_done, void* user) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  if (!layers || !grads || !d_saved || !d_dhidden || n_layers <= 0) return fail(PMB_ERR_ARG, "stack_bwd: bad argument");
  return stack_bwd(static_cast<cudaStream_t>(stream), d, n_layers, layers, nullptr, grads, d_saved, d_dhidden, d_ws, ws_bytes,
                   on_layer_done, user);
}

// ---- bf16-storage variants (block.rs:24-42: activations and the two projections in bf16, islands in fp32)
extern "C" pmb_status pmb_cast_f32_to_bf16(void* stream, const float* d_src, uint16_t* d_dst, int64_t n) {
  if (!d_src || !d_dst || n <= 0) return fail(PMB_ERR_ARG, "cast_f32_to_bf16: bad argument");
  return cast_f32_bf16(static_cast<cudaStream_t>(stream), d_src, d_dst, n);
}

extern "C" size_t pmb_mamba2_block_workspace_bytes_bf16(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen) {
  Dims d;
  if (make_dims(cfg, batch, seqlen, &d) != PMB_OK) return 0;
  return block_ws_bytes(d, true);
}

static pmb_status check_bf16_dims(const Dims& d) {
  if ((d.D % 8) || (d.J % 8) || (d.I % 8)) return fail(PMB_ERR_SHAPE, "bf16 storage needs d_model, d_inner and in_proj_dim to be multiples of 8");
  return PMB_OK;
}

extern "C" pmb_status pmb_mamba2_block_fwd_bf16(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                                const uint16_t* d_in_proj_bf16, const uint16_t* d_out_proj_bf16,
                                                int32_t batch, int32_t seqlen, const uint16_t* d_x, const uint16_t* d_residual,
                                                uint16_t* d_out, void* d_ws, size_t ws_bytes) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  PMB_TRY(check_bf16_dims(d));
  if (!params || !d_in_proj_bf16 || !d_out_proj_bf16 || !d_x || !d_out) return fail(PMB_ERR_ARG, "block_fwd_bf16: NULL argument");
  Weights16 w16{d_in_proj_bf16, d_out_proj_bf16};
  return block_fwd(static_cast<cudaStream_t>(stream), d, *params, d_x, d_residual, d_out, d_ws, ws_bytes, &w16);
}

extern "C" pmb_status pmb_mamba2_block_bwd_bf16(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                                const uint16_t* d_in_proj_bf16, const uint16_t* d_out_proj_bf16,
                                                int32_t batch, int32_t seqlen, const uint16_t* d_x, const uint16_t* d_dout,
                                                const uint16_t* d_dx_accum, uint16_t* d_dx, const pmb_block_grads* grads,
                                                void* d_ws, size_t ws_bytes) {
  Dims d;
  PMB_TRY(make_dims(cfg, batch, seqlen, &d));
  PMB_TRY(check_bf16_dims(d));
  if (!params || !grads || !d_in_proj_bf16 || !d_out_proj_bf16 || !d_x || !d_dout || !d_dx) return fail(PMB_ERR_ARG, "block_bwd_bf16: NULL argument");
  Weights16 w16{d_in_proj_bf16, d_out_proj_bf16};
  return block_bwd(static_cast<cudaStream_t>(stream), d, *params, d_x, d_dout, d_dx_accum, d_dx, *grads, d_ws, ws_bytes, &w16);
}
