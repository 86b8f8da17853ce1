/*
 * pm_b200 — C ABI of the B200 (sm_100a) Mamba2 SSD block backend.
 *
 * Every entry point takes plain pointers and sizes.  Pointers named d_* are device
 * pointers on the current CUDA device; h_* are host pointers.  `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).  All tensors are
 * row-major (last axis fastest) unless a leading dimension is given.  Every function
 * returns a pmb_status; pmb_last_error() returns the text of the last failure on the
 * calling thread.  Nothing here falls back to the CPU: an unsupported request is an
 * error.  The library is not re-entrant per model handle (one host thread per GPU
 * rank, like the reference's single-threaded step loop, crates/pm-cli/src/train_cmd.rs:220).
 *
 * Symbols and the reference interface each one stands behind (paths relative to the
 * reference checkout):
 *   pmb_gemm_f32              Ops::matmul                 crates/pm-core/src/ops.rs (matmul), block.rs:143-144,224-225
 *   pmb_conv_silu_dt_fwd/bwd  Ops::conv1d+silu+softplus   crates/pm-core/src/mamba2/block.rs:150-163,184-188
 *   pmb_ssd_scan_fwd/bwd      Ops::ssd_scan               crates/pm-core/src/ops.rs:345-352, mamba2/ssd_ops.rs:61-284
 *   pmb_gated_rmsnorm_fwd/bwd silu/mul/Ops::rmsnorm       crates/pm-core/src/mamba2/block.rs:216-222, ops.rs:91-96
 *   pmb_mamba2_block_fwd/bwd  Mamba2Block::forward + its autograd backward   mamba2/block.rs:118-226
 *   pmb_mamba2_step           Mamba2Block::step           crates/pm-core/src/mamba2/block.rs:278-417
 *   pmb_stack_fwd_ckpt/bwd    ContextEncoder::forward_checkpointed + checkpoint_backward
 *                                                         photon/encoder.rs:73-87, checkpoint.rs:68-135
 *   pmb_lm_*                  FlatMamba::forward_checkpointed_hidden + fused CE + backward
 *                                                         flat.rs:122-161, pm-train/src/loss.rs:39-69,121-138
 */
#ifndef PM_B200_H
#define PM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pmb_status {
  PMB_OK = 0,
  PMB_ERR_SHAPE = 1,        /* dimension / divisibility / alignment violation */
  PMB_ERR_UNSUPPORTED = 2,  /* dtype or feature this build does not implement */
  PMB_ERR_CUDA = 3,         /* a CUDA runtime or driver call failed */
  PMB_ERR_WORKSPACE = 4,    /* caller-provided workspace too small */
  PMB_ERR_DEVICE_STATUS = 5,/* a kernel gave up on a bounded wait and raised its status word */
  PMB_ERR_ARG = 6           /* NULL pointer or invalid enum */
} pmb_status;

/* Mirror of Mamba2Config (crates/pm-core/src/mamba2/block.rs:48-57). */
typedef struct pmb_mamba2_config {
  int32_t d_model;
  int32_t d_state;     /* N */
  int32_t d_head;      /* P */
  int32_t n_heads;     /* H */
  int32_t n_groups;    /* 1 or n_heads */
  int32_t d_conv;      /* K, 2..8 */
  int32_t block_len;   /* SSD chunk length Q */
  float   rmsnorm_eps;
} pmb_mamba2_config;

/* Parameter order of Mamba2Block::append_params (block.rs:440-450). All fp32. */
typedef struct pmb_block_params {
  const float* in_proj_weight;   /* (D, J)  used as x @ W */
  const float* conv1d_weight;    /* (X, 1, K) */
  const float* conv1d_bias;      /* (X) */
  const float* a_log;            /* (H) */
  const float* d_skip;           /* (H) */
  const float* dt_bias;          /* (H) */
  const float* norm_weight;      /* (I) */
  const float* out_proj_weight;  /* (I, D) */
} pmb_block_params;

typedef struct pmb_block_grads {
  float* in_proj_weight;
  float* conv1d_weight;
  float* conv1d_bias;
  float* a_log;
  float* d_skip;
  float* dt_bias;
  float* norm_weight;
  float* out_proj_weight;
} pmb_block_grads;

const char* pmb_last_error(void);
/* Library build string ("pm_b200 <ver> sm_100a"). */
const char* pmb_version(void);
/* Number of kernels this library has launched since load (all threads). */
int64_t pmb_launch_count(void);
/* Optional per-kernel timing for benchmarks (no reference counterpart; the reference's analogue is its
 * env-gated op profiler, crates/pm-cuda/src/profiler.rs).  Between start and stop every kernel group is
 * bracketed by CUDA events on its launching stream; stop synchronises the device and writes a JSON array
 * [{"name","launches","ms","flops","bytes"}] of per-name totals (algorithmic FLOPs / bytes) into h_json. */
void pmb_profile_start(void);
pmb_status pmb_profile_stop(char* h_json, size_t capacity);
/* on = 0: the library stops using its internal side streams (recompute-ahead, concurrent scan chains, deferred
 * gradient GEMMs and reductions) and enqueues everything on the caller's stream, in the same order; results do not
 * change.  For per-kernel timing and for callers that want plain single-stream behaviour.  Default on. */
void pmb_set_concurrency(int32_t on);

/* Reads and clears the device status word (0 = no kernel gave up on a bounded wait). */
pmb_status pmb_device_status(int32_t* h_word_out);
/* Self-tests (no reference counterpart; the reference guards its GPU tests with host-side deadlines,
 * crates/pm-cuda/tests/conv1d_depthwise_bwd_gpu.rs:186-212).  pmb_selftest_bounded_wait launches one thread that
 * waits on a barrier nothing arms, gives up after `polls` polls (1..2^20) and raises bit 15 of the status word
 * (0x8000): the path every tensor-core kernel here takes instead of hanging.  pmb_selftest_device_once checks the
 * per-device "done once" table on the host and returns the number of failed checks (no GPU needed). */
pmb_status pmb_selftest_bounded_wait(void* stream, uint32_t polls);
int32_t pmb_selftest_device_once(void);

/* ---- GEMM (Ops::matmul).  C[M,N] = op(A)·op(B) (+ R).  fp32 storage.
 * trans_a = 0: A is (M,K) row-major with leading dimension lda; 1: A is stored (K,M).
 * trans_b = 0: B is (K,N) row-major with ldb;                   1: B is stored (N,K).
 * d_R (may be NULL) is added to the product (same shape/ld as C); d_R may equal d_C.
 * engine: 0 = auto, 1 = fp32 FMA, 2 = tcgen05 3xTF32 with 128x128 tiles, 3 = tcgen05 3xTF32 with 128x64 tiles,
 * 4 / 5 / 6 = tcgen05 bf16 pairs with 128x128 tiles on the persistent single-CTA kernel / 256x256 / 256x128 CTA-pair
 * tiles (cta_group::2): both operands are split into (hi, lo) bf16 pairs (hi + lo carries 16 mantissa bits) and each
 * k-step issues hi*hi + lo*hi + hi*lo with kind::f16, fp32 accumulation.  Error ~1e-5 of the result's scale (the
 * 3xTF32 kernels: ~1e-6), about twice their speed.  Auto takes the pair engine when the operands are 16-byte aligned
 * with row lengths that are multiples of 8 (a persistent kernel of 256x256 CTA-pair tiles when M > 128 and the product
 * has at least 18 such tiles -- PMB_GEMM_PAIR_MIN changes the 18 -- else the persistent single-CTA kernel), else 3xTF32
 * when its alignment rules hold, else FMA; the environment variable
 * PMB_GEMM_ENGINE=tf32 keeps auto off engine 4, =simt forces FMA.  Engine 4 keeps the split operands in a
 * library-owned scratch buffer that grows on demand (cudaMalloc inside the call); pmb_gemm_reserve_scratch() sizes it
 * ahead of time: 4*(|A| + |B|) bytes of the largest product. */
pmb_status pmb_gemm_reserve_scratch(size_t bytes);
pmb_status pmb_gemm_f32(void* stream, int32_t trans_a, int32_t trans_b, int64_t M, int64_t N, int64_t K,
                        const float* d_A, int64_t lda, const float* d_B, int64_t ldb,
                        float* d_C, int64_t ldc, const float* d_R, int32_t engine);

/* bf16 GEMM for the bf16-storage configurations (block.rs:24-42): A, B are bf16 bit patterns, accumulation is
 * fp32 on the tensor cores; d_C and d_R are fp32 (out_bf16 = 0) or bf16 (out_bf16 = 1).  Operand bases must be
 * 16-byte aligned and lda, ldb multiples of 8 elements. */
pmb_status pmb_gemm_bf16(void* stream, int32_t trans_a, int32_t trans_b, int64_t M, int64_t N, int64_t K,
                         const uint16_t* d_A, int64_t lda, const uint16_t* d_B, int64_t ldb,
                         void* d_C, int64_t ldc, const void* d_R, int32_t out_bf16);
/* Ops::to_dtype(F32 -> BF16) (ops.rs:54-73), round to nearest even. */
pmb_status pmb_cast_f32_to_bf16(void* stream, const float* d_src, uint16_t* d_dst, int64_t n);

/* ---- conv1d + SiLU + dt softplus (block.rs:150-163,184-188).
 * d_xzd (B,T,J): columns [0,I) z, [I,I+X) xBC pre-conv, [I+X,J) dt_raw.
 * d_act (B,T,X) = silu(causal depthwise conv + bias); d_dt (B,T,H) = softplus(dt_raw + dt_bias). */
pmb_status pmb_conv_silu_dt_fwd(void* stream, const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen,
                                const float* d_xzd, const float* d_conv_w, const float* d_conv_b,
                                const float* d_dt_bias, float* d_act, float* d_dt);
/* Backward of the conv+SiLU part.  d_dact (B,T,X) is the gradient w.r.t. d_act.  Writes the xBC
 * columns of d_dxzd (B,T,J) and d_dconv_w (X,K), d_dconv_b (X).  d_ws: workspace of
 * pmb_conv_bwd_workspace_bytes() bytes. */
size_t pmb_conv_bwd_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen);
pmb_status pmb_conv_silu_bwd(void* stream, const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen,
                             const float* d_xzd, const float* d_conv_w, const float* d_conv_b,
                             const float* d_dact, float* d_dxzd, float* d_dconv_w, float* d_dconv_b,
                             void* d_ws, size_t ws_bytes);

/* ---- SSD scan (Ops::ssd_scan, ops.rs:345-352).  y[b,t,h,:] = sum_{s<=t} exp(sum_{k=s+1..t} a_k)(C_t·B_s) x_s.
 * x (B,T,H,P) with row stride ldx between tokens (ldx >= H*P), a (B,T,H), b/c (B,T,G,N) with token
 * stride ldbc (G = n_groups in {1,H}: groups are NOT broadcast in memory), y (B,T,H,P) stride ldy.
 * T must be a multiple of block_len (the reference routes other T to its dense O(T^2) path; pass
 * block_len = T for that case).  d_init_state / d_final_state (B,H,N,P) may be NULL.
 * d_ws: workspace of pmb_ssd_workspace_bytes(); after the call it holds the per-chunk cumulative
 * sums and entering states that pmb_ssd_scan_bwd reads (keep it untouched between the two). */
size_t pmb_ssd_workspace_bytes(int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                               int32_t d_state, int32_t n_groups, int32_t block_len);
pmb_status pmb_ssd_scan_fwd(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                            int32_t d_state, int32_t n_groups, int32_t block_len,
                            const float* d_x, int64_t ldx, const float* d_a,
                            const float* d_b, const float* d_c, int64_t ldbc,
                            const float* d_init_state, float* d_y, int64_t ldy, float* d_final_state,
                            void* d_ws, size_t ws_bytes);
/* Backward: given dy, writes dx (stride lddx), da (B,T,H), db, dc (B,T,G,N; stride lddbc). */
pmb_status pmb_ssd_scan_bwd(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                            int32_t d_state, int32_t n_groups, int32_t block_len,
                            const float* d_x, int64_t ldx, const float* d_a,
                            const float* d_b, const float* d_c, int64_t ldbc,
                            const float* d_y, int64_t ldy, const float* d_dy, int64_t lddy,
                            float* d_dx, int64_t lddx, float* d_da, float* d_db, float* d_dc, int64_t lddbc,
                            void* d_ws, size_t ws_bytes);

/* Scan with bf16 inputs and fp32 state (the reference upcasts to F32 around Ops::ssd_scan, block.rs:203-208):
 * x, b, c, y and dy, dx, db, dc are contiguous bf16 (B,T,H,P) / (B,T,G,N); a, da and the states are fp32.
 * The backward reads x, b, c from the workspace the forward left behind (keep it untouched in between).
 * With d_head 64, d_state 64 or 128, block_len a multiple of 128 and at most 64 chunks per sequence the bf16 tensors
 * are the tensor-core operands as they are (one kind::f16 MMA per product; cumulative sums, decay factors, chunk
 * states and accumulators in fp32; y and dx written as bf16 by the kernels that form them) and the eight bf16
 * pointers must be 16-byte aligned.  Other shapes widen to fp32, run the fp32 scan and round the results. */
size_t pmb_ssd_workspace_bytes_bf16(int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                    int32_t d_state, int32_t n_groups, int32_t block_len);
pmb_status pmb_ssd_scan_fwd_bf16(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                 int32_t d_state, int32_t n_groups, int32_t block_len,
                                 const uint16_t* d_x, const float* d_a, const uint16_t* d_b, const uint16_t* d_c,
                                 const float* d_init_state, uint16_t* d_y, float* d_final_state,
                                 void* d_ws, size_t ws_bytes);
pmb_status pmb_ssd_scan_bwd_bf16(void* stream, int32_t batch, int32_t seqlen, int32_t n_heads, int32_t d_head,
                                 int32_t d_state, int32_t n_groups, int32_t block_len,
                                 const float* d_a, const uint16_t* d_dy,
                                 uint16_t* d_dx, float* d_da, uint16_t* d_db, uint16_t* d_dc,
                                 void* d_ws, size_t ws_bytes);

/* ---- gated RMSNorm (block.rs:216-222): out = rmsnorm(y * silu(z), w, eps) over the last axis (I).
 * z has token stride ldz (it lives inside xzd).  d_rstd (rows) receives 1/sqrt(mean+eps). */
pmb_status pmb_gated_rmsnorm_fwd(void* stream, int64_t rows, int32_t width, float eps,
                                 const float* d_y, const float* d_z, int64_t ldz, const float* d_w,
                                 float* d_out, float* d_rstd);
size_t pmb_gated_rmsnorm_bwd_workspace_bytes(int64_t rows, int32_t width);
pmb_status pmb_gated_rmsnorm_bwd(void* stream, int64_t rows, int32_t width,
                                 const float* d_dout, const float* d_y, const float* d_z, int64_t ldz,
                                 const float* d_w, const float* d_rstd,
                                 float* d_dy, float* d_dz, int64_t lddz, float* d_dw,
                                 void* d_ws, size_t ws_bytes);

/* Same backward for callers that cannot allocate device memory (no counterpart in the reference).
 * Hosts that gave the whole GPU to their own pool at start-up, or that must keep out of the driver's
 * allocator on a latency-critical path, have no workspace to pass.  This variant takes none: the
 * weight-gradient partials go to a 4 MiB array built into the library image (held by every GPU that
 * loads the library until exit), so ceil(rows/4) * width * 4 bytes must not exceed
 * pmb_gated_rmsnorm_bwd_static_max_bytes(); larger problems get PMB_ERR_SHAPE.  It calls no cudaMalloc /
 * cudaFree.  The first call on each device resolves the array's device address (make that call outside
 * stream capture).  All calls share the array: calls that may overlap on the GPU race and must be
 * ordered by the caller.  Results equal pmb_gated_rmsnorm_bwd's. */
size_t pmb_gated_rmsnorm_bwd_static_max_bytes(void);
pmb_status pmb_gated_rmsnorm_bwd_static(void* stream, int64_t rows, int32_t width,
                                        const float* d_dout, const float* d_y, const float* d_z, int64_t ldz,
                                        const float* d_w, const float* d_rstd,
                                        float* d_dy, float* d_dz, int64_t lddz, float* d_dw);

/* ---- one Mamba2 block (block.rs:118-226) and its backward with in-call recompute.
 * fwd: out (B,T,D) = Block(x); if d_residual != NULL, out = residual + Block(x) (the caller's
 * `h + Block(h)`, photon/encoder.rs:54-59; d_residual may equal d_x).  Nothing is kept for backward.
 * bwd: recomputes the block from x (the only stored activation), then writes dx (B,T,D) — added to
 * d_dx_accum when that is non-NULL (dx = dx_accum + dBlock/dx; may alias d_dx) — and all 8 parameter
 * gradients (overwritten, not accumulated). */
size_t pmb_mamba2_block_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen);
pmb_status pmb_mamba2_block_fwd(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                int32_t batch, int32_t seqlen, const float* d_x, const float* d_residual,
                                float* d_out, void* d_ws, size_t ws_bytes);
pmb_status pmb_mamba2_block_bwd(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                int32_t batch, int32_t seqlen, const float* d_x, const float* d_dout,
                                const float* d_dx_accum, float* d_dx, const pmb_block_grads* grads,
                                void* d_ws, size_t ws_bytes);

/* bf16-storage block ("compute dtype" bf16, block.rs:24-42): x, residual, out, dout, dx are bf16; parameters stay
 * fp32 and the caller supplies bf16 copies of the two projection weights (pmb_cast_f32_to_bf16, refreshed whenever
 * the fp32 masters change).  The projections run as bf16 GEMMs with fp32 accumulation; conv, softplus, exp, the
 * scan's recurrence (cumulative sums, decay factors, chunk states, accumulators) and the norm run in fp32 as in the
 * reference; on the shapes the fused scan kernels take (block_len a multiple of 128, d_state = d_head = 64) the
 * scan's tensor-core products read their operands rounded to bf16.  Parameter gradients are fp32.  Needs d_model,
 * d_inner and in_proj_dim to be multiples of 8. */
size_t pmb_mamba2_block_workspace_bytes_bf16(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen);
pmb_status pmb_mamba2_block_fwd_bf16(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                     const uint16_t* d_in_proj_bf16, const uint16_t* d_out_proj_bf16,
                                     int32_t batch, int32_t seqlen, const uint16_t* d_x, const uint16_t* d_residual,
                                     uint16_t* d_out, void* d_ws, size_t ws_bytes);
pmb_status pmb_mamba2_block_bwd_bf16(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                                     const uint16_t* d_in_proj_bf16, const uint16_t* d_out_proj_bf16,
                                     int32_t batch, int32_t seqlen, const uint16_t* d_x, const uint16_t* d_dout,
                                     const uint16_t* d_dx_accum, uint16_t* d_dx, const pmb_block_grads* grads,
                                     void* d_ws, size_t ws_bytes);

/* ---- one-token decode (Mamba2Block::step, block.rs:278-417).  x_t (B,1,D) -> y_t (B,1,D);
 * ssm_state (B,H,N,P) and conv_window (B,X,K-1) are updated in place. */
size_t pmb_mamba2_step_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch);
pmb_status pmb_mamba2_step(void* stream, const pmb_mamba2_config* cfg, const pmb_block_params* params,
                           int32_t batch, const float* d_x_t, float* d_ssm_state, float* d_conv_window,
                           float* d_y_t, void* d_ws, size_t ws_bytes);

/* ---- residual stack with the re-planned checkpoint policy (encoder.rs:73-87, checkpoint.rs:68-135).
 * Stored across the stack: the input of every block, d_saved (n_layers+1, B,T,D) (slot l = input of
 * block l, slot n_layers = stack output).  Backward walks blocks last to first, recomputing each one.
 * d_dhidden (B,T,D) is the gradient w.r.t. the stack output and is overwritten with the gradient
 * w.r.t. the stack input.  `on_layer_done(layer, user)` (may be NULL) is called on the host right
 * after layer `layer`'s gradient kernels have been enqueued (data-parallel callers enqueue that
 * layer's gradient all-reduce from it).
 * Workspace: pmb_mamba2_block_workspace_bytes() is enough.  With pmb_stack_workspace_bytes() (a second copy of the
 * forward part of the block workspace) pmb_stack_bwd enqueues the recompute of block l-1 on an internal second
 * stream while block l's gradient kernels run; results are identical.  The internal streams and events are
 * created on the first call on a device (make that call outside stream capture).  One host thread per device.
 * Captured into a CUDA graph, every GEMM launch of the library keeps a tile-scheduler counter of its own for the life
 * of the graph (a few bytes of device memory, never recycled): replay one instantiation of a captured graph at a
 * time, not two copies of it concurrently. */
typedef void (*pmb_layer_callback)(int32_t layer, void* user);
size_t pmb_stack_workspace_bytes(const pmb_mamba2_config* cfg, int32_t batch, int32_t seqlen);
pmb_status pmb_stack_fwd_ckpt(void* stream, const pmb_mamba2_config* cfg, int32_t n_layers,
                              const pmb_block_params* layers, int32_t batch, int32_t seqlen,
                              float* d_saved, void* d_ws, size_t ws_bytes);
pmb_status pmb_stack_bwd(void* stream, const pmb_mamba2_config* cfg, int32_t n_layers,
                         const pmb_block_params* layers, const pmb_block_grads* grads,
                         int32_t batch, int32_t seqlen, const float* d_saved, float* d_dhidden,
                         void* d_ws, size_t ws_bytes, pmb_layer_callback on_layer_done, void* user);

/* ---- flat Mamba2 LM training step (flat.rs:122-161 + pm-train/src/loss.rs:121-138): tied embedding ->
 * checkpointed stack -> tied head -> mean cross-entropy, forward + backward (no optimizer).
 * The model handle owns activations and workspaces (cudaMalloc at create).  Parameters and gradients
 * live in two caller-visible flat fp32 device buffers with identical layout:
 *   [embedding (V,D)] then per layer the 8 tensors in append_params order, each 256-byte aligned;
 * pmb_lm_param_offset() gives element offsets.  Ids/targets are int64 (crates/pm-core/src/dtype.rs I64). */
typedef struct pmb_lm pmb_lm;
pmb_status pmb_lm_create(const pmb_mamba2_config* cfg, int32_t n_layers, int32_t vocab,
                         int32_t batch, int32_t seqlen, pmb_lm** out);
/* Same with the storage dtype chosen: bf16_storage != 0 keeps activations (block inputs, hidden, gradient stream)
 * and the GEMM operands in bf16 with fp32 accumulation, islands and logits in fp32 (FlatMamba::with_compute_dtype,
 * flat.rs:74-78); parameters and gradients stay fp32. */
pmb_status pmb_lm_create_dtype(const pmb_mamba2_config* cfg, int32_t n_layers, int32_t vocab,
                               int32_t batch, int32_t seqlen, int32_t bf16_storage, pmb_lm** out);
/* Two-level variant (built from the same blocks; no counterpart wiring in the reference, whose
 * PHOTON glue is crates/pm-core/src/model.rs): level 0 = n_layers_level0 blocks at token rate; groups of `group`
 * hidden states are mean-pooled and projected by a (D,D) matrix into level 1 (n_layers_level1 blocks at 1/group
 * rate); level-1 outputs are repeated `group` times, shifted by one group, and added back before the tied head.
 * Flat parameter layout: embedding, level-0 layers, projection, level-1 layers; pmb_lm_param_offset(lm, -2, 0)
 * gives the projection, layer indices run over both levels.  seqlen/group must satisfy the block's chunk rules. */
pmb_status pmb_lm_create_hier(const pmb_mamba2_config* cfg, int32_t n_layers_level0, int32_t n_layers_level1,
                              int32_t group, int32_t vocab, int32_t batch, int32_t seqlen, int32_t bf16_storage,
                              pmb_lm** out);
void       pmb_lm_destroy(pmb_lm* lm);
int64_t    pmb_lm_param_count(const pmb_lm* lm);                 /* elements in the flat buffer (with padding) */
int64_t    pmb_lm_param_offset(const pmb_lm* lm, int32_t layer, int32_t which); /* layer=-1: embedding, -2: level-1 projection; which 0..7 */
float*     pmb_lm_params(pmb_lm* lm);                            /* device pointer, pmb_lm_param_count() floats */
float*     pmb_lm_grads(pmb_lm* lm);                             /* device pointer, same layout */
int64_t    pmb_lm_activation_bytes(const pmb_lm* lm);            /* stored activations + transient workspace */
/* h_out3 = { bytes stored for backward (block inputs), one block's transient workspace, LM-head transients } */
void       pmb_lm_activation_detail(const pmb_lm* lm, int64_t* h_out3);
/* One fwd+bwd step with inputs already on the device.  Loss is left in a device scalar (pmb_lm_loss_device). */
pmb_status pmb_lm_step_device(pmb_lm* lm, void* stream, const int64_t* d_ids, const int64_t* d_targets,
                              pmb_layer_callback on_layer_done, void* user);
const float* pmb_lm_loss_device(const pmb_lm* lm);
/* Token ids or targets outside [0, vocab) (on which the reference's gather / cross-entropy fail, photon/embedding.rs:
 * 54-66, pm-train/src/loss.rs:39-69) do not fault here: a bad id reads embedding row 0, a bad target contributes no
 * loss and no one-hot term, and a flag word on the device records it (bit 0: an id, bit 1: a target).
 * pmb_lm_step_host checks the word after every step; callers of pmb_lm_step_device and of captured graphs poll it
 * here (waits for `stream`, reads and clears the word). */
pmb_status pmb_lm_bad_tokens(pmb_lm* lm, void* stream, int32_t* h_flags_out);
/* Same step through host buffers: copies ids/targets (pinned or pageable host memory) to the device,
 * runs the step, copies the loss back and synchronises the stream.  This is the call a host trainer makes. */
pmb_status pmb_lm_step_host(pmb_lm* lm, void* stream, const int64_t* h_ids, const int64_t* h_targets,
                            float* h_loss, pmb_layer_callback on_layer_done, void* user);

/* ---- primitive ops: what the rest of pm_core::Ops needs on the device when an op sequence is not the fused block
 * (crates/pm-core/src/ops.rs): contiguous fp32 tensors unless a stride is given; every result is a new buffer the
 * caller owns.  Views (Ops::narrow / transpose / broadcast_as / reshape / concat, ops.rs:123-148) are one strided
 * copy: describe the source view by extents, element strides (0 broadcasts) and a start offset; concat is one copy
 * per input into an offset of the output.  pmb_unary_f32 serves neg / exp / sqrt / silu / sigmoid / softplus /
 * mul_scalar / add_scalar (ops.rs:80,98-100,166,310-319) and plain copies; pmb_binary_f32 serves add / sub / mul /
 * div (ops.rs:77-79,316) on equal shapes (broadcast the smaller operand with pmb_strided_copy_f32 first). */
enum { PMB_MAX_RANK = 6 };
enum { PMB_OP_COPY = 0, PMB_OP_NEG = 1, PMB_OP_EXP = 2, PMB_OP_SQRT = 3, PMB_OP_SILU = 4, PMB_OP_SIGMOID = 5, PMB_OP_SOFTPLUS = 6,
       PMB_OP_MUL_SCALAR = 7, PMB_OP_ADD_SCALAR = 8,
       PMB_OP_ADD = 16, PMB_OP_SUB = 17, PMB_OP_MUL = 18, PMB_OP_DIV = 19 };
pmb_status pmb_unary_f32(void* stream, int32_t op, const float* d_x, float scalar, float* d_out, int64_t n);
pmb_status pmb_binary_f32(void* stream, int32_t op, const float* d_a, const float* d_b, float* d_out, int64_t n);
pmb_status pmb_strided_copy_f32(void* stream, const float* d_src, int32_t rank, const int64_t* h_shape,
                                const int64_t* h_strides, int64_t offset, float* d_out);
/* Ops::embedding (ops.rs:158-164): out[r,:] = table[ids[r],:]; an id outside [0, vocab) yields a zero row and sets
 * *d_bad_flag (a device word the caller clears and polls), since the reference fails on such input. */
pmb_status pmb_embedding_f32(void* stream, const float* d_table, int64_t vocab, int64_t width, const int64_t* d_ids,
                             int64_t rows, float* d_out, uint32_t* d_bad_flag);
/* Ops::gather along the last axis with one index per row (ops.rs:296-302): out[r] = x[r, index[r]]. */
pmb_status pmb_gather_last_f32(void* stream, const float* d_x, const int64_t* d_index, int64_t rows, int64_t width,
                               float* d_out, uint32_t* d_bad_flag);
/* Ops::log_softmax over the last axis (ops.rs:292). */
pmb_status pmb_log_softmax_f32(void* stream, const float* d_x, int64_t rows, int64_t width, float* d_out);
/* Ops::sum_all / mean_all (ops.rs:304-307): a device scalar, two fixed-order passes. */
size_t     pmb_sum_workspace_bytes(void);
pmb_status pmb_sum_all_f32(void* stream, const float* d_x, int64_t n, int32_t mean, float* d_out, void* d_ws, size_t ws_bytes);
/* Ops::cumsum (ops.rs:120) along an axis of length `len` of a tensor viewed as (outer, len, inner). */
pmb_status pmb_cumsum_f32(void* stream, const float* d_x, int64_t outer, int64_t len, int64_t inner, float* d_out);

/* ---- data parallelism (no counterpart in the reference, which drives one device: crates/pm-cli/src/train_cmd.rs:50).
 * The path shards over batch with no data-path collective; the one exchange per step is the average of the parameter
 * gradients.  One process (or host thread) per GPU: rank 0 obtains an id with pmb_dp_unique_id and hands its 128 bytes
 * to the other ranks by any host channel; every rank calls pmb_dp_init with its device current (a collective call:
 * all ranks must enter it).  NCCL is loaded at run time (libnccl.so.2, or the name in PMB_NCCL_LIB).
 * pmb_dp_allreduce_async orders an in-place average of `count` floats after everything already enqueued on `stream`
 * and runs it on the communicator's own stream; pmb_dp_allgather_async does the same for an all-gather of `bytes`
 * bytes per rank (d_recv holds world_size * bytes, rank r's block at r * bytes); pmb_dp_sync makes `stream` wait for
 * all of them.
 * pmb_lm_step_device_dp is pmb_lm_step_device with one such all-reduce per layer bucket (the layer's 8 gradient
 * tensors, contiguous in the flat buffer), enqueued the moment the layer's gradient kernels are, and the final wait:
 * on return `stream` sees averaged gradients.  The embedding bucket is exchanged in two parts: the tied head's share
 * (the whole table, complete right after the head's backward) is all-reduced while the stack backward runs, and the
 * token-lookup share, which exists only when the backward ends and touches at most batch * seqlen rows per rank,
 * travels as an all-gather of those rows and their token ids and is scatter-added by every rank.  Every rank must make the same calls in the
 * same order.  With two ranks the communicator is created with at most 8 NCCL CTAs (ncclConfig_t::maxCTAs: the
 * all-reduces run beside compute kernels that want whole SMs); larger worlds keep NCCL's choice; the environment
 * variable PMB_DP_MAX_CTAS overrides both (0 = NCCL's default).  These calls may be captured into a CUDA graph (after one eager step, which lets NCCL set up its
 * connections); NCCL then keeps the communicator alive for that graph, so destroy such graphs before pmb_dp_destroy,
 * which otherwise waits for them. */
typedef struct pmb_dp pmb_dp;
pmb_status pmb_dp_unique_id(void* h_id128);
pmb_status pmb_dp_init(int32_t nranks, int32_t rank, const void* h_id128, pmb_dp** out);
void       pmb_dp_destroy(pmb_dp* dp);
int32_t    pmb_dp_world_size(const pmb_dp* dp);
pmb_status pmb_dp_allreduce_async(pmb_dp* dp, void* stream, float* d_buf, int64_t count);
pmb_status pmb_dp_allgather_async(pmb_dp* dp, void* stream, const void* d_send, void* d_recv, int64_t bytes);
pmb_status pmb_dp_sync(pmb_dp* dp, void* stream);
pmb_status pmb_lm_step_device_dp(pmb_lm* lm, void* stream, const int64_t* d_ids, const int64_t* d_targets, pmb_dp* dp);

/* ---- optimizer on the flat parameter buffer (outside the benchmarked metric; pm-train/src/clip.rs:13-53,
 * pm-train/src/optim.rs:104-157).  pmb_grad_sumsq leaves sum(g^2) in a device scalar (two passes, fixed order, no
 * host sync); pmb_adamw_step applies global-norm clipping (when max_norm > 0: g *= max_norm/norm if norm > max_norm,
 * read from d_sumsq on the device), decoupled weight decay, the moment updates and the parameter update for all n
 * elements in one kernel.  `step` is 1-based.  Gradients are not rewritten. */
size_t pmb_grad_sumsq_workspace_bytes(void);
pmb_status pmb_grad_sumsq(void* stream, int64_t n, const float* d_grads, float* d_sumsq_out, void* d_ws, size_t ws_bytes);
pmb_status pmb_adamw_step(void* stream, int64_t n, float* d_params, const float* d_grads, float* d_m, float* d_v,
                          float lr, float beta1, float beta2, float eps, float weight_decay, int32_t step,
                          float max_norm, const float* d_sumsq);

/* ---- weights checkpoint I/O in the reference's format (pm-train/src/checkpoint.rs:25-97): a safetensors file with
 * the parameters by position, "p_0000", "p_0001", ... in append_params order (embedding (V,D), then per block
 * in_proj (D,J), conv1d_weight (X,1,K), conv1d_bias (X), a_log (H), d_skip (H), dt_bias (H), norm_weight (I),
 * out_proj (I,D); the two-level model has its (D,D) projection between the two stacks), all F32.  Load requires
 * the same tensor count, dtype and shapes and changes nothing when it fails.  Host-side file code; the stream is
 * synchronised before the device copy.  The two *_f32 entry points are the format code alone, on host buffers:
 * shapes_flat holds the extents of all tensors back to back, ranks[i] how many belong to tensor i. */
pmb_status pmb_lm_save_safetensors(pmb_lm* lm, void* stream, const char* path);
pmb_status pmb_lm_load_safetensors(pmb_lm* lm, void* stream, const char* path);
pmb_status pmb_safetensors_save_f32(const char* path, int32_t n_tensors, const int64_t* shapes_flat, const int32_t* ranks,
                                    const float* const* h_data);
pmb_status pmb_safetensors_load_f32(const char* path, int32_t n_tensors, const int64_t* shapes_flat, const int32_t* ranks,
                                    float* const* h_data);

#ifdef __cplusplus
}
#endif
#endif /* PM_B200_H */
