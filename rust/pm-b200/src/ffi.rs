//! Raw bindings of `include/pm_b200.h` (the C ABI of `libpm_b200.so`), one declaration per exported symbol.
//!
//! NOT COMPILED: the environment this crate was written in has no Rust toolchain.  The list below is checked
//! against the header by `tests/test_abi.py::test_rust_ffi_declares_every_symbol` (names only); the argument types
//! follow the header one to one (`void*` = `*mut c_void`, `int64_t` = `i64`, `size_t` = `usize`, `pmb_status` = `i32`).
#![allow(non_camel_case_types, clippy::too_many_arguments)]
use std::os::raw::{c_char, c_void};

/// `pmb_mamba2_config`: mirror of `Mamba2Config` (crates/pm-core/src/mamba2/block.rs:48-57).
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct PmbConfig {
    pub d_model: i32,
    pub d_state: i32,
    pub d_head: i32,
    pub n_heads: i32,
    pub n_groups: i32,
    pub d_conv: i32,
    pub block_len: i32,
    pub rmsnorm_eps: f32,
}

/// `pmb_block_params` / `pmb_block_grads`: the 8 tensors of a block in `append_params` order (block.rs:440-450).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct PmbBlockParams {
    pub p: [*const f32; 8],
}
#[repr(C)]
#[derive(Clone, Copy)]
pub struct PmbBlockGrads {
    pub g: [*mut f32; 8],
}

/// Opaque handles.
#[repr(C)]
pub struct PmbLm {
    _private: [u8; 0],
}
#[repr(C)]
pub struct PmbDp {
    _private: [u8; 0],
}

pub type LayerCb = Option<extern "C" fn(layer: i32, user: *mut c_void)>;

pub const PMB_OK: i32 = 0;
pub const PMB_ERR_SHAPE: i32 = 1;
pub const PMB_ERR_UNSUPPORTED: i32 = 2;
pub const PMB_ERR_CUDA: i32 = 3;
pub const PMB_ERR_WORKSPACE: i32 = 4;
pub const PMB_ERR_DEVICE_STATUS: i32 = 5;
pub const PMB_ERR_ARG: i32 = 6;

pub const PMB_OP_COPY: i32 = 0;
pub const PMB_OP_NEG: i32 = 1;
pub const PMB_OP_EXP: i32 = 2;
pub const PMB_OP_SQRT: i32 = 3;
pub const PMB_OP_SILU: i32 = 4;
pub const PMB_OP_SIGMOID: i32 = 5;
pub const PMB_OP_SOFTPLUS: i32 = 6;
pub const PMB_OP_MUL_SCALAR: i32 = 7;
pub const PMB_OP_ADD_SCALAR: i32 = 8;
pub const PMB_OP_ADD: i32 = 16;
pub const PMB_OP_SUB: i32 = 17;
pub const PMB_OP_MUL: i32 = 18;
pub const PMB_OP_DIV: i32 = 19;

#[link(name = "pm_b200")]
extern "C" {
    pub fn pmb_last_error() -> *const c_char;
    pub fn pmb_version() -> *const c_char;
    pub fn pmb_launch_count() -> i64;
    pub fn pmb_profile_start();
    pub fn pmb_profile_stop(h_json: *mut c_char, capacity: usize) -> i32;
    pub fn pmb_set_concurrency(on: i32);
    pub fn pmb_device_status(h_word_out: *mut i32) -> i32;
    pub fn pmb_selftest_bounded_wait(stream: *mut c_void, polls: u32) -> i32;
    pub fn pmb_selftest_device_once() -> i32;
    pub fn pmb_gemm_reserve_scratch(bytes: usize) -> i32;
    pub fn pmb_gemm_f32(stream: *mut c_void, trans_a: i32, trans_b: i32, M: i64, N: i64, K: i64, d_A: *const f32, lda: i64, d_B: *const f32, ldb: i64, d_C: *mut f32, ldc: i64, d_R: *const f32, engine: i32) -> i32;
    pub fn pmb_gemm_bf16(stream: *mut c_void, trans_a: i32, trans_b: i32, M: i64, N: i64, K: i64, d_A: *const u16, lda: i64, d_B: *const u16, ldb: i64, d_C: *mut c_void, ldc: i64, d_R: *const c_void, out_bf16: i32) -> i32;
    pub fn pmb_cast_f32_to_bf16(stream: *mut c_void, d_src: *const f32, d_dst: *mut u16, n: i64) -> i32;
    pub fn pmb_conv_silu_dt_fwd(stream: *mut c_void, cfg: *const PmbConfig, batch: i32, seqlen: i32, d_xzd: *const f32, d_conv_w: *const f32, d_conv_b: *const f32, d_dt_bias: *const f32, d_act: *mut f32, d_dt: *mut f32) -> i32;
    pub fn pmb_conv_bwd_workspace_bytes(cfg: *const PmbConfig, batch: i32, seqlen: i32) -> usize;
    pub fn pmb_conv_silu_bwd(stream: *mut c_void, cfg: *const PmbConfig, batch: i32, seqlen: i32, d_xzd: *const f32, d_conv_w: *const f32, d_conv_b: *const f32, d_dact: *const f32, d_dxzd: *mut f32, d_dconv_w: *mut f32, d_dconv_b: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_ssd_workspace_bytes(batch: i32, seqlen: i32, n_heads: i32, d_head: i32, d_state: i32, n_groups: i32, block_len: i32) -> usize;
    pub fn pmb_ssd_scan_fwd(stream: *mut c_void, batch: i32, seqlen: i32, n_heads: i32, d_head: i32, d_state: i32, n_groups: i32, block_len: i32, d_x: *const f32, ldx: i64, d_a: *const f32, d_b: *const f32, d_c: *const f32, ldbc: i64, d_init_state: *const f32, d_y: *mut f32, ldy: i64, d_final_state: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_ssd_scan_bwd(stream: *mut c_void, batch: i32, seqlen: i32, n_heads: i32, d_head: i32, d_state: i32, n_groups: i32, block_len: i32, d_x: *const f32, ldx: i64, d_a: *const f32, d_b: *const f32, d_c: *const f32, ldbc: i64, d_y: *const f32, ldy: i64, d_dy: *const f32, lddy: i64, d_dx: *mut f32, lddx: i64, d_da: *mut f32, d_db: *mut f32, d_dc: *mut f32, lddbc: i64, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_ssd_workspace_bytes_bf16(batch: i32, seqlen: i32, n_heads: i32, d_head: i32, d_state: i32, n_groups: i32, block_len: i32) -> usize;
    pub fn pmb_ssd_scan_fwd_bf16(stream: *mut c_void, batch: i32, seqlen: i32, n_heads: i32, d_head: i32, d_state: i32, n_groups: i32, block_len: i32, d_x: *const u16, d_a: *const f32, d_b: *const u16, d_c: *const u16, d_init_state: *const f32, d_y: *mut u16, d_final_state: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_ssd_scan_bwd_bf16(stream: *mut c_void, batch: i32, seqlen: i32, n_heads: i32, d_head: i32, d_state: i32, n_groups: i32, block_len: i32, d_a: *const f32, d_dy: *const u16, d_dx: *mut u16, d_da: *mut f32, d_db: *mut u16, d_dc: *mut u16, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_gated_rmsnorm_fwd(stream: *mut c_void, rows: i64, width: i32, eps: f32, d_y: *const f32, d_z: *const f32, ldz: i64, d_w: *const f32, d_out: *mut f32, d_rstd: *mut f32) -> i32;
    pub fn pmb_gated_rmsnorm_bwd_workspace_bytes(rows: i64, width: i32) -> usize;
    pub fn pmb_gated_rmsnorm_bwd(stream: *mut c_void, rows: i64, width: i32, d_dout: *const f32, d_y: *const f32, d_z: *const f32, ldz: i64, d_w: *const f32, d_rstd: *const f32, d_dy: *mut f32, d_dz: *mut f32, lddz: i64, d_dw: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_gated_rmsnorm_bwd_static_max_bytes() -> usize;
    pub fn pmb_gated_rmsnorm_bwd_static(stream: *mut c_void, rows: i64, width: i32, d_dout: *const f32, d_y: *const f32, d_z: *const f32, ldz: i64, d_w: *const f32, d_rstd: *const f32, d_dy: *mut f32, d_dz: *mut f32, lddz: i64, d_dw: *mut f32) -> i32;
    pub fn pmb_mamba2_block_workspace_bytes(cfg: *const PmbConfig, batch: i32, seqlen: i32) -> usize;
    pub fn pmb_mamba2_block_fwd(stream: *mut c_void, cfg: *const PmbConfig, params: *const PmbBlockParams, batch: i32, seqlen: i32, d_x: *const f32, d_residual: *const f32, d_out: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_mamba2_block_bwd(stream: *mut c_void, cfg: *const PmbConfig, params: *const PmbBlockParams, batch: i32, seqlen: i32, d_x: *const f32, d_dout: *const f32, d_dx_accum: *const f32, d_dx: *mut f32, grads: *const PmbBlockGrads, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_mamba2_block_workspace_bytes_bf16(cfg: *const PmbConfig, batch: i32, seqlen: i32) -> usize;
    pub fn pmb_mamba2_block_fwd_bf16(stream: *mut c_void, cfg: *const PmbConfig, params: *const PmbBlockParams, d_in_proj_bf16: *const u16, d_out_proj_bf16: *const u16, batch: i32, seqlen: i32, d_x: *const u16, d_residual: *const u16, d_out: *mut u16, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_mamba2_block_bwd_bf16(stream: *mut c_void, cfg: *const PmbConfig, params: *const PmbBlockParams, d_in_proj_bf16: *const u16, d_out_proj_bf16: *const u16, batch: i32, seqlen: i32, d_x: *const u16, d_dout: *const u16, d_dx_accum: *const u16, d_dx: *mut u16, grads: *const PmbBlockGrads, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_mamba2_step_workspace_bytes(cfg: *const PmbConfig, batch: i32) -> usize;
    pub fn pmb_mamba2_step(stream: *mut c_void, cfg: *const PmbConfig, params: *const PmbBlockParams, batch: i32, d_x_t: *const f32, d_ssm_state: *mut f32, d_conv_window: *mut f32, d_y_t: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_stack_workspace_bytes(cfg: *const PmbConfig, batch: i32, seqlen: i32) -> usize;
    pub fn pmb_stack_fwd_ckpt(stream: *mut c_void, cfg: *const PmbConfig, n_layers: i32, layers: *const PmbBlockParams, batch: i32, seqlen: i32, d_saved: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_stack_bwd(stream: *mut c_void, cfg: *const PmbConfig, n_layers: i32, layers: *const PmbBlockParams, grads: *const PmbBlockGrads, batch: i32, seqlen: i32, d_saved: *const f32, d_dhidden: *mut f32, d_ws: *mut c_void, ws_bytes: usize, on_layer_done: LayerCb, user: *mut c_void) -> i32;
    pub fn pmb_lm_create(cfg: *const PmbConfig, n_layers: i32, vocab: i32, batch: i32, seqlen: i32, out: *mut *mut PmbLm) -> i32;
    pub fn pmb_lm_create_dtype(cfg: *const PmbConfig, n_layers: i32, vocab: i32, batch: i32, seqlen: i32, bf16_storage: i32, out: *mut *mut PmbLm) -> i32;
    pub fn pmb_lm_create_hier(cfg: *const PmbConfig, n_layers_level0: i32, n_layers_level1: i32, group: i32, vocab: i32, batch: i32, seqlen: i32, bf16_storage: i32, out: *mut *mut PmbLm) -> i32;
    pub fn pmb_lm_destroy(lm: *mut PmbLm);
    pub fn pmb_lm_param_count(lm: *const PmbLm) -> i64;
    pub fn pmb_lm_param_offset(lm: *const PmbLm, layer: i32, which: i32) -> i64;
    pub fn pmb_lm_params(lm: *mut PmbLm) -> *mut f32;
    pub fn pmb_lm_grads(lm: *mut PmbLm) -> *mut f32;
    pub fn pmb_lm_activation_bytes(lm: *const PmbLm) -> i64;
    pub fn pmb_lm_activation_detail(lm: *const PmbLm, h_out3: *mut i64);
    pub fn pmb_lm_step_device(lm: *mut PmbLm, stream: *mut c_void, d_ids: *const i64, d_targets: *const i64, on_layer_done: LayerCb, user: *mut c_void) -> i32;
    pub fn pmb_lm_loss_device(lm: *const PmbLm) -> *const f32;
    pub fn pmb_lm_bad_tokens(lm: *mut PmbLm, stream: *mut c_void, h_flags_out: *mut i32) -> i32;
    pub fn pmb_lm_step_host(lm: *mut PmbLm, stream: *mut c_void, h_ids: *const i64, h_targets: *const i64, h_loss: *mut f32, on_layer_done: LayerCb, user: *mut c_void) -> i32;
    pub fn pmb_unary_f32(stream: *mut c_void, op: i32, d_x: *const f32, scalar: f32, d_out: *mut f32, n: i64) -> i32;
    pub fn pmb_binary_f32(stream: *mut c_void, op: i32, d_a: *const f32, d_b: *const f32, d_out: *mut f32, n: i64) -> i32;
    pub fn pmb_strided_copy_f32(stream: *mut c_void, d_src: *const f32, rank: i32, h_shape: *const i64, h_strides: *const i64, offset: i64, d_out: *mut f32) -> i32;
    pub fn pmb_embedding_f32(stream: *mut c_void, d_table: *const f32, vocab: i64, width: i64, d_ids: *const i64, rows: i64, d_out: *mut f32, d_bad_flag: *mut u32) -> i32;
    pub fn pmb_gather_last_f32(stream: *mut c_void, d_x: *const f32, d_index: *const i64, rows: i64, width: i64, d_out: *mut f32, d_bad_flag: *mut u32) -> i32;
    pub fn pmb_log_softmax_f32(stream: *mut c_void, d_x: *const f32, rows: i64, width: i64, d_out: *mut f32) -> i32;
    pub fn pmb_sum_workspace_bytes() -> usize;
    pub fn pmb_sum_all_f32(stream: *mut c_void, d_x: *const f32, n: i64, mean: i32, d_out: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_cumsum_f32(stream: *mut c_void, d_x: *const f32, outer: i64, len: i64, inner: i64, d_out: *mut f32) -> i32;
    pub fn pmb_dp_unique_id(h_id128: *mut c_void) -> i32;
    pub fn pmb_dp_init(nranks: i32, rank: i32, h_id128: *const c_void, out: *mut *mut PmbDp) -> i32;
    pub fn pmb_dp_destroy(dp: *mut PmbDp);
    pub fn pmb_dp_world_size(dp: *const PmbDp) -> i32;
    pub fn pmb_dp_allreduce_async(dp: *mut PmbDp, stream: *mut c_void, d_buf: *mut f32, count: i64) -> i32;
    pub fn pmb_dp_allgather_async(dp: *mut PmbDp, stream: *mut c_void, d_send: *const c_void, d_recv: *mut c_void, bytes: i64) -> i32;
    pub fn pmb_dp_sync(dp: *mut PmbDp, stream: *mut c_void) -> i32;
    pub fn pmb_lm_step_device_dp(lm: *mut PmbLm, stream: *mut c_void, d_ids: *const i64, d_targets: *const i64, dp: *mut PmbDp) -> i32;
    pub fn pmb_grad_sumsq_workspace_bytes() -> usize;
    pub fn pmb_grad_sumsq(stream: *mut c_void, n: i64, d_grads: *const f32, d_sumsq_out: *mut f32, d_ws: *mut c_void, ws_bytes: usize) -> i32;
    pub fn pmb_adamw_step(stream: *mut c_void, n: i64, d_params: *mut f32, d_grads: *const f32, d_m: *mut f32, d_v: *mut f32, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, step: i32, max_norm: f32, d_sumsq: *const f32) -> i32;
    pub fn pmb_lm_save_safetensors(lm: *mut PmbLm, stream: *mut c_void, path: *const c_char) -> i32;
    pub fn pmb_lm_load_safetensors(lm: *mut PmbLm, stream: *mut c_void, path: *const c_char) -> i32;
    pub fn pmb_safetensors_save_f32(path: *const c_char, n_tensors: i32, shapes_flat: *const i64, ranks: *const i32, h_data: *const *const f32) -> i32;
    pub fn pmb_safetensors_load_f32(path: *const c_char, n_tensors: i32, shapes_flat: *const i64, ranks: *const i32, h_data: *const *mut f32) -> i32;
}
