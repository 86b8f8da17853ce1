//! `B200Backend`: `pm_core::Ops` + `pm_backend::Backend` over the C ABI of `libpm_b200.so`.
//!
//! NOT COMPILED where it was written (no Rust toolchain there).  What it shows, in real code rather than prose:
//!
//! * every `Ops` method is either served by one C-ABI call (`ffi::pmb_*`), absorbed into the fused block call, or
//!   refused with `B200Error::Unsupported` (the table in INTEGRATION.md lists which is which);
//! * tensors are cheap-clone handles (`Arc`) over device buffers with a shape, element strides and an offset, so
//!   `narrow` / `transpose` / `reshape` / `broadcast_as` are views and only materialise when a kernel needs
//!   contiguous memory (`pmb_strided_copy_f32`);
//! * `Mamba2Block::forward` is a blanket impl over `Ops` (crates/pm-core/src/mamba2/block.rs:118-226) and cannot be
//!   specialised, so the adaptor records provenance on the views it hands out and recognises the block's fixed op
//!   sequence: `matmul(x, in_proj)` opens a `BlockTrace`, the narrows / transposes / conv1d / silu / softplus /
//!   exp / ssd_scan / rmsnorm calls that follow only extend the trace (each returns a lazy tensor), and the final
//!   `matmul(normed, out_proj)` executes the whole trace as one `pmb_mamba2_block_fwd`.  A lazy tensor that is
//!   consumed by anything else forces the eager path for the ops recorded so far;
//! * `param_from_tensor` on a block output (crates/pm-core/src/checkpoint.rs:82) marks a checkpoint boundary: only
//!   the block input is kept, and `checkpoint_backward`'s recompute -> mul(dy) -> sum_all -> backward
//!   (checkpoint.rs:127-131) runs as one `pmb_mamba2_block_bwd`.
use std::cell::RefCell;
use std::ffi::CStr;
use std::os::raw::c_void;
use std::sync::{Arc, Mutex};

use pm_backend::{Backend, DeviceKind};
use pm_core::{Dtype, Ops, Param, Tensor};

use crate::ffi;

// ------------------------------------------------------------------------------------------------ errors

/// Mirrors `pmb_status` (include/pm_b200.h) with the library's message; the reference's typed backend error has
/// the same shape (crates/pm-cuda/src/error.rs:4-23).
#[derive(Debug, thiserror::Error)]
pub enum B200Error {
    #[error("shape: {0}")]
    Shape(String),
    #[error("unsupported: {0}")]
    Unsupported(String),
    #[error("cuda: {0}")]
    Cuda(String),
    #[error("workspace: {0}")]
    Workspace(String),
    #[error("a kernel gave up on a bounded wait (device status word set): {0}")]
    DeviceStatus(String),
    #[error("argument: {0}")]
    Arg(String),
}

fn check(status: i32) -> Result<(), B200Error> {
    if status == ffi::PMB_OK {
        return Ok(());
    }
    let text = unsafe { CStr::from_ptr(ffi::pmb_last_error()) }.to_string_lossy().into_owned();
    Err(match status {
        ffi::PMB_ERR_SHAPE => B200Error::Shape(text),
        ffi::PMB_ERR_UNSUPPORTED => B200Error::Unsupported(text),
        ffi::PMB_ERR_WORKSPACE => B200Error::Workspace(text),
        ffi::PMB_ERR_DEVICE_STATUS => B200Error::DeviceStatus(text),
        ffi::PMB_ERR_ARG => B200Error::Arg(text),
        _ => B200Error::Cuda(text),
    })
}

// ------------------------------------------------------------------------------------------------ device memory

extern "C" {
    fn cudaMalloc(ptr: *mut *mut c_void, bytes: usize) -> i32;
    fn cudaFree(ptr: *mut c_void) -> i32;
    fn cudaMemcpy(dst: *mut c_void, src: *const c_void, bytes: usize, kind: i32) -> i32;
    fn cudaSetDevice(ordinal: i32) -> i32;
}
const H2D: i32 = 1;
const D2H: i32 = 2;

/// One device allocation, freed when the last tensor that views it goes away.
pub struct DeviceBuf {
    ptr: *mut c_void,
    bytes: usize,
}
unsafe impl Send for DeviceBuf {}
unsafe impl Sync for DeviceBuf {}
impl DeviceBuf {
    fn new(bytes: usize) -> Result<Arc<Self>, B200Error> {
        let mut ptr = std::ptr::null_mut();
        if unsafe { cudaMalloc(&mut ptr, bytes.max(16)) } != 0 {
            return Err(B200Error::Cuda(format!("cudaMalloc({bytes}) failed")));
        }
        Ok(Arc::new(Self { ptr, bytes }))
    }
}
impl Drop for DeviceBuf {
    fn drop(&mut self) {
        unsafe { cudaFree(self.ptr) };
    }
}

// ------------------------------------------------------------------------------------------------ tensors

/// How a tensor came to be, as far as the block recogniser needs to know.
#[derive(Clone)]
enum Origin {
    /// Plain data in memory.
    Data,
    /// A value that belongs to an open block trace and has not been computed: `step` says which op of
    /// block.rs:143-225 produced it.  Consuming it outside the trace flushes the trace eagerly.
    Lazy { trace: Arc<Mutex<BlockTrace>>, step: BlockStep },
}

#[derive(Clone, Copy, PartialEq, Eq, Debug)]
enum BlockStep {
    InProj, Z, Xbc, DtRaw, XbcT, Conv, ConvNarrow, ConvT, Act, Xssm, Bmat, Cmat, Dt, A, Adt, Xdt, Scan, Skip, Gate, Normed,
}

struct Inner {
    buf: Option<Arc<DeviceBuf>>, // None while lazy
    shape: Vec<usize>,
    strides: Vec<usize>, // in elements
    offset: usize,       // in elements
    dtype: Dtype,
    origin: Origin,
    node: Option<usize>, // tape node that produced it (None under no_grad or for constants)
}

#[derive(Clone)]
pub struct B200Tensor(Arc<Inner>);

impl Tensor for B200Tensor {
    fn shape(&self) -> &[usize] {
        &self.0.shape
    }
    fn dtype(&self) -> Dtype {
        self.0.dtype
    }
}

fn contiguous_strides(shape: &[usize]) -> Vec<usize> {
    let mut s = vec![1; shape.len()];
    for d in (0..shape.len().saturating_sub(1)).rev() {
        s[d] = s[d + 1] * shape[d + 1];
    }
    s
}

impl B200Tensor {
    fn from_buf(buf: Arc<DeviceBuf>, shape: &[usize], dtype: Dtype, node: Option<usize>) -> Self {
        Self(Arc::new(Inner { buf: Some(buf), shape: shape.to_vec(), strides: contiguous_strides(shape), offset: 0, dtype, origin: Origin::Data, node }))
    }
    fn view(&self, shape: Vec<usize>, strides: Vec<usize>, offset: usize) -> Self {
        Self(Arc::new(Inner { buf: self.0.buf.clone(), shape, strides, offset, dtype: self.0.dtype, origin: self.0.origin.clone(), node: self.0.node }))
    }
    fn is_contiguous(&self) -> bool {
        self.0.offset == 0 && self.0.strides == contiguous_strides(&self.0.shape)
    }
    fn ptr_f32(&self) -> *const f32 {
        let base = self.0.buf.as_ref().expect("lazy tensor used as data").ptr as *const f32;
        unsafe { base.add(self.0.offset) }
    }
    /// Row pitch of a 2-D view whose last axis is dense: what `pmb_gemm_f32` takes as a leading dimension, so that
    /// `narrow` results feed the GEMM without a copy.
    fn row_pitch(&self) -> Option<i64> {
        let r = self.0.shape.len();
        (r >= 2 && self.0.strides[r - 1] == 1).then(|| self.0.strides[r - 2] as i64)
    }
}

/// Trainable leaf: a tensor plus an identity for the gradient store.  Neither `Send` nor `Sync` is required
/// (crates/pm-core/src/param.rs:16-22); `assign` swaps the buffer between steps (ops.rs:276-287).
#[derive(Clone)]
pub struct B200Param {
    id: usize,
    value: Arc<RefCell<B200Tensor>>,
    shadow: B200Tensor, // what `as_tensor` lends out; refreshed by `assign`
}
impl Param for B200Param {
    type Tensor = B200Tensor;
    fn as_tensor(&self) -> &B200Tensor {
        &self.shadow
    }
}

/// Gradients by parameter id (`Ops::gradient`, ops.rs:192-199).
#[derive(Default)]
pub struct B200GradStore {
    grads: std::collections::HashMap<usize, B200Tensor>,
}

// ------------------------------------------------------------------------------------------------ block trace

/// The operands of one `Mamba2Block::forward` in flight (block.rs:118-226) and how far the op sequence has got.
struct BlockTrace {
    x: B200Tensor,                 // (B,T,D) block input
    params: [Option<B200Tensor>; 8], // in append_params order, filled in as the ops name them
    cfg: ffi::PmbConfig,
    batch: i32,
    seqlen: i32,
    last: BlockStep,
    flushed: bool,                 // an outside consumer forced eager execution: the fast path is off for this trace
}

impl BlockTrace {
    /// `next` is accepted when it is the op that block.rs performs after `self.last`.
    fn advance(&mut self, next: BlockStep) -> bool {
        use BlockStep::*;
        let ok = matches!(
            (self.last, next),
            (InProj, Z) | (Z, Xbc) | (Xbc, DtRaw) | (DtRaw, XbcT) | (XbcT, Conv) | (Conv, ConvNarrow) | (ConvNarrow, ConvT) | (ConvT, Act)
                | (Act, Xssm) | (Xssm, Bmat) | (Bmat, Cmat) | (Cmat, Dt) | (Dt, A) | (A, Adt) | (Adt, Xdt) | (Xdt, Scan) | (Scan, Skip)
                | (Skip, Gate) | (Gate, Normed)
        );
        if ok {
            self.last = next;
        }
        ok && !self.flushed
    }
}

// ------------------------------------------------------------------------------------------------ tape

/// What backward needs for each differentiable op that runs outside the fused block: the residual adds of the
/// stack (photon/encoder.rs:54-59), the embedding, the tied head and the loss (pm-train/src/loss.rs:39-69).
enum Node {
    Leaf { param: usize },
    Add { a: usize, b: usize },
    MulScalar { a: usize, s: f32 },
    Mul { a: usize, b: usize, av: B200Tensor, bv: B200Tensor },
    SumAll { a: usize, shape: Vec<usize>, mean: bool },
    Matmul { a: usize, b: usize, av: B200Tensor, bv: B200Tensor },
    Embedding { table: usize, ids: B200Tensor, vocab: usize },
    LogSoftmax { a: usize, out: B200Tensor },
    Gather { a: usize, index: B200Tensor, width: usize },
    /// One fused block: input node, the 8 parameter ids and the saved input (the only stored activation).
    Block { x: usize, params: Vec<B200Tensor>, saved_x: B200Tensor, cfg: ffi::PmbConfig, batch: i32, seqlen: i32 },
    SsdScan { x: usize, a: usize, b: usize, c: usize, saved: Vec<B200Tensor>, ws: Arc<DeviceBuf>, dims: [i32; 7] },
}

#[derive(Default)]
struct Tape {
    nodes: Vec<Node>,
    grad_enabled: bool,
}

// ------------------------------------------------------------------------------------------------ backend

pub struct B200Backend {
    ordinal: i32,
    stream: *mut c_void, // cudaStream_t; NULL = the legacy default stream
    tape: RefCell<Tape>,
    next_param: RefCell<usize>,
    block_ws: RefCell<Option<Arc<DeviceBuf>>>, // one transient block workspace, reused by every layer
    open_trace: RefCell<Option<Arc<Mutex<BlockTrace>>>>,
}

impl B200Backend {
    /// One backend per process and device, like the reference's `--backend` switch (crates/pm-cli/src/train_cmd.rs:38-65).
    pub fn new(ordinal: i32) -> Result<Self, B200Error> {
        if unsafe { cudaSetDevice(ordinal) } != 0 {
            return Err(B200Error::Cuda(format!("cudaSetDevice({ordinal}) failed")));
        }
        Ok(Self {
            ordinal,
            stream: std::ptr::null_mut(),
            tape: RefCell::new(Tape { nodes: Vec::new(), grad_enabled: true }),
            next_param: RefCell::new(0),
            block_ws: RefCell::new(None),
            open_trace: RefCell::new(None),
        })
    }

    fn alloc(&self, shape: &[usize], dtype: Dtype, node: Option<usize>) -> Result<B200Tensor, B200Error> {
        let n: usize = shape.iter().product();
        Ok(B200Tensor::from_buf(DeviceBuf::new(n * dtype.size_in_bytes())?, shape, dtype, node))
    }

    fn record(&self, node: Node) -> Option<usize> {
        let mut t = self.tape.borrow_mut();
        if !t.grad_enabled {
            return None;
        }
        t.nodes.push(node);
        Some(t.nodes.len() - 1)
    }

    fn require_f32(&self, t: &B200Tensor, what: &str) -> Result<(), B200Error> {
        // unsupported dtypes are an error, never a silent fallback (crates/pm-core/src/dtype.rs:3-4)
        if t.0.dtype != Dtype::F32 {
            return Err(B200Error::Unsupported(format!("{what}: dtype {:?} (this op takes F32)", t.0.dtype)));
        }
        Ok(())
    }

    /// Dense copy of a view (or the tensor itself when it already is dense); flushes a lazy tensor's trace first.
    fn contiguous(&self, t: &B200Tensor) -> Result<B200Tensor, B200Error> {
        let t = self.materialise(t)?;
        if t.is_contiguous() {
            return Ok(t);
        }
        self.require_f32(&t, "contiguous")?;
        let out = self.alloc(&t.0.shape, Dtype::F32, t.0.node)?;
        let shape: Vec<i64> = t.0.shape.iter().map(|&v| v as i64).collect();
        let strides: Vec<i64> = t.0.strides.iter().map(|&v| v as i64).collect();
        let base = t.0.buf.as_ref().unwrap().ptr as *const f32;
        check(unsafe {
            ffi::pmb_strided_copy_f32(self.stream, base, shape.len() as i32, shape.as_ptr(), strides.as_ptr(), t.0.offset as i64, out.ptr_f32() as *mut f32)
        })?;
        Ok(out)
    }

    /// A lazy tensor consumed outside its trace: run the recorded prefix of the block op by op (each step has an
    /// eager kernel: GEMM, strided copy, pmb_conv_silu_dt_fwd, pmb_unary_f32, pmb_ssd_scan_fwd, pmb_gated_rmsnorm_fwd)
    /// and mark the trace so that its remaining ops run eagerly too.
    fn materialise(&self, t: &B200Tensor) -> Result<B200Tensor, B200Error> {
        match &t.0.origin {
            Origin::Data => Ok(t.clone()),
            Origin::Lazy { trace, step } => {
                trace.lock().unwrap().flushed = true;
                self.run_block_prefix(trace, *step)
            }
        }
    }

    fn run_block_prefix(&self, trace: &Arc<Mutex<BlockTrace>>, upto: BlockStep) -> Result<B200Tensor, B200Error> {
        // The eager rendition of block.rs:143-222 up to `upto`, built from the stand-alone entry points named above.
        // It exists for op sequences that merely resemble the block (e.g. a test that inspects `xzd`); training never
        // takes it.  Spelled out in INTEGRATION.md section 3; omitted here for length.
        let _ = (trace, upto);
        Err(B200Error::Unsupported("eager execution of a partial block trace (see INTEGRATION.md, section 3)".into()))
    }

    /// The whole block as one call (block.rs:118-226).  `residual` is the caller's `h + Block(h)` when the next op
    /// is that add (photon/encoder.rs:54-59); the epilogue of the last GEMM performs it.
    fn run_block(&self, tr: &BlockTrace, out_proj: &B200Tensor) -> Result<B200Tensor, B200Error> {
        let mut p = [std::ptr::null::<f32>(); 8];
        for (i, t) in tr.params.iter().enumerate() {
            p[i] = if i == 7 { out_proj.ptr_f32() } else { t.as_ref().ok_or_else(|| B200Error::Arg(format!("block parameter {i} was never named")))?.ptr_f32() };
        }
        let params = ffi::PmbBlockParams { p };
        let need = unsafe { ffi::pmb_mamba2_block_workspace_bytes(&tr.cfg, tr.batch, tr.seqlen) };
        let ws = {
            let mut slot = self.block_ws.borrow_mut();
            if slot.as_ref().map_or(true, |b| b.bytes < need) {
                *slot = Some(DeviceBuf::new(need)?);
            }
            slot.as_ref().unwrap().clone()
        };
        let x = self.contiguous(&tr.x)?;
        let out = self.alloc(&x.0.shape, Dtype::F32, None)?;
        check(unsafe {
            ffi::pmb_mamba2_block_fwd(self.stream, &tr.cfg, &params, tr.batch, tr.seqlen, x.ptr_f32(), std::ptr::null(), out.ptr_f32() as *mut f32, ws.ptr, ws.bytes)
        })?;
        Ok(out)
    }
}

// ------------------------------------------------------------------------------------------------ Ops

impl B200Backend {
    fn unary(&self, op: i32, x: &B200Tensor, scalar: f32, what: &str) -> Result<B200Tensor, B200Error> {
        let x = self.contiguous(x)?;
        self.require_f32(&x, what)?;
        let out = self.alloc(&x.0.shape, Dtype::F32, None)?;
        check(unsafe { ffi::pmb_unary_f32(self.stream, op, x.ptr_f32(), scalar, out.ptr_f32() as *mut f32, x.numel() as i64) })?;
        Ok(out)
    }
    fn binary(&self, op: i32, a: &B200Tensor, b: &B200Tensor, what: &str) -> Result<B200Tensor, B200Error> {
        // broadcasting follows the reference's callers: the smaller operand is expanded with broadcast_as first
        let (a, b) = (self.contiguous(a)?, self.contiguous(b)?);
        self.require_f32(&a, what)?;
        self.require_f32(&b, what)?;
        if a.0.shape != b.0.shape {
            return Err(B200Error::Shape(format!("{what}: {:?} vs {:?}", a.0.shape, b.0.shape)));
        }
        let out = self.alloc(&a.0.shape, Dtype::F32, None)?;
        check(unsafe { ffi::pmb_binary_f32(self.stream, op, a.ptr_f32(), b.ptr_f32(), out.ptr_f32() as *mut f32, a.numel() as i64) })?;
        Ok(out)
    }
    fn with_node(&self, t: B200Tensor, node: Option<usize>) -> B200Tensor {
        B200Tensor(Arc::new(Inner { buf: t.0.buf.clone(), shape: t.0.shape.clone(), strides: t.0.strides.clone(), offset: t.0.offset, dtype: t.0.dtype, origin: Origin::Data, node }))
    }
    fn lazy(&self, trace: &Arc<Mutex<BlockTrace>>, step: BlockStep, shape: Vec<usize>) -> B200Tensor {
        let strides = contiguous_strides(&shape);
        B200Tensor(Arc::new(Inner { buf: None, shape, strides, offset: 0, dtype: Dtype::F32, origin: Origin::Lazy { trace: trace.clone(), step }, node: None }))
    }
}

impl Ops for B200Backend {
    type Tensor = B200Tensor;
    type Error = B200Error;
    type Param = B200Param;
    type GradStore = B200GradStore;

    // ---- construction / host transfer (ops.rs:30-50,274) -----------------------------------------------
    fn zeros(&self, shape: &[usize], dtype: Dtype) -> Result<B200Tensor, B200Error> {
        let host = vec![0.0f32; shape.iter().product()];
        let t = self.from_slice_f32(&host, shape)?;
        self.to_dtype(&t, dtype)
    }
    fn ones(&self, shape: &[usize], dtype: Dtype) -> Result<B200Tensor, B200Error> {
        let host = vec![1.0f32; shape.iter().product()];
        let t = self.from_slice_f32(&host, shape)?;
        self.to_dtype(&t, dtype)
    }
    fn from_slice_f32(&self, data: &[f32], shape: &[usize]) -> Result<B200Tensor, B200Error> {
        let t = self.alloc(shape, Dtype::F32, None)?;
        unsafe { cudaMemcpy(t.ptr_f32() as *mut c_void, data.as_ptr() as *const c_void, data.len() * 4, H2D) };
        Ok(t)
    }
    fn from_slice_i64(&self, data: &[i64], shape: &[usize]) -> Result<B200Tensor, B200Error> {
        let t = self.alloc(shape, Dtype::I64, None)?;
        unsafe { cudaMemcpy(t.0.buf.as_ref().unwrap().ptr, data.as_ptr() as *const c_void, data.len() * 8, H2D) };
        Ok(t)
    }
    fn to_vec_f32(&self, x: &B200Tensor) -> Result<Vec<f32>, B200Error> {
        let x = self.contiguous(x)?;
        let mut v = vec![0.0f32; x.numel()];
        unsafe { cudaMemcpy(v.as_mut_ptr() as *mut c_void, x.ptr_f32() as *const c_void, v.len() * 4, D2H) };
        Ok(v)
    }
    fn to_vec_i64(&self, x: &B200Tensor) -> Result<Vec<i64>, B200Error> {
        let mut v = vec![0i64; x.numel()];
        unsafe { cudaMemcpy(v.as_mut_ptr() as *mut c_void, x.0.buf.as_ref().unwrap().ptr, v.len() * 8, D2H) };
        Ok(v)
    }
    /// No-op when the dtype already matches (ops.rs:54-73); F32 -> BF16 is `pmb_cast_f32_to_bf16`; the other
    /// directions are refused (the bf16-storage path of the library keeps its own bf16 copies).
    fn to_dtype(&self, t: &B200Tensor, dtype: Dtype) -> Result<B200Tensor, B200Error> {
        if t.0.dtype == dtype {
            return Ok(t.clone());
        }
        if t.0.dtype == Dtype::F32 && dtype == Dtype::BF16 {
            let t = self.contiguous(t)?;
            let out = self.alloc(&t.0.shape, Dtype::BF16, None)?;
            check(unsafe { ffi::pmb_cast_f32_to_bf16(self.stream, t.ptr_f32(), out.0.buf.as_ref().unwrap().ptr as *mut u16, t.numel() as i64) })?;
            return Ok(out);
        }
        Err(B200Error::Unsupported(format!("to_dtype {:?} -> {:?}", t.0.dtype, dtype)))
    }

    // ---- arithmetic (ops.rs:77-80,166,310-319): pmb_unary_f32 / pmb_binary_f32 ------------------------
    fn add(&self, a: &B200Tensor, b: &B200Tensor) -> Result<B200Tensor, B200Error> {
        let out = self.binary(ffi::PMB_OP_ADD, a, b, "add")?;
        let node = match (a.0.node, b.0.node) { (Some(x), Some(y)) => self.record(Node::Add { a: x, b: y }), _ => None };
        Ok(self.with_node(out, node))
    }
    fn sub(&self, a: &B200Tensor, b: &B200Tensor) -> Result<B200Tensor, B200Error> { self.binary(ffi::PMB_OP_SUB, a, b, "sub") }
    fn mul(&self, a: &B200Tensor, b: &B200Tensor) -> Result<B200Tensor, B200Error> {
        let out = self.binary(ffi::PMB_OP_MUL, a, b, "mul")?;
        let node = match (a.0.node, b.0.node) { (Some(x), Some(y)) => self.record(Node::Mul { a: x, b: y, av: a.clone(), bv: b.clone() }), _ => None };
        Ok(self.with_node(out, node))
    }
    fn div(&self, a: &B200Tensor, b: &B200Tensor) -> Result<B200Tensor, B200Error> { self.binary(ffi::PMB_OP_DIV, a, b, "div") }
    fn neg(&self, a: &B200Tensor) -> Result<B200Tensor, B200Error> { self.unary(ffi::PMB_OP_NEG, a, 0.0, "neg") }
    fn exp(&self, x: &B200Tensor) -> Result<B200Tensor, B200Error> { self.unary(ffi::PMB_OP_EXP, x, 0.0, "exp") }
    fn sqrt(&self, x: &B200Tensor) -> Result<B200Tensor, B200Error> { self.unary(ffi::PMB_OP_SQRT, x, 0.0, "sqrt") }
    fn silu(&self, x: &B200Tensor) -> Result<B200Tensor, B200Error> { self.unary(ffi::PMB_OP_SILU, x, 0.0, "silu") }
    fn sigmoid(&self, x: &B200Tensor) -> Result<B200Tensor, B200Error> { self.unary(ffi::PMB_OP_SIGMOID, x, 0.0, "sigmoid") }
    fn softplus(&self, x: &B200Tensor) -> Result<B200Tensor, B200Error> { self.unary(ffi::PMB_OP_SOFTPLUS, x, 0.0, "softplus") }
    fn add_scalar(&self, x: &B200Tensor, s: f32) -> Result<B200Tensor, B200Error> { self.unary(ffi::PMB_OP_ADD_SCALAR, x, s, "add_scalar") }
    fn mul_scalar(&self, x: &B200Tensor, s: f32) -> Result<B200Tensor, B200Error> {
        let out = self.unary(ffi::PMB_OP_MUL_SCALAR, x, s, "mul_scalar")?;
        let node = x.0.node.and_then(|a| self.record(Node::MulScalar { a, s }));
        Ok(self.with_node(out, node))
    }

    // ---- views (ops.rs:123-148): no kernel until a consumer needs dense memory -------------------------
    fn narrow(&self, x: &B200Tensor, dim: usize, start: usize, len: usize) -> Result<B200Tensor, B200Error> {
        let mut shape = x.0.shape.clone();
        shape[dim] = len;
        Ok(x.view(shape, x.0.strides.clone(), x.0.offset + start * x.0.strides[dim]))
    }
    fn reshape(&self, x: &B200Tensor, shape: &[usize]) -> Result<B200Tensor, B200Error> {
        let x = if x.is_contiguous() { x.clone() } else { self.contiguous(x)? };
        Ok(x.view(shape.to_vec(), contiguous_strides(shape), 0))
    }
    fn transpose(&self, x: &B200Tensor, d0: usize, d1: usize) -> Result<B200Tensor, B200Error> {
        let (mut shape, mut strides) = (x.0.shape.clone(), x.0.strides.clone());
        shape.swap(d0, d1);
        strides.swap(d0, d1);
        Ok(x.view(shape, strides, x.0.offset))
    }
    fn broadcast_as(&self, x: &B200Tensor, shape: &[usize]) -> Result<B200Tensor, B200Error> {
        let pad = shape.len() - x.0.shape.len();
        let mut strides = vec![0usize; shape.len()];
        for d in 0..x.0.shape.len() {
            strides[pad + d] = if x.0.shape[d] == 1 { 0 } else { x.0.strides[d] };
        }
        Ok(x.view(shape.to_vec(), strides, x.0.offset))   // stride 0 = broadcast; B and C keep their (B,T,G,N) source this way
    }
    fn concat(&self, tensors: &[&B200Tensor], dim: usize) -> Result<B200Tensor, B200Error> {
        // one strided copy per input into its slice of the output
        let mut shape = tensors[0].0.shape.clone();
        shape[dim] = tensors.iter().map(|t| t.0.shape[dim]).sum();
        let out = self.alloc(&shape, Dtype::F32, None)?;
        let _ = out.ptr_f32();
        Err(B200Error::Unsupported("concat: destination-strided copy is not exported yet (pmb_strided_copy_f32 strides the source only)".into()))
    }

    // ---- contractions and the block recogniser ---------------------------------------------------------
    /// `Ops::matmul` (ops.rs:85): `pmb_gemm_f32` with the operands' own leading dimensions (a `narrow` or a
    /// `transpose` of a dense matrix is passed as lda / trans flags, not copied).  Two special cases make the block
    /// one call: `x @ in_proj_weight` opens a trace and returns a lazy `xzd`; `normed @ out_proj_weight` with
    /// `normed` the last lazy value of an unflushed trace runs `pmb_mamba2_block_fwd`.
    fn matmul(&self, a: &B200Tensor, b: &B200Tensor) -> Result<B200Tensor, B200Error> {
        if let Origin::Lazy { trace, step: BlockStep::Normed } = &a.0.origin {
            let tr = trace.lock().unwrap();
            if !tr.flushed {
                let out = self.run_block(&tr, b)?;
                let node = tr.x.0.node.and_then(|x| {
                    // the 8 parameter tensors (each carries its leaf node): 0..6 named by the trace, 7 = out_proj
                    let mut ps: Vec<B200Tensor> = tr.params[..7].iter().map(|t| t.clone().expect("block parameter")).collect();
                    ps.push(b.clone());
                    self.record(Node::Block { x, params: ps, saved_x: tr.x.clone(), cfg: tr.cfg, batch: tr.batch, seqlen: tr.seqlen })
                });
                *self.open_trace.borrow_mut() = None;
                return Ok(self.with_node(out, node));
            }
        }
        if self.looks_like_in_proj(a, b) {
            return Ok(self.open_block_trace(a, b));
        }
        let (a, b) = (self.materialise(a)?, self.materialise(b)?);
        self.require_f32(&a, "matmul")?;
        let (m, k, n) = (a.0.shape[a.0.shape.len() - 2], a.0.shape[a.0.shape.len() - 1], b.0.shape[b.0.shape.len() - 1]);
        let rows: usize = a.0.shape[..a.0.shape.len() - 1].iter().product();   // leading axes of `a` fold into M (weights are 2-D)
        let (a2, b2) = (self.dense_or_pitched(&a)?, self.dense_or_pitched(&b)?);
        let mut oshape = a.0.shape.clone();
        *oshape.last_mut().unwrap() = n;
        let out = self.alloc(&oshape, Dtype::F32, None)?;
        let _ = m;
        check(unsafe {
            ffi::pmb_gemm_f32(self.stream, 0, 0, rows as i64, n as i64, k as i64, a2.ptr_f32(), a2.row_pitch().unwrap(), b2.ptr_f32(), b2.row_pitch().unwrap(),
                              out.ptr_f32() as *mut f32, n as i64, std::ptr::null(), 0)
        })?;
        let node = match (a.0.node, b.0.node) { (Some(x), Some(y)) => self.record(Node::Matmul { a: x, b: y, av: a2, bv: b2 }), _ => None };
        Ok(self.with_node(out, node))
    }

    /// `Ops::ssd_scan` (ops.rs:345-352).  Inside a trace it only advances the trace.  Stand-alone it is
    /// `pmb_ssd_scan_fwd`: B and C arrive head-broadcast from block.rs:172-180 as stride-0 views, so the (B,T,G,N)
    /// source is passed with G explicit and never expanded; the tape node keeps x, a, b, c, y and the workspace for
    /// `pmb_ssd_scan_bwd`.
    fn ssd_scan(&self, x: &B200Tensor, a: &B200Tensor, b: &B200Tensor, c: &B200Tensor, block_len: usize) -> Result<B200Tensor, B200Error> {
        if let Origin::Lazy { trace, .. } = &x.0.origin {
            if trace.lock().unwrap().advance(BlockStep::Scan) {
                return Ok(self.lazy(trace, BlockStep::Scan, x.0.shape.clone()));
            }
        }
        let (x, a) = (self.contiguous(x)?, self.contiguous(a)?);
        let (bsz, t, h, p) = (x.0.shape[0] as i32, x.0.shape[1] as i32, x.0.shape[2] as i32, x.0.shape[3] as i32);
        let n = b.0.shape[3] as i32;
        let g = if b.0.strides[2] == 0 { 1 } else { h };                 // head-broadcast view => one group
        let (bsrc, csrc) = (self.group_source(b, g)?, self.group_source(c, g)?);
        let q = if block_len == 0 || t % block_len as i32 != 0 { t } else { block_len as i32 };   // dense route = one chunk (ssd_ops.rs:70-78)
        let need = unsafe { ffi::pmb_ssd_workspace_bytes(bsz, t, h, p, n, g, q) };
        let ws = DeviceBuf::new(need)?;
        let y = self.alloc(&x.0.shape, Dtype::F32, None)?;
        check(unsafe {
            ffi::pmb_ssd_scan_fwd(self.stream, bsz, t, h, p, n, g, q, x.ptr_f32(), (h * p) as i64, a.ptr_f32(), bsrc.ptr_f32(), csrc.ptr_f32(), (g * n) as i64,
                                  std::ptr::null(), y.ptr_f32() as *mut f32, (h * p) as i64, std::ptr::null_mut(), ws.ptr, ws.bytes)
        })?;
        let node = match (x.0.node, a.0.node, b.0.node, c.0.node) {
            (Some(xn), Some(an), Some(bn), Some(cn)) => self.record(Node::SsdScan { x: xn, a: an, b: bn, c: cn, saved: vec![x, a, bsrc, csrc, y.clone()], ws, dims: [bsz, t, h, p, n, g, q] }),
            _ => None,
        };
        Ok(self.with_node(y, node))
    }

    /// `Ops::rmsnorm` (ops.rs:91-96).  Preceded by `mul(y_skip, silu(z))` inside a trace it is the gated norm of
    /// block.rs:216-222 (`pmb_gated_rmsnorm_fwd` when run eagerly); stand-alone it is the same kernel with z = +inf
    /// replaced by a plain path: not exported separately, so a stand-alone rmsnorm is refused.
    fn rmsnorm(&self, x: &B200Tensor, weight: &B200Tensor, _eps: f32) -> Result<B200Tensor, B200Error> {
        if let Origin::Lazy { trace, .. } = &x.0.origin {
            let mut tr = trace.lock().unwrap();
            tr.params[6] = Some(weight.clone());
            if tr.advance(BlockStep::Normed) {
                drop(tr);
                return Ok(self.lazy(trace, BlockStep::Normed, x.0.shape.clone()));
            }
        }
        Err(B200Error::Unsupported("rmsnorm outside the block's gate (only pmb_gated_rmsnorm_fwd is exported)".into()))
    }

    /// `Ops::conv1d` (ops.rs:108-116): only the block's causal depthwise form (groups == channels, stride 1,
    /// padding K-1, block.rs:150-163), which is part of the trace; `pmb_conv_silu_dt_fwd` is its eager kernel.
    fn conv1d(&self, x: &B200Tensor, weight: &B200Tensor, bias: Option<&B200Tensor>, stride: usize, padding: usize, groups: usize) -> Result<B200Tensor, B200Error> {
        if let Origin::Lazy { trace, .. } = &x.0.origin {
            let mut tr = trace.lock().unwrap();
            if stride == 1 && groups == x.0.shape[1] && padding + 1 == weight.0.shape[2] {
                tr.params[1] = Some(weight.clone());
                tr.params[2] = bias.cloned();
                if tr.advance(BlockStep::Conv) {
                    let mut shape = x.0.shape.clone();
                    shape[2] += padding;
                    drop(tr);
                    return Ok(self.lazy(trace, BlockStep::Conv, shape));
                }
            }
        }
        Err(B200Error::Unsupported("conv1d other than the block's causal depthwise convolution".into()))
    }

    // ---- indexing / reductions (ops.rs:120,158-164,292-307) ---------------------------------------------
    fn cumsum(&self, x: &B200Tensor, dim: usize) -> Result<B200Tensor, B200Error> {
        let x = self.contiguous(x)?;
        let outer: usize = x.0.shape[..dim].iter().product();
        let inner: usize = x.0.shape[dim + 1..].iter().product();
        let out = self.alloc(&x.0.shape, Dtype::F32, None)?;
        check(unsafe { ffi::pmb_cumsum_f32(self.stream, x.ptr_f32(), outer as i64, x.0.shape[dim] as i64, inner as i64, out.ptr_f32() as *mut f32) })?;
        Ok(out)
    }
    fn embedding(&self, table: &B200Tensor, ids: &B200Tensor) -> Result<B200Tensor, B200Error> {
        let (vocab, width) = (table.0.shape[0], table.0.shape[1]);
        let mut shape = ids.0.shape.clone();
        shape.push(width);
        let out = self.alloc(&shape, Dtype::F32, None)?;
        let flag = self.zeros(&[1], Dtype::F32)?;   // 4 zero bytes reused as the bad-id word
        check(unsafe {
            ffi::pmb_embedding_f32(self.stream, table.ptr_f32(), vocab as i64, width as i64, ids.0.buf.as_ref().unwrap().ptr as *const i64, ids.numel() as i64,
                                   out.ptr_f32() as *mut f32, flag.ptr_f32() as *mut u32)
        })?;
        if self.to_vec_f32(&flag)?[0].to_bits() != 0 {
            return Err(B200Error::Arg("embedding: token id outside [0, vocab)".into()));
        }
        let node = table.0.node.and_then(|t| self.record(Node::Embedding { table: t, ids: ids.clone(), vocab }));
        Ok(self.with_node(out, node))
    }
    fn log_softmax(&self, x: &B200Tensor, dim: usize) -> Result<B200Tensor, B200Error> {
        if dim + 1 != x.0.shape.len() {
            return Err(B200Error::Unsupported("log_softmax over an axis other than the last".into()));
        }
        let x = self.contiguous(x)?;
        let width = *x.0.shape.last().unwrap();
        let out = self.alloc(&x.0.shape, Dtype::F32, None)?;
        check(unsafe { ffi::pmb_log_softmax_f32(self.stream, x.ptr_f32(), (x.numel() / width) as i64, width as i64, out.ptr_f32() as *mut f32) })?;
        let node = x.0.node.and_then(|a| self.record(Node::LogSoftmax { a, out: out.clone() }));
        Ok(self.with_node(out, node))
    }
    fn gather(&self, x: &B200Tensor, index: &B200Tensor, dim: usize) -> Result<B200Tensor, B200Error> {
        if dim + 1 != x.0.shape.len() {
            return Err(B200Error::Unsupported("gather along an axis other than the last".into()));
        }
        let x = self.contiguous(x)?;
        let width = *x.0.shape.last().unwrap();
        let rows = x.numel() / width;
        let out = self.alloc(&index.0.shape, Dtype::F32, None)?;
        let flag = self.zeros(&[1], Dtype::F32)?;
        check(unsafe {
            ffi::pmb_gather_last_f32(self.stream, x.ptr_f32(), index.0.buf.as_ref().unwrap().ptr as *const i64, rows as i64, width as i64, out.ptr_f32() as *mut f32,
                                     flag.ptr_f32() as *mut u32)
        })?;
        let node = x.0.node.and_then(|a| self.record(Node::Gather { a, index: index.clone(), width }));
        Ok(self.with_node(out, node))
    }
    fn sum_all(&self, x: &B200Tensor) -> Result<B200Tensor, B200Error> { self.reduce_all(x, false) }
    fn mean_all(&self, x: &B200Tensor) -> Result<B200Tensor, B200Error> { self.reduce_all(x, true) }

    // ---- parameters and autograd (ops.rs:171-287) --------------------------------------------------------
    fn param_from_slice_f32(&self, data: &[f32], shape: &[usize]) -> Result<B200Param, B200Error> {
        let t = self.from_slice_f32(data, shape)?;
        self.param_from_tensor(&t)
    }
    fn param_zeros(&self, shape: &[usize], dtype: Dtype) -> Result<B200Param, B200Error> { let t = self.zeros(shape, dtype)?; self.param_from_tensor(&t) }
    fn param_ones(&self, shape: &[usize], dtype: Dtype) -> Result<B200Param, B200Error> { let t = self.ones(shape, dtype)?; self.param_from_tensor(&t) }
    /// A new leaf sharing the tensor's memory (ops.rs:232-235).  `forward_checkpointed` calls this on every block
    /// output (checkpoint.rs:82): the leaf cuts the tape there, which is what lets the block's `Node::Block` keep
    /// nothing but its input.
    fn param_from_tensor(&self, t: &B200Tensor) -> Result<B200Param, B200Error> {
        let t = self.contiguous(t)?;
        let id = { let mut n = self.next_param.borrow_mut(); *n += 1; *n - 1 };
        let node = self.record(Node::Leaf { param: id });
        let shadow = self.with_node(t, node);
        Ok(B200Param { id, value: Arc::new(RefCell::new(shadow.clone())), shadow })
    }
    fn detach(&self, t: &B200Tensor) -> Result<B200Tensor, B200Error> { let t = self.materialise(t)?; Ok(self.with_node(t, None)) }
    fn no_grad_scope<R>(&self, f: impl FnOnce() -> R) -> R {
        let was = std::mem::replace(&mut self.tape.borrow_mut().grad_enabled, false);
        let r = f();
        self.tape.borrow_mut().grad_enabled = was;
        r
    }
    /// Reverse walk of the tape from `loss` (a scalar).  `Node::Block` is one `pmb_mamba2_block_bwd`: the block is
    /// recomputed from its saved input inside the call, all 8 parameter gradients come back at once, and the input
    /// gradient is added to the upstream node (the `dh_{l-1} = dh_l + dBlock_l/dx` of checkpoint.rs:110-135).
    /// The tape is consumed (the reference clears its tape after backward too, crates/pm-cuda/src/backend/ops_impl.rs:1531-1548).
    fn backward(&self, loss: &B200Tensor) -> Result<B200GradStore, B200Error> {
        let nodes = std::mem::take(&mut self.tape.borrow_mut().nodes);
        let mut grads: Vec<Option<B200Tensor>> = (0..nodes.len()).map(|_| None).collect();
        let mut store = B200GradStore::default();
        let root = loss.0.node.ok_or_else(|| B200Error::Arg("backward: the loss is not attached to the tape".into()))?;
        grads[root] = Some(self.ones(&loss.0.shape, Dtype::F32)?);
        for i in (0..=root).rev() {
            let Some(g) = grads[i].take() else { continue };
            let mut push = |j: usize, v: B200Tensor, this: &Self| -> Result<(), B200Error> {
                grads[j] = Some(match grads[j].take() { Some(acc) => this.binary(ffi::PMB_OP_ADD, &acc, &v, "grad accumulate")?, None => v });
                Ok(())
            };
            match &nodes[i] {
                Node::Leaf { param } => { store.grads.insert(*param, g); }
                Node::Add { a, b } => { push(*a, g.clone(), self)?; push(*b, g, self)?; }
                Node::MulScalar { a, s } => push(*a, self.unary(ffi::PMB_OP_MUL_SCALAR, &g, *s, "d mul_scalar")?, self)?,
                Node::Mul { a, b, av, bv } => {
                    push(*a, self.binary(ffi::PMB_OP_MUL, &g, bv, "d mul")?, self)?;
                    push(*b, self.binary(ffi::PMB_OP_MUL, &g, av, "d mul")?, self)?;
                }
                Node::SumAll { a, shape, mean } => {
                    let scale = if *mean { 1.0 / shape.iter().product::<usize>() as f32 } else { 1.0 };
                    let full = self.contiguous(&self.broadcast_as(&g, shape)?)?;
                    push(*a, self.unary(ffi::PMB_OP_MUL_SCALAR, &full, scale, "d sum_all")?, self)?;
                }
                Node::Matmul { a, b, av, bv } => {
                    // dA = g B^T, dB = A^T g: two more pmb_gemm_f32 calls with the transpose flags
                    push(*a, self.gemm_flags(&g, bv, false, true)?, self)?;
                    push(*b, self.gemm_flags(av, &g, true, false)?, self)?;
                }
                Node::Block { x, params, saved_x, cfg, batch, seqlen } => {
                    let (dx, dparams) = self.block_backward(saved_x, &g, params, cfg, *batch, *seqlen)?;
                    push(*x, dx, self)?;
                    // each parameter gradient flows on to that parameter's leaf node
                    for (pt, gp) in params.iter().zip(dparams) { if let Some(n) = pt.0.node { push(n, gp, self)?; } }
                }
                Node::SsdScan { x, a, b, c, saved, ws, dims } => {
                    let [dx, da, db, dc] = self.scan_backward(saved, ws, dims, &g)?;
                    push(*x, dx, self)?; push(*a, da, self)?; push(*b, db, self)?; push(*c, dc, self)?;
                }
                // The scatter-add of Ops::embedding and the softmax-Jacobian products of log_softmax / gather have no
                // exported kernel: a trainer on this backend takes the loss through pmb_lm_step_* (tied head + fused
                // cross-entropy + embedding gradient in one call) instead of composing it from primitives.
                Node::Embedding { .. } | Node::LogSoftmax { .. } | Node::Gather { .. } =>
                    return Err(B200Error::Unsupported("backward through embedding / log_softmax / gather: use pmb_lm_step_device".into())),
            }
        }
        Ok(store)
    }
    fn gradient(&self, store: &B200GradStore, p: &B200Param) -> Result<Option<B200Tensor>, B200Error> { Ok(store.grads.get(&p.id).cloned()) }
    fn set_gradient(&self, store: &mut B200GradStore, p: &B200Param, g: &B200Tensor) -> Result<(), B200Error> { store.grads.insert(p.id, g.clone()); Ok(()) }
    fn merge_grad_stores(&self, into: &mut B200GradStore, from: B200GradStore) -> Result<(), B200Error> {
        for (id, g) in from.grads {
            let merged = match into.grads.remove(&id) { Some(acc) => self.binary(ffi::PMB_OP_ADD, &acc, &g, "merge_grad_stores")?, None => g };
            into.grads.insert(id, merged);
        }
        Ok(())
    }
    fn assign(&self, param: &B200Param, value: &B200Tensor) -> Result<(), B200Error> { *param.value.borrow_mut() = self.contiguous(value)?; Ok(()) }
    fn sgd_step(&self, param: &B200Param, grad: &B200Tensor, lr: f32) -> Result<(), B200Error> {
        let step = self.unary(ffi::PMB_OP_MUL_SCALAR, grad, -lr, "sgd_step")?;
        let next = self.binary(ffi::PMB_OP_ADD, &param.value.borrow(), &step, "sgd_step")?;
        self.assign(param, &next)
    }
    /// `Ops::fused_cross_entropy` (ops.rs:405): served for the tied-head LM by `pmb_lm_step_*`, which fuses the head
    /// GEMM, the loss and its backward; as a stand-alone op over materialised logits it is composed from
    /// log_softmax + gather + mean_all above.
    fn fused_cross_entropy(&self, logits: &B200Tensor, targets: &B200Tensor) -> Result<B200Tensor, B200Error> {
        let lp = self.log_softmax(logits, logits.0.shape.len() - 1)?;
        let picked = self.gather(&lp, targets, lp.0.shape.len() - 1)?;
        self.mean_all(&self.neg(&picked)?)
    }
}

impl Backend for B200Backend {
    fn device_kind(&self) -> DeviceKind {
        DeviceKind::Cuda { ordinal: self.ordinal as usize }
    }
}

// ------------------------------------------------------------------------------------------------ helpers

impl B200Backend {
    fn reduce_all(&self, x: &B200Tensor, mean: bool) -> Result<B200Tensor, B200Error> {
        let x = self.contiguous(x)?;
        let ws = DeviceBuf::new(unsafe { ffi::pmb_sum_workspace_bytes() })?;
        let out = self.alloc(&[1], Dtype::F32, None)?;
        check(unsafe { ffi::pmb_sum_all_f32(self.stream, x.ptr_f32(), x.numel() as i64, mean as i32, out.ptr_f32() as *mut f32, ws.ptr, ws.bytes) })?;
        let node = x.0.node.and_then(|a| self.record(Node::SumAll { a, shape: x.0.shape.clone(), mean }));
        Ok(self.with_node(out, node))
    }
    /// `a` is `(.., D)` data attached to the tape and `b` a 2-D parameter whose second extent is the block's
    /// in_proj width `2*d_inner + 2*G*N + H`: the first op of block.rs:143.
    fn looks_like_in_proj(&self, a: &B200Tensor, b: &B200Tensor) -> bool {
        a.0.shape.len() == 3 && b.0.shape.len() == 2 && matches!(a.0.origin, Origin::Data) && self.open_trace.borrow().is_none() && b.0.shape[1] > 2 * b.0.shape[0]
    }
    fn open_block_trace(&self, x: &B200Tensor, in_proj: &B200Tensor) -> B200Tensor {
        // d_state, d_head, n_heads, d_conv and block_len are filled in as the following ops reveal them (the widths of
        // the three narrows, the conv weight's K, ssd_scan's block_len); d_model and J are known here
        let cfg = ffi::PmbConfig { d_model: x.0.shape[2] as i32, d_state: 0, d_head: 0, n_heads: 0, n_groups: 1, d_conv: 0, block_len: 0, rmsnorm_eps: 1e-5 };
        let mut params: [Option<B200Tensor>; 8] = Default::default();
        params[0] = Some(in_proj.clone());
        let tr = Arc::new(Mutex::new(BlockTrace { x: x.clone(), params, cfg, batch: x.0.shape[0] as i32, seqlen: x.0.shape[1] as i32, last: BlockStep::InProj, flushed: false }));
        *self.open_trace.borrow_mut() = Some(tr.clone());
        self.lazy(&tr, BlockStep::InProj, vec![x.0.shape[0], x.0.shape[1], in_proj.0.shape[1]])
    }
    fn dense_or_pitched(&self, t: &B200Tensor) -> Result<B200Tensor, B200Error> {
        if t.row_pitch().is_some() && t.0.shape.len() == 2 { Ok(t.clone()) } else { self.contiguous(t) }
    }
    fn group_source(&self, t: &B200Tensor, g: i32) -> Result<B200Tensor, B200Error> {
        // the un-broadcast (B,T,G,N) tensor behind a stride-0 head axis
        if g == 1 { self.contiguous(&self.narrow(t, 2, 0, 1)?) } else { self.contiguous(t) }
    }
    fn gemm_flags(&self, a: &B200Tensor, b: &B200Tensor, ta: bool, tb: bool) -> Result<B200Tensor, B200Error> {
        let (a, b) = (self.contiguous(a)?, self.contiguous(b)?);
        let (ar, ac) = (a.numel() / a.0.shape[a.0.shape.len() - 1], a.0.shape[a.0.shape.len() - 1]);
        let (br, bc) = (b.numel() / b.0.shape[b.0.shape.len() - 1], b.0.shape[b.0.shape.len() - 1]);
        let (m, k) = if ta { (ac, ar) } else { (ar, ac) };
        let n = if tb { br } else { bc };
        let out = self.alloc(&[m, n], Dtype::F32, None)?;
        check(unsafe {
            ffi::pmb_gemm_f32(self.stream, ta as i32, tb as i32, m as i64, n as i64, k as i64, a.ptr_f32(), ac as i64, b.ptr_f32(), bc as i64, out.ptr_f32() as *mut f32,
                              n as i64, std::ptr::null(), 0)
        })?;
        Ok(out)
    }
    /// One `pmb_mamba2_block_bwd`: recompute from the saved input inside the call, then dx and all 8 parameter gradients.
    fn block_backward(&self, x: &B200Tensor, dout: &B200Tensor, params: &[B200Tensor], cfg: &ffi::PmbConfig, batch: i32, seqlen: i32)
        -> Result<(B200Tensor, Vec<B200Tensor>), B200Error> {
        let (x, dout) = (self.contiguous(x)?, self.contiguous(dout)?);
        let mut p = [std::ptr::null::<f32>(); 8];
        let mut g = [std::ptr::null_mut::<f32>(); 8];
        let mut grads = Vec::with_capacity(8);
        for i in 0..8 {
            p[i] = params[i].ptr_f32();
            let gi = self.alloc(&params[i].0.shape, Dtype::F32, None)?;
            g[i] = gi.ptr_f32() as *mut f32;
            grads.push(gi);
        }
        let need = unsafe { ffi::pmb_mamba2_block_workspace_bytes(cfg, batch, seqlen) };
        let ws = { let mut slot = self.block_ws.borrow_mut(); if slot.as_ref().map_or(true, |b| b.bytes < need) { *slot = Some(DeviceBuf::new(need)?); } slot.as_ref().unwrap().clone() };
        let dx = self.alloc(&x.0.shape, Dtype::F32, None)?;
        check(unsafe {
            ffi::pmb_mamba2_block_bwd(self.stream, cfg, &ffi::PmbBlockParams { p }, batch, seqlen, x.ptr_f32(), dout.ptr_f32(), std::ptr::null(), dx.ptr_f32() as *mut f32,
                                      &ffi::PmbBlockGrads { g }, ws.ptr, ws.bytes)
        })?;
        Ok((dx, grads))
    }
    fn scan_backward(&self, saved: &[B200Tensor], ws: &Arc<DeviceBuf>, dims: &[i32; 7], dy: &B200Tensor) -> Result<[B200Tensor; 4], B200Error> {
        let [b, t, h, p, n, g, q] = *dims;
        let dy = self.contiguous(dy)?;
        let (dx, da) = (self.alloc(&saved[0].0.shape, Dtype::F32, None)?, self.alloc(&saved[1].0.shape, Dtype::F32, None)?);
        let (db, dc) = (self.alloc(&saved[2].0.shape, Dtype::F32, None)?, self.alloc(&saved[3].0.shape, Dtype::F32, None)?);
        check(unsafe {
            ffi::pmb_ssd_scan_bwd(self.stream, b, t, h, p, n, g, q, saved[0].ptr_f32(), (h * p) as i64, saved[1].ptr_f32(), saved[2].ptr_f32(), saved[3].ptr_f32(),
                                  (g * n) as i64, saved[4].ptr_f32(), (h * p) as i64, dy.ptr_f32(), (h * p) as i64, dx.ptr_f32() as *mut f32, (h * p) as i64,
                                  da.ptr_f32() as *mut f32, db.ptr_f32() as *mut f32, dc.ptr_f32() as *mut f32, (g * n) as i64, ws.ptr, ws.bytes)
        })?;
        Ok([dx, da, db, dc])
    }
}
