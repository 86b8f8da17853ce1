"""Host-side mirror of the reference's operator interface for the Mamba2 SSD block path,
bound to libpm_b200.so (hand-written sm_100a CUDA) through its C ABI with ctypes.

Names follow the reference: `Mamba2Config` / `Mamba2Block.forward` / `Mamba2Block.step`
(crates/pm-core/src/mamba2/block.rs:48-88,118-226,278-417), `ssd_scan` (crates/pm-core/src/ops.rs:345-352),
`ContextEncoder.forward_checkpointed` + `checkpoint_backward` (photon/encoder.rs:73-87, checkpoint.rs:110-135),
`FlatMamba` (flat.rs:89-161).  torch is used only to own device memory and streams; every computation is a
call into the library, and there is no CPU or eager-PyTorch fallback: a missing library raises ImportError.
"""
from __future__ import annotations

import ctypes as C
import pathlib
from dataclasses import dataclass

import torch

_HERE = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libpm_b200.so"

PARAM_ORDER = ("in_proj_weight", "conv1d_weight", "conv1d_bias", "a_log", "d_skip", "dt_bias",
               "norm_weight", "out_proj_weight")


class PmbError(RuntimeError):
    """Raised when a library call returns a non-zero pmb_status (the reference's typed backend error,
    crates/pm-cuda/src/error.rs:4-23)."""

    def __init__(self, status: int, text: str):
        super().__init__(f"pm_b200 status {status}: {text}")
        self.status = status


class _Cfg(C.Structure):
    _fields_ = [("d_model", C.c_int32), ("d_state", C.c_int32), ("d_head", C.c_int32), ("n_heads", C.c_int32),
                ("n_groups", C.c_int32), ("d_conv", C.c_int32), ("block_len", C.c_int32), ("rmsnorm_eps", C.c_float)]


class _Params(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in PARAM_ORDER]


LAYER_CALLBACK = C.CFUNCTYPE(None, C.c_int32, C.c_void_p)


def _load():
    if not _LIB_PATH.exists():
        raise ImportError(f"{_LIB_PATH} is missing: build it with `python photon-mamba2-llm_b200/build.py` "
                          "(there is no fallback path)")
    lib = C.CDLL(str(_LIB_PATH))
    vp, i32, i64, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
    cfgp = C.POINTER(_Cfg)
    sig = {
        "pmb_last_error": (C.c_char_p, []),
        "pmb_version": (C.c_char_p, []),
        "pmb_launch_count": (i64, []),
        "pmb_device_status": (i32, [C.POINTER(i32)]),
        "pmb_profile_start": (None, []),
        "pmb_profile_stop": (i32, [C.c_char_p, sz]),
        "pmb_gemm_f32": (i32, [vp, i32, i32, i64, i64, i64, vp, i64, vp, i64, vp, i64, vp, i32]),
        "pmb_gemm_reserve_scratch": (i32, [C.c_size_t]),
        "pmb_set_concurrency": (None, [i32]),
        "pmb_gemm_bf16": (i32, [vp, i32, i32, i64, i64, i64, vp, i64, vp, i64, vp, i64, vp, i32]),
        "pmb_cast_f32_to_bf16": (i32, [vp, vp, vp, i64]),
        "pmb_mamba2_block_workspace_bytes_bf16": (sz, [cfgp, i32, i32]),
        "pmb_mamba2_block_fwd_bf16": (i32, [vp, cfgp, C.POINTER(_Params), vp, vp, i32, i32, vp, vp, vp, vp, sz]),
        "pmb_mamba2_block_bwd_bf16": (i32, [vp, cfgp, C.POINTER(_Params), vp, vp, i32, i32, vp, vp, vp, vp, C.POINTER(_Params), vp, sz]),
        "pmb_conv_silu_dt_fwd": (i32, [vp, cfgp, i32, i32, vp, vp, vp, vp, vp, vp]),
        "pmb_conv_bwd_workspace_bytes": (sz, [cfgp, i32, i32]),
        "pmb_conv_silu_bwd": (i32, [vp, cfgp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, sz]),
        "pmb_ssd_workspace_bytes": (sz, [i32] * 7),
        "pmb_ssd_scan_fwd": (i32, [vp] + [i32] * 7 + [vp, i64, vp, vp, vp, i64, vp, vp, i64, vp, vp, sz]),
        "pmb_ssd_scan_bwd": (i32, [vp] + [i32] * 7 + [vp, i64, vp, vp, vp, i64, vp, i64, vp, i64, vp, i64, vp, vp, vp, i64, vp, sz]),
        "pmb_ssd_workspace_bytes_bf16": (sz, [i32] * 7),
        "pmb_ssd_scan_fwd_bf16": (i32, [vp] + [i32] * 7 + [vp, vp, vp, vp, vp, vp, vp, vp, sz]),
        "pmb_ssd_scan_bwd_bf16": (i32, [vp] + [i32] * 7 + [vp, vp, vp, vp, vp, vp, vp, sz]),
        "pmb_gated_rmsnorm_fwd": (i32, [vp, i64, i32, f32, vp, vp, i64, vp, vp, vp]),
        "pmb_gated_rmsnorm_bwd_workspace_bytes": (sz, [i64, i32]),
        "pmb_gated_rmsnorm_bwd": (i32, [vp, i64, i32, vp, vp, vp, i64, vp, vp, vp, vp, i64, vp, vp, sz]),
        "pmb_gated_rmsnorm_bwd_static_max_bytes": (sz, []),
        "pmb_gated_rmsnorm_bwd_static": (i32, [vp, i64, i32, vp, vp, vp, i64, vp, vp, vp, vp, i64, vp]),
        "pmb_mamba2_block_workspace_bytes": (sz, [cfgp, i32, i32]),
        "pmb_stack_workspace_bytes": (sz, [cfgp, i32, i32]),
        "pmb_lm_save_safetensors": (i32, [vp, vp, C.c_char_p]),
        "pmb_lm_load_safetensors": (i32, [vp, vp, C.c_char_p]),
        "pmb_safetensors_save_f32": (i32, [C.c_char_p, i32, C.POINTER(i64), C.POINTER(i32), C.POINTER(vp)]),
        "pmb_safetensors_load_f32": (i32, [C.c_char_p, i32, C.POINTER(i64), C.POINTER(i32), C.POINTER(vp)]),
        "pmb_mamba2_block_fwd": (i32, [vp, cfgp, C.POINTER(_Params), i32, i32, vp, vp, vp, vp, sz]),
        "pmb_mamba2_block_bwd": (i32, [vp, cfgp, C.POINTER(_Params), i32, i32, vp, vp, vp, vp, C.POINTER(_Params), vp, sz]),
        "pmb_mamba2_step_workspace_bytes": (sz, [cfgp, i32]),
        "pmb_mamba2_step": (i32, [vp, cfgp, C.POINTER(_Params), i32, vp, vp, vp, vp, vp, sz]),
        "pmb_stack_fwd_ckpt": (i32, [vp, cfgp, i32, C.POINTER(_Params), i32, i32, vp, vp, sz]),
        "pmb_stack_bwd": (i32, [vp, cfgp, i32, C.POINTER(_Params), C.POINTER(_Params), i32, i32, vp, vp, vp, sz, LAYER_CALLBACK, vp]),
        "pmb_grad_sumsq_workspace_bytes": (sz, []),
        "pmb_grad_sumsq": (i32, [vp, i64, vp, vp, vp, sz]),
        "pmb_adamw_step": (i32, [vp, i64, vp, vp, vp, vp, f32, f32, f32, f32, f32, i32, f32, vp]),
        "pmb_lm_create": (i32, [cfgp, i32, i32, i32, i32, C.POINTER(vp)]),
        "pmb_lm_create_dtype": (i32, [cfgp, i32, i32, i32, i32, i32, C.POINTER(vp)]),
        "pmb_lm_create_hier": (i32, [cfgp, i32, i32, i32, i32, i32, i32, i32, C.POINTER(vp)]),
        "pmb_lm_destroy": (None, [vp]),
        "pmb_lm_param_count": (i64, [vp]),
        "pmb_lm_param_offset": (i64, [vp, i32, i32]),
        "pmb_lm_params": (vp, [vp]),
        "pmb_lm_grads": (vp, [vp]),
        "pmb_lm_activation_bytes": (i64, [vp]),
        "pmb_lm_activation_detail": (None, [vp, C.POINTER(i64)]),
        "pmb_lm_step_device": (i32, [vp, vp, vp, vp, LAYER_CALLBACK, vp]),
        "pmb_lm_loss_device": (vp, [vp]),
        "pmb_lm_step_host": (i32, [vp, vp, vp, vp, C.POINTER(f32), LAYER_CALLBACK, vp]),
        "pmb_lm_bad_tokens": (i32, [vp, vp, C.POINTER(i32)]),
        "pmb_unary_f32": (i32, [vp, i32, vp, f32, vp, i64]),
        "pmb_binary_f32": (i32, [vp, i32, vp, vp, vp, i64]),
        "pmb_strided_copy_f32": (i32, [vp, vp, i32, C.POINTER(i64), C.POINTER(i64), i64, vp]),
        "pmb_embedding_f32": (i32, [vp, vp, i64, i64, vp, i64, vp, vp]),
        "pmb_gather_last_f32": (i32, [vp, vp, vp, i64, i64, vp, vp]),
        "pmb_log_softmax_f32": (i32, [vp, vp, i64, i64, vp]),
        "pmb_sum_workspace_bytes": (sz, []),
        "pmb_sum_all_f32": (i32, [vp, vp, i64, i32, vp, vp, sz]),
        "pmb_cumsum_f32": (i32, [vp, vp, i64, i64, i64, vp]),
        "pmb_dp_unique_id": (i32, [vp]),
        "pmb_dp_init": (i32, [i32, i32, vp, C.POINTER(vp)]),
        "pmb_dp_destroy": (None, [vp]),
        "pmb_dp_world_size": (i32, [vp]),
        "pmb_dp_allreduce_async": (i32, [vp, vp, vp, i64]),
        "pmb_dp_allgather_async": (i32, [vp, vp, vp, vp, i64]),
        "pmb_dp_sync": (i32, [vp, vp]),
        "pmb_lm_step_device_dp": (i32, [vp, vp, vp, vp, vp]),
        "pmb_selftest_bounded_wait": (i32, [vp, C.c_uint32]),
        "pmb_selftest_device_once": (i32, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)   # AttributeError here = the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib, sorted(sig)


lib, EXPORTED = _load()


def _check(status: int):
    if status != 0:
        raise PmbError(status, lib.pmb_last_error().decode())


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def _dev(t: torch.Tensor, name: str) -> torch.Tensor:
    if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise PmbError(2, f"{name}: expected a contiguous float32 CUDA tensor, got {t.dtype} on {t.device}")
    return t


def launch_count() -> int:
    return int(lib.pmb_launch_count())


def device_status() -> int:
    w = C.c_int32(0)
    _check(lib.pmb_device_status(C.byref(w)))
    return w.value


def set_concurrency(on: bool):
    """False: everything runs on the caller's stream (no internal side streams); results are unchanged."""
    lib.pmb_set_concurrency(1 if on else 0)


def profile_start():
    lib.pmb_profile_start()


def profile_stop() -> list:
    """Per-kernel totals since profile_start(): list of dicts (name, launches, ms, flops, bytes)."""
    import json
    buf = C.create_string_buffer(1 << 16)
    _check(lib.pmb_profile_stop(buf, len(buf)))
    return json.loads(buf.value.decode())


@dataclass
class Mamba2Config:
    """crates/pm-core/src/mamba2/block.rs:48-72."""
    d_model: int
    d_state: int
    d_head: int
    n_heads: int
    n_groups: int = 1
    d_conv: int = 4
    block_len: int = 64
    rmsnorm_eps: float = 1e-5

    @property
    def d_inner(self): return self.n_heads * self.d_head
    @property
    def xbc_dim(self): return self.d_inner + 2 * self.n_groups * self.d_state
    @property
    def in_proj_dim(self): return self.d_inner + self.xbc_dim + self.n_heads

    def c(self) -> _Cfg:
        return _Cfg(self.d_model, self.d_state, self.d_head, self.n_heads, self.n_groups, self.d_conv,
                    self.block_len, self.rmsnorm_eps)

    def param_shapes(self):
        return {"in_proj_weight": (self.d_model, self.in_proj_dim), "conv1d_weight": (self.xbc_dim, 1, self.d_conv),
                "conv1d_bias": (self.xbc_dim,), "a_log": (self.n_heads,), "d_skip": (self.n_heads,),
                "dt_bias": (self.n_heads,), "norm_weight": (self.d_inner,), "out_proj_weight": (self.d_inner, self.d_model)}


def init_block_params(config: Mamba2Config, seed: int) -> dict:
    """Random-init block parameters (CPU float32 tensors) with the distributions the benchmark configurations
    name: projection and conv weights uniform in +-1/sqrt(fan_in) (fan_in = d_model, d_inner, d_conv),
    conv bias 0, A = -exp(U[log 1, log 16]) (so a_log = U[0, log 16]), dt_bias = softplus^-1(U[1e-3, 1e-1]),
    D = 1, norm weight 1.  One torch.Generator per tensor, seeded from `seed`."""
    import math
    sh = config.param_shapes()

    def gen(k):
        g = torch.Generator(); g.manual_seed(seed * 1000003 + k)
        return g

    def uni(shape, bound, k):
        return (torch.rand(shape, generator=gen(k)) * 2 - 1) * bound

    dt = torch.rand(sh["dt_bias"], generator=gen(5)) * (1e-1 - 1e-3) + 1e-3
    return {
        "in_proj_weight": uni(sh["in_proj_weight"], 1 / math.sqrt(config.d_model), 0),
        "conv1d_weight": uni(sh["conv1d_weight"], 1 / math.sqrt(config.d_conv), 1),
        "conv1d_bias": torch.zeros(sh["conv1d_bias"]),
        "a_log": torch.rand(sh["a_log"], generator=gen(3)) * math.log(16.0),
        "d_skip": torch.ones(sh["d_skip"]),
        "dt_bias": dt + torch.log(-torch.expm1(-dt)),          # softplus^-1(dt)
        "norm_weight": torch.ones(sh["norm_weight"]),
        "out_proj_weight": uni(sh["out_proj_weight"], 1 / math.sqrt(config.d_inner), 7),
    }


# ---- primitive ops (the rest of pm_core::Ops; see include/pm_b200.h)
UNARY = {"copy": 0, "neg": 1, "exp": 2, "sqrt": 3, "silu": 4, "sigmoid": 5, "softplus": 6, "mul_scalar": 7, "add_scalar": 8}
BINARY = {"add": 16, "sub": 17, "mul": 18, "div": 19}


def unary(op: str, x: torch.Tensor, scalar: float = 0.0) -> torch.Tensor:
    x = _dev(x, "x"); out = torch.empty_like(x)
    _check(lib.pmb_unary_f32(_stream(), UNARY[op], x.data_ptr(), scalar, out.data_ptr(), x.numel()))
    return out


def binary(op: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    a, b = _dev(a, "a"), _dev(b, "b")
    if a.shape != b.shape:
        raise PmbError(1, f"binary {op}: shapes differ {tuple(a.shape)} vs {tuple(b.shape)}")
    out = torch.empty_like(a)
    _check(lib.pmb_binary_f32(_stream(), BINARY[op], a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel()))
    return out


def strided_copy(src: torch.Tensor, shape, strides, offset: int = 0) -> torch.Tensor:
    """narrow / transpose / broadcast_as as one copy: `shape`, element `strides` (0 broadcasts) and start `offset`
    describe the view of the contiguous fp32 buffer `src`."""
    src = _dev(src, "src")
    out = torch.empty(tuple(shape), device=src.device, dtype=torch.float32)
    sh = (C.c_int64 * len(shape))(*shape); st = (C.c_int64 * len(shape))(*strides)
    _check(lib.pmb_strided_copy_f32(_stream(), src.data_ptr(), len(shape), sh, st, offset, out.data_ptr()))
    return out


def embedding(table: torch.Tensor, ids: torch.Tensor):
    table = _dev(table, "table")
    out = torch.empty(ids.numel(), table.shape[1], device=table.device, dtype=torch.float32)
    bad = torch.zeros(1, device=table.device, dtype=torch.int32)
    _check(lib.pmb_embedding_f32(_stream(), table.data_ptr(), table.shape[0], table.shape[1], ids.data_ptr(), ids.numel(), out.data_ptr(), bad.data_ptr()))
    return out.reshape(*ids.shape, table.shape[1]), bad


def gather_last(x: torch.Tensor, index: torch.Tensor):
    x = _dev(x, "x")
    out = torch.empty(x.shape[0], device=x.device, dtype=torch.float32)
    bad = torch.zeros(1, device=x.device, dtype=torch.int32)
    _check(lib.pmb_gather_last_f32(_stream(), x.data_ptr(), index.data_ptr(), x.shape[0], x.shape[1], out.data_ptr(), bad.data_ptr()))
    return out, bad


def log_softmax(x: torch.Tensor) -> torch.Tensor:
    x = _dev(x, "x"); out = torch.empty_like(x)
    _check(lib.pmb_log_softmax_f32(_stream(), x.data_ptr(), x.numel() // x.shape[-1], x.shape[-1], out.data_ptr()))
    return out


def sum_all(x: torch.Tensor, mean: bool = False) -> torch.Tensor:
    x = _dev(x, "x")
    out = torch.empty(1, device=x.device, dtype=torch.float32)
    ws = torch.empty(lib.pmb_sum_workspace_bytes(), device=x.device, dtype=torch.uint8)
    _check(lib.pmb_sum_all_f32(_stream(), x.data_ptr(), x.numel(), int(mean), out.data_ptr(), ws.data_ptr(), ws.numel()))
    return out


def cumsum(x: torch.Tensor, dim: int) -> torch.Tensor:
    x = _dev(x, "x"); out = torch.empty_like(x)
    outer = 1
    for s_ in x.shape[:dim]:
        outer *= s_
    inner = 1
    for s_ in x.shape[dim + 1:]:
        inner *= s_
    _check(lib.pmb_cumsum_f32(_stream(), x.data_ptr(), outer, x.shape[dim], inner, out.data_ptr()))
    return out


def selftest_bounded_wait(polls: int = 4096):
    """Launches the library's one-thread bounded-wait self-test on the current stream."""
    _check(lib.pmb_selftest_bounded_wait(_stream(), polls))


def _params_struct(p: dict) -> _Params:
    s = _Params()
    for n in PARAM_ORDER:
        setattr(s, n, _dev(p[n], n).data_ptr())
    return s


# ------------------------------------------------------------------------------------------------
# primitive ops
# ------------------------------------------------------------------------------------------------

def matmul(a: torch.Tensor, b: torch.Tensor, *, trans_a=False, trans_b=False, residual=None, engine=0, out=None):
    """Ops::matmul on 2-D operands.  C = op(a) @ op(b) (+ residual)."""
    _dev(a, "a"); _dev(b, "b")
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    K2, N = (b.shape[1], b.shape[0]) if trans_b else b.shape
    if K != K2:
        raise PmbError(1, f"matmul: inner dimensions differ ({K} vs {K2})")
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=torch.float32)
    _check(lib.pmb_gemm_f32(_stream(), int(trans_a), int(trans_b), M, N, K, a.data_ptr(), a.stride(0), b.data_ptr(),
                            b.stride(0), out.data_ptr(), out.stride(0), _ptr(residual), engine))
    return out


def matmul_bf16(a: torch.Tensor, b: torch.Tensor, *, trans_a=False, trans_b=False, residual=None, out_dtype=torch.float32):
    """bf16 x bf16 -> fp32-accumulated product; result (and residual) fp32 or bf16."""
    for t, n in ((a, "a"), (b, "b")):
        if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
            raise PmbError(2, f"{n}: expected a contiguous bfloat16 CUDA tensor, got {t.dtype}")
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    K2, N = (b.shape[1], b.shape[0]) if trans_b else b.shape
    if K != K2:
        raise PmbError(1, f"matmul_bf16: inner dimensions differ ({K} vs {K2})")
    out = torch.empty(M, N, device=a.device, dtype=out_dtype)
    if residual is not None and residual.dtype != out_dtype:
        raise PmbError(2, "matmul_bf16: residual dtype must equal the output dtype")
    _check(lib.pmb_gemm_bf16(_stream(), int(trans_a), int(trans_b), M, N, K, a.data_ptr(), a.stride(0), b.data_ptr(),
                             b.stride(0), out.data_ptr(), out.stride(0), _ptr(residual), int(out_dtype == torch.bfloat16)))
    return out


def to_bf16(t: torch.Tensor) -> torch.Tensor:
    """Ops::to_dtype(F32 -> BF16) on the device."""
    _dev(t, "t")
    out = torch.empty(t.shape, device=t.device, dtype=torch.bfloat16)
    _check(lib.pmb_cast_f32_to_bf16(_stream(), t.data_ptr(), out.data_ptr(), t.numel()))
    return out


def conv_silu_dt_fwd(cfg: Mamba2Config, xzd, conv_w, conv_b, dt_bias):
    B, T, J = xzd.shape
    act = torch.empty(B, T, cfg.xbc_dim, device=xzd.device, dtype=torch.float32)
    dt = torch.empty(B, T, cfg.n_heads, device=xzd.device, dtype=torch.float32)
    _check(lib.pmb_conv_silu_dt_fwd(_stream(), C.byref(cfg.c()), B, T, _dev(xzd, "xzd").data_ptr(), conv_w.data_ptr(),
                                    _ptr(conv_b), dt_bias.data_ptr(), act.data_ptr(), dt.data_ptr()))
    return act, dt


def conv_silu_bwd(cfg: Mamba2Config, xzd, conv_w, conv_b, dact):
    B, T, J = xzd.shape
    dxzd = torch.zeros_like(xzd)
    dw = torch.empty_like(conv_w)
    db = torch.empty(cfg.xbc_dim, device=xzd.device, dtype=torch.float32)
    n = lib.pmb_conv_bwd_workspace_bytes(C.byref(cfg.c()), B, T)
    ws = torch.empty(n, device=xzd.device, dtype=torch.uint8)
    _check(lib.pmb_conv_silu_bwd(_stream(), C.byref(cfg.c()), B, T, xzd.data_ptr(), conv_w.data_ptr(), _ptr(conv_b),
                                 _dev(dact, "dact").data_ptr(), dxzd.data_ptr(), dw.data_ptr(), db.data_ptr(), ws.data_ptr(), n))
    return dxzd, dw, db


class SsdScan:
    """`Ops::ssd_scan` with its backward.  x (B,T,H,P), a (B,T,H), b/c (B,T,G,N), G in {1,H}."""

    def __init__(self, x, a, b, c, block_len):
        self.x, self.a, self.b, self.c = (_dev(t, n) for t, n in ((x, "x"), (a, "a"), (b, "b"), (c, "c")))
        self.B, self.T, self.H, self.P = x.shape
        self.G, self.N = b.shape[2], b.shape[3]
        q = block_len
        if q <= 0 or q >= self.T or self.T % q != 0:   # the reference's dense route (ssd_ops.rs:70-78)
            q = self.T
        self.Q = q
        self.dims = (self.B, self.T, self.H, self.P, self.N, self.G, self.Q)
        n = lib.pmb_ssd_workspace_bytes(*self.dims)
        if n == 0:
            raise PmbError(1, lib.pmb_last_error().decode())
        self.ws = torch.empty(n, device=x.device, dtype=torch.uint8)
        self.y = None

    def forward(self, init_state=None, want_final_state=False):
        x, b = self.x, self.b
        self.y = torch.empty_like(x)
        fs = torch.empty(self.B, self.H, self.N, self.P, device=x.device, dtype=torch.float32) if want_final_state else None
        _check(lib.pmb_ssd_scan_fwd(_stream(), *self.dims, x.data_ptr(), self.H * self.P, self.a.data_ptr(),
                                    b.data_ptr(), self.c.data_ptr(), self.G * self.N, _ptr(init_state), self.y.data_ptr(),
                                    self.H * self.P, _ptr(fs), self.ws.data_ptr(), self.ws.numel()))
        return (self.y, fs) if want_final_state else self.y

    def backward(self, dy):
        x = self.x
        dx, da, db, dc = torch.empty_like(x), torch.empty_like(self.a), torch.empty_like(self.b), torch.empty_like(self.c)
        hp, gn = self.H * self.P, self.G * self.N
        _check(lib.pmb_ssd_scan_bwd(_stream(), *self.dims, x.data_ptr(), hp, self.a.data_ptr(), self.b.data_ptr(),
                                    self.c.data_ptr(), gn, self.y.data_ptr(), hp, _dev(dy, "dy").data_ptr(), hp,
                                    dx.data_ptr(), hp, da.data_ptr(), db.data_ptr(), dc.data_ptr(), gn,
                                    self.ws.data_ptr(), self.ws.numel()))
        return dx, da, db, dc


class SsdScanBf16:
    """`Ops::ssd_scan` with bf16 x/B/C/y (and gradients) and fp32 a / state."""

    def __init__(self, x, a, b, c, block_len):
        for t, n in ((x, "x"), (b, "b"), (c, "c")):
            if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
                raise PmbError(2, f"{n}: expected a contiguous bfloat16 CUDA tensor, got {t.dtype}")
        self.x, self.a, self.b, self.c = x, _dev(a, "a"), b, c
        self.B, self.T, self.H, self.P = x.shape
        self.G, self.N = b.shape[2], b.shape[3]
        q = block_len
        if q <= 0 or q >= self.T or self.T % q != 0:
            q = self.T
        self.dims = (self.B, self.T, self.H, self.P, self.N, self.G, q)
        n = lib.pmb_ssd_workspace_bytes_bf16(*self.dims)
        if n == 0:
            raise PmbError(1, lib.pmb_last_error().decode())
        self.ws = torch.empty(n, device=x.device, dtype=torch.uint8)

    def forward(self, init_state=None, want_final_state=False):
        y = torch.empty_like(self.x)
        fs = torch.empty(self.B, self.H, self.N, self.P, device=y.device, dtype=torch.float32) if want_final_state else None
        _check(lib.pmb_ssd_scan_fwd_bf16(_stream(), *self.dims, self.x.data_ptr(), self.a.data_ptr(), self.b.data_ptr(),
                                         self.c.data_ptr(), _ptr(init_state), y.data_ptr(), _ptr(fs), self.ws.data_ptr(), self.ws.numel()))
        return (y, fs) if want_final_state else y

    def backward(self, dy):
        dx, da, db, dc = torch.empty_like(self.x), torch.empty_like(self.a), torch.empty_like(self.b), torch.empty_like(self.c)
        _check(lib.pmb_ssd_scan_bwd_bf16(_stream(), *self.dims, self.a.data_ptr(), dy.data_ptr(), dx.data_ptr(), da.data_ptr(),
                                         db.data_ptr(), dc.data_ptr(), self.ws.data_ptr(), self.ws.numel()))
        return dx, da, db, dc


def ssd_scan(x, a, b, c, block_len):
    return SsdScan(x, a, b, c, block_len).forward()


def gated_rmsnorm_fwd(y, z, w, eps):
    rows, width = y.shape
    out = torch.empty_like(y)
    rstd = torch.empty(rows, device=y.device, dtype=torch.float32)
    _check(lib.pmb_gated_rmsnorm_fwd(_stream(), rows, width, eps, _dev(y, "y").data_ptr(), z.data_ptr(), z.stride(0),
                                     w.data_ptr(), out.data_ptr(), rstd.data_ptr()))
    return out, rstd


def gated_rmsnorm_bwd(dout, y, z, w, rstd):
    rows, width = y.shape
    dy, dz, dw = torch.empty_like(y), torch.empty(rows, width, device=y.device, dtype=torch.float32), torch.empty_like(w)
    n = lib.pmb_gated_rmsnorm_bwd_workspace_bytes(rows, width)
    ws = torch.empty(n, device=y.device, dtype=torch.uint8)
    _check(lib.pmb_gated_rmsnorm_bwd(_stream(), rows, width, _dev(dout, "dout").data_ptr(), y.data_ptr(), z.data_ptr(),
                                     z.stride(0), w.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dz.data_ptr(), width,
                                     dw.data_ptr(), ws.data_ptr(), n))
    return dy, dz, dw


def gated_rmsnorm_bwd_static(dout, y, z, w, rstd):
    """Gated RMSNorm backward without any device allocation by the library: for hosts that cannot
    call cudaMalloc where they need it (all memory already in their own pool, or an allocator-free
    hot loop).  The scratch is a fixed 4 MiB array inside the library, so ceil(rows/4)*width*4 bytes
    must fit; calls share it and must not overlap on the GPU.  Output buffers are the caller's."""
    rows, width = y.shape
    dy, dz, dw = torch.empty_like(y), torch.empty(rows, width, device=y.device, dtype=torch.float32), torch.empty_like(w)
    _check(lib.pmb_gated_rmsnorm_bwd_static(_stream(), rows, width, _dev(dout, "dout").data_ptr(), y.data_ptr(), z.data_ptr(),
                                            z.stride(0), w.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dz.data_ptr(), width,
                                            dw.data_ptr()))
    return dy, dz, dw


# ------------------------------------------------------------------------------------------------
# Mamba2Block
# ------------------------------------------------------------------------------------------------

class Mamba2Block:
    """One block: parameters are a dict of fp32 CUDA tensors in `PARAM_ORDER`."""

    def __init__(self, config: Mamba2Config, params: dict, compute_dtype=torch.float32):
        """`compute_dtype` mirrors the reference's ambient dtype (`x.dtype()`, block.rs:137): float32, or bfloat16
        for bf16 storage with fp32 islands.  Parameters are always fp32."""
        self.config = config
        self.params = {k: _dev(params[k], k) for k in PARAM_ORDER}
        for k, shp in config.param_shapes().items():
            if tuple(self.params[k].shape) != tuple(shp):
                raise PmbError(1, f"{k}: shape {tuple(self.params[k].shape)} != {shp}")
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise PmbError(2, f"compute dtype {compute_dtype} is not supported")
        self.bf16 = compute_dtype == torch.bfloat16
        self._ws = None
        self.refresh_weights()

    def refresh_weights(self):
        """Re-derives the bf16 copies of the projection weights after the fp32 masters changed."""
        if self.bf16:
            self.w_in16 = to_bf16(self.params["in_proj_weight"])
            self.w_out16 = to_bf16(self.params["out_proj_weight"])

    def _io(self, t, name):
        want = torch.bfloat16 if self.bf16 else torch.float32
        if not (t.is_cuda and t.dtype == want and t.is_contiguous()):
            raise PmbError(2, f"{name}: expected a contiguous {want} CUDA tensor, got {t.dtype}")
        return t

    def _workspace(self, B, T, device):
        fn = lib.pmb_mamba2_block_workspace_bytes_bf16 if self.bf16 else lib.pmb_mamba2_block_workspace_bytes
        n = fn(C.byref(self.config.c()), B, T)
        if n == 0:
            raise PmbError(1, lib.pmb_last_error().decode())
        if self._ws is None or self._ws.numel() < n:
            self._ws = torch.empty(n, device=device, dtype=torch.uint8)
        return self._ws

    def forward(self, x, residual=None):
        B, T, D = x.shape
        ws = self._workspace(B, T, x.device)
        out = torch.empty_like(x)
        ps = _params_struct(self.params)
        self._io(x, "x")
        if self.bf16:
            _check(lib.pmb_mamba2_block_fwd_bf16(_stream(), C.byref(self.config.c()), C.byref(ps), self.w_in16.data_ptr(),
                                                 self.w_out16.data_ptr(), B, T, x.data_ptr(), _ptr(residual), out.data_ptr(),
                                                 ws.data_ptr(), ws.numel()))
        else:
            _check(lib.pmb_mamba2_block_fwd(_stream(), C.byref(self.config.c()), C.byref(ps), B, T, x.data_ptr(),
                                            _ptr(residual), out.data_ptr(), ws.data_ptr(), ws.numel()))
        return out

    def backward(self, x, dout, dx_accum=None):
        """Recomputes the block from `x` and returns (dx, {param gradients})."""
        B, T, D = x.shape
        ws = self._workspace(B, T, x.device)
        dx = torch.empty_like(x)
        grads = {k: torch.empty_like(v) for k, v in self.params.items()}
        ps, gs = _params_struct(self.params), _params_struct(grads)
        self._io(x, "x"); self._io(dout, "dout")
        if self.bf16:
            _check(lib.pmb_mamba2_block_bwd_bf16(_stream(), C.byref(self.config.c()), C.byref(ps), self.w_in16.data_ptr(),
                                                 self.w_out16.data_ptr(), B, T, x.data_ptr(), dout.data_ptr(), _ptr(dx_accum),
                                                 dx.data_ptr(), C.byref(gs), ws.data_ptr(), ws.numel()))
        else:
            _check(lib.pmb_mamba2_block_bwd(_stream(), C.byref(self.config.c()), C.byref(ps), B, T, x.data_ptr(),
                                            dout.data_ptr(), _ptr(dx_accum), dx.data_ptr(), C.byref(gs),
                                            ws.data_ptr(), ws.numel()))
        return dx, grads

    def zero_state(self, batch, device="cuda"):
        cfg = self.config
        return {"ssm_state": torch.zeros(batch, cfg.n_heads, cfg.d_state, cfg.d_head, device=device),
                "conv_window": torch.zeros(batch, cfg.xbc_dim, cfg.d_conv - 1, device=device)}

    def step(self, x_t, state):
        """`Mamba2Block::step`: x_t (B,1,D); the state dict is updated in place and returned."""
        B = x_t.shape[0]
        n = lib.pmb_mamba2_step_workspace_bytes(C.byref(self.config.c()), B)
        ws = torch.empty(n, device=x_t.device, dtype=torch.uint8)
        y = torch.empty_like(x_t)
        ps = _params_struct(self.params)
        _check(lib.pmb_mamba2_step(_stream(), C.byref(self.config.c()), C.byref(ps), B, _dev(x_t, "x_t").data_ptr(),
                                   state["ssm_state"].data_ptr(), state["conv_window"].data_ptr(), y.data_ptr(),
                                   ws.data_ptr(), n))
        return y, state


class ContextEncoder:
    """Residual stack h_l = h_{l-1} + Block_l(h_{l-1}) with the re-planned checkpoint policy."""

    def __init__(self, config: Mamba2Config, layers: list):
        self.config = config
        self.layers = [{k: _dev(p[k], k) for k in PARAM_ORDER} for p in layers]
        self._ws = None

    def _arrays(self, dicts):
        arr = (_Params * len(dicts))()
        for i, p in enumerate(dicts):
            arr[i] = _params_struct(p)
        return arr

    def forward_checkpointed(self, x):
        B, T, D = x.shape
        L = len(self.layers)
        n = lib.pmb_stack_workspace_bytes(C.byref(self.config.c()), B, T)   # two forward slots: recompute one block ahead
        if self._ws is None or self._ws.numel() < n:
            self._ws = torch.empty(n, device=x.device, dtype=torch.uint8)
        saved = torch.empty(L + 1, B, T, D, device=x.device, dtype=torch.float32)
        saved[0].copy_(x)
        _check(lib.pmb_stack_fwd_ckpt(_stream(), C.byref(self.config.c()), L, self._arrays(self.layers), B, T,
                                      saved.data_ptr(), self._ws.data_ptr(), self._ws.numel()))
        return saved[L], saved

    def checkpoint_backward(self, saved, dhidden, on_layer_done=None):
        L, B, T, D = saved.shape[0] - 1, saved.shape[1], saved.shape[2], saved.shape[3]
        grads = [{k: torch.empty_like(v) for k, v in p.items()} for p in self.layers]
        dh = dhidden.clone()
        cb = LAYER_CALLBACK(on_layer_done) if on_layer_done else C.cast(None, LAYER_CALLBACK)
        _check(lib.pmb_stack_bwd(_stream(), C.byref(self.config.c()), L, self._arrays(self.layers), self._arrays(grads),
                                 B, T, saved.data_ptr(), dh.data_ptr(), self._ws.data_ptr(), self._ws.numel(), cb, None))
        return dh, grads


class FlatMamba:
    """Flat LM (tied embedding -> stack -> tied head -> mean CE).  Owns a library model handle whose flat
    parameter/gradient buffers are exposed as torch views."""

    def __init__(self, config: Mamba2Config, n_layers: int, vocab: int, batch: int, seqlen: int, compute_dtype=torch.float32,
                 level1_layers: int = 0, group: int = 4):
        """`level1_layers > 0` selects the two-level wiring (n_layers blocks at token rate, level1_layers blocks at
        1/group rate); layer indices then run over both levels and `view(flat, -2)` is the (D,D) projection."""
        self.config, self.vocab, self.batch, self.seqlen = config, vocab, batch, seqlen
        self.n_layers = n_layers + level1_layers
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise PmbError(2, f"compute dtype {compute_dtype} is not supported")
        h = C.c_void_p()
        if level1_layers > 0:
            _check(lib.pmb_lm_create_hier(C.byref(config.c()), n_layers, level1_layers, group, vocab, batch, seqlen,
                                          int(compute_dtype == torch.bfloat16), C.byref(h)))
        else:
            _check(lib.pmb_lm_create_dtype(C.byref(config.c()), n_layers, vocab, batch, seqlen,
                                           int(compute_dtype == torch.bfloat16), C.byref(h)))
        self._h = h
        n = lib.pmb_lm_param_count(h)
        self.flat_params = _as_tensor(lib.pmb_lm_params(h), n)
        self.flat_grads = _as_tensor(lib.pmb_lm_grads(h), n)
        self.loss_dev = _as_tensor(lib.pmb_lm_loss_device(h), 1)

    def view(self, flat, layer, which=0):
        """Tensor view of one parameter (layer=-1: embedding (V,D))."""
        off = lib.pmb_lm_param_offset(self._h, layer, which)
        if layer == -2:
            shp = (self.config.d_model, self.config.d_model)
        elif layer < 0:
            shp = (self.vocab, self.config.d_model)
        else:
            shp = self.config.param_shapes()[PARAM_ORDER[which]]
        n = 1
        for s in shp:
            n *= s
        return flat[off:off + n].view(*shp)

    def load(self, embed, layers, wproj=None):
        self.view(self.flat_params, -1).copy_(embed)
        if wproj is not None:
            self.view(self.flat_params, -2).copy_(wproj)
        for l, p in enumerate(layers):
            for w, name in enumerate(PARAM_ORDER):
                self.view(self.flat_params, l, w).copy_(p[name])

    def grads(self):
        g_embed = self.view(self.flat_grads, -1)
        g_layers = [{name: self.view(self.flat_grads, l, w) for w, name in enumerate(PARAM_ORDER)} for l in range(self.n_layers)]
        return g_embed, g_layers

    @property
    def activation_bytes(self):
        return int(lib.pmb_lm_activation_bytes(self._h))

    @property
    def activation_detail(self):
        out = (C.c_int64 * 3)()
        lib.pmb_lm_activation_detail(self._h, out)
        return {"stored_for_backward": out[0], "block_workspace": out[1], "lm_head_transient": out[2]}

    def step_device(self, ids, targets, on_layer_done=None):
        cb = LAYER_CALLBACK(on_layer_done) if on_layer_done else C.cast(None, LAYER_CALLBACK)
        _check(lib.pmb_lm_step_device(self._h, _stream(), ids.data_ptr(), targets.data_ptr(), cb, None))
        return self.loss_dev

    def step_device_dp(self, ids, targets, dp: "DataParallel"):
        """The step with the per-layer gradient all-reduce over `dp` (NCCL behind the C ABI) overlapped with the
        backward; on return the current stream sees averaged gradients."""
        _check(lib.pmb_lm_step_device_dp(self._h, _stream(), ids.data_ptr(), targets.data_ptr(), dp._h))
        return self.loss_dev

    def capture_step(self, on_layer_done=None, after=None, dp=None):
        """One training step (forward + checkpointed backward) captured into a CUDA graph.

        Returns a callable `step(ids, targets) -> loss` (0-d device tensor): it copies the int64 token tensors
        (device, or pinned host for an asynchronous copy) into the graph's static input buffers and replays the
        graph, so the ~1000 launches of a step cost one launch.  The graph holds this rank's compute only.
        `on_layer_done` / `after` are called while capturing; whatever they enqueue on the capturing stream becomes
        part of the graph.  They must not issue collectives: asynchronous NCCL work enqueued from these callbacks
        on another stream, with its `Work.wait()` and the process group's watchdog polling events of a stream that is
        still capturing, did not finish when it was tried, so with an initialised process group of more than one
        rank a callback is refused here.  Average the gradients after the replay instead (see `bench.py`).
        Two warm-up steps run first on a side stream: the library creates its internal streams, events and scratch
        on first use, which a capture must not contain."""
        if on_layer_done is not None or after is not None:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                raise PmbError(2, "capture_step: callbacks are refused while a process group with more than one rank is "
                                  "initialised (collectives inside the capture are not supported); all-reduce after the replay")
        return _GraphStep(self, on_layer_done, after, dp)

    def bad_tokens(self) -> int:
        """Reads and clears the flag word for out-of-range input (bit 0: a token id, bit 1: a target); the step
        entry points other than `step_host` do not check it themselves."""
        w = C.c_int32(0)
        _check(lib.pmb_lm_bad_tokens(self._h, _stream(), C.byref(w)))
        return w.value

    def step_host(self, ids_host, targets_host, on_layer_done=None):
        """ids/targets: int64 CPU tensors (pinned for an asynchronous copy).  Returns the loss as a float."""
        loss = C.c_float(0)
        cb = LAYER_CALLBACK(on_layer_done) if on_layer_done else C.cast(None, LAYER_CALLBACK)
        _check(lib.pmb_lm_step_host(self._h, _stream(), ids_host.data_ptr(), targets_host.data_ptr(), C.byref(loss), cb, None))
        return loss.value

    def save_checkpoint(self, path: str):
        """Write the parameters as the reference's positional safetensors checkpoint (pm-train/src/checkpoint.rs:25-52)."""
        _check(lib.pmb_lm_save_safetensors(self._h, _stream(), str(path).encode()))

    def load_checkpoint(self, path: str):
        """Read such a checkpoint; count, dtype and shapes must match (pm-train/src/checkpoint.rs:56-97)."""
        _check(lib.pmb_lm_load_safetensors(self._h, _stream(), str(path).encode()))

    def close(self):
        if self._h:
            lib.pmb_lm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DataParallel:
    """NCCL communicator of the library (pmb_dp_*).  `unique_id()` on rank 0, hand the 128 bytes to the other ranks,
    then every rank constructs `DataParallel(nranks, rank, id)` with its device current."""

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        _check(lib.pmb_dp_unique_id(buf))
        return buf.raw

    def __init__(self, nranks: int, rank: int, unique_id: bytes):
        h = C.c_void_p()
        buf = C.create_string_buffer(bytes(unique_id), 128)
        _check(lib.pmb_dp_init(nranks, rank, buf, C.byref(h)))
        self._h, self.nranks, self.rank = h, nranks, rank

    def all_reduce_async(self, t: torch.Tensor):
        _check(lib.pmb_dp_allreduce_async(self._h, _stream(), _dev(t, "tensor").data_ptr(), t.numel()))

    def all_gather_async(self, send: torch.Tensor, recv: torch.Tensor):
        """recv (nranks * send.numel() elements of send's dtype) receives every rank's `send`, rank r's block at r."""
        for t, name in ((send, "send"), (recv, "recv")):      # any dtype: the exchange is by bytes
            if not (t.is_cuda and t.is_contiguous()):
                raise PmbError(2, f"{name}: expected a contiguous CUDA tensor")
        nbytes = send.numel() * send.element_size()
        if recv.numel() * recv.element_size() != self.nranks * nbytes:
            raise ValueError("all_gather_async: recv must hold nranks blocks of send's size")
        _check(lib.pmb_dp_allgather_async(self._h, _stream(), send.data_ptr(), recv.data_ptr(), nbytes))

    def sync(self):
        _check(lib.pmb_dp_sync(self._h, _stream()))

    def close(self):
        if self._h:
            lib.pmb_dp_destroy(self._h)
            self._h = None


class _GraphStep:
    def __init__(self, lm: "FlatMamba", on_layer_done, after, dp=None):
        if dp is not None:
            # the whole data-parallel step is one library call: no host callback and no torch process group inside
            # the capture, only this library's streams, events and NCCL's own kernels
            step_fn = lambda: lm.step_device_dp(self.ids, self.targets, dp)
        else:
            step_fn = lambda: lm.step_device(self.ids, self.targets, on_layer_done)
        dev = lm.loss_dev.device
        self.ids = torch.zeros(lm.batch, lm.seqlen, dtype=torch.int64, device=dev)
        self.targets = torch.zeros_like(self.ids)
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):
                step_fn()
                if after:
                    after()
        cur.wait_stream(side)
        torch.cuda.synchronize()
        n0 = launch_count()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = step_fn()
            if after:
                after()
        self.launches_per_step = launch_count() - n0     # kernels of this library inside one replay

    def __call__(self, ids, targets):
        self.ids.copy_(ids.view_as(self.ids), non_blocking=True)
        self.targets.copy_(targets.view_as(self.targets), non_blocking=True)
        self.graph.replay()
        return self.loss


def _tensor_table(arrays):
    n = len(arrays)
    shapes = [int(s) for a in arrays for s in a.shape]
    sh = (C.c_int64 * max(1, len(shapes)))(*shapes)
    rk = (C.c_int32 * max(1, n))(*[a.ndim for a in arrays])
    ptrs = (C.c_void_p * max(1, n))(*[a.ctypes.data for a in arrays])
    return n, sh, rk, ptrs


def save_checkpoint_f32(path: str, arrays):
    """Host-side format code alone: `arrays` (C-contiguous float32 numpy arrays) become p_0000, p_0001, ..."""
    import numpy as np
    arrays = [np.ascontiguousarray(a, dtype=np.float32) for a in arrays]
    n, sh, rk, ptrs = _tensor_table(arrays)
    _check(lib.pmb_safetensors_save_f32(str(path).encode(), n, sh, rk, ptrs))


def load_checkpoint_f32(path: str, shapes):
    """Reads p_0000.. into new float32 arrays of the given shapes; raises PmbError on any count / dtype / shape mismatch."""
    import numpy as np
    arrays = [np.zeros(s, dtype=np.float32) for s in shapes]
    n, sh, rk, ptrs = _tensor_table(arrays)
    _check(lib.pmb_safetensors_load_f32(str(path).encode(), n, sh, rk, ptrs))
    return arrays


class AdamW:
    """`AdamW` + `clip_grad_norm` of the reference (pm-train/src/optim.rs:104-157, clip.rs:13-53) over one flat
    fp32 parameter buffer; the gradient norm never leaves the device."""

    def __init__(self, flat_params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        self.p = _dev(flat_params, "flat_params")
        self.m, self.v = torch.zeros_like(self.p), torch.zeros_like(self.p)
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay
        self.t = 0
        self.sumsq = torch.zeros(1, device=self.p.device, dtype=torch.float32)
        self._ws = torch.empty(lib.pmb_grad_sumsq_workspace_bytes(), device=self.p.device, dtype=torch.uint8)

    def step(self, flat_grads, max_norm=0.0):
        """Returns the device scalar holding sum(g^2) (its square root is the unclipped global norm)."""
        g = _dev(flat_grads, "flat_grads")
        self.t += 1
        _check(lib.pmb_grad_sumsq(_stream(), g.numel(), g.data_ptr(), self.sumsq.data_ptr(), self._ws.data_ptr(), self._ws.numel()))
        _check(lib.pmb_adamw_step(_stream(), g.numel(), self.p.data_ptr(), g.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                                  self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.t, max_norm,
                                  self.sumsq.data_ptr()))
        return self.sumsq


def _as_tensor(ptr: int, n: int) -> torch.Tensor:
    """Wraps library-owned device memory (fp32) as a torch tensor without copying."""
    class _Iface:
        pass
    o = _Iface()
    o.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 2}
    return torch.as_tensor(o, device="cuda")
