//! `pm-b200`: the B200 (sm_100a) backend of the Mamba2 SSD block path behind `pm_core::Ops` / `pm_backend::Backend`.
//!
//! NOT COMPILED where it was written (no Rust toolchain); the executable verification of the library is through the
//! same C ABI from Python.  `ffi` binds every symbol of `include/pm_b200.h`; `backend` holds `B200Backend`.
pub mod backend;
pub mod ffi;

pub use backend::{B200Backend, B200Error, B200GradStore, B200Param, B200Tensor};
