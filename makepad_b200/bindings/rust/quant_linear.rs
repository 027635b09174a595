// Safe wrapper over mpq_sys.rs: the operator surface a Rust runtime would call.
// Source only (no rustc on the image this library is built on).
use std::ffi::{c_void, CStr};
use std::ptr::null_mut;
use std::rc::Rc;

use crate::mpq_sys::*;

#[derive(Debug)]
pub struct MpqError {
    pub status: i32,
    pub text: String,
}

pub struct Context {
    lib: Rc<LibMpq>,
    raw: *mut mpq_context,
}

impl Context {
    pub fn new(lib: Rc<LibMpq>, device: i32) -> Result<Context, MpqError> {
        let mut raw = null_mut();
        let st = unsafe { (lib.mpq_context_create)(device, &mut raw) };
        if st != MPQ_OK {
            return Err(MpqError { status: st, text: lib.status_text(st) });
        }
        Ok(Context { lib, raw })
    }

    fn check(&self, st: i32) -> Result<(), MpqError> {
        if st == MPQ_OK {
            return Ok(());
        }
        let detail = unsafe { CStr::from_ptr((self.lib.mpq_last_error)(self.raw)).to_string_lossy().into_owned() };
        Err(MpqError { status: st, text: format!("{}: {}", self.lib.status_text(st), detail) })
    }

    /// Reports a device-side bounded wait that ran out since the last poll (synchronises).
    pub fn poll_status(&self) -> Result<(), MpqError> {
        self.check(unsafe { (self.lib.mpq_context_poll_status)(self.raw) })
    }
}

impl Drop for Context {
    fn drop(&mut self) {
        unsafe { (self.lib.mpq_context_destroy)(self.raw) };
    }
}

/// A quantised weight resident on the GPU in the layout the kernels stream.
pub struct QuantWeight<'c> {
    ctx: &'c Context,
    raw: *mut mpq_weight,
    pub n: i64,
    pub k: i64,
    pub fmt: i32,
}

impl<'c> QuantWeight<'c> {
    /// codes: N*K/2 bytes, element 2j in the low nibble; scales: N*K/32 fp16 bit patterns.
    pub fn q4(ctx: &'c Context, n: i64, k: i64, codes: &[u8], scales: &[u16], tp_mode: i32, rank: i32, world: i32)
        -> Result<QuantWeight<'c>, MpqError> {
        if codes.len() as i64 != n * k / 2 || scales.len() as i64 != n * k / 32 {
            return Err(MpqError { status: MPQ_ERR_SHAPE, text: "codes/scales length does not match N, K".into() });
        }
        let mut raw = null_mut();
        ctx.check(unsafe { (ctx.lib.mpq_q4_weight_create)(ctx.raw, n, k, codes.as_ptr(), scales.as_ptr(), tp_mode, rank, world, &mut raw) })?;
        let (mut sn, mut sk, mut fmt) = (0i64, 0i64, 0i32);
        unsafe { (ctx.lib.mpq_weight_shape)(raw, &mut sn, &mut sk, &mut fmt) };
        Ok(QuantWeight { ctx, raw, n: sn, k: sk, fmt })
    }

    pub fn nvfp4(ctx: &'c Context, n: i64, k: i64, codes: &[u8], sf: &[u8], tensor_scale: f32) -> Result<QuantWeight<'c>, MpqError> {
        if codes.len() as i64 != n * k / 2 || sf.len() as i64 != n * k / 16 {
            return Err(MpqError { status: MPQ_ERR_SHAPE, text: "codes/sf length does not match N, K".into() });
        }
        let mut raw = null_mut();
        ctx.check(unsafe { (ctx.lib.mpq_nvfp4_weight_create)(ctx.raw, n, k, codes.as_ptr(), sf.as_ptr(), tensor_scale, &mut raw) })?;
        Ok(QuantWeight { ctx, raw, n, k, fmt: MPQ_FMT_NVFP4 })
    }
}

impl<'c> Drop for QuantWeight<'c> {
    fn drop(&mut self) {
        unsafe { (self.ctx.lib.mpq_weight_destroy)(self.raw) };
    }
}

/// Device memory owned by the caller's runtime; the library only reads or writes through it.
#[derive(Clone, Copy)]
pub struct DevicePtr(pub *mut c_void);

pub struct QuantLinear<'c> {
    pub weight: QuantWeight<'c>,
}

impl<'c> QuantLinear<'c> {
    /// Q4: y[M][N] = x[M][K] . W^T, fp32 in and out, enqueued on `stream`.
    pub fn forward_q4(&self, x: DevicePtr, m: i64, y: DevicePtr, stream: *mut c_void) -> Result<(), MpqError> {
        let c = self.weight.ctx;
        c.check(unsafe { (c.lib.mpq_q4_linear_forward)(c.raw, self.weight.raw, x.0 as *const f32, m, y.0 as *mut f32, stream) })
    }

    /// NVFP4: C[M][N] bf16 = tsA * tsB * A . B^T with A = (codes, e4m3 scales, tensor scale) on the device.
    pub fn forward_nvfp4(&self, a_codes: DevicePtr, a_sf: DevicePtr, a_tensor_scale: f32, m: i64, c_bf16: DevicePtr,
                         stream: *mut c_void) -> Result<(), MpqError> {
        let c = self.weight.ctx;
        c.check(unsafe {
            (c.lib.mpq_nvfp4_gemm_forward)(c.raw, self.weight.raw, a_codes.0 as *const u8, a_sf.0 as *const u8, a_tensor_scale, m,
                                           c_bf16.0 as *mut u16, stream)
        })
    }

    /// Q4 without any allocation by the library (static device scratch; launches beyond its 512 CTAs are refused).
    /// `status_dev`, when not null, is a caller-owned device int a kernel sets when one of its bounded waits runs out.
    pub fn forward_q4_static(&self, x: DevicePtr, m: i64, y: DevicePtr, status_dev: DevicePtr, stream: *mut c_void) -> Result<(), MpqError> {
        let c = self.weight.ctx;
        c.check(unsafe {
            (c.lib.mpq_q4_linear_forward_static)(c.raw, self.weight.raw, x.0 as *const f32, m, y.0 as *mut f32, status_dev.0 as *mut i32, stream)
        })
    }

    /// Q4 down projection with SwiGLU in front: y = (silu(gate) * up) . W^T for gate_up[M][2K] = [gate | up] on the device.
    pub fn forward_q4_swiglu(&self, gate_up: DevicePtr, m: i64, y: DevicePtr, stream: *mut c_void) -> Result<(), MpqError> {
        let c = self.weight.ctx;
        c.check(unsafe { (c.lib.mpq_q4_linear_forward_swiglu)(c.raw, self.weight.raw, gate_up.0 as *const f32, m, y.0 as *mut f32, stream) })
    }

    /// Host-buffer convenience path (copies in, runs, copies out, synchronises).
    pub fn forward_q4_host(&self, x: &[f32], m: i64, y: &mut [f32]) -> Result<(), MpqError> {
        let c = self.weight.ctx;
        if x.len() as i64 != m * self.weight.k || y.len() as i64 != m * self.weight.n {
            return Err(MpqError { status: MPQ_ERR_SHAPE, text: "x/y length does not match M, K, N".into() });
        }
        c.check(unsafe { (c.lib.mpq_q4_linear_forward_host)(c.raw, self.weight.raw, x.as_ptr(), m, y.as_mut_ptr()) })
    }
}

/// Activations for the NVFP4 GEMM, quantised on the device: x[M][K] (fp32, or bf16 bits) -> codes [M][K/2], sf [M][K/16].
/// With `swiglu` the input is [M][2K] = [gate | up] and silu(gate) * up is what gets quantised.
pub fn nvfp4_quantize(ctx: &Context, x: DevicePtr, x_is_bf16: bool, swiglu: bool, m: i64, k: i64, tensor_scale: f32, codes: DevicePtr,
                      sf: DevicePtr, stream: *mut c_void) -> Result<(), MpqError> {
    let f = if swiglu { ctx.lib.mpq_nvfp4_quantize_swiglu } else { ctx.lib.mpq_nvfp4_quantize_activations };
    ctx.check(unsafe { f(ctx.raw, x.0 as *const c_void, x_is_bf16 as i32, m, k, tensor_scale, codes.0 as *mut u8, sf.0 as *mut u8, stream) })
}

/// out[M][F] = silu(gate) * up for gate_up[M][2F] = [gate | up], fp32 on the device.
pub fn swiglu(ctx: &Context, gate_up: DevicePtr, m: i64, f: i64, out: DevicePtr, stream: *mut c_void) -> Result<(), MpqError> {
    ctx.check(unsafe { (ctx.lib.mpq_swiglu)(ctx.raw, gate_up.0 as *const f32, m, f, out.0 as *mut f32, stream) })
}
