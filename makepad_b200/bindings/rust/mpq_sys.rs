// Raw binding of libmpq.so (include/mpq.h), written the way makepad binds its
// native libraries: a hand-written *_sys file, no bindgen, no libc crate, a
// loader struct of typed extern "C" function pointers filled by dlopen/dlsym
// (compare platform/src/os/linux/module_loader.rs:5-41 and egl_sys.rs:311-375
// in makepad).  Source only: the image this library is built on has no rustc,
// so this file has not been compiled.
#![allow(non_camel_case_types, non_snake_case, dead_code)]

use std::ffi::{c_char, c_void, CStr, CString};

pub const MPQ_OK: i32 = 0;
pub const MPQ_ERR_INVALID_ARG: i32 = -1;
pub const MPQ_ERR_SHAPE: i32 = -2;
pub const MPQ_ERR_ALIGN: i32 = -3;
pub const MPQ_ERR_CUDA: i32 = -4;
pub const MPQ_ERR_UNSUPPORTED: i32 = -5;
pub const MPQ_ERR_PEER_TIMEOUT: i32 = -6;
pub const MPQ_ERR_STATE: i32 = -7;
pub const MPQ_ERR_FORMAT: i32 = -8;
pub const MPQ_ERR_IO: i32 = -9;

pub const MPQ_FILE_CANONICAL: i32 = 1;
pub const MPQ_FILE_DEVICE: i32 = 2;

pub const MPQ_FMT_Q4: i32 = 1;
pub const MPQ_FMT_NVFP4: i32 = 2;
pub const MPQ_TP_NONE: i32 = 0;
pub const MPQ_TP_COLUMN: i32 = 1;
pub const MPQ_TP_ROW: i32 = 2;

#[repr(C)] pub struct mpq_context { _private: [u8; 0] }
#[repr(C)] pub struct mpq_weight { _private: [u8; 0] }
#[repr(C)] pub struct mpq_exchange { _private: [u8; 0] }

#[repr(C)]
#[derive(Clone, Copy, Default, Debug)]
pub struct mpq_device_info {
    pub device: i32,
    pub sm_count: i32,
    pub cc_major: i32,
    pub cc_minor: i32,
    pub l2_bytes: i64,
    pub total_mem_bytes: i64,
    pub sm_clock_khz: i32,
    pub mem_clock_khz: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Default, Debug)]
pub struct mpq_file_info_t {
    pub kind: i32,
    pub fmt: i32,
    pub layout_version: i32,
    pub reserved: i32,
    pub N: i64,
    pub K: i64,
    pub bytes_a: i64,
    pub bytes_b: i64,
    pub tensor_scale: f32,
    pub reserved2: i32,
}

extern "C" {
    fn dlopen(filename: *const c_char, flag: i32) -> *mut c_void;
    fn dlsym(handle: *mut c_void, symbol: *const c_char) -> *mut c_void;
    fn dlclose(handle: *mut c_void) -> i32;
}
const RTLD_NOW: i32 = 2;

pub struct LibMpq {
    pub mpq_context_create: unsafe extern "C" fn(i32, *mut *mut mpq_context) -> i32,
    pub mpq_context_destroy: unsafe extern "C" fn(*mut mpq_context) -> i32,
    pub mpq_context_info: unsafe extern "C" fn(*const mpq_context, *mut mpq_device_info) -> i32,
    pub mpq_status_string: unsafe extern "C" fn(i32) -> *const c_char,
    pub mpq_last_error: unsafe extern "C" fn(*const mpq_context) -> *const c_char,
    pub mpq_context_poll_status: unsafe extern "C" fn(*mut mpq_context) -> i32,
    pub mpq_context_launch_count: unsafe extern "C" fn(*const mpq_context) -> i64,
    pub mpq_q4_weight_create: unsafe extern "C" fn(*mut mpq_context, i64, i64, *const u8, *const u16, i32, i32, i32, *mut *mut mpq_weight) -> i32,
    pub mpq_q4_weight_create_dev: unsafe extern "C" fn(*mut mpq_context, i64, i64, *const u8, *const u16, *mut *mut mpq_weight) -> i32,
    pub mpq_nvfp4_weight_create: unsafe extern "C" fn(*mut mpq_context, i64, i64, *const u8, *const u8, f32, *mut *mut mpq_weight) -> i32,
    pub mpq_weight_shape: unsafe extern "C" fn(*const mpq_weight, *mut i64, *mut i64, *mut i32) -> i32,
    pub mpq_weight_dequantize: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *mut f32, *mut c_void) -> i32,
    pub mpq_weight_device_bytes: unsafe extern "C" fn(*const mpq_weight) -> i64,
    pub mpq_weight_destroy: unsafe extern "C" fn(*mut mpq_weight) -> i32,
    pub mpq_q4_linear_forward: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *const f32, i64, *mut f32, *mut c_void) -> i32,
    pub mpq_q4_linear_forward_static: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *const f32, i64, *mut f32, *mut i32, *mut c_void) -> i32,
    pub mpq_q4_linear_forward_host: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *const f32, i64, *mut f32) -> i32,
    pub mpq_exchange_create: unsafe extern "C" fn(*mut mpq_context, i32, i32, i64, *mut *mut mpq_exchange) -> i32,
    pub mpq_exchange_ipc_handle: unsafe extern "C" fn(*mut mpq_exchange, *mut u8) -> i32,
    pub mpq_exchange_attach: unsafe extern "C" fn(*mut mpq_exchange, *const u8) -> i32,
    pub mpq_exchange_attach_pointers: unsafe extern "C" fn(*mut mpq_exchange, *const *mut c_void) -> i32,
    pub mpq_exchange_buffer: unsafe extern "C" fn(*mut mpq_exchange, *mut *mut c_void, *mut i64) -> i32,
    pub mpq_exchange_set_wait_limit: unsafe extern "C" fn(*mut mpq_exchange, u32) -> i32,
    pub mpq_exchange_graph_check: unsafe extern "C" fn(*mut mpq_exchange) -> i32,
    pub mpq_exchange_destroy: unsafe extern "C" fn(*mut mpq_exchange) -> i32,
    pub mpq_q4_linear_forward_allreduce: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *mut mpq_exchange, *const f32, i64, *mut f32, *mut c_void) -> i32,
    pub mpq_nvfp4_gemm_forward: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *const u8, *const u8, f32, i64, *mut u16, *mut c_void) -> i32,
    pub mpq_nvfp4_dequantize: unsafe extern "C" fn(*mut mpq_context, i64, i64, *const u8, *const u8, f32, *mut f32, *mut c_void) -> i32,
    pub mpq_nvfp4_quantize_activations: unsafe extern "C" fn(*mut mpq_context, *const c_void, i32, i64, i64, f32, *mut u8, *mut u8, *mut c_void) -> i32,
    pub mpq_nvfp4_quantize_swiglu: unsafe extern "C" fn(*mut mpq_context, *const c_void, i32, i64, i64, f32, *mut u8, *mut u8, *mut c_void) -> i32,
    pub mpq_swiglu: unsafe extern "C" fn(*mut mpq_context, *const f32, i64, i64, *mut f32, *mut c_void) -> i32,
    pub mpq_q4_linear_forward_swiglu: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *const f32, i64, *mut f32, *mut c_void) -> i32,
    pub mpq_file_info: unsafe extern "C" fn(*const c_char, *mut mpq_file_info_t) -> i32,
    pub mpq_canonical_save: unsafe extern "C" fn(*const c_char, i32, i64, i64, *const u8, *const c_void, f32) -> i32,
    pub mpq_canonical_load: unsafe extern "C" fn(*const c_char, *mut u8, i64, *mut c_void, i64, *mut f32) -> i32,
    pub mpq_weight_save: unsafe extern "C" fn(*mut mpq_context, *const mpq_weight, *const c_char) -> i32,
    pub mpq_weight_load: unsafe extern "C" fn(*mut mpq_context, *const c_char, *mut *mut mpq_weight) -> i32,
    pub mpq_probe_hbm_read: unsafe extern "C" fn(*mut mpq_context, *const c_void, i64, *mut u32, *mut c_void) -> i32,
    pub mpq_probe_fp4_mma: unsafe extern "C" fn(*mut mpq_context, i32, *mut f64, *mut c_void) -> i32,
    pub mpq_probe_f16_mma: unsafe extern "C" fn(*mut mpq_context, i32, i32, i32, *mut f64) -> i32,
    _keep_module_alive: *mut c_void,
}

macro_rules! sym {
    ($h:expr, $name:literal) => {{
        let c = CString::new($name).unwrap();
        let p = dlsym($h, c.as_ptr());
        if p.is_null() {
            dlclose($h);
            return Err(format!("libmpq: symbol {} not found", $name));
        }
        std::mem::transmute(p)
    }};
}

impl LibMpq {
    /// Loads the library; a missing file or symbol is an `Err`, never a panic.
    pub fn try_load(path: &str) -> Result<LibMpq, String> {
        unsafe {
            let c = CString::new(path).map_err(|e| e.to_string())?;
            let h = dlopen(c.as_ptr(), RTLD_NOW);
            if h.is_null() {
                return Err(format!("libmpq: cannot load {}", path));
            }
            Ok(LibMpq {
                mpq_context_create: sym!(h, "mpq_context_create"),
                mpq_context_destroy: sym!(h, "mpq_context_destroy"),
                mpq_context_info: sym!(h, "mpq_context_info"),
                mpq_status_string: sym!(h, "mpq_status_string"),
                mpq_last_error: sym!(h, "mpq_last_error"),
                mpq_context_poll_status: sym!(h, "mpq_context_poll_status"),
                mpq_context_launch_count: sym!(h, "mpq_context_launch_count"),
                mpq_q4_weight_create: sym!(h, "mpq_q4_weight_create"),
                mpq_q4_weight_create_dev: sym!(h, "mpq_q4_weight_create_dev"),
                mpq_nvfp4_weight_create: sym!(h, "mpq_nvfp4_weight_create"),
                mpq_weight_shape: sym!(h, "mpq_weight_shape"),
                mpq_weight_dequantize: sym!(h, "mpq_weight_dequantize"),
                mpq_weight_device_bytes: sym!(h, "mpq_weight_device_bytes"),
                mpq_weight_destroy: sym!(h, "mpq_weight_destroy"),
                mpq_q4_linear_forward: sym!(h, "mpq_q4_linear_forward"),
                mpq_q4_linear_forward_static: sym!(h, "mpq_q4_linear_forward_static"),
                mpq_q4_linear_forward_host: sym!(h, "mpq_q4_linear_forward_host"),
                mpq_exchange_create: sym!(h, "mpq_exchange_create"),
                mpq_exchange_ipc_handle: sym!(h, "mpq_exchange_ipc_handle"),
                mpq_exchange_attach: sym!(h, "mpq_exchange_attach"),
                mpq_exchange_attach_pointers: sym!(h, "mpq_exchange_attach_pointers"),
                mpq_exchange_buffer: sym!(h, "mpq_exchange_buffer"),
                mpq_exchange_set_wait_limit: sym!(h, "mpq_exchange_set_wait_limit"),
                mpq_exchange_graph_check: sym!(h, "mpq_exchange_graph_check"),
                mpq_exchange_destroy: sym!(h, "mpq_exchange_destroy"),
                mpq_q4_linear_forward_allreduce: sym!(h, "mpq_q4_linear_forward_allreduce"),
                mpq_nvfp4_gemm_forward: sym!(h, "mpq_nvfp4_gemm_forward"),
                mpq_nvfp4_dequantize: sym!(h, "mpq_nvfp4_dequantize"),
                mpq_nvfp4_quantize_activations: sym!(h, "mpq_nvfp4_quantize_activations"),
                mpq_nvfp4_quantize_swiglu: sym!(h, "mpq_nvfp4_quantize_swiglu"),
                mpq_swiglu: sym!(h, "mpq_swiglu"),
                mpq_q4_linear_forward_swiglu: sym!(h, "mpq_q4_linear_forward_swiglu"),
                mpq_file_info: sym!(h, "mpq_file_info"),
                mpq_canonical_save: sym!(h, "mpq_canonical_save"),
                mpq_canonical_load: sym!(h, "mpq_canonical_load"),
                mpq_weight_save: sym!(h, "mpq_weight_save"),
                mpq_weight_load: sym!(h, "mpq_weight_load"),
                mpq_probe_hbm_read: sym!(h, "mpq_probe_hbm_read"),
                mpq_probe_fp4_mma: sym!(h, "mpq_probe_fp4_mma"),
                mpq_probe_f16_mma: sym!(h, "mpq_probe_f16_mma"),
                _keep_module_alive: h,
            })
        }
    }

    pub fn status_text(&self, status: i32) -> String {
        unsafe { CStr::from_ptr((self.mpq_status_string)(status)).to_string_lossy().into_owned() }
    }
}
