//! Unsafe bindings to `libdyninfer_cuda`, the C ABI of the B200 (`sm_100a`) `cuda` target.
//!
//! One declaration per export of `include/dyninfer_cuda.h`, written by hand (the header is
//! small and stable; no bindgen step). The session half mirrors what
//! `crates/iree-runtime-sys/src/lib.rs:53-145` declares for the IREE wrapper; the operator half
//! and the `tp_*` / batching entry points are extensions of the cuda target.
//!
//! Not compiled in this repository's build image (no `rustc`); the same ABI is driven from C by
//! `tests/abi_driver.c` and from Python by `dyninfer_b200/_lib.py`.

#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_void};

pub const DYNINFER_CUDA_ABI_VERSION: c_int = 1;

pub const DYNINFER_ENC_F32: i32 = 0;
pub const DYNINFER_ENC_F16: i32 = 1;
pub const DYNINFER_ENC_BF16: i32 = 2;
pub const DYNINFER_ENC_Q4_0: i32 = 3;
pub const DYNINFER_ENC_Q4_1: i32 = 4;
pub const DYNINFER_ENC_Q8_0: i32 = 5;
pub const DYNINFER_ENC_Q6_K: i32 = 6;
pub const DYNINFER_ENC_MLX_U4: i32 = 7;
pub const DYNINFER_ENC_Q4_K: i32 = 8;
pub const DYNINFER_ENC_Q5_K: i32 = 9;
pub const DYNINFER_ENC_IQ4_XS: i32 = 10;

/// Opaque session: one KV cache, one parameter arena, one stream.
#[repr(C)]
pub struct dyninfer_cuda_session_t {
    _private: [u8; 0],
}

/// One `[rows, cols]` parameter as its verbatim checkpoint bytes in device memory.
#[repr(C)]
#[derive(Debug, Clone, Copy)]
pub struct dyninfer_cuda_weight_t {
    pub encoding: i32,
    pub aux_type: i32,
    pub group: i32,
    pub reserved: i32,
    pub rows: i64,
    pub cols: i64,
    pub data: *const c_void,
    pub scales: *const c_void,
    pub biases: *const c_void,
}

#[repr(C)]
pub struct dyninfer_cuda_parameter_file_t {
    pub path: *const c_char,
}

#[repr(C)]
pub struct dyninfer_cuda_file_param_t {
    pub key: *const c_char,
    pub source_file_index: usize,
    pub offset: u64,
    pub length: u64,
}

#[repr(C)]
#[derive(Debug, Default, Clone, Copy)]
pub struct dyninfer_cuda_allocator_statistics_t {
    pub host_bytes_peak: u64,
    pub host_bytes_allocated: u64,
    pub host_bytes_freed: u64,
    pub device_bytes_peak: u64,
    pub device_bytes_allocated: u64,
    pub device_bytes_freed: u64,
}

unsafe extern "C" {
    // ---- library
    pub fn dyninfer_cuda_abi_version() -> c_int;
    pub fn dyninfer_cuda_last_error() -> *const c_char;
    pub fn dyninfer_cuda_device_count(out_count: *mut c_int) -> c_int;
    pub fn dyninfer_cuda_row_bytes(encoding: c_int, cols: i64) -> u64;
    pub fn dyninfer_cuda_check_device_error() -> c_int;
    pub fn dyninfer_cuda_free(p: *mut c_void);

    // ---- single operators (device pointers, asynchronous on `stream`)
    pub fn dyninfer_cuda_dequant(w: *const dyninfer_cuda_weight_t, out_dev: *mut f32, stream: *mut c_void) -> c_int;
    pub fn dyninfer_cuda_embedding_gather(
        w: *const dyninfer_cuda_weight_t,
        tokens_dev: *const i64,
        count: i64,
        out_dev: *mut f32,
        stream: *mut c_void,
    ) -> c_int;
    pub fn dyninfer_cuda_linear(
        w: *const dyninfer_cuda_weight_t,
        x_dev: *const c_void,
        x_type: c_int,
        m: i64,
        y_dev: *mut f32,
        stream: *mut c_void,
    ) -> c_int;
    pub fn dyninfer_cuda_rms_norm(
        x_dev: *const f32,
        w_dev: *const c_void,
        w_type: c_int,
        rows: i64,
        width: i64,
        eps: f32,
        y_dev: *mut f32,
        stream: *mut c_void,
    ) -> c_int;
    pub fn dyninfer_cuda_rope(
        x_dev: *mut f32,
        s: i64,
        heads: i64,
        d: i64,
        start_pos: i64,
        theta: f32,
        stream: *mut c_void,
    ) -> c_int;
    pub fn dyninfer_cuda_silu_mul(
        gate_dev: *const f32,
        up_dev: *const f32,
        n: i64,
        y_dev: *mut f32,
        stream: *mut c_void,
    ) -> c_int;
    pub fn dyninfer_cuda_attention(
        q_dev: *const f32,
        k_cache_dev: *const c_void,
        v_cache_dev: *const c_void,
        kv_type: c_int,
        s: i64,
        heads: i64,
        kv_heads: i64,
        d: i64,
        kv_cap: i64,
        start_pos: i64,
        ctx_dev: *mut f32,
        stream: *mut c_void,
    ) -> c_int;
    pub fn dyninfer_cuda_argmax_scratch_bytes(n: i64) -> usize;
    pub fn dyninfer_cuda_argmax(
        v_dev: *const f32,
        n: i64,
        out_index_dev: *mut i64,
        scratch_dev: *mut c_void,
        stream: *mut c_void,
    ) -> c_int;
    pub fn dyninfer_cuda_argmax_static_max_n() -> i64;
    pub fn dyninfer_cuda_argmax_static(
        v_dev: *const f32,
        n: i64,
        out_index_dev: *mut i64,
        stream: *mut c_void,
    ) -> c_int;

    // ---- session (paged-KV ABI; third_party/iree_runtime_c_api/wrapper.h:46-122)
    pub fn dyninfer_cuda_session_create_with_file_params(
        device_uri: *const c_char,
        model_desc_json: *const c_char,
        files: *const dyninfer_cuda_parameter_file_t,
        file_count: usize,
        params: *const dyninfer_cuda_file_param_t,
        param_count: usize,
        out_session: *mut *mut dyninfer_cuda_session_t,
    ) -> c_int;
    pub fn dyninfer_cuda_session_destroy(session: *mut dyninfer_cuda_session_t);
    pub fn dyninfer_cuda_session_configure_paged_kv(
        session: *mut dyninfer_cuda_session_t,
        layer_count: usize,
        page_size: usize,
        kv_head_count: usize,
        head_dim: usize,
        kv_element_byte_count: usize,
        chunk_size: usize,
        vocab_size: usize,
    ) -> c_int;
    pub fn dyninfer_cuda_session_ensure_kv_pages(session: *mut dyninfer_cuda_session_t, page_count: usize) -> c_int;
    pub fn dyninfer_cuda_session_invoke_paged_chunk(
        session: *mut dyninfer_cuda_session_t,
        tokens: *const i64,
        token_count: usize,
        last: i64,
        start_pos: i64,
        out_logits: *mut *mut f32,
        out_count: *mut usize,
        out_token: *mut i64,
        want_logits: c_int,
    ) -> c_int;
    pub fn dyninfer_cuda_session_reset_paged_kv(session: *mut dyninfer_cuda_session_t) -> c_int;
    pub fn dyninfer_cuda_session_kv_page_count(session: *const dyninfer_cuda_session_t) -> usize;
    pub fn dyninfer_cuda_session_kv_allocated_bytes(session: *const dyninfer_cuda_session_t) -> usize;
    pub fn dyninfer_cuda_session_allocator_statistics(
        session: *const dyninfer_cuda_session_t,
        out_stats: *mut dyninfer_cuda_allocator_statistics_t,
    ) -> c_int;

    // ---- batching
    pub fn dyninfer_cuda_session_invoke_paged_chunk_slot(
        session: *mut dyninfer_cuda_session_t,
        tokens: *const i64,
        token_count: usize,
        last: i64,
        start_pos: i64,
        slot: i64,
        out_logits: *mut *mut f32,
        out_count: *mut usize,
        out_token: *mut i64,
        want_logits: c_int,
    ) -> c_int;
    pub fn dyninfer_cuda_session_decode_batch(
        session: *mut dyninfer_cuda_session_t,
        tokens: *const i64,
        positions: *const i64,
        slots: *const i64,
        count: usize,
        out_tokens: *mut i64,
        out_logits: *mut *mut f32,
        want_logits: c_int,
    ) -> c_int;

    // ---- tensor parallelism
    pub fn dyninfer_cuda_tp_unique_id_bytes() -> usize;
    pub fn dyninfer_cuda_tp_unique_id(out_id: *mut u8, byte_count: usize) -> c_int;
    pub fn dyninfer_cuda_session_tp_init(session: *mut dyninfer_cuda_session_t, id: *const u8, byte_count: usize) -> c_int;
    pub fn dyninfer_cuda_tp_peer_handle_bytes() -> usize;
    pub fn dyninfer_cuda_session_tp_peer_handle(
        session: *mut dyninfer_cuda_session_t,
        out_handle: *mut u8,
        byte_count: usize,
    ) -> c_int;
    pub fn dyninfer_cuda_session_tp_peer_attach(
        session: *mut dyninfer_cuda_session_t,
        handles: *const u8,
        byte_count: usize,
    ) -> c_int;
    pub fn dyninfer_cuda_tp_exchange_wait_probe(hidden: c_int, rows: i64, spin_limit: i64) -> c_int;

    // ---- session extensions
    pub fn dyninfer_cuda_session_weight_bytes(session: *const dyninfer_cuda_session_t) -> u64;
    pub fn dyninfer_cuda_session_decode_weight_bytes(session: *const dyninfer_cuda_session_t) -> u64;
    pub fn dyninfer_cuda_session_decode_loop(
        session: *mut dyninfer_cuda_session_t,
        first_token: i64,
        start_pos: i64,
        steps: usize,
        out_tokens: *mut i64,
        out_device_ms: *mut f32,
    ) -> c_int;
    pub fn dyninfer_cuda_session_uses_persistent_kernel(session: *const dyninfer_cuda_session_t) -> c_int;
    pub fn dyninfer_cuda_session_decode_phase_profile(
        session: *mut dyninfer_cuda_session_t,
        out_us: *mut f64,
        count: usize,
    ) -> c_int;
    pub fn dyninfer_cuda_session_decode_trace(
        session: *mut dyninfer_cuda_session_t,
        out: *mut u64,
        count: usize,
        out_needed: *mut usize,
    ) -> c_int;
    pub fn dyninfer_cuda_session_launch_count(session: *const dyninfer_cuda_session_t) -> u64;
    pub fn dyninfer_cuda_session_timer(session: *mut dyninfer_cuda_session_t, stop: c_int, out_ms: *mut f32) -> c_int;
}
