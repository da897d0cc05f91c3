//! Safe host side of the B200 `cuda` target: one [`Context`] = one native session = one KV cache.
//!
//! Counterpart of `crates/iree-runtime/src/lib.rs` for `libdyninfer_cuda`:
//! * [`FileRanges`] owns the C strings of the `(key, file, offset, length)` provider plan
//!   (`crates/iree-runtime/src/lib.rs:139-215` validates the same way: non-empty keys, file index
//!   in range, no interior NULs; payload bytes are never read on the Rust side);
//! * [`Context`] creates the native session lazily under a `Mutex`, because a session is
//!   thread-compatible, not thread-safe (`crates/iree-runtime/src/lib.rs:110-121,268-277`);
//! * every failing call becomes `DynInferError::IreeRuntime`-shaped runtime error carrying the
//!   library's thread-local message and the return code (`:645-650`);
//! * logits are session-owned scratch borrowed until the next invoke, so they are copied into a
//!   `Vec<f32>` before the lock is released (`:652-667`).
//!
//! Not compiled in this repository's build image (no `rustc`). `tests/abi_driver.c` drives the
//! same sequence of calls from C on a GPU.

pub mod session;

use dyninfer_cuda_sys as sys;
use dyninfer_error::{DynInferError, IreeRuntimeError, Result};
use std::ffi::{CStr, CString};
use std::path::{Path, PathBuf};
use std::ptr::{self, NonNull};
use std::sync::{Arc, Mutex};

pub use session::CudaSession;

fn runtime_error(message: impl Into<String>, status_code: Option<i32>) -> DynInferError {
    DynInferError::IreeRuntime(IreeRuntimeError {
        message: message.into(),
        status_code,
    })
}

/// The library's thread-local message for the call that just failed on this thread.
fn last_error_string() -> String {
    // SAFETY: the pointer is either null or a NUL-terminated string owned by the library and
    // valid until the next failing call on this thread.
    unsafe {
        let p = sys::dyninfer_cuda_last_error();
        if p.is_null() {
            "unknown dyninfer-cuda error".to_owned()
        } else {
            CStr::from_ptr(p).to_string_lossy().into_owned()
        }
    }
}

fn native_error(code: i32) -> DynInferError {
    runtime_error(last_error_string(), Some(code))
}

fn check(code: i32) -> Result<()> {
    if code == 0 { Ok(()) } else { Err(native_error(code)) }
}

/// Communicator id for a tensor-parallel group: created on rank 0 and handed to every rank (over
/// whatever channel the launcher has) for `Context::with_tensor_parallel`.
pub fn tp_unique_id() -> Result<Vec<u8>> {
    // SAFETY: plain query.
    let mut id = vec![0u8; unsafe { sys::dyninfer_cuda_tp_unique_id_bytes() }];
    // SAFETY: `id` holds the advertised number of bytes.
    check(unsafe { sys::dyninfer_cuda_tp_unique_id(id.as_mut_ptr(), id.len()) })?;
    Ok(id)
}

/// Number of usable CUDA devices. Fails (never falls back to a CPU) when there is none.
pub fn device_count() -> Result<usize> {
    let mut n = 0;
    // SAFETY: plain out-parameter.
    check(unsafe { sys::dyninfer_cuda_device_count(&mut n) })?;
    Ok(n.max(0) as usize)
}

/// One contiguous byte range of an original checkpoint file behind a stable external key
/// (`"{scope}::{canonical}::{component}"`, `crates/dyninfer-binding/src/lib.rs:247-250`).
#[derive(Debug, Clone, PartialEq, Eq)]
pub struct FileRange {
    pub key: String,
    pub source_file_index: usize,
    pub offset: u64,
    pub length: u64,
}

/// Owns the strings handed to the native session; shared by independent sessions.
#[derive(Debug)]
pub struct FileRanges {
    files: Vec<CString>,
    keys: Vec<CString>,
    ranges: Vec<FileRange>,
}

impl FileRanges {
    pub fn new(files: &[PathBuf], ranges: Vec<FileRange>) -> Result<Self> {
        if files.is_empty() {
            return Err(runtime_error("parameter provider has no source files", None));
        }
        let c_files = files
            .iter()
            .map(|p| path_cstring(p))
            .collect::<Result<Vec<_>>>()?;
        let mut keys = Vec::with_capacity(ranges.len());
        for r in &ranges {
            if r.key.is_empty() {
                return Err(runtime_error("parameter key is empty", None));
            }
            if r.source_file_index >= files.len() {
                return Err(runtime_error(
                    format!(
                        "parameter `{}` names source file {} of {}",
                        r.key,
                        r.source_file_index,
                        files.len()
                    ),
                    None,
                ));
            }
            if r.offset.checked_add(r.length).is_none() {
                return Err(runtime_error(format!("parameter `{}` byte range overflows", r.key), None));
            }
            keys.push(
                CString::new(r.key.as_str())
                    .map_err(|e| runtime_error(format!("parameter key `{}`: {e}", r.key), None))?,
            );
        }
        Ok(Self { files: c_files, keys, ranges })
    }

    pub fn len(&self) -> usize {
        self.ranges.len()
    }

    pub fn is_empty(&self) -> bool {
        self.ranges.is_empty()
    }
}

fn path_cstring(p: &Path) -> Result<CString> {
    CString::new(p.to_string_lossy().as_bytes())
        .map_err(|e| runtime_error(format!("path {}: {e}", p.display()), None))
}

/// Allocator counters of one session (`AllocatorMetrics`, `crates/dyninfer-runtime/src/lib.rs:100-117`).
pub type AllocatorStatistics = sys::dyninfer_cuda_allocator_statistics_t;

struct NativeSession(NonNull<sys::dyninfer_cuda_session_t>);

// SAFETY: a native session may be used from any thread as long as calls do not overlap; the
// `Mutex` in `Context` guarantees that (same contract as `crates/iree-runtime/src/lib.rs:92-95`).
unsafe impl Send for NativeSession {}

impl Drop for NativeSession {
    fn drop(&mut self) {
        // SAFETY: created by session_create_with_file_params and destroyed exactly once.
        unsafe { sys::dyninfer_cuda_session_destroy(self.0.as_ptr()) };
    }
}

/// Geometry handed to `configure_paged_kv` (`KvCacheDescriptor` with `KvCacheStorage::Paged`).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub struct PagedKvGeometry {
    pub layer_count: usize,
    pub page_size: usize,
    pub kv_head_count: usize,
    pub head_dim: usize,
    /// 4 = f32 cache, 2 = the 2-byte type the model descriptor names (bf16 by default).
    pub element_bytes: usize,
    pub chunk_size: usize,
    pub vocab_size: usize,
}

/// Execution context of the cuda target. Cheap to share behind an `Arc`; the native session is
/// created on first use.
pub struct Context {
    device_uri: CString,
    /// Model geometry plus per-parameter encoding and logical shape: what the compiled module
    /// carries on the IREE targets (`include/dyninfer_cuda.h`, session_create_with_file_params).
    model_descriptor: CString,
    ranges: Arc<FileRanges>,
    geometry: PagedKvGeometry,
    /// Communicator id of the tensor-parallel group this context is one rank of (the descriptor
    /// then carries `tp_rank` / `tp_world` and the ranges are the rank's slices).
    tp_unique_id: Option<Vec<u8>>,
    session: Mutex<Option<NativeSession>>,
}

impl Context {
    pub fn new(
        device_uri: &str,
        model_descriptor_json: &str,
        ranges: Arc<FileRanges>,
        geometry: PagedKvGeometry,
    ) -> Result<Self> {
        Ok(Self {
            device_uri: CString::new(device_uri)
                .map_err(|e| runtime_error(format!("invalid device string: {e}"), None))?,
            model_descriptor: CString::new(model_descriptor_json)
                .map_err(|e| runtime_error(format!("invalid model descriptor: {e}"), None))?,
            ranges,
            geometry,
            tp_unique_id: None,
            session: Mutex::new(None),
        })
    }

    /// Makes this context one rank of a tensor-parallel group. `unique_id` is what `tp_unique_id()`
    /// returned on rank 0, handed to every rank by the launcher; the group is joined when the native
    /// session is created (every rank must then create its session: the call is collective).
    pub fn with_tensor_parallel(mut self, unique_id: Vec<u8>) -> Self {
        self.tp_unique_id = Some(unique_id);
        self
    }

    /// Runs `f` with the native handle, creating and configuring the session on first use.
    fn with_session<R>(&self, f: impl FnOnce(*mut sys::dyninfer_cuda_session_t) -> Result<R>) -> Result<R> {
        let mut guard = self
            .session
            .lock()
            .map_err(|_| runtime_error("dyninfer-cuda session mutex poisoned", None))?;
        if guard.is_none() {
            let files: Vec<sys::dyninfer_cuda_parameter_file_t> = self
                .ranges
                .files
                .iter()
                .map(|p| sys::dyninfer_cuda_parameter_file_t { path: p.as_ptr() })
                .collect();
            let params: Vec<sys::dyninfer_cuda_file_param_t> = self
                .ranges
                .ranges
                .iter()
                .zip(&self.ranges.keys)
                .map(|(r, key)| sys::dyninfer_cuda_file_param_t {
                    key: key.as_ptr(),
                    source_file_index: r.source_file_index,
                    offset: r.offset,
                    length: r.length,
                })
                .collect();
            let mut raw = ptr::null_mut();
            // SAFETY: all pointers outlive the call; the library copies what it keeps.
            let rc = unsafe {
                sys::dyninfer_cuda_session_create_with_file_params(
                    self.device_uri.as_ptr(),
                    self.model_descriptor.as_ptr(),
                    files.as_ptr(),
                    files.len(),
                    params.as_ptr(),
                    params.len(),
                    &mut raw,
                )
            };
            let handle = match NonNull::new(raw) {
                Some(h) if rc == 0 => NativeSession(h),
                _ => return Err(native_error(rc)),
            };
            if let Some(id) = &self.tp_unique_id {
                // SAFETY: valid handle; `id` outlives the call. Must precede the KV configuration.
                check(unsafe { sys::dyninfer_cuda_session_tp_init(handle.0.as_ptr(), id.as_ptr(), id.len()) })?;
            }
            let g = self.geometry;
            // SAFETY: valid handle; plain integers.
            check(unsafe {
                sys::dyninfer_cuda_session_configure_paged_kv(
                    handle.0.as_ptr(),
                    g.layer_count,
                    g.page_size,
                    g.kv_head_count,
                    g.head_dim,
                    g.element_bytes,
                    g.chunk_size,
                    g.vocab_size,
                )
            })?;
            *guard = Some(handle);
        }
        let handle = guard.as_ref().map(|s| s.0.as_ptr()).unwrap_or(ptr::null_mut());
        f(handle)
    }

    pub fn ensure_kv_pages(&self, page_count: usize) -> Result<()> {
        // SAFETY: valid handle.
        self.with_session(|s| check(unsafe { sys::dyninfer_cuda_session_ensure_kv_pages(s, page_count) }))
    }

    pub fn reset_paged_kv(&self) -> Result<()> {
        // SAFETY: valid handle.
        self.with_session(|s| check(unsafe { sys::dyninfer_cuda_session_reset_paged_kv(s) }))
    }

    /// `(page_count, allocated_bytes)` of the KV pool.
    pub fn paged_kv_metrics(&self) -> Result<(usize, usize)> {
        self.with_session(|s| {
            // SAFETY: valid handle; both calls only read.
            Ok(unsafe {
                (
                    sys::dyninfer_cuda_session_kv_page_count(s),
                    sys::dyninfer_cuda_session_kv_allocated_bytes(s),
                )
            })
        })
    }

    pub fn allocator_statistics(&self) -> Result<AllocatorStatistics> {
        self.with_session(|s| {
            let mut st = AllocatorStatistics::default();
            // SAFETY: valid handle and out-parameter.
            check(unsafe { sys::dyninfer_cuda_session_allocator_statistics(s, &mut st) })?;
            Ok(st)
        })
    }

    /// One chunk of the sequence: `tokens.len()` is the chunk size or 1, rows `0..=last` are real,
    /// positions start at `start_pos`. Returns the logits of row `last` (only when asked: the
    /// vocabulary-sized copy is skipped otherwise) and the first strict maximum of those logits.
    pub fn invoke_paged_chunk_ex(
        &self,
        tokens: &[i64],
        last: i64,
        start_pos: i64,
        want_logits: bool,
    ) -> Result<(Option<Vec<f32>>, i64)> {
        self.with_session(|s| {
            let mut view: *mut f32 = ptr::null_mut();
            let mut count = 0usize;
            let mut token = -1i64;
            // SAFETY: `tokens` outlives the call; out-parameters are local; NULL logits
            // pointers are allowed when want_logits = 0.
            let rc = unsafe {
                sys::dyninfer_cuda_session_invoke_paged_chunk(
                    s,
                    tokens.as_ptr(),
                    tokens.len(),
                    last,
                    start_pos,
                    if want_logits { &mut view } else { ptr::null_mut() },
                    if want_logits { &mut count } else { ptr::null_mut() },
                    &mut token,
                    want_logits as i32,
                )
            };
            check(rc)?;
            let logits = if want_logits {
                if view.is_null() {
                    return Err(runtime_error("null logits pointer from the cuda session", None));
                }
                // SAFETY: the library guarantees `count` floats at `view` until the next invoke
                // on this session; we still hold the session lock, and copy before releasing it.
                let values = unsafe { std::slice::from_raw_parts(view, count) }.to_vec();
                // SAFETY: a no-op for session scratch, kept for symmetry with the IREE wrapper.
                unsafe { sys::dyninfer_cuda_free(view.cast()) };
                Some(values)
            } else {
                None
            };
            Ok((logits, token))
        })
    }

    pub fn invoke_paged_chunk(&self, tokens: &[i64], last: i64, start_pos: i64) -> Result<Vec<f32>> {
        let (logits, _) = self.invoke_paged_chunk_ex(tokens, last, start_pos, true)?;
        logits.ok_or_else(|| runtime_error("logits were requested but not returned", None))
    }

    /// `invoke_paged_chunk_ex` for KV slot `slot` of a session whose descriptor sets `"batch"` > 1.
    /// Sequences in different slots are independent; each has its own positions.
    pub fn invoke_paged_chunk_slot(
        &self,
        tokens: &[i64],
        last: i64,
        start_pos: i64,
        slot: i64,
        want_logits: bool,
    ) -> Result<(Option<Vec<f32>>, i64)> {
        self.with_session(|s| {
            let mut view: *mut f32 = ptr::null_mut();
            let mut count = 0usize;
            let mut token = -1i64;
            // SAFETY: as in `invoke_paged_chunk_ex`.
            check(unsafe {
                sys::dyninfer_cuda_session_invoke_paged_chunk_slot(
                    s,
                    tokens.as_ptr(),
                    tokens.len(),
                    last,
                    start_pos,
                    slot,
                    if want_logits { &mut view } else { ptr::null_mut() },
                    if want_logits { &mut count } else { ptr::null_mut() },
                    &mut token,
                    want_logits as i32,
                )
            })?;
            let logits = if want_logits && !view.is_null() {
                // SAFETY: `count` floats at `view` until the next invoke; copied under the lock.
                Some(unsafe { std::slice::from_raw_parts(view, count) }.to_vec())
            } else {
                None
            };
            Ok((logits, token))
        })
    }

    /// One decode step for several slots in one pass over the weights: row `i` feeds `tokens[i]` at
    /// `positions[i]` into KV slot `slots[i]`. Returns the next token of every row and, when asked,
    /// the logits as `tokens.len()` rows of `vocab` values.
    pub fn decode_batch(
        &self,
        tokens: &[i64],
        positions: &[i64],
        slots: &[i64],
        want_logits: bool,
    ) -> Result<(Vec<i64>, Option<Vec<f32>>)> {
        if tokens.len() != positions.len() || tokens.len() != slots.len() {
            return Err(runtime_error("decode_batch: tokens, positions and slots differ in length", None));
        }
        let vocab = self.geometry.vocab_size;
        self.with_session(|s| {
            let mut out = vec![-1i64; tokens.len()];
            let mut view: *mut f32 = ptr::null_mut();
            // SAFETY: the three inputs and `out` hold `tokens.len()` entries each.
            check(unsafe {
                sys::dyninfer_cuda_session_decode_batch(
                    s,
                    tokens.as_ptr(),
                    positions.as_ptr(),
                    slots.as_ptr(),
                    tokens.len(),
                    out.as_mut_ptr(),
                    if want_logits { &mut view } else { ptr::null_mut() },
                    want_logits as i32,
                )
            })?;
            let logits = if want_logits && !view.is_null() {
                // SAFETY: session scratch of rows x vocab floats, valid until the next call; copied
                // while the lock is held.
                Some(unsafe { std::slice::from_raw_parts(view, tokens.len() * vocab) }.to_vec())
            } else {
                None
            };
            Ok((out, logits))
        })
    }

    /// This rank's exchange-region handle for the fused peer-memory exchange (after the KV pool is
    /// configured, i.e. after first use). The launcher gathers every rank's handle, in rank order.
    pub fn tp_peer_handle(&self) -> Result<Vec<u8>> {
        self.with_session(|s| {
            // SAFETY: plain query.
            let mut buf = vec![0u8; unsafe { sys::dyninfer_cuda_tp_peer_handle_bytes() }];
            // SAFETY: `buf` holds the advertised number of bytes.
            check(unsafe { sys::dyninfer_cuda_session_tp_peer_handle(s, buf.as_mut_ptr(), buf.len()) })?;
            Ok(buf)
        })
    }

    /// Maps the peers' exchange regions: `handles` = all ranks' handles concatenated in rank order.
    /// Without this call the partial sums go through NCCL.
    pub fn tp_peer_attach(&self, handles: &[u8]) -> Result<()> {
        // SAFETY: valid handle; `handles` outlives the call.
        self.with_session(|s| check(unsafe { sys::dyninfer_cuda_session_tp_peer_attach(s, handles.as_ptr(), handles.len()) }))
    }

    /// Device-resident greedy loop (no host round trip per token). Returns the tokens produced and
    /// the CUDA-event time of the loop in milliseconds.
    pub fn decode_loop(&self, first_token: i64, start_pos: i64, steps: usize) -> Result<(Vec<i64>, f32)> {
        self.with_session(|s| {
            let mut out = vec![0i64; steps];
            let mut ms = 0f32;
            // SAFETY: `out` holds `steps` entries.
            check(unsafe {
                sys::dyninfer_cuda_session_decode_loop(s, first_token, start_pos, steps, out.as_mut_ptr(), &mut ms)
            })?;
            Ok((out, ms))
        })
    }

    /// Bytes of parameters one decode step reads (for `eff_weight_bw_gbs`,
    /// `crates/dyninfer-runtime/src/perf.rs:298-305`).
    pub fn decode_weight_bytes(&self) -> Result<u64> {
        // SAFETY: valid handle; read only.
        self.with_session(|s| Ok(unsafe { sys::dyninfer_cuda_session_decode_weight_bytes(s) }))
    }

    /// Starts the device-side stopwatch on the session's stream (after the work queued so far).
    pub fn timer_start(&self) -> Result<()> {
        // SAFETY: valid handle; a null output is allowed when `stop` is 0.
        self.with_session(|s| check(unsafe { sys::dyninfer_cuda_session_timer(s, 0, std::ptr::null_mut()) }))
    }

    /// Stops the stopwatch, waits for the stream and returns the milliseconds it spent since `timer_start`.
    pub fn timer_stop(&self) -> Result<f32> {
        self.with_session(|s| {
            let mut ms = 0f32;
            // SAFETY: `ms` outlives the call.
            check(unsafe { sys::dyninfer_cuda_session_timer(s, 1, &mut ms) })?;
            Ok(ms)
        })
    }

    pub fn uses_persistent_kernel(&self) -> Result<bool> {
        // SAFETY: valid handle; read only.
        self.with_session(|s| Ok(unsafe { sys::dyninfer_cuda_session_uses_persistent_kernel(s) } != 0))
    }
}
