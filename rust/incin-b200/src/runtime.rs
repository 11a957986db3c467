//! The native host runtime: plan-hash digest, batch loader, telemetry sink (csrc/runtime of `libincin_host.so`).
use core::ffi::c_void;
use std::ffi::CString;
use std::path::Path;

use incin_b200_sys as sys;

/// Streaming FNV-1a 64 with the field encoding of the plan hash: `number` = 8 little-endian bytes, `field` =
/// number(length) + bytes, `text` = field(utf-8).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub struct Digest {
    state: u64,
}

impl Default for Digest {
    fn default() -> Self {
        Digest::new()
    }
}

impl Digest {
    pub fn new() -> Self {
        // SAFETY: no arguments.
        Digest { state: unsafe { sys::incin_digest_init() } }
    }

    pub fn bytes(mut self, b: &[u8]) -> Self {
        // SAFETY: pointer and length describe `b`.
        self.state = unsafe { sys::incin_digest_bytes(self.state, b.as_ptr() as *const c_void, b.len() as i64) };
        self
    }

    pub fn number(mut self, v: u64) -> Self {
        // SAFETY: plain arithmetic.
        self.state = unsafe { sys::incin_digest_number(self.state, v) };
        self
    }

    pub fn field(mut self, b: &[u8]) -> Self {
        // SAFETY: pointer and length describe `b`.
        self.state = unsafe { sys::incin_digest_field(self.state, b.as_ptr() as *const c_void, b.len() as i64) };
        self
    }

    pub fn text(self, t: &str) -> Self {
        self.field(t.as_bytes())
    }

    pub fn finish(self) -> u64 {
        self.state
    }
}

/// Batches of `f32` rows (and optional `i64` targets) gathered by native worker threads, delivered in order.
/// The batch sequence depends on (seed, epoch, batch size) only, not on the number of workers.
pub struct BatchLoader<'a> {
    handle: i64,
    row_len: usize,
    batch: usize,
    has_targets: bool,
    _data: core::marker::PhantomData<&'a [f32]>,
}

/// One delivered batch.
#[derive(Debug, Clone, PartialEq)]
pub struct LoadedBatch {
    pub rows: usize,
    pub inputs: Vec<f32>,
    pub targets: Vec<i64>,
}

impl<'a> BatchLoader<'a> {
    /// `inputs` holds `n * row_len` values, `targets` (if any) `n`.  The slices must outlive the loader, which the
    /// lifetime enforces.
    pub fn new(inputs: &'a [f32], row_len: usize, targets: Option<&'a [i64]>, batch: usize, shuffle: bool, drop_last: bool,
               seed: u64, workers: usize, prefetch: usize) -> Option<Self> {
        if row_len == 0 || batch == 0 || inputs.len() % row_len != 0 {
            return None;
        }
        let n = inputs.len() / row_len;
        if let Some(t) = targets {
            if t.len() != n {
                return None;
            }
        }
        let tptr = targets.map_or(core::ptr::null(), |t| t.as_ptr() as *const c_void);
        // SAFETY: the arrays are valid for the lifetime 'a, which outlives the loader.
        let handle = unsafe {
            sys::incin_loader_create(inputs.as_ptr() as *const c_void, (row_len * 4) as i64, tptr, 8, n as i64, batch as i64,
                                     shuffle as i32, drop_last as i32, seed, workers as i32, (prefetch + 1) as i32)
        };
        if handle == 0 {
            return None;
        }
        Some(BatchLoader { handle, row_len, batch, has_targets: targets.is_some(), _data: core::marker::PhantomData })
    }

    /// Start epoch `epoch`; returns its number of batches.
    pub fn start(&mut self, epoch: u64) -> usize {
        // SAFETY: valid handle.
        let n = unsafe { sys::incin_loader_start(self.handle, epoch) };
        if n < 0 {
            0
        } else {
            n as usize
        }
    }

    /// The next batch of the running epoch, `None` at its end.
    pub fn next_batch(&mut self) -> Option<LoadedBatch> {
        let mut inputs = vec![0.0f32; self.batch * self.row_len];
        let mut targets = vec![0i64; if self.has_targets { self.batch } else { 0 }];
        let mut rows: i64 = 0;
        let tptr = if self.has_targets { targets.as_mut_ptr() as *mut c_void } else { core::ptr::null_mut() };
        // SAFETY: both buffers hold a full batch.
        let rc = unsafe { sys::incin_loader_next(self.handle, inputs.as_mut_ptr() as *mut c_void, tptr, &mut rows) };
        if rc != 1 {
            return None;
        }
        let rows = rows as usize;
        inputs.truncate(rows * self.row_len);
        if self.has_targets {
            targets.truncate(rows);
        }
        Some(LoadedBatch { rows, inputs, targets })
    }
}

impl<'a> Drop for BatchLoader<'a> {
    fn drop(&mut self) {
        // SAFETY: destroyed exactly once; joins the worker threads.
        unsafe { sys::incin_loader_destroy(self.handle) }
    }
}

/// JSON-lines telemetry sink with a bounded queue and a background writer; a full queue drops and counts.
pub struct TelemetrySink {
    handle: i64,
}

impl TelemetrySink {
    pub fn open(path: &Path, capacity: usize) -> Option<Self> {
        let c = CString::new(path.to_string_lossy().as_bytes()).ok()?;
        // SAFETY: NUL-terminated path.
        let handle = unsafe { sys::incin_telemetry_open(c.as_ptr(), capacity as i64) };
        if handle == 0 {
            None
        } else {
            Some(TelemetrySink { handle })
        }
    }

    /// `true` when queued, `false` when dropped.
    pub fn scalar(&self, name: &str, value: f64, step: i64) -> bool {
        match CString::new(name) {
            // SAFETY: NUL-terminated name.
            Ok(c) => unsafe { sys::incin_telemetry_scalar(self.handle, c.as_ptr(), value, step) == 1 },
            Err(_) => false,
        }
    }

    /// Wait until everything queued is on disk; returns the number of dropped events so far.
    pub fn flush(&self) -> i64 {
        // SAFETY: valid handle.
        unsafe { sys::incin_telemetry_flush(self.handle) }
    }
}

impl Drop for TelemetrySink {
    fn drop(&mut self) {
        // SAFETY: closed exactly once.
        unsafe {
            sys::incin_telemetry_close(self.handle);
        }
    }
}
