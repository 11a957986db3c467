//! The tape: `loss.backward()? -> Gradients`.
//!
//! Thin, safe layer over the thread-local tape of `libincin_host.so` (csrc/cpu_ref/tape.cpp), which follows the
//! reference's autograd core (crates/incin-core/src/exec/tape.rs:49-306): every differentiable op records a node while
//! gradient mode is on, `backward` seeds ones at the root, walks the nodes in reverse and accumulates fan-out.
//! Values on the tape are matrices (`rows x cols`); handles are only valid on the thread that created them and until
//! [`reset`].
use core::fmt;

use incin_b200_sys as sys;

/// Errors of tape operations.
#[derive(Debug, Clone, PartialEq, Eq)]
pub enum TapeError {
    /// Operand shapes do not fit the operation (or a handle is stale).
    Shape(&'static str),
    /// A class index is outside `[0, classes)`.
    Target,
    /// `backward` met a non-finite gradient while the NaN policy was "report".
    NonFinite,
    /// The variable is not on a path to the root that was differentiated.
    NoGradient,
}

impl fmt::Display for TapeError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        match self {
            TapeError::Shape(what) => write!(f, "shape mismatch or stale handle in {what}"),
            TapeError::Target => write!(f, "a target class is out of range"),
            TapeError::NonFinite => write!(f, "backward produced a non-finite gradient"),
            TapeError::NoGradient => write!(f, "no gradient was computed for this variable"),
        }
    }
}

impl std::error::Error for TapeError {}

/// A value on the tape.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub struct Var {
    handle: i64,
    rows: usize,
    cols: usize,
}

impl Var {
    /// A leaf holding `data` (`rows x cols`, row-major).  Parameters pass `requires_grad = true`.
    pub fn leaf(data: &[f32], rows: usize, cols: usize, requires_grad: bool) -> Result<Var, TapeError> {
        if data.len() != rows * cols {
            return Err(TapeError::Shape("leaf"));
        }
        // SAFETY: `data` holds rows * cols floats; the library copies them.
        let handle = unsafe { sys::incin_tape_tensor(data.as_ptr(), rows as i64, cols as i64, requires_grad as i32) };
        if handle == 0 {
            return Err(TapeError::Shape("leaf"));
        }
        Ok(Var { handle, rows, cols })
    }

    pub fn rows(&self) -> usize {
        self.rows
    }

    pub fn cols(&self) -> usize {
        self.cols
    }

    /// Process-unique id of the underlying tensor (what gradients are keyed by).
    pub fn id(&self) -> u64 {
        // SAFETY: a stale handle yields 0.
        unsafe { sys::incin_tape_tensor_id(self.handle) }
    }

    /// `self [M, K] x weight [N, K]^T + bias [N]`.
    pub fn linear(&self, weight: &Var, bias: Option<&Var>) -> Result<Var, TapeError> {
        // SAFETY: handles are validated by the library; 0 means "no bias".
        let h = unsafe { sys::incin_tape_linear(self.handle, weight.handle, bias.map_or(0, |b| b.handle)) };
        if h == 0 {
            return Err(TapeError::Shape("linear"));
        }
        Ok(Var { handle: h, rows: self.rows, cols: weight.rows })
    }

    pub fn relu(&self) -> Result<Var, TapeError> {
        // SAFETY: as above.
        let h = unsafe { sys::incin_tape_relu(self.handle) };
        if h == 0 {
            return Err(TapeError::Shape("relu"));
        }
        Ok(Var { handle: h, rows: self.rows, cols: self.cols })
    }

    /// Mean softmax cross-entropy of logits `[rows, classes]` against one class index per row.
    pub fn cross_entropy(&self, targets: &[i64]) -> Result<Var, TapeError> {
        if targets.len() != self.rows {
            return Err(TapeError::Shape("cross_entropy"));
        }
        if targets.iter().any(|&t| t < 0 || t as usize >= self.cols) {
            return Err(TapeError::Target);
        }
        // SAFETY: `targets` holds one index per row.
        let h = unsafe { sys::incin_tape_cross_entropy(self.handle, targets.as_ptr()) };
        if h == 0 {
            return Err(TapeError::Shape("cross_entropy"));
        }
        Ok(Var { handle: h, rows: 1, cols: 1 })
    }

    /// Copy the value out.
    pub fn value(&self) -> Result<Vec<f32>, TapeError> {
        let mut out = vec![0.0f32; self.rows * self.cols];
        // SAFETY: the buffer matches the recorded extents.
        let rc = unsafe { sys::incin_tape_read(self.handle, out.as_mut_ptr()) };
        if rc != 0 {
            return Err(TapeError::Shape("value"));
        }
        Ok(out)
    }

    /// Differentiate this (scalar) value with respect to every leaf that requires a gradient.  Drains the tape.
    pub fn backward(&self) -> Result<Gradients, TapeError> {
        // SAFETY: handle validated by the library.
        match unsafe { sys::incin_tape_backward(self.handle) } {
            0 => Ok(Gradients { _private: () }),
            2 => Err(TapeError::NonFinite),
            _ => Err(TapeError::Shape("backward")),
        }
    }
}

/// The gradients of the last `backward` on this thread.
#[derive(Debug)]
pub struct Gradients {
    _private: (),
}

impl Gradients {
    /// Gradient of the differentiated root with respect to `var` (same extents as `var`).
    pub fn get(&self, var: &Var) -> Result<Vec<f32>, TapeError> {
        let mut out = vec![0.0f32; var.rows * var.cols];
        // SAFETY: the buffer matches the recorded extents.
        match unsafe { sys::incin_tape_grad(var.handle, out.as_mut_ptr()) } {
            0 => Ok(out),
            2 => Err(TapeError::NoGradient),
            _ => Err(TapeError::Shape("gradient")),
        }
    }
}

/// Number of nodes currently recorded.
pub fn depth() -> usize {
    // SAFETY: no arguments.
    unsafe { sys::incin_tape_depth() as usize }
}

/// Drop every handle, node and gradient of this thread's tape (between training steps).
pub fn reset() {
    // SAFETY: no arguments.
    unsafe { sys::incin_tape_reset() }
}

/// Report non-finite gradients from `backward` (`true`) or let them through (`false`).
pub fn check_gradients(report: bool) {
    // SAFETY: plain setter.
    unsafe { sys::incin_tape_set_nan_policy(report as i32) }
}

/// Run `f` without recording (inference, metric evaluation); gradient mode is switched back on afterwards.
pub fn no_grad<T>(f: impl FnOnce() -> T) -> T {
    // SAFETY: plain setters.
    unsafe { sys::incin_tape_set_grad_mode(0) };
    let out = f();
    unsafe { sys::incin_tape_set_grad_mode(1) };
    out
}
