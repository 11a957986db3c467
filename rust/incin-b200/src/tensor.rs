//! `Tensor<S>`: fp32 data on the host with its shape in the type, computed by the C++ CPU oracle.
//!
//! The CPU backend is the default backend and the correctness oracle of the framework (as in the reference:
//! crates/incin/src/lib.rs:143-167); the GPU kernels are validated against exactly these functions.
use core::marker::PhantomData;
use core::ops::{Range, RangeFrom, RangeFull, RangeTo};

use incin_b200_sys as sys;

use crate::shape::{self, DynShape, Shape, Shape2, ShapeError};

/// Elementwise functions of the oracle (`incin_cpu_unary_f32`).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Unary {
    Relu = 0,
    Gelu = 1,
    GeluTanh = 2,
    Silu = 3,
    Sigmoid = 4,
    Tanh = 5,
    Exp = 6,
    Log = 7,
    Sqrt = 8,
    Neg = 9,
    Abs = 10,
    Mish = 11,
    Elu = 12,
    Softplus = 13,
    Sign = 14,
}

/// Row-major fp32 tensor whose shape type `S` is checked against its run-time extents at construction.
#[derive(Debug, Clone, PartialEq)]
pub struct Tensor<S: Shape = DynShape> {
    data: Vec<f32>,
    dims: Vec<usize>,
    _shape: PhantomData<S>,
}

impl<S: Shape> Tensor<S> {
    /// Wrap existing data; the extents must match both the type and the data length.
    pub fn from_vec(data: Vec<f32>, dims: &[usize]) -> Result<Self, ShapeError> {
        S::check(dims)?;
        if shape::numel(dims) != data.len() {
            return Err(ShapeError::Numel { expected: shape::numel(dims), got: data.len() });
        }
        Ok(Tensor { data, dims: dims.to_vec(), _shape: PhantomData })
    }

    /// Zeros with run-time extents (needed when `S` has a `dyn` axis).
    pub fn zeros_dyn(dims: &[usize]) -> Result<Self, ShapeError> {
        Self::from_vec(vec![0.0; shape::numel(dims)], dims)
    }

    /// Zeros of a fully static shape.
    pub fn zeros() -> Self {
        let dims = S::static_dims().expect("Tensor::zeros needs a shape without dyn axes; use zeros_dyn");
        Tensor { data: vec![0.0; shape::numel(&dims)], dims, _shape: PhantomData }
    }

    /// Standard-normal entries from the Philox generator the device kernels use (same seed, same numbers).
    pub fn randn_dyn(dims: &[usize], seed: u64) -> Result<Self, ShapeError> {
        let mut t = Self::zeros_dyn(dims)?;
        // SAFETY: the buffer holds exactly `len` floats.
        unsafe { sys::incin_cpu_philox_normal_f32(t.data.as_mut_ptr(), t.data.len() as i64, seed, 0, 0.0, 1.0) };
        Ok(t)
    }

    pub fn randn(seed: u64) -> Self {
        let dims = S::static_dims().expect("Tensor::randn needs a shape without dyn axes; use randn_dyn");
        Self::randn_dyn(&dims, seed).expect("static extents always match their own type")
    }

    /// Uniform [0, 1) entries from the same generator.
    pub fn rand_dyn(dims: &[usize], seed: u64) -> Result<Self, ShapeError> {
        let mut t = Self::zeros_dyn(dims)?;
        // SAFETY: as above.
        unsafe { sys::incin_cpu_philox_uniform_f32(t.data.as_mut_ptr(), t.data.len() as i64, seed, 0) };
        Ok(t)
    }

    pub fn dims(&self) -> &[usize] {
        &self.dims
    }

    pub fn numel(&self) -> usize {
        self.data.len()
    }

    pub fn as_slice(&self) -> &[f32] {
        &self.data
    }

    pub fn to_vec(&self) -> Vec<f32> {
        self.data.clone()
    }

    /// The single value of a one-element tensor.
    pub fn to_scalar(&self) -> Result<f32, ShapeError> {
        if self.data.len() == 1 {
            Ok(self.data[0])
        } else {
            Err(ShapeError::Numel { expected: 1, got: self.data.len() })
        }
    }

    /// Forget the static shape.
    pub fn into_dyn(self) -> Tensor<DynShape> {
        Tensor { data: self.data, dims: self.dims, _shape: PhantomData }
    }

    /// Re-type the same data as shape `T` (extents are checked, the element count must be unchanged).
    pub fn reshape<T: Shape>(self, target: &[isize]) -> Result<Tensor<T>, ShapeError> {
        let dims = shape::reshape_infer(self.data.len(), target)?;
        Tensor::<T>::from_vec(self.data, &dims)
    }

    /// Apply an elementwise function.
    pub fn unary(&self, op: Unary) -> Self {
        let mut out = vec![0.0f32; self.data.len()];
        // SAFETY: both buffers hold `len` floats.
        unsafe { sys::incin_cpu_unary_f32(self.data.as_ptr(), out.as_mut_ptr(), out.len() as i64, op as i32) };
        Tensor { data: out, dims: self.dims.clone(), _shape: PhantomData }
    }

    pub fn relu(&self) -> Self {
        self.unary(Unary::Relu)
    }

    pub fn gelu(&self) -> Self {
        self.unary(Unary::Gelu)
    }

    fn rows_cols(&self) -> (i64, i64) {
        let c = *self.dims.last().unwrap_or(&1);
        ((self.data.len() / c.max(1)) as i64, c as i64)
    }

    /// Softmax (or log-softmax) over the last axis.
    pub fn softmax(&self, log: bool) -> Self {
        let (rows, c) = self.rows_cols();
        let mut out = vec![0.0f32; self.data.len()];
        // SAFETY: `rows * c == len` by construction.
        unsafe { sys::incin_cpu_softmax_f32(self.data.as_ptr(), out.as_mut_ptr(), rows, c, log as i32) };
        Tensor { data: out, dims: self.dims.clone(), _shape: PhantomData }
    }

    /// LayerNorm (`rms = false`, `beta` optional) or RMSNorm (`rms = true`) over the last axis.
    pub fn normalize(&self, gamma: &[f32], beta: Option<&[f32]>, eps: f32, rms: bool) -> Result<Self, ShapeError> {
        let (rows, c) = self.rows_cols();
        if gamma.len() as i64 != c {
            return Err(ShapeError::Extent { axis: self.dims.len().saturating_sub(1), expected: c as usize, got: gamma.len() });
        }
        if let Some(b) = beta {
            if b.len() as i64 != c {
                return Err(ShapeError::Extent { axis: self.dims.len().saturating_sub(1), expected: c as usize, got: b.len() });
            }
        }
        let mut out = vec![0.0f32; self.data.len()];
        let bptr = beta.map_or(core::ptr::null(), |b| b.as_ptr());
        // SAFETY: lengths checked above.
        unsafe {
            sys::incin_cpu_layernorm_f32(self.data.as_ptr(), gamma.as_ptr(), bptr, out.as_mut_ptr(), rows, c, eps, rms as i32)
        };
        Ok(Tensor { data: out, dims: self.dims.clone(), _shape: PhantomData })
    }

    /// Bounds-checked slicing; integer items drop their axis, ranges keep it.  The result is dynamically shaped.
    pub fn slice(&self, spec: &IndexSpec) -> Result<Tensor<DynShape>, ShapeError> {
        let plan = spec.resolve(&self.dims)?;
        let st = shape::strides(&self.dims);
        let out_dims: Vec<usize> = plan.iter().filter(|a| a.keep).map(|a| a.len).collect();
        let total: usize = plan.iter().map(|a| a.len).product();
        let mut out = Vec::with_capacity(total);
        let mut counter = vec![0usize; plan.len()];
        for _ in 0..total {
            let mut off = 0usize;
            for (axis, a) in plan.iter().enumerate() {
                off += (a.start + counter[axis]) * st[axis];
            }
            out.push(self.data[off]);
            for axis in (0..plan.len()).rev() {
                counter[axis] += 1;
                if counter[axis] < plan[axis].len {
                    break;
                }
                counter[axis] = 0;
            }
        }
        Tensor::<DynShape>::from_vec(out, &out_dims)
    }
}

impl<const M: usize, const K: usize> Tensor<Shape2<M, K>> {
    /// `[M, K] x [K, N] -> [M, N]`.  The inner extent is one const parameter shared by both operand types, so a
    /// mismatch of static extents does not compile; `dyn` extents are compared here.
    pub fn matmul<const N: usize>(&self, rhs: &Tensor<Shape2<K, N>>) -> Result<Tensor<Shape2<M, N>>, ShapeError> {
        let (m, k) = (self.dims[0], self.dims[1]);
        let (k2, n) = (rhs.dims[0], rhs.dims[1]);
        if k != k2 {
            return Err(ShapeError::Inner { left: k, right: k2 });
        }
        let mut out = vec![0.0f32; m * n];
        // SAFETY: row-major operands with the strides given; extents were validated when the tensors were built.
        unsafe {
            // (batch, M, N, K), A strides (batch, row, col), B strides (batch, k, n), C strides (batch, row), alpha, beta
            sys::incin_cpu_gemm_f32(self.data.as_ptr(), rhs.data.as_ptr(), out.as_mut_ptr(), 1, m as i64, n as i64,
                                    k as i64, 0, k as i64, 1, 0, n as i64, 1, 0, n as i64, 1.0, 0.0)
        };
        Tensor::<Shape2<M, N>>::from_vec(out, &[m, n])
    }
}

/// One item of a slicing specification.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Idx {
    /// One entry; negative counts from the end.  Drops the axis.
    At(isize),
    /// `start..stop`.
    Range(usize, usize),
    /// `start..`.
    From(usize),
    /// `..stop`.
    To(usize),
    /// `..`: the whole axis.
    Full,
    /// As many whole axes as are needed to fill the rank.
    Ellipsis,
}

impl From<isize> for Idx {
    fn from(i: isize) -> Self {
        Idx::At(i)
    }
}
impl From<Range<usize>> for Idx {
    fn from(r: Range<usize>) -> Self {
        Idx::Range(r.start, r.end)
    }
}
impl From<RangeFrom<usize>> for Idx {
    fn from(r: RangeFrom<usize>) -> Self {
        Idx::From(r.start)
    }
}
impl From<RangeTo<usize>> for Idx {
    fn from(r: RangeTo<usize>) -> Self {
        Idx::To(r.end)
    }
}
impl From<RangeFull> for Idx {
    fn from(_: RangeFull) -> Self {
        Idx::Full
    }
}

#[derive(Debug, Clone, Copy)]
pub(crate) struct AxisPlan {
    start: usize,
    len: usize,
    keep: bool,
}

/// A list of [`Idx`] items, built by `idx![...]`.
#[derive(Debug, Clone, PartialEq, Eq)]
pub struct IndexSpec {
    items: Vec<Idx>,
}

impl IndexSpec {
    pub fn new(items: Vec<Idx>) -> Self {
        IndexSpec { items }
    }

    /// Per axis of `dims`: first index, number of entries, and whether the axis survives.  Every bound is checked
    /// (a range that reaches past the axis is an error, not a clamp).
    pub(crate) fn resolve(&self, dims: &[usize]) -> Result<Vec<AxisPlan>, ShapeError> {
        let explicit = self.items.iter().filter(|i| **i != Idx::Ellipsis).count();
        if explicit > dims.len() {
            return Err(ShapeError::TooManyIndices { rank: dims.len(), got: explicit });
        }
        let mut plan = Vec::with_capacity(dims.len());
        let mut axis = 0usize;
        let mut seen_ellipsis = false;
        for item in &self.items {
            if *item == Idx::Ellipsis {
                if !seen_ellipsis {
                    seen_ellipsis = true;
                    for _ in 0..(dims.len() - explicit) {
                        plan.push(AxisPlan { start: 0, len: dims[axis], keep: true });
                        axis += 1;
                    }
                }
                continue;
            }
            let ext = dims[axis];
            let oob = |start: isize, stop: isize| ShapeError::OutOfBounds { axis, extent: ext, start, stop };
            let p = match *item {
                Idx::At(i) => {
                    let j = if i < 0 { i + ext as isize } else { i };
                    if j < 0 || j >= ext as isize {
                        return Err(oob(i, i + 1));
                    }
                    AxisPlan { start: j as usize, len: 1, keep: false }
                }
                Idx::Range(a, b) => {
                    if a > b || b > ext {
                        return Err(oob(a as isize, b as isize));
                    }
                    AxisPlan { start: a, len: b - a, keep: true }
                }
                Idx::From(a) => {
                    if a > ext {
                        return Err(oob(a as isize, ext as isize));
                    }
                    AxisPlan { start: a, len: ext - a, keep: true }
                }
                Idx::To(b) => {
                    if b > ext {
                        return Err(oob(0, b as isize));
                    }
                    AxisPlan { start: 0, len: b, keep: true }
                }
                Idx::Full | Idx::Ellipsis => AxisPlan { start: 0, len: ext, keep: true },
            };
            plan.push(p);
            axis += 1;
        }
        while axis < dims.len() {
            plan.push(AxisPlan { start: 0, len: dims[axis], keep: true });
            axis += 1;
        }
        Ok(plan)
    }
}
