//! Shapes as types, with a run-time escape hatch per axis.
//!
//! An extent is a const generic; [`DYN`] marks an axis whose extent is only known at run time.  The counterpart in the
//! reference is the typenum-based shape algebra of crates/incin-core/src/shapes; const generics state the same proofs
//! without type-level arithmetic: equal inner extents of a product are one shared const parameter, and whatever
//! involves a `DYN` axis is checked when the tensor is built or the operation runs.
use core::fmt;
use std::collections::HashMap;

/// Marker extent of an axis that is sized at run time.
pub const DYN: usize = usize::MAX;

/// What went wrong, with the axis and both extents, so that the message can say it in one sentence.
#[derive(Debug, Clone, PartialEq, Eq)]
pub enum ShapeError {
    Rank { expected: usize, got: usize },
    Extent { axis: usize, expected: usize, got: usize },
    Numel { expected: usize, got: usize },
    Inner { left: usize, right: usize },
    Broadcast { axis: usize, left: usize, right: usize },
    OutOfBounds { axis: usize, extent: usize, start: isize, stop: isize },
    TooManyIndices { rank: usize, got: usize },
    NamedAxis { name: &'static str, bound: usize, got: usize },
    Infer { numel: usize, known: usize },
}

impl fmt::Display for ShapeError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        match self {
            ShapeError::Rank { expected, got } => write!(f, "expected rank {expected}, got rank {got}"),
            ShapeError::Extent { axis, expected, got } => {
                write!(f, "axis {axis} must have extent {expected}, got {got}")
            }
            ShapeError::Numel { expected, got } => write!(f, "{got} elements cannot be viewed as {expected}"),
            ShapeError::Inner { left, right } => {
                write!(f, "matmul needs [M, K] x [K, N]: inner extents {left} and {right} differ")
            }
            ShapeError::Broadcast { axis, left, right } => {
                write!(f, "cannot broadcast axis {axis}: {left} against {right} (extents must be equal or 1)")
            }
            ShapeError::OutOfBounds { axis, extent, start, stop } => {
                write!(f, "range {start}..{stop} is out of bounds for axis {axis} of extent {extent}")
            }
            ShapeError::TooManyIndices { rank, got } => write!(f, "{got} indices for a rank-{rank} tensor"),
            ShapeError::NamedAxis { name, bound, got } => {
                write!(f, "axis {name} is bound to {bound} but was used with {got}")
            }
            ShapeError::Infer { numel, known } => {
                write!(f, "cannot infer an extent: {numel} elements are not divisible by {known}")
            }
        }
    }
}

impl std::error::Error for ShapeError {}

/// A shape type.  `EXTENTS` lists the static extents ([`DYN`] where the axis is dynamic); `None` rank means the
/// rank itself is dynamic ([`DynShape`]).
pub trait Shape: Copy + Default + fmt::Debug + 'static {
    /// `Some(rank)` for the fixed-rank shapes.
    const RANK: Option<usize>;

    /// The static extents, [`DYN`] for run-time axes; empty for [`DynShape`].
    fn extents() -> Vec<usize>;

    /// Check run-time extents against the type.
    fn check(dims: &[usize]) -> Result<(), ShapeError> {
        if let Some(rank) = Self::RANK {
            if dims.len() != rank {
                return Err(ShapeError::Rank { expected: rank, got: dims.len() });
            }
            for (axis, (&want, &got)) in Self::extents().iter().zip(dims.iter()).enumerate() {
                if want != DYN && want != got {
                    return Err(ShapeError::Extent { axis, expected: want, got });
                }
            }
        }
        Ok(())
    }

    /// The extents when every axis is static.
    fn static_dims() -> Option<Vec<usize>> {
        Self::RANK?;
        let e = Self::extents();
        if e.iter().any(|&d| d == DYN) {
            None
        } else {
            Some(e)
        }
    }
}

/// Fully dynamic shape: rank and extents are run-time values.
#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct DynShape;

impl Shape for DynShape {
    const RANK: Option<usize> = None;
    fn extents() -> Vec<usize> {
        Vec::new()
    }
}

#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct Shape1<const A: usize>;
#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct Shape2<const A: usize, const B: usize>;
#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct Shape3<const A: usize, const B: usize, const C: usize>;
#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct Shape4<const A: usize, const B: usize, const C: usize, const D: usize>;

impl<const A: usize> Shape for Shape1<A> {
    const RANK: Option<usize> = Some(1);
    fn extents() -> Vec<usize> {
        vec![A]
    }
}
impl<const A: usize, const B: usize> Shape for Shape2<A, B> {
    const RANK: Option<usize> = Some(2);
    fn extents() -> Vec<usize> {
        vec![A, B]
    }
}
impl<const A: usize, const B: usize, const C: usize> Shape for Shape3<A, B, C> {
    const RANK: Option<usize> = Some(3);
    fn extents() -> Vec<usize> {
        vec![A, B, C]
    }
}
impl<const A: usize, const B: usize, const C: usize, const D: usize> Shape for Shape4<A, B, C, D> {
    const RANK: Option<usize> = Some(4);
    fn extents() -> Vec<usize> {
        vec![A, B, C, D]
    }
}

/// Number of elements of run-time extents.
pub fn numel(dims: &[usize]) -> usize {
    dims.iter().product()
}

/// Row-major strides of run-time extents.
pub fn strides(dims: &[usize]) -> Vec<usize> {
    let mut st = vec![1usize; dims.len()];
    for i in (0..dims.len().saturating_sub(1)).rev() {
        st[i] = st[i + 1] * dims[i + 1];
    }
    st
}

/// Resolve at most one `-1` of a reshape target against an element count.
pub fn reshape_infer(numel_in: usize, target: &[isize]) -> Result<Vec<usize>, ShapeError> {
    let mut known = 1usize;
    let mut unknown: Option<usize> = None;
    for (i, &d) in target.iter().enumerate() {
        if d == -1 {
            if unknown.is_some() {
                return Err(ShapeError::Infer { numel: numel_in, known: 0 });
            }
            unknown = Some(i);
        } else if d < 0 {
            return Err(ShapeError::Infer { numel: numel_in, known: 0 });
        } else {
            known *= d as usize;
        }
    }
    let mut out: Vec<usize> = target.iter().map(|&d| if d < 0 { 0 } else { d as usize }).collect();
    match unknown {
        Some(i) => {
            if known == 0 || numel_in % known != 0 {
                return Err(ShapeError::Infer { numel: numel_in, known });
            }
            out[i] = numel_in / known;
        }
        None => {
            if known != numel_in {
                return Err(ShapeError::Numel { expected: known, got: numel_in });
            }
        }
    }
    Ok(out)
}

/// Extents of `a` broadcast against `b` (aligned from the last axis; extents must be equal or 1).
pub fn broadcast(a: &[usize], b: &[usize]) -> Result<Vec<usize>, ShapeError> {
    let rank = a.len().max(b.len());
    let mut out = vec![0usize; rank];
    for i in 0..rank {
        let da = if i < a.len() { a[a.len() - 1 - i] } else { 1 };
        let db = if i < b.len() { b[b.len() - 1 - i] } else { 1 };
        out[rank - 1 - i] = if da == db || db == 1 {
            da
        } else if da == 1 {
            db
        } else {
            return Err(ShapeError::Broadcast { axis: rank - 1 - i, left: da, right: db });
        };
    }
    Ok(out)
}

/// A named axis declared with `dim!`.
pub trait NamedAxis: 'static {
    const NAME: &'static str;
}

/// Run-time sizes of named axes: the first `bind` of an axis fixes its extent, later ones must agree.
#[derive(Debug, Clone, Default)]
pub struct Axes {
    sizes: HashMap<&'static str, usize>,
}

impl Axes {
    pub fn new() -> Self {
        Axes::default()
    }

    pub fn bind<A: NamedAxis>(mut self, extent: usize) -> Result<Self, ShapeError> {
        self.bind_mut::<A>(extent)?;
        Ok(self)
    }

    pub fn bind_mut<A: NamedAxis>(&mut self, extent: usize) -> Result<(), ShapeError> {
        match self.sizes.get(A::NAME) {
            Some(&bound) if bound != extent => Err(ShapeError::NamedAxis { name: A::NAME, bound, got: extent }),
            Some(_) => Ok(()),
            None => {
                self.sizes.insert(A::NAME, extent);
                Ok(())
            }
        }
    }

    pub fn get<A: NamedAxis>(&self) -> Option<usize> {
        self.sizes.get(A::NAME).copied()
    }
}
