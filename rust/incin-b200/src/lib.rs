//! Rust facade over the incin-b200 libraries.
//!
//! It keeps the vocabulary of the `incin` crate (crates/incin/src/lib.rs:143-189 of the reference): tensors whose
//! shape is part of their type (`s![2, 3]`, `s![dyn, 784]`), named run-time axes (`dim!`), bounds-checked slicing
//! (`idx!`), a tape with `backward()`, layer builders, `AdamW` / `Sgd`, a `Trainer` with a plan, and a
//! `DistributedContext::from_env()` with typed meshes (`mesh!`) and placements.  The default backend is the CPU one:
//! everything in [`tensor`], [`autograd`], [`nn`], [`optim`] and [`train`] runs on the C++ CPU oracle and tape of
//! `libincin_host.so`; [`io`] reads and writes safetensors files with the tensor names of the Python package;
//! [`runtime`] wraps the native digest, batch loader and telemetry sink; [`dist`] wraps its TCP rendezvous and the reference (host-memory) collective transport; [`gpu`] is the typed
//! front end of the sm_100a kernels in `libincin_sm100.so`, which work on device pointers the caller owns.
//!
//! ```ignore
//! use incin_b200::prelude::*;
//!
//! let x: Tensor<s![dyn, 784]> = Tensor::randn_dyn(&[64, 784], 0)?;
//! let w: Tensor<s![784, 128]> = Tensor::randn(1);
//! let h = x.matmul(&w)?.relu();                       // Tensor<s![dyn, 128]>; inner extents checked by the types
//! let first = h.slice(&idx![0..5, ..])?;              // bounds checked
//!
//! let plan = Trainer::plan().devices(DeviceSet::cpu()).epochs(2).build()?;
//! let mut model = Mlp::build((784, 256, 10), 0);
//! let mut opt = AdamW::new(model.num_parameters(), 1e-3);
//! let losses = Trainer::new(plan).fit(&mut model, &mut opt, &batches)?;
//! ```
pub mod autograd;
pub mod dist;
pub mod gpu;
pub mod io;
pub mod nn;
pub mod optim;
pub mod runtime;
pub mod shape;
pub mod tensor;
pub mod train;

pub mod prelude {
    pub use crate::autograd::{no_grad, Gradients, Var};
    pub use crate::dist::{DistributedContext, Mesh, Placement, ReduceOp, ReferenceTransport, Rendezvous};
    pub use crate::io::{load_safetensors, save_safetensors, Format, NamedTensor};
    pub use crate::nn::{Linear, Mlp, Module};
    pub use crate::optim::{AdamW, Optimizer, Sgd};
    pub use crate::shape::{DynShape, Shape, Shape1, Shape2, Shape3, Shape4, ShapeError, DYN};
    pub use crate::tensor::{Idx, IndexSpec, Tensor, Unary};
    pub use crate::train::{Batch, DeviceSet, Plan, TrainError, Trainer};
    pub use crate::{dim, idx, mesh, s};
}

/// A shape as a type: `s![2, 3]` is `Shape2<2, 3>`, `s![dyn, 784]` is `Shape2<DYN, 784>` (first extent known at run
/// time only), `s![]` is the fully dynamic [`shape::DynShape`].  Up to rank 4.
#[macro_export]
macro_rules! s {
    () => { $crate::shape::DynShape };
    ($a:tt) => { $crate::shape::Shape1<{ $crate::__extent!($a) }> };
    ($a:tt, $b:tt) => { $crate::shape::Shape2<{ $crate::__extent!($a) }, { $crate::__extent!($b) }> };
    ($a:tt, $b:tt, $c:tt) => {
        $crate::shape::Shape3<{ $crate::__extent!($a) }, { $crate::__extent!($b) }, { $crate::__extent!($c) }>
    };
    ($a:tt, $b:tt, $c:tt, $d:tt) => {
        $crate::shape::Shape4<{ $crate::__extent!($a) }, { $crate::__extent!($b) }, { $crate::__extent!($c) },
                              { $crate::__extent!($d) }>
    };
}

#[doc(hidden)]
#[macro_export]
macro_rules! __extent {
    (dyn) => { $crate::shape::DYN };
    ($n:expr) => { $n };
}

/// A slicing specification: `idx![0..5, .., 15..30]`, `idx![3, ..]`, `idx![..4, Idx::Ellipsis, -1]`.  Integers pick one
/// entry (negative counts from the end) and drop the axis; ranges keep it.  Applied with [`tensor::Tensor::slice`],
/// which checks every bound.
#[macro_export]
macro_rules! idx {
    ($($e:expr),* $(,)?) => { $crate::tensor::IndexSpec::new(vec![$($crate::tensor::Idx::from($e)),*]) };
}

/// Named axes whose extents are run-time values: `dim!(Batch, Seq);` declares the marker types, and
/// `shape::Axes::new().bind::<Batch>(32)` gives them sizes that every later use has to agree with.
#[macro_export]
macro_rules! dim {
    ($($name:ident),+ $(,)?) => {
        $(
            #[derive(Debug, Clone, Copy, PartialEq, Eq)]
            pub struct $name;
            impl $crate::shape::NamedAxis for $name {
                const NAME: &'static str = stringify!($name);
            }
        )+
    };
}

/// A device mesh: `mesh![dp = 2, tp = 4]` (missing axes are 1).  [`dist::Mesh::validate`] checks it against a world size.
#[macro_export]
macro_rules! mesh {
    ($($axis:ident = $n:expr),+ $(,)?) => {{
        let mut m = $crate::dist::Mesh::single();
        $( m = m.with_axis(stringify!($axis), $n); )+
        m
    }};
}
