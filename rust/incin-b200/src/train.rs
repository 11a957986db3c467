//! `Trainer::plan().devices(..).epochs(n).build()? -> Plan`, `Trainer::new(plan).fit(..)`.
//!
//! Same shape as the reference's trainer (crates/incin/src/train.rs:546-617 and its `TrainError`, :220-255): a plan is
//! validated before anything runs, a multi-device plan without a collective transport is an error, a failing step is
//! reported with its index.  This crate trains on the CPU backend (tape + oracle); multi-GPU training is driven from
//! the Python package, one process per GPU.
use core::fmt;

use incin_b200_sys as sys;

use crate::autograd::{self, TapeError, Var};
use crate::nn::Module;
use crate::optim::Optimizer;

/// Devices a plan may use.
#[derive(Debug, Clone, PartialEq, Eq)]
pub enum DeviceSet {
    Cpu,
    /// CUDA device indices.
    Cuda(Vec<u32>),
}

impl DeviceSet {
    pub fn cpu() -> Self {
        DeviceSet::Cpu
    }

    pub fn cuda(indices: core::ops::Range<u32>) -> Result<Self, TrainError> {
        let v: Vec<u32> = indices.collect();
        if v.is_empty() {
            return Err(TrainError::NoDevices);
        }
        Ok(DeviceSet::Cuda(v))
    }

    pub fn len(&self) -> usize {
        match self {
            DeviceSet::Cpu => 1,
            DeviceSet::Cuda(v) => v.len(),
        }
    }

    pub fn is_empty(&self) -> bool {
        self.len() == 0
    }
}

#[derive(Debug)]
pub enum TrainError {
    /// The plan names no device.
    NoDevices,
    /// `epochs(0)`.
    NoEpochs,
    /// More than one device but no process group / transport to reduce gradients with.
    CollectivesUnavailable { devices: usize },
    /// This front end executes on the CPU backend only.
    UnsupportedDevice,
    /// Step `index` failed.
    Step { index: usize, source: TapeError },
}

impl fmt::Display for TrainError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        match self {
            TrainError::NoDevices => write!(f, "the plan names no device"),
            TrainError::NoEpochs => write!(f, "the plan runs zero epochs"),
            TrainError::CollectivesUnavailable { devices } => {
                write!(f, "a {devices}-device plan needs one process per device and a collective transport")
            }
            TrainError::UnsupportedDevice => write!(f, "this front end trains on the CPU backend"),
            TrainError::Step { index, source } => write!(f, "step {index} failed: {source}"),
        }
    }
}

impl std::error::Error for TrainError {}

/// A validated training plan.
#[derive(Debug, Clone, PartialEq, Eq)]
pub struct Plan {
    pub devices: DeviceSet,
    pub epochs: usize,
}

impl Plan {
    pub fn is_multi_device(&self) -> bool {
        self.devices.len() > 1
    }
}

#[derive(Debug, Clone)]
pub struct PlanBuilder {
    devices: Option<DeviceSet>,
    epochs: usize,
}

impl PlanBuilder {
    pub fn devices(mut self, d: DeviceSet) -> Self {
        self.devices = Some(d);
        self
    }

    pub fn epochs(mut self, n: usize) -> Self {
        self.epochs = n;
        self
    }

    pub fn build(self) -> Result<Plan, TrainError> {
        let devices = self.devices.unwrap_or(DeviceSet::Cpu);
        if devices.is_empty() {
            return Err(TrainError::NoDevices);
        }
        if self.epochs == 0 {
            return Err(TrainError::NoEpochs);
        }
        Ok(Plan { devices, epochs: self.epochs })
    }
}

/// One batch: `inputs` is `[rows, features]` row-major, `targets` one class per row.
#[derive(Debug, Clone)]
pub struct Batch {
    pub inputs: Vec<f32>,
    pub rows: usize,
    pub features: usize,
    pub targets: Vec<i64>,
}

pub struct Trainer {
    plan: Plan,
}

impl Trainer {
    pub fn plan() -> PlanBuilder {
        PlanBuilder { devices: None, epochs: 1 }
    }

    pub fn new(plan: Plan) -> Self {
        Trainer { plan }
    }

    /// Cross-entropy training of `model` over `batches`, `plan.epochs` times; returns the loss of every step.
    pub fn fit<M: Module, O: Optimizer>(&self, model: &mut M, opt: &mut O, batches: &[Batch]) -> Result<Vec<f32>, TrainError> {
        if self.plan.is_multi_device() {
            return Err(TrainError::CollectivesUnavailable { devices: self.plan.devices.len() });
        }
        if self.plan.devices != DeviceSet::Cpu {
            return Err(TrainError::UnsupportedDevice);
        }
        let mut losses = Vec::with_capacity(self.plan.epochs * batches.len());
        let mut index = 0usize;
        for _ in 0..self.plan.epochs {
            for b in batches {
                let loss = Self::one_step(model, opt, b).map_err(|source| TrainError::Step { index, source })?;
                losses.push(loss);
                index += 1;
            }
        }
        Ok(losses)
    }

    fn one_step<M: Module, O: Optimizer>(model: &mut M, opt: &mut O, b: &Batch) -> Result<f32, TapeError> {
        autograd::reset();
        let x = Var::leaf(&b.inputs, b.rows, b.features, false)?;
        let logits = model.forward(&x)?;
        let loss = logits.cross_entropy(&b.targets)?;
        let value = loss.value()?[0];
        let grads = loss.backward()?;
        let flat = model.collect_gradients(&grads)?;
        opt.step(model, &flat);
        Ok(value)
    }
}

/// The CPU benchmark configuration end to end in native code (784 -> 256 -> 10 MLP, batch 64, SGD on synthetic
/// Philox data): returns the loss of every step.  `python -m incin_b200` reports the same curve.
pub fn native_mlp_benchmark(steps: usize, batch: usize, dims: (usize, usize, usize), lr: f32, seed: u64) -> Option<Vec<f32>> {
    let (i, h, o) = dims;
    let mut losses = vec![0.0f32; steps];
    // SAFETY: `losses` holds one float per step; a null parameter pointer means "do not return the parameters".
    let rc = unsafe {
        sys::incin_cpu_mlp_train(steps as i32, batch as i32, i as i32, h as i32, o as i32, lr, seed, losses.as_mut_ptr(),
                                 core::ptr::null_mut())
    };
    if rc == 0 {
        Some(losses)
    } else {
        None
    }
}
