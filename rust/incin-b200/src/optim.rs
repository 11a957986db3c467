//! Optimisers over a model's flat parameter list.
//!
//! Defaults follow the reference (`AdamW::new(model.parameters(), lr)`: betas (0.9, 0.999), eps 1e-8, weight decay
//! 0.01, bias-corrected; crates/incin-core/src/optim/mod.rs:112-124).  The update itself is the oracle's
//! `incin_cpu_adamw_f32` / `incin_cpu_sgd_f32`, the same arithmetic the flat device optimiser implements.
use incin_b200_sys as sys;

use crate::nn::Module;

/// `step` consumes the gradients of one backward pass, concatenated in parameter order.
pub trait Optimizer {
    fn step<M: Module>(&mut self, model: &mut M, gradients: &[f32]);
}

/// Plain SGD.
#[derive(Debug, Clone)]
pub struct Sgd {
    pub lr: f32,
}

impl Sgd {
    pub fn new(lr: f32) -> Self {
        Sgd { lr }
    }
}

impl Optimizer for Sgd {
    fn step<M: Module>(&mut self, model: &mut M, gradients: &[f32]) {
        let mut offset = 0usize;
        for p in model.parameters_mut() {
            let g = &gradients[offset..offset + p.len()];
            // SAFETY: `p` and `g` have the same length.
            unsafe { sys::incin_cpu_sgd_f32(p.as_mut_ptr(), g.as_ptr(), p.len() as i64, self.lr) };
            offset += p.len();
        }
    }
}

/// AdamW with decoupled weight decay and bias correction; first and second moments are flat like the parameters.
#[derive(Debug, Clone)]
pub struct AdamW {
    pub lr: f32,
    pub betas: (f32, f32),
    pub eps: f32,
    pub weight_decay: f32,
    m: Vec<f32>,
    v: Vec<f32>,
    steps: i32,
}

impl AdamW {
    /// `num_parameters` is `model.num_parameters()`.
    pub fn new(num_parameters: usize, lr: f32) -> Self {
        AdamW {
            lr,
            betas: (0.9, 0.999),
            eps: 1e-8,
            weight_decay: 0.01,
            m: vec![0.0; num_parameters],
            v: vec![0.0; num_parameters],
            steps: 0,
        }
    }

    pub fn betas(mut self, b1: f32, b2: f32) -> Self {
        self.betas = (b1, b2);
        self
    }

    pub fn weight_decay(mut self, wd: f32) -> Self {
        self.weight_decay = wd;
        self
    }

    pub fn steps_taken(&self) -> i32 {
        self.steps
    }
}

impl Optimizer for AdamW {
    fn step<M: Module>(&mut self, model: &mut M, gradients: &[f32]) {
        self.steps += 1;
        let mut offset = 0usize;
        for p in model.parameters_mut() {
            let n = p.len();
            let g = &gradients[offset..offset + n];
            let m = &mut self.m[offset..offset + n];
            let v = &mut self.v[offset..offset + n];
            // SAFETY: all four slices have length `n`.
            unsafe {
                sys::incin_cpu_adamw_f32(p.as_mut_ptr(), m.as_mut_ptr(), v.as_mut_ptr(), g.as_ptr(), n as i64, self.lr,
                                         self.betas.0, self.betas.1, self.eps, self.weight_decay, self.steps)
            };
            offset += n;
        }
    }
}
