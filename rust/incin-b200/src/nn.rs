//! Layers with builder tuples, parameters as flat fp32 slices.
//!
//! `Linear::build((784, 128), seed)` mirrors the reference's compressed builder arguments
//! (`Linear::<Dyn, B>::build((784, 128))`, crates/incin-core/src/nn); initialisation is Kaiming-uniform with
//! a = sqrt(5) (bound 1 / sqrt(fan_in)) from the Philox generator, one stream offset per parameter tensor.
use incin_b200_sys as sys;

use crate::autograd::{Gradients, TapeError, Var};

/// What the optimisers and the trainer need from a model: its parameters as one ordered list of flat slices.
pub trait Module {
    /// Parameters in a fixed order (the order of `parameters_mut`, `bind` and `collect_gradients`).
    fn parameters(&self) -> Vec<&[f32]>;
    fn parameters_mut(&mut self) -> Vec<&mut [f32]>;

    fn num_parameters(&self) -> usize {
        self.parameters().iter().map(|p| p.len()).sum()
    }

    /// Put the parameters on the tape as leaves for one step and run the forward pass on `x`.
    fn forward(&mut self, x: &Var) -> Result<Var, TapeError>;

    /// After `backward`: the gradients of the leaves bound by the last `forward`, in parameter order, concatenated.
    fn collect_gradients(&self, grads: &Gradients) -> Result<Vec<f32>, TapeError>;
}

fn uniform(n: usize, bound: f32, seed: u64, stream: u64) -> Vec<f32> {
    let mut v = vec![0.0f32; n];
    // SAFETY: the buffer holds `n` floats.
    unsafe { sys::incin_cpu_philox_uniform_f32(v.as_mut_ptr(), n as i64, seed, stream) };
    for x in v.iter_mut() {
        *x = (2.0 * *x - 1.0) * bound;
    }
    v
}

/// `y = x W^T + b` with `W: [out, in]`.
#[derive(Debug, Clone)]
pub struct Linear {
    pub weight: Vec<f32>,
    pub bias: Vec<f32>,
    pub in_features: usize,
    pub out_features: usize,
    bound: Option<(Var, Var)>,
}

impl Linear {
    /// `(in_features, out_features)`, a seed, and the Philox stream offset of this layer (two streams are used).
    pub fn build(dims: (usize, usize), seed: u64, stream: u64) -> Self {
        let (inf, outf) = dims;
        let bound = 1.0 / (inf as f32).sqrt();
        Linear {
            weight: uniform(inf * outf, bound, seed, stream),
            bias: uniform(outf, bound, seed, stream + 1),
            in_features: inf,
            out_features: outf,
            bound: None,
        }
    }

    pub fn forward(&mut self, x: &Var) -> Result<Var, TapeError> {
        let w = Var::leaf(&self.weight, self.out_features, self.in_features, true)?;
        let b = Var::leaf(&self.bias, 1, self.out_features, true)?;
        let y = x.linear(&w, Some(&b))?;
        self.bound = Some((w, b));
        Ok(y)
    }

    fn gradients_into(&self, grads: &Gradients, out: &mut Vec<f32>) -> Result<(), TapeError> {
        let (w, b) = self.bound.as_ref().ok_or(TapeError::NoGradient)?;
        out.extend(grads.get(w)?);
        out.extend(grads.get(b)?);
        Ok(())
    }
}

/// `Linear -> ReLU -> Linear`: the model of the CPU benchmark configuration (784 -> 256 -> 10).
#[derive(Debug, Clone)]
pub struct Mlp {
    pub fc1: Linear,
    pub fc2: Linear,
}

impl Mlp {
    /// `(inputs, hidden, outputs)` and a seed.
    pub fn build(dims: (usize, usize, usize), seed: u64) -> Self {
        let (i, h, o) = dims;
        Mlp { fc1: Linear::build((i, h), seed, 0), fc2: Linear::build((h, o), seed, 2) }
    }
}

impl Module for Mlp {
    fn parameters(&self) -> Vec<&[f32]> {
        vec![&self.fc1.weight[..], &self.fc1.bias[..], &self.fc2.weight[..], &self.fc2.bias[..]]
    }

    fn parameters_mut(&mut self) -> Vec<&mut [f32]> {
        let Mlp { fc1, fc2 } = self;
        vec![&mut fc1.weight[..], &mut fc1.bias[..], &mut fc2.weight[..], &mut fc2.bias[..]]
    }

    fn forward(&mut self, x: &Var) -> Result<Var, TapeError> {
        let h = self.fc1.forward(x)?.relu()?;
        self.fc2.forward(&h)
    }

    fn collect_gradients(&self, grads: &Gradients) -> Result<Vec<f32>, TapeError> {
        let mut out = Vec::with_capacity(self.num_parameters());
        self.fc1.gradients_into(grads, &mut out)?;
        self.fc2.gradients_into(grads, &mut out)?;
        Ok(out)
    }
}
