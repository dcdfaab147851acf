//! `Sequential` and `sequential!` (src/module/sequential.rs:11-110): forward folds left,
//! backward folds right and returns dX of the network input, `parameters` concatenates in
//! layer order.
//!
//! Fusion is a peephole over adjacent layers and changes no result: a `Linear` directly
//! followed by a `ReLU` applies the ReLU in its GEMM epilogue, and a `Linear` directly
//! behind a `ReLU` applies that ReLU's backward in its dX epilogue.  Layers called on their
//! own keep the unfused kernels.
use std::fmt::Debug;

use crate::module::{FusionRole, Module, Parameters};
use crate::tensor::Tensor;

pub trait ModuleDebug: Module + Debug {}
impl<T: Module + Debug> ModuleDebug for T {}

#[derive(Debug, Default)]
pub struct Sequential {
    layers: Vec<Box<dyn ModuleDebug>>,
}

impl Sequential {
    #[inline]
    #[must_use]
    pub fn new(layers: Vec<Box<dyn ModuleDebug>>) -> Sequential {
        Sequential { layers }
    }

    #[inline]
    pub fn push<M: ModuleDebug + 'static>(&mut self, layer: M) {
        self.layers.push(Box::new(layer));
    }

    #[inline]
    pub fn insert<M: ModuleDebug + 'static>(&mut self, index: usize, layer: M) {
        self.layers.insert(index, Box::new(layer));
    }

    #[inline]
    #[must_use]
    pub fn len(&self) -> usize {
        self.layers.len()
    }

    #[inline]
    #[must_use]
    pub fn is_empty(&self) -> bool {
        self.layers.is_empty()
    }

    #[inline]
    pub fn remove(&mut self, index: usize) -> Option<Box<dyn ModuleDebug>> {
        if index >= self.len() {
            None
        } else {
            Some(self.layers.remove(index))
        }
    }

    #[inline]
    pub fn push_box(&mut self, layer: Box<dyn ModuleDebug>) {
        self.layers.push(layer);
    }

    #[inline]
    pub fn insert_box(&mut self, index: usize, layer: Box<dyn ModuleDebug>) {
        self.layers.insert(index, layer);
    }

    #[inline]
    fn role(&self, index: usize) -> FusionRole {
        self.layers[index].fusion_role()
    }
}

#[macro_export]
macro_rules! sequential {
    ($ ($layer:ident ($($arg:expr),* $(,)?) ),* $(,)?) => (
        $crate::Sequential::new(vec![$(Box::new($layer::new($($arg,)*)),)*])
    );
    ($($layer:expr),* $(,)?) => (
        $crate::Sequential::new(vec![$(Box::new($layer),)*])
    );
}

impl Module for Sequential {
    fn forward(&mut self, input: Tensor) -> Tensor {
        let n = self.layers.len();
        let mut x = input;
        let mut i = 0;
        while i < n {
            if self.role(i) == FusionRole::Linear && i + 1 < n && self.role(i + 1) == FusionRole::ReLU {
                x = self.layers[i].forward_fused(x, true);
                self.layers[i + 1].note_fused(&x); // sign pattern of the pre-activation
                i += 2;
            } else {
                x = self.layers[i].forward(x);
                i += 1;
            }
        }
        x
    }

    fn backward(&mut self, gradient: Tensor) -> Tensor {
        let mut g = gradient;
        let mut i = self.layers.len();
        while i > 0 {
            i -= 1;
            if self.role(i) == FusionRole::Linear && i > 0 && self.role(i - 1) == FusionRole::ReLU {
                g = self.layers[i].backward_fused(g, true);
                self.layers[i - 1].discard_cache(); // its mask was applied in the epilogue above
                i -= 1;
            } else {
                g = self.layers[i].backward(g);
            }
        }
        g
    }

    fn parameters(&mut self) -> Parameters<'_> {
        self.layers
            .iter_mut()
            .fold(Parameters::new(0), |acc, layer| acc.extend(layer.parameters()))
    }

    fn train(&mut self) {
        self.layers.iter_mut().for_each(|layer| layer.train());
    }

    fn eval(&mut self) {
        self.layers.iter_mut().for_each(|layer| layer.eval());
    }
}
