//! `Sequential` and `sequential!` (src/module/sequential.rs:11-110): forward folds left,
//! backward folds right and returns dX of the network input, `parameters` concatenates in
//! layer order.
//!
//! Fusion is a peephole over adjacent layers and changes no result: a `Linear` directly
//! followed by a `ReLU` applies the ReLU in its GEMM epilogue, and a `Linear` directly
//! behind a `ReLU` applies that ReLU's backward in its dX epilogue.  Layers called on their
//! own keep the unfused kernels.
use std::fmt::Debug;

use crate::ffi;
use crate::module::{FusionRole, Module, Parameters};
use crate::tensor::Tensor;

/// Layers above this many weight elements keep the layer-by-layer backward.
const CHAIN_MAX_WEIGHT_ELEMS: usize = 1 << 20;

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

    /// Index of the first layer of a trailing `Linear, (ReLU, Linear)*` run of small plain
    /// layers that, apart from leading `Identity` layers, is the whole container.
    fn small_linear_chain(&mut self) -> Option<usize> {
        let first = (0..self.layers.len()).find(|&i| self.role(i) != FusionRole::Identity)?;
        let n = self.layers.len() - first;
        if n < 3 || n % 2 == 0 {
            return None;
        }
        for k in 0..n {
            if k % 2 == 0 {
                let small = self.layers[first + k].as_linear().map(|l| l.weight_elems() <= CHAIN_MAX_WEIGHT_ELEMS);
                if small != Some(true) {
                    return None;
                }
            } else if self.role(first + k) != FusionRole::ReLU {
                return None;
            }
        }
        Some(first)
    }

    /// The whole backward as one library call: the dependent dX products first, then every
    /// dW/db product in one launch.
    fn backward_chain(&mut self, first: usize, gradient: &Tensor) -> Tensor {
        let n = (self.layers.len() - first + 1) / 2;
        let ctx = gradient.context().clone();
        let (mut xs, mut dxs) = (Vec::with_capacity(n), Vec::with_capacity(n));
        let (mut hx, mut hw, mut hdw, mut hdb, mut hdx, mut mask) =
            (Vec::new(), Vec::new(), Vec::new(), Vec::new(), Vec::new(), Vec::new());
        for l in 0..n {
            if l > 0 {
                self.layers[first + 2 * l - 1].discard_cache();
            }
            let (x, w, dw, db) = self.layers[first + 2 * l].as_linear().unwrap().chain_slot();
            let dx = x.empty_like();
            hx.push(x.raw() as *const ffi::rst_tensor);
            hw.push(w);
            hdw.push(dw);
            hdb.push(db);
            hdx.push(dx.raw());
            mask.push(u8::from(l > 0));
            xs.push(x);
            dxs.push(dx);
        }
        ctx.check(unsafe {
            ffi::rst_linear_backward_chain(ctx.raw(), n as i32, gradient.raw(), hx.as_ptr(), hw.as_ptr(),
                                           mask.as_ptr(), hdw.as_ptr(), hdb.as_ptr(), hdx.as_ptr())
        });
        dxs.swap_remove(0)
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
        if let Some(first) = self.small_linear_chain() {
            return self.backward_chain(first, &gradient);
        }
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
