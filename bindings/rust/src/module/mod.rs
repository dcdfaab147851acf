//! `Module`, `Parameter`, `Parameters` with the reference's shapes and names
//! (src/module/mod.rs:16-56); only the matrix type changes, from `Array2<f64>` to the
//! device [`Tensor`].
use crate::tensor::Tensor;

pub mod activation;
pub mod init;
pub(crate) mod linear;
pub(crate) mod sequential;

pub use activation::{Identity, ReLU, Softmax};
pub use linear::Linear;
pub use sequential::{ModuleDebug, Sequential};

pub struct Parameter<'a> {
    pub parm: &'a mut Tensor,
    pub grad: &'a mut Tensor,
}

pub struct Parameters<'a> {
    parms: Vec<Parameter<'a>>,
}

impl<'a> Parameters<'a> {
    pub(crate) fn new(size: usize) -> Self {
        Self { parms: Vec::with_capacity(size) }
    }

    pub fn add(mut self, parm: &'a mut Tensor, grad: &'a mut Tensor) -> Self {
        self.parms.push(Parameter { parm, grad });
        self
    }

    pub(crate) fn extend(mut self, other: Parameters<'a>) -> Self {
        self.parms.extend(other.parms);
        self
    }

    pub fn iter(self) -> impl Iterator<Item = Parameter<'a>> {
        self.parms.into_iter()
    }
}

/// What `Sequential` needs to know about a layer to fuse a `Linear` with the `ReLU`
/// behind it.  Layers outside this crate keep the default and are never fused.
#[doc(hidden)]
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum FusionRole {
    Other,
    Identity,
    Linear,
    ReLU,
}

pub trait Module {
    /// (batch_size, input_size) -> (batch_size, output_size)
    fn forward(&mut self, input: Tensor) -> Tensor;

    /// (batch_size, output_size) -> (batch_size, input_size)
    fn backward(&mut self, gradient: Tensor) -> Tensor;

    fn parameters(&mut self) -> Parameters<'_>;

    #[inline]
    fn train(&mut self) {}

    #[inline]
    fn eval(&mut self) {}

    #[doc(hidden)]
    #[inline]
    fn fusion_role(&self) -> FusionRole {
        FusionRole::Other
    }

    /// `Linear` only: forward with the ReLU that follows applied in the GEMM epilogue.
    #[doc(hidden)]
    fn forward_fused(&mut self, input: Tensor, _relu_after: bool) -> Tensor {
        self.forward(input)
    }

    /// `Linear` only: backward with the backward of the ReLU in front applied in the dX
    /// epilogue (the cached input of this layer is that ReLU's output, and
    /// `max(x, 0) > 0` exactly when `x > 0`).
    #[doc(hidden)]
    fn backward_fused(&mut self, gradient: Tensor, _relu_before: bool) -> Tensor {
        self.backward(gradient)
    }

    /// `Linear` only: the layer itself, for the whole-chain backward of `Sequential`.
    #[doc(hidden)]
    fn as_linear(&mut self) -> Option<&mut Linear> {
        None
    }

    /// `ReLU` only: the layer in front produced `output` with this ReLU already applied;
    /// keep it as the cache a later stand-alone `backward` masks with.
    #[doc(hidden)]
    fn note_fused(&mut self, _output: &Tensor) {}

    /// `ReLU` only: the layer behind applied this ReLU's backward; drop the cache the way
    /// `backward` would have (`take()`, src/module/activation/relu.rs:26).
    #[doc(hidden)]
    fn discard_cache(&mut self) {}
}
