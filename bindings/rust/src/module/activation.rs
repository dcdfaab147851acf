//! `Identity`, `ReLU`, `Softmax` (src/module/activation/{identity,relu,softmax}.rs).
use crate::ffi;
use crate::module::{FusionRole, Module, Parameters};
use crate::tensor::Tensor;

/// Pass-through in both directions (identity.rs:15-29).
#[derive(Debug, Default)]
pub struct Identity;

impl Identity {
    #[inline]
    #[must_use]
    pub fn new() -> Self {
        Identity
    }
}

impl Module for Identity {
    #[inline]
    fn forward(&mut self, input: Tensor) -> Tensor {
        input
    }

    #[inline]
    fn backward(&mut self, gradient: Tensor) -> Tensor {
        gradient
    }

    #[inline]
    fn parameters(&mut self) -> Parameters<'_> {
        Parameters::new(0)
    }

    #[inline]
    fn fusion_role(&self) -> FusionRole {
        FusionRole::Identity
    }
}

/// `max(x, 0)`; backward multiplies by `(x > 0)` (relu.rs:17-32).  The cache is any tensor
/// with the pre-activation's sign pattern: the pre-activation itself when the layer runs on
/// its own, the post-ReLU output when `Sequential` ran the forward inside the `Linear` in
/// front of it.
#[derive(Debug, Default)]
pub struct ReLU {
    prev_input: Option<Tensor>,
}

impl ReLU {
    #[inline]
    #[must_use]
    pub fn new() -> Self {
        ReLU { prev_input: None }
    }
}

impl Module for ReLU {
    fn forward(&mut self, input: Tensor) -> Tensor {
        let ctx = input.context().clone();
        let out = input.empty_like();
        ctx.check(unsafe { ffi::rst_relu_forward(ctx.raw(), input.raw(), out.raw()) });
        self.prev_input = Some(input); // the reference keeps a clone (relu.rs:20); a handle is enough here
        out
    }

    fn backward(&mut self, gradient: Tensor) -> Tensor {
        let prev = self.prev_input.take().unwrap(); // same panic as relu.rs:26
        let ctx = gradient.context().clone();
        let out = gradient.empty_like();
        ctx.check(unsafe { ffi::rst_relu_backward(ctx.raw(), gradient.raw(), prev.raw(), out.raw()) });
        out
    }

    #[inline]
    fn parameters(&mut self) -> Parameters<'_> {
        Parameters::new(0)
    }

    #[inline]
    fn fusion_role(&self) -> FusionRole {
        FusionRole::ReLU
    }

    #[inline]
    fn note_fused(&mut self, output: &Tensor) {
        self.prev_input = Some(output.clone());
    }

    #[inline]
    fn discard_cache(&mut self) {
        self.prev_input.take().unwrap();
    }
}

/// Softmax as a layer (softmax.rs:5-34, 55-78).  The backward is the reference's, kept as
/// written: a Jacobian `-(Oᵀ·O)` over the whole batch with the diagonal replaced by
/// `s(1-s)`, applied as `gradient · jacobian`.
#[derive(Debug)]
pub struct Softmax {
    output: Option<Tensor>,
    axis: usize,
}

impl Default for Softmax {
    #[inline]
    fn default() -> Self {
        Self::new()
    }
}

impl Softmax {
    #[inline]
    #[must_use]
    pub fn with_axis(axis: usize) -> Self {
        Softmax { output: None, axis }
    }

    #[inline]
    #[must_use]
    pub fn new() -> Self {
        Self::with_axis(1)
    }
}

impl Module for Softmax {
    fn forward(&mut self, input: Tensor) -> Tensor {
        let ctx = input.context().clone();
        let out = input.empty_like();
        let status = match self.axis {
            0 => unsafe { ffi::rst_softmax_axis0(ctx.raw(), input.raw(), out.raw()) },
            1 => unsafe { ffi::rst_softmax(ctx.raw(), input.raw(), out.raw()) },
            a => panic!("axis {a} out of range for a 2-D array"),
        };
        ctx.check(status);
        self.output = Some(out.clone());
        out
    }

    fn backward(&mut self, gradient: Tensor) -> Tensor {
        let output = self.output.take().unwrap(); // same panic as softmax.rs:63
        let ctx = gradient.context().clone();
        let dx = ctx.empty(gradient.nrows(), output.ncols());
        ctx.check(unsafe { ffi::rst_softmax_backward(ctx.raw(), output.raw(), gradient.raw(), dx.raw()) });
        dx
    }

    #[inline]
    fn parameters(&mut self) -> Parameters<'_> {
        Parameters::new(0)
    }
}
