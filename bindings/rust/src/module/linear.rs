//! `Linear` (src/module/linear.rs): `y = x·Wᵀ + b`, `weight` is `(out, in)`, `bias` `(1, out)`.
use crate::ffi;
use crate::module::init::{InitParameters, KaimingNormal};
use crate::module::{FusionRole, Module, Parameters};
use crate::tensor::{Context, Tensor};

#[derive(Debug)]
pub struct Linear {
    weight: Tensor,
    bias: Option<Tensor>,

    prev_input: Option<Tensor>,
    grad_weight: Option<Tensor>,
    grad_bias: Option<Tensor>,
}

impl Linear {
    /// Builds the layer on the calling thread's current context with weights from `init`
    /// (linear.rs:20-33); the bias is always present, as through the reference's public
    /// constructors.
    #[must_use]
    pub fn new_with_kernel<I: InitParameters>(input_size: usize, output_size: usize, init: I) -> Linear {
        let ctx = Context::current();
        Linear {
            weight: ctx.tensor(&init.weight(input_size, output_size)),
            bias: Some(ctx.tensor(&init.bias(input_size, output_size))),
            prev_input: None,
            grad_weight: None,
            grad_bias: None,
        }
    }

    #[inline]
    #[must_use]
    pub fn new(input_size: usize, output_size: usize) -> Linear {
        Linear::new_with_kernel(input_size, output_size, KaimingNormal)
    }

    /// A layer whose `bias` is `None`: the reference's struct holds `Option<Array2<f64>>` and
    /// branches on it (linear.rs:51-53, 65-67, 74-77) although its public constructors always
    /// fill it (:27).  `y = x·Wᵀ`, no `db`, one parameter pair.
    #[must_use]
    pub fn without_bias<I: InitParameters>(input_size: usize, output_size: usize, init: I) -> Linear {
        let ctx = Context::current();
        Linear {
            weight: ctx.tensor(&init.weight(input_size, output_size)),
            bias: None,
            prev_input: None,
            grad_weight: None,
            grad_bias: None,
        }
    }

    /// Host copies, for tests and checkpoints.
    #[must_use]
    pub fn weight(&self) -> &Tensor {
        &self.weight
    }

    #[must_use]
    pub fn bias(&self) -> Option<&Tensor> {
        self.bias.as_ref()
    }

    #[must_use]
    pub fn grad_weight(&self) -> Option<&Tensor> {
        self.grad_weight.as_ref()
    }

    #[must_use]
    pub fn grad_bias(&self) -> Option<&Tensor> {
        self.grad_bias.as_ref()
    }

    /// Number of weight elements, for `Sequential`'s "small layer" test.
    pub(crate) fn weight_elems(&self) -> usize {
        self.weight.nrows() * self.weight.ncols()
    }

    /// What the whole-chain backward needs from this layer: the cached input (taken, with
    /// the reference's panic when it is missing, linear.rs:61) and the handles of W, dW, db.
    pub(crate) fn chain_slot(&mut self) -> (Tensor, *const ffi::rst_tensor, *mut ffi::rst_tensor, *mut ffi::rst_tensor) {
        let x = self.prev_input.take().unwrap();
        let ctx = x.context().clone();
        let (out_size, in_size) = (self.weight.nrows(), self.weight.ncols());
        let dw = self.grad_weight.get_or_insert_with(|| ctx.empty(out_size, in_size)).raw();
        let db = match &self.bias {
            Some(_) => self.grad_bias.get_or_insert_with(|| ctx.empty(1, out_size)).raw(),
            None => std::ptr::null_mut(),
        };
        (x, self.weight.raw() as *const ffi::rst_tensor, dw, db)
    }

    fn run_forward(&mut self, input: Tensor, relu: bool) -> Tensor {
        let ctx = input.context().clone();
        let out = ctx.empty(input.nrows(), self.weight.nrows());
        let bias = self.bias.as_ref().map_or(std::ptr::null(), |b| b.raw() as *const ffi::rst_tensor);
        ctx.check(unsafe {
            ffi::rst_linear_forward(ctx.raw(), input.raw(), self.weight.raw(), bias, relu as i32, out.raw())
        });
        self.prev_input = Some(input); // moved in, not copied (linear.rs:55)
        out
    }

    fn run_backward(&mut self, gradient: Tensor, relu_before: bool) -> Tensor {
        let x = self.prev_input.take().unwrap(); // same panic as linear.rs:61
        let ctx = x.context().clone();
        let (out_size, in_size) = (self.weight.nrows(), self.weight.ncols());
        // gradients are overwritten, never accumulated (linear.rs:63,66); the buffers are
        // kept so that the optimiser's pointer table stays valid from step to step
        let dw = self.grad_weight.get_or_insert_with(|| ctx.empty(out_size, in_size)).raw();
        let db = match &self.bias {
            Some(_) => self.grad_bias.get_or_insert_with(|| ctx.empty(1, out_size)).raw(),
            None => std::ptr::null_mut(),
        };
        let dx = x.empty_like();
        let mask = if relu_before { x.raw() as *const ffi::rst_tensor } else { std::ptr::null() };
        ctx.check(unsafe {
            ffi::rst_linear_backward(ctx.raw(), gradient.raw(), x.raw(), self.weight.raw(), mask, dw, db, dx.raw())
        });
        dx
    }
}

impl Module for Linear {
    #[inline]
    fn forward(&mut self, input: Tensor) -> Tensor {
        self.run_forward(input, false)
    }

    #[inline]
    fn backward(&mut self, gradient: Tensor) -> Tensor {
        self.run_backward(gradient, false)
    }

    fn parameters(&mut self) -> Parameters<'_> {
        // panics before the first backward, like linear.rs:72,75
        let p = Parameters::new(2).add(&mut self.weight, self.grad_weight.as_mut().unwrap());
        match &mut self.bias {
            Some(bias) => p.add(bias, self.grad_bias.as_mut().unwrap()),
            None => p,
        }
    }

    #[inline]
    fn fusion_role(&self) -> FusionRole {
        FusionRole::Linear
    }

    #[inline]
    fn as_linear(&mut self) -> Option<&mut Linear> {
        Some(self)
    }

    #[inline]
    fn forward_fused(&mut self, input: Tensor, relu_after: bool) -> Tensor {
        self.run_forward(input, relu_after)
    }

    #[inline]
    fn backward_fused(&mut self, gradient: Tensor, relu_before: bool) -> Tensor {
        self.run_backward(gradient, relu_before)
    }
}
