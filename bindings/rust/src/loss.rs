//! `Loss` and `CrossEntropyLoss` (src/loss/mod.rs:6-11, src/loss/cross_entropy.rs:32-48).
use crate::ffi;
use crate::tensor::Tensor;

pub trait Loss {
    /// (batch_size, input_size)
    fn forward(&mut self, input: Tensor, truth: Tensor) -> f64;
    /// (batch_size, input_size)
    fn backward(&mut self) -> Tensor;
}

/// One kernel pass computes `p = softmax(pred)`, `loss = -(Σ t·ln p) / B`, the gradient
/// `p - t` (no 1/B: that factor lives in `Linear::backward`) and the number of rows whose
/// argmax matches the truth's; `forward` blocks on the loss, as a function returning `f64`
/// must.
pub struct CrossEntropyLoss {
    grad: Option<Tensor>,
    last_accuracy: f64,
}

impl CrossEntropyLoss {
    #[inline]
    #[must_use]
    pub fn new() -> Self {
        Self { grad: None, last_accuracy: f64::NAN }
    }

    /// `accuracy(pred, truth)` of the batch the last `forward` saw, for loops that want it
    /// without a second pass over the logits.
    #[inline]
    #[must_use]
    pub fn last_accuracy(&self) -> f64 {
        self.last_accuracy
    }
}

impl Default for CrossEntropyLoss {
    #[inline]
    fn default() -> Self {
        Self::new()
    }
}

impl Loss for CrossEntropyLoss {
    fn forward(&mut self, pred: Tensor, truth: Tensor) -> f64 {
        let ctx = pred.context().clone();
        let grad = pred.empty_like();
        let (mut loss, mut acc) = (0.0f64, 0.0f64);
        ctx.check(unsafe { ffi::rst_xent_forward_backward(ctx.raw(), pred.raw(), truth.raw(), grad.raw(), 0) });
        // RST_ERR_NAN here is the reference's panic on a NaN logit (softmax.rs:38)
        ctx.check(unsafe { ffi::rst_xent_result(ctx.raw(), 0, &mut loss, &mut acc) });
        self.grad = Some(grad);
        self.last_accuracy = acc;
        loss
    }

    fn backward(&mut self) -> Tensor {
        self.grad.take().unwrap() // same panic as cross_entropy.rs:46
    }
}
