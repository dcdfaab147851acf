//! `BasicModel` (src/model.rs:4-32): a module, a loss and an optimiser bundled into the
//! reference's own statement of the training step and of inference.
use crate::loss::Loss;
use crate::module::Module;
use crate::optim::Optimizer;
use crate::tensor::Tensor;

pub struct BasicModel<M, L, O> {
    pub module: M,
    pub loss: L,
    pub optim: O,
}

impl<M: Module, L: Loss, O: Optimizer> BasicModel<M, L, O> {
    #[must_use]
    pub fn new(module: M, loss: L, optim: O) -> Self {
        Self { module, loss, optim }
    }

    /// forward, loss.forward, loss.backward, backward, optim.step (model.rs:19-27).
    pub fn step(&mut self, input: Tensor, truth: Tensor) {
        let input = self.module.forward(input);
        self.loss.forward(input, truth);

        let gradient = self.loss.backward();
        self.module.backward(gradient);

        self.optim.step(&mut self.module);
    }

    /// `module.forward(input)` (model.rs:29-31).
    pub fn predict(&mut self, input: Tensor) -> Tensor {
        self.module.forward(input)
    }
}
