//! `Optimizer` and `SGD` (src/optim/mod.rs:6-8, src/optim/sgd.rs:6-25).
use crate::ffi;
use crate::module::Module;

pub trait Optimizer {
    fn step<M: Module>(&mut self, module: &mut M);
}

/// `parm = parm - (lr * grad)` for every pair of `module.parameters()`, the product rounded
/// and then the difference rounded as the reference's two array operations do, in one
/// kernel launch over all tensors.  The library caches the pointer table of a parameter
/// list on the context, so a steady-state step uploads nothing.
#[allow(clippy::upper_case_acronyms)]
pub struct SGD {
    lr: f64,
}

impl SGD {
    #[inline]
    #[must_use]
    pub fn new(lr: f64) -> Self {
        Self { lr }
    }
}

impl Optimizer for SGD {
    fn step<M: Module>(&mut self, module: &mut M) {
        let mut ctx = None;
        let (params, grads): (Vec<_>, Vec<_>) = module
            .parameters()
            .iter()
            .map(|p| {
                ctx.get_or_insert_with(|| p.parm.context().clone());
                (p.parm.raw(), p.grad.raw())
            })
            .unzip();
        if let Some(ctx) = ctx {
            ctx.check(unsafe {
                ffi::rst_sgd_step(ctx.raw(), params.len() as i32, params.as_ptr(), grads.as_ptr(), self.lr)
            });
        }
    }
}
