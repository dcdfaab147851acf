//! Data-parallel gradient exchange, one process per GPU (no counterpart in the reference,
//! which is single-threaded).  Each rank runs the step on `B / world` rows; because
//! `Linear::backward` divides by the local row count, the average over ranks of every
//! dW/db is the full-batch gradient.
use crate::ffi;
use crate::module::Module;
use crate::tensor::Context;

pub struct Communicator {
    h: *mut ffi::rst_comm,
    ctx: Context,
}

impl Communicator {
    /// Rank 0 calls this and ships the bytes to the other ranks by any channel.
    #[must_use]
    pub fn unique_id() -> [u8; ffi::RST_COMM_ID_BYTES] {
        let mut id = [0u8; ffi::RST_COMM_ID_BYTES];
        ffi::check(std::ptr::null(), unsafe { ffi::rst_comm_get_id(id.as_mut_ptr().cast()) });
        id
    }

    #[must_use]
    pub fn new(ctx: &Context, id: &[u8; ffi::RST_COMM_ID_BYTES], rank: usize, world: usize) -> Communicator {
        let mut h = std::ptr::null_mut();
        ctx.check(unsafe { ffi::rst_comm_create(ctx.raw(), id.as_ptr().cast(), rank as i32, world as i32, &mut h) });
        Communicator { h, ctx: ctx.clone() }
    }

    /// Averages every gradient of `module` over the ranks on the communication stream and
    /// makes the compute stream wait for the result; call it between `backward` and
    /// `Optimizer::step`.
    pub fn average_gradients<M: Module>(&self, module: &mut M) {
        let grads: Vec<_> = module.parameters().iter().map(|p| p.grad.raw()).collect();
        self.ctx.check(unsafe { ffi::rst_allreduce_avg(self.h, grads.len() as i32, grads.as_ptr()) });
        self.ctx.check(unsafe { ffi::rst_comm_join(self.h) });
    }
}

impl Drop for Communicator {
    fn drop(&mut self) {
        unsafe { ffi::rst_comm_destroy(self.h) };
    }
}
