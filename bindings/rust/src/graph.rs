//! Whole-step replay: everything queued on the context between `Context::capture_begin`
//! and `Context::capture_end` becomes a CUDA graph (the batch-32 step is nine short
//! kernels; replaying them as one graph removes their launch cost from the host).
use crate::ffi;
use crate::tensor::Context;

pub struct Graph {
    h: *mut ffi::rst_graph,
    ctx: Context,
}

impl Context {
    /// Starts recording.  Calls that block or that allocate from the driver are refused
    /// until `capture_end`: run the step once before capturing it.
    pub fn capture_begin(&self) {
        self.check(unsafe { ffi::rst_graph_capture_begin(self.raw()) });
    }

    #[must_use]
    pub fn capture_end(&self) -> Graph {
        let mut h = std::ptr::null_mut();
        self.check(unsafe { ffi::rst_graph_capture_end(self.raw(), &mut h) });
        Graph { h, ctx: self.clone() }
    }
}

impl Graph {
    /// Queues one replay on the compute stream.
    pub fn launch(&self) {
        self.ctx.check(unsafe { ffi::rst_graph_launch(self.h) });
    }
}

impl Drop for Graph {
    fn drop(&mut self) {
        unsafe { ffi::rst_graph_destroy(self.h) };
    }
}
