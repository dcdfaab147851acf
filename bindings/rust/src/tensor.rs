//! The device tensor that takes the place of `Array2<f64>` in the crate's `Module`, `Loss`
//! and `Optimizer` signatures (src/module/mod.rs:42-56), and the per-GPU context it lives in.
use std::cell::RefCell;
use std::fmt;
use std::rc::Rc;

use ndarray::Array2;

use crate::ffi;

struct ContextInner {
    h: *mut ffi::rst_ctx,
}

impl Drop for ContextInner {
    fn drop(&mut self) {
        unsafe { ffi::rst_ctx_destroy(self.h) };
    }
}

/// One GPU: streams, caching allocator, result ring.  Cheap to clone; the GPU state is
/// released when the last clone and the last tensor made from it are gone.
#[derive(Clone)]
pub struct Context {
    inner: Rc<ContextInner>,
}

thread_local! {
    static CURRENT: RefCell<Option<Context>> = RefCell::new(None);
}

impl Context {
    /// Creates the context of CUDA device `device`.  Panics without a usable GPU: there is
    /// no CPU path behind this crate.
    #[must_use]
    pub fn new(device: i32) -> Context {
        let mut h = std::ptr::null_mut();
        let status = unsafe { ffi::rst_ctx_create(device, &mut h) };
        ffi::check(std::ptr::null(), status);
        Context { inner: Rc::new(ContextInner { h }) }
    }

    /// The context that `Linear::new`, `Tensor::from(array)` and the data loader use when
    /// none is given, so that the reference's constructors keep their signatures.  Created
    /// on first use for the device named by `RSTORCH_B200_DEVICE` (default 0).
    #[must_use]
    pub fn current() -> Context {
        CURRENT.with(|c| {
            c.borrow_mut()
                .get_or_insert_with(|| {
                    let device = std::env::var("RSTORCH_B200_DEVICE").ok().and_then(|v| v.parse().ok()).unwrap_or(0);
                    Context::new(device)
                })
                .clone()
        })
    }

    /// Makes `ctx` the calling thread's default (one rank per GPU: call it once with the
    /// rank's device before building the model).
    pub fn set_current(ctx: &Context) {
        CURRENT.with(|c| *c.borrow_mut() = Some(ctx.clone()));
    }

    #[inline]
    pub(crate) fn raw(&self) -> *mut ffi::rst_ctx {
        self.inner.h
    }

    #[inline]
    pub(crate) fn check(&self, status: i32) {
        ffi::check(self.inner.h, status);
    }

    /// Blocks until everything queued on this GPU has finished.
    pub fn synchronize(&self) {
        self.check(unsafe { ffi::rst_ctx_synchronize(self.raw()) });
    }

    /// Panics if a kernel's bounded wait ran out since the last call.
    pub fn check_device(&self) {
        self.check(unsafe { ffi::rst_ctx_check_device(self.raw()) });
    }

    /// Uninitialised `(rows, cols)` tensor from the caching allocator.
    #[must_use]
    pub fn empty(&self, rows: usize, cols: usize) -> Tensor {
        let mut h = std::ptr::null_mut();
        self.check(unsafe { ffi::rst_tensor_alloc(self.raw(), rows as i64, cols as i64, &mut h) });
        Tensor { inner: Rc::new(TensorInner { h, owns: true, ctx: self.clone() }), rows, cols }
    }

    #[must_use]
    pub fn zeros(&self, rows: usize, cols: usize) -> Tensor {
        let t = self.empty(rows, cols);
        self.check(unsafe { ffi::rst_tensor_fill(t.raw(), 0.0) });
        t
    }

    /// Copies a host matrix into HBM (standard layout first, as the crate's own `dot`
    /// operands are).
    #[must_use]
    pub fn tensor(&self, a: &Array2<f64>) -> Tensor {
        let a = a.as_standard_layout();
        let t = self.empty(a.nrows(), a.ncols());
        self.check(unsafe { ffi::rst_tensor_upload(t.raw(), a.as_ptr()) });
        t
    }

    /// Wraps a handle the library keeps ownership of (the tensors of a staging slot).
    pub(crate) fn borrowed(&self, h: *mut ffi::rst_tensor) -> Tensor {
        let (mut rows, mut cols) = (0i64, 0i64);
        self.check(unsafe { ffi::rst_tensor_shape(h, &mut rows, &mut cols) });
        Tensor { inner: Rc::new(TensorInner { h, owns: false, ctx: self.clone() }), rows: rows as usize, cols: cols as usize }
    }
}

struct TensorInner {
    h: *mut ffi::rst_tensor,
    owns: bool,
    ctx: Context,
}

impl Drop for TensorInner {
    fn drop(&mut self) {
        if self.owns {
            // back to the caching allocator, ordered on the compute stream
            unsafe { ffi::rst_tensor_free(self.h) };
        }
    }
}

/// Dense row-major f64 matrix in HBM.  A `Tensor` is a shared handle: `clone()` copies the
/// handle, not the data, which is what lets `loss.forward(pred.clone(), y.clone())` of the
/// README loop stay free of device copies.  Kernels never write into a tensor they were
/// given as an input, so sharing is not observable.
#[derive(Clone)]
pub struct Tensor {
    inner: Rc<TensorInner>,
    rows: usize,
    cols: usize,
}

impl Tensor {
    #[inline]
    #[must_use]
    pub fn nrows(&self) -> usize {
        self.rows
    }

    #[inline]
    #[must_use]
    pub fn ncols(&self) -> usize {
        self.cols
    }

    #[inline]
    #[must_use]
    pub fn shape(&self) -> [usize; 2] {
        [self.rows, self.cols]
    }

    #[inline]
    #[must_use]
    pub fn context(&self) -> &Context {
        &self.inner.ctx
    }

    #[inline]
    pub(crate) fn raw(&self) -> *mut ffi::rst_tensor {
        self.inner.h
    }

    /// Same shape, uninitialised, same GPU.
    #[must_use]
    pub fn empty_like(&self) -> Tensor {
        self.inner.ctx.empty(self.rows, self.cols)
    }

    /// Blocking copy back to the host.
    #[must_use]
    pub fn to_array(&self) -> Array2<f64> {
        let mut v = vec![0.0f64; self.rows * self.cols];
        self.inner.ctx.check(unsafe { ffi::rst_tensor_download(self.raw(), v.as_mut_ptr()) });
        Array2::from_shape_vec((self.rows, self.cols), v).expect("shape matches the buffer")
    }

    /// Overwrites the contents from a host matrix of the same shape.
    pub fn assign(&mut self, a: &Array2<f64>) {
        assert_eq!(a.shape(), &[self.rows, self.cols], "shape mismatch in Tensor::assign");
        let a = a.as_standard_layout();
        self.inner.ctx.check(unsafe { ffi::rst_tensor_upload(self.raw(), a.as_ptr()) });
    }
}

impl From<Array2<f64>> for Tensor {
    fn from(a: Array2<f64>) -> Tensor {
        Context::current().tensor(&a)
    }
}

impl From<&Array2<f64>> for Tensor {
    fn from(a: &Array2<f64>) -> Tensor {
        Context::current().tensor(a)
    }
}

impl From<Tensor> for Array2<f64> {
    fn from(t: Tensor) -> Array2<f64> {
        t.to_array()
    }
}

impl fmt::Debug for Tensor {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "Tensor({}x{} f64 @ {:p})", self.rows, self.cols, self.inner.h)
    }
}
