//! `accuracy`, `argmax`, `one_hot`, `flatten`, `normalize_zero_one` (src/utils.rs:5-65).
use ndarray::{Array, Array0, Array1, Dimension};

use crate::ffi;
use crate::tensor::Tensor;

/// Per row, the index of the maximum; the first maximum wins and a NaN never replaces the
/// running maximum (utils.rs:44-53).  Blocking.
#[must_use]
pub fn argmax(arr: Tensor) -> Array1<usize> {
    let ctx = arr.context().clone();
    let mut idx = vec![0i64; arr.nrows()];
    ctx.check(unsafe { ffi::rst_argmax(ctx.raw(), arr.raw(), idx.as_mut_ptr()) });
    idx.into_iter().map(|i| i as usize).collect()
}

/// Fraction of rows whose argmax agrees between `pred` and `truth` (utils.rs:55-65).
/// Blocking.
#[must_use]
pub fn accuracy(pred: Tensor, truth: Tensor) -> f64 {
    let ctx = pred.context().clone();
    let mut acc = 0.0f64;
    ctx.check(unsafe { ffi::rst_accuracy(ctx.raw(), pred.raw(), truth.raw(), &mut acc) });
    acc
}

/// Host-side transforms of one sample, for datasets that are not resident in HBM (a
/// resident dataset applies them inside its gather kernel).
pub fn flatten<A, D: Dimension>(x: Array<A, D>) -> Array1<A> {
    x.into_iter().collect()
}

pub fn one_hot<A: Into<usize>>(x: Array0<A>, n: usize) -> Array1<f64> {
    let mut encoded = Array1::zeros(n);
    encoded[x.into_scalar().into()] = 1.0;
    encoded
}

/// Min-max scaling of one sample to [0, 1] by its own minimum and maximum (utils.rs:5-18);
/// a constant sample gives 0/0 = NaN, as in the reference.
pub fn normalize_zero_one<A: Into<f64> + Copy, D: Dimension>(x: Array<A, D>) -> Array<f64, D> {
    let x = x.mapv(|v| v.into());
    let min = x.iter().copied().fold(f64::INFINITY, f64::min);
    let max = x.iter().copied().fold(f64::NEG_INFINITY, f64::max);
    x.mapv(|v| (v - min) / (max - min))
}
