//! Weight initialisers (src/module/init/mod.rs:11-18, he.rs:9-15, xavier.rs, sigma.rs).
//!
//! The reference draws from a thread-seeded generator and cannot be reproduced; here the
//! draws come from the library's counter-based streams (`rst_synth_normal`), keyed by a
//! process-wide seed and a per-thread layer counter, so that two runs of one program build
//! the same model.  The distributions are the reference's.
use std::cell::Cell;

use ndarray::Array2;

use crate::ffi;

pub trait InitParameters {
    fn weight(&self, input_size: usize, output_size: usize) -> Array2<f64>;

    #[inline]
    fn bias(&self, _input_size: usize, output_size: usize) -> Array2<f64> {
        Array2::zeros((1, output_size))
    }
}

thread_local! {
    static SEED: Cell<u64> = Cell::new(
        std::env::var("RSTORCH_B200_SEED").ok().and_then(|v| v.parse().ok()).unwrap_or(0));
    static LAYER: Cell<u64> = Cell::new(0);
}

/// Restarts the initialiser streams of the calling thread at `seed`.
pub fn set_seed(seed: u64) {
    SEED.with(|s| s.set(seed));
    LAYER.with(|l| l.set(0));
}

fn mix(mut z: u64) -> u64 {
    // splitmix64 finaliser
    z = (z ^ (z >> 30)).wrapping_mul(0xBF58_476D_1CE4_E5B9);
    z = (z ^ (z >> 27)).wrapping_mul(0x94D0_49BB_1331_11EB);
    z ^ (z >> 31)
}

/// Key of the next layer's stream for initialiser family `tag`.
fn next_stream(tag: u64) -> u64 {
    let seed = SEED.with(|s| s.get());
    let layer = LAYER.with(|l| {
        let v = l.get();
        l.set(v + 1);
        v
    });
    mix(mix(seed ^ tag.wrapping_mul(0x9E37_79B9_7F4A_7C15)).wrapping_add(layer))
}

fn normal_matrix(tag: u64, rows: usize, cols: usize, mean: f64, stddev: f64) -> Array2<f64> {
    let mut v = vec![0.0f64; rows * cols];
    let status = unsafe { ffi::rst_synth_normal(next_stream(tag), v.len() as u64, 0, mean, stddev, v.as_mut_ptr()) };
    ffi::check(std::ptr::null(), status);
    Array2::from_shape_vec((rows, cols), v).expect("shape matches the buffer")
}

/// N(0, 1/sqrt(input_size)) weights, zero bias (he.rs:9-15).
#[derive(Debug, Default, Clone, Copy)]
pub struct KaimingNormal;

impl InitParameters for KaimingNormal {
    fn weight(&self, input_size: usize, output_size: usize) -> Array2<f64> {
        let sigma = 1.0 / f64::sqrt(input_size as f64);
        normal_matrix(1, output_size, input_size, 0.0, sigma)
    }
}

/// N(0, sqrt(2 / (input_size + output_size))) weights (xavier.rs).
#[derive(Debug, Default, Clone, Copy)]
pub struct XavierNormal;

impl InitParameters for XavierNormal {
    fn weight(&self, input_size: usize, output_size: usize) -> Array2<f64> {
        let sigma = f64::sqrt(2.0 / (input_size as f64 + output_size as f64));
        normal_matrix(2, output_size, input_size, 0.0, sigma)
    }
}

/// N(mean, std) weights (sigma.rs); the constructors refuse a non-finite deviation.
#[derive(Debug, Clone, Copy)]
pub struct Normal {
    mean: f64,
    std: f64,
}

impl Normal {
    #[must_use]
    pub fn new(mean: f64, std: f64) -> Option<Normal> {
        std.is_finite().then_some(Normal { mean, std })
    }

    #[must_use]
    pub fn new_std(std: f64) -> Option<Normal> {
        Normal::new(0.0, std)
    }
}

impl InitParameters for Normal {
    fn weight(&self, input_size: usize, output_size: usize) -> Array2<f64> {
        normal_matrix(3, output_size, input_size, self.mean, self.std)
    }
}
