//! `Dataset`, `Sampler`, `DataLoader::iter_array` (src/data/dataset/mod.rs:15-57,
//! src/data/sampler.rs:6-43, src/data/data_loader.rs:42-93,180-208).
//!
//! `iter_array` yields device tensors.  Where the reference `append`s `batch_size` samples
//! to two fresh arrays, the iterator here writes them straight into a pinned host slot,
//! starts the host-to-device copy on the copy stream and hands out the tensors of the slot
//! that was filled one batch earlier, so the copy of batch k+1 overlaps the step on batch k.
use std::ops::Range;

use ndarray::{Array, Dimension};

use crate::ffi;
use crate::tensor::{Context, Tensor};

pub trait Dataset {
    type Item;

    fn get(&self, index: usize) -> Option<Self::Item>;
    fn len(&self) -> usize;

    #[inline]
    fn is_empty(&self) -> bool {
        self.len() == 0
    }

    #[inline]
    fn transform<B, F>(self, f: F) -> Transform<Self, F>
    where
        Self: Sized,
        F: Fn(Self::Item) -> B,
    {
        Transform { dataset: self, f }
    }
}

/// Dataset over a vector of items.
pub struct Basic<T> {
    items: Vec<T>,
}

impl<T: Clone> Basic<T> {
    #[inline]
    #[must_use]
    pub fn new(items: Vec<T>) -> Self {
        Self { items }
    }
}

impl<T: Clone> Dataset for Basic<T> {
    type Item = T;

    #[inline]
    fn get(&self, index: usize) -> Option<T> {
        self.items.get(index).cloned()
    }

    #[inline]
    fn len(&self) -> usize {
        self.items.len()
    }
}

/// `dataset.transform(f)`: `f` applied to every item on access.
pub struct Transform<D, F> {
    dataset: D,
    f: F,
}

impl<D: Dataset, B, F: Fn(D::Item) -> B> Dataset for Transform<D, F> {
    type Item = B;

    #[inline]
    fn get(&self, index: usize) -> Option<B> {
        self.dataset.get(index).map(&self.f)
    }

    #[inline]
    fn len(&self) -> usize {
        self.dataset.len()
    }
}

pub trait Sampler {
    type Iter: Iterator<Item = usize>;

    fn iter(&mut self) -> Self::Iter;

    fn len(&self) -> usize;

    #[inline]
    fn is_empty(&self) -> bool {
        self.len() == 0
    }
}

pub struct SequentialSampler {
    size: usize,
}

impl SequentialSampler {
    #[inline]
    #[must_use]
    pub fn new(size: usize) -> Self {
        Self { size }
    }
}

impl Sampler for SequentialSampler {
    type Iter = Range<usize>;

    #[inline]
    fn iter(&mut self) -> Range<usize> {
        0..self.size
    }

    #[inline]
    fn len(&self) -> usize {
        self.size
    }
}

struct Stager {
    h: *mut ffi::rst_stager,
    ctx: Context,
    x_cols: usize,
    t_cols: usize,
}

impl Drop for Stager {
    fn drop(&mut self) {
        unsafe { ffi::rst_stager_destroy(self.h) };
    }
}

const SLOTS: usize = 2;

pub struct DataLoader<D, S> {
    dataset: D,
    batch_size: usize,
    sampler: S,
    /// `Some(permutation)` when shuffling: index i of the sampler maps to `permutation[i]`
    /// (the role of `Shuffler`, src/data/dataset/shuffler.rs:15-25).
    permutation: Option<Vec<usize>>,
    shuffle_state: u64,
    stager: Option<Stager>,
}

impl<D: Dataset, S: Sampler> DataLoader<D, S> {
    #[inline]
    #[must_use]
    pub fn new(dataset: D, batch_size: usize, shuffle: bool, sampler: S) -> Self {
        let permutation = shuffle.then(|| (0..dataset.len()).collect());
        Self { dataset, batch_size, sampler, permutation, shuffle_state: 0x5EED, stager: None }
    }

    /// Seeds the permutation stream (the reference shuffles with an unseedable thread
    /// generator; a seeded stream makes an epoch order repeatable).
    pub fn seed_shuffle(&mut self, seed: u64) {
        self.shuffle_state = seed;
    }

    /// Redraws the permutation (Fisher-Yates over a splitmix64 stream).
    pub fn shuffle(&mut self) {
        if let Some(p) = &mut self.permutation {
            for i in (1..p.len()).rev() {
                self.shuffle_state = self.shuffle_state.wrapping_add(0x9E37_79B9_7F4A_7C15);
                let mut z = self.shuffle_state;
                z = (z ^ (z >> 30)).wrapping_mul(0xBF58_476D_1CE4_E5B9);
                z = (z ^ (z >> 27)).wrapping_mul(0x94D0_49BB_1331_11EB);
                z ^= z >> 31;
                let j = (z % (i as u64 + 1)) as usize;
                p.swap(i, j);
            }
        }
    }

    #[inline]
    #[must_use]
    pub fn len(&self) -> usize {
        self.dataset.len() / self.batch_size
    }

    #[inline]
    #[must_use]
    pub fn is_empty(&self) -> bool {
        // the remainder that does not fill a batch is ignored, as in the reference
        self.dataset.len() < self.batch_size
    }

    fn item(&self, index: usize) -> Option<D::Item> {
        match &self.permutation {
            Some(p) => self.dataset.get(*p.get(index)?),
            None => self.dataset.get(index),
        }
    }
}

impl<D, D1, D2, S> DataLoader<D, S>
where
    D: Dataset<Item = (Array<f64, D1>, Array<f64, D2>)>,
    S: Sampler,
    D1: Dimension,
    D2: Dimension,
{
    /// Batches of `(X, T)` on the calling thread's current context: `X` is
    /// `(batch_size, sample elements)`, `T` is `(batch_size, target elements)`.
    pub fn iter_array(&mut self) -> ArrayDataLoaderIter<'_, D, S> {
        self.shuffle();
        let iter = self.sampler.iter();
        ArrayDataLoaderIter { data_loader: self, iter, filled: [false; SLOTS], next_slot: 0, primed: false }
    }
}

pub struct ArrayDataLoaderIter<'a, D, S: Sampler> {
    data_loader: &'a mut DataLoader<D, S>,
    iter: S::Iter,
    filled: [bool; SLOTS],
    next_slot: usize,
    primed: bool,
}

impl<'a, D, D1, D2, S> ArrayDataLoaderIter<'a, D, S>
where
    D: Dataset<Item = (Array<f64, D1>, Array<f64, D2>)>,
    S: Sampler,
    D1: Dimension,
    D2: Dimension,
{
    /// Writes the next `batch_size` samples into pinned slot `slot` and starts its copy.
    /// Returns false (and starts nothing) if the sampler or the dataset ran out first: the
    /// partial batch is dropped (data_loader.rs:192-207).
    fn fill(&mut self, slot: usize) -> bool {
        let b = self.data_loader.batch_size;
        for row in 0..b {
            let Some(index) = self.iter.next() else { return false };
            let Some((sample, target)) = self.data_loader.item(index) else { return false };
            if self.data_loader.stager.is_none() {
                let ctx = Context::current();
                let mut h = std::ptr::null_mut();
                ctx.check(unsafe {
                    ffi::rst_stager_create(ctx.raw(), b as i64, sample.len() as i64, target.len() as i64,
                                           SLOTS as i32, &mut h)
                });
                self.data_loader.stager = Some(Stager { h, ctx, x_cols: sample.len(), t_cols: target.len() });
            }
            let st = self.data_loader.stager.as_ref().unwrap();
            assert_eq!(sample.len(), st.x_cols, "samples of one loader must have one size");
            assert_eq!(target.len(), st.t_cols, "targets of one loader must have one size");
            let (mut px, mut pt) = (std::ptr::null_mut(), std::ptr::null_mut());
            st.ctx.check(unsafe { ffi::rst_stager_host(st.h, slot as i32, &mut px, &mut pt) });
            // logical (row-major) order, whatever the item's memory layout
            for (k, v) in sample.iter().enumerate() {
                unsafe { *px.add(row * st.x_cols + k) = *v };
            }
            for (k, v) in target.iter().enumerate() {
                unsafe { *pt.add(row * st.t_cols + k) = *v };
            }
        }
        let st = self.data_loader.stager.as_ref().unwrap();
        st.ctx.check(unsafe { ffi::rst_stager_submit(st.h, slot as i32) });
        true
    }
}

impl<'a, D, D1, D2, S> Iterator for ArrayDataLoaderIter<'a, D, S>
where
    D: Dataset<Item = (Array<f64, D1>, Array<f64, D2>)>,
    S: Sampler,
    D1: Dimension,
    D2: Dimension,
{
    type Item = (Tensor, Tensor);

    fn next(&mut self) -> Option<(Tensor, Tensor)> {
        if !self.primed {
            self.primed = true;
            self.filled[0] = self.fill(0);
        }
        let slot = self.next_slot;
        if !self.filled[slot] {
            return None;
        }
        let st = self.data_loader.stager.as_ref().unwrap();
        let (mut hx, mut ht) = (std::ptr::null_mut(), std::ptr::null_mut());
        st.ctx.check(unsafe { ffi::rst_stager_acquire(st.h, slot as i32, &mut hx, &mut ht) });
        let batch = (st.ctx.borrowed(hx), st.ctx.borrowed(ht));
        // the other slot was consumed one batch ago: refill it while this batch is in use
        self.filled[slot] = false;
        let other = (slot + 1) % SLOTS;
        self.filled[other] = self.fill(other);
        self.next_slot = other;
        Some(batch)
    }
}
