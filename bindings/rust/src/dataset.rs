//! A u8 dataset resident in HBM with the README transform
//! `(flatten(normalize_zero_one(x)), one_hot(y, classes))` (README.md:44, src/utils.rs:5-42)
//! applied by the kernel that builds a batch: what `Transform` + `ArrayDataLoaderIter::next`
//! (src/data/data_loader.rs:192-207) do on the host for the MNIST item type
//! (src/data/dataset/hub/mnist.rs:181-194).
use crate::ffi;
use crate::tensor::{Context, Tensor};

pub struct DeviceDataset {
    h: *mut ffi::rst_dataset,
    ctx: Context,
    len: usize,
    features: usize,
    classes: usize,
}

impl DeviceDataset {
    /// `images` holds `labels.len()` samples of `features` bytes each, row-major.
    /// Panics if a label is `>= classes` (the reference's `one_hot` panics on it).
    #[must_use]
    pub fn new(ctx: &Context, images: &[u8], labels: &[u8], features: usize, classes: usize) -> DeviceDataset {
        assert_eq!(images.len(), labels.len() * features, "images and labels differ in length");
        let mut h = std::ptr::null_mut();
        ctx.check(unsafe {
            ffi::rst_dataset_create_u8(ctx.raw(), images.as_ptr(), labels.as_ptr(), labels.len() as i64,
                                       features as i64, classes as i64, &mut h)
        });
        DeviceDataset { h, ctx: ctx.clone(), len: labels.len(), features, classes }
    }

    #[inline]
    #[must_use]
    pub fn len(&self) -> usize {
        self.len
    }

    #[inline]
    #[must_use]
    pub fn is_empty(&self) -> bool {
        self.len == 0
    }

    /// The batch of the given sample indices: `(X (n, features), T (n, classes))`.
    #[must_use]
    pub fn gather(&self, indices: &[i64]) -> (Tensor, Tensor) {
        let x = self.ctx.empty(indices.len(), self.features);
        let t = self.ctx.empty(indices.len(), self.classes);
        self.ctx.check(unsafe {
            ffi::rst_dataset_gather(self.h, indices.as_ptr(), indices.len() as i64, x.raw(), t.raw())
        });
        (x, t)
    }

    /// The dataset's pinned index buffer: write the next batch's indices into it, then call
    /// `gather_staged` (directly, or by replaying a graph that captured it).  The slice is
    /// valid until a larger batch is asked for.
    pub fn index_stage(&mut self, batch: usize) -> &mut [i64] {
        let mut p: *mut i64 = std::ptr::null_mut();
        self.ctx.check(unsafe { ffi::rst_dataset_index_stage(self.h, batch as i64, &mut p) });
        unsafe { std::slice::from_raw_parts_mut(p, batch) }
    }

    /// Builds into `x`, `t` the batch of the indices the stage holds when the work runs; reads
    /// no index on the host, so it may be captured into a graph.
    pub fn gather_staged(&self, batch: usize, x: &Tensor, t: &Tensor) {
        self.ctx.check(unsafe { ffi::rst_dataset_gather_staged(self.h, batch as i64, x.raw(), t.raw()) });
    }

    /// Draws the order of the next epoch on the device (`Shuffler::shuffle`,
    /// src/data/dataset/shuffler.rs:22-25), seeded where the reference's `thread_rng` is not.
    pub fn shuffle(&mut self, seed: u64) {
        self.ctx.check(unsafe { ffi::rst_dataset_shuffle(self.h, seed) });
    }

    /// The batch of epoch positions `[first, first + batch)` (`Shuffler::get`, shuffler.rs:31-33).
    #[must_use]
    pub fn gather_epoch(&self, first: usize, batch: usize) -> (Tensor, Tensor) {
        let x = self.ctx.empty(batch, self.features);
        let t = self.ctx.empty(batch, self.classes);
        self.ctx.check(unsafe { ffi::rst_dataset_gather_epoch(self.h, first as i64, batch as i64, x.raw(), t.raw()) });
        (x, t)
    }

    /// The current epoch's order of the samples (identity before the first shuffle).
    #[must_use]
    pub fn epoch_order(&self) -> Vec<i64> {
        let mut order = vec![0i64; self.len];
        self.ctx.check(unsafe { ffi::rst_dataset_epoch_order(self.h, order.as_mut_ptr()) });
        order
    }
}

impl Drop for DeviceDataset {
    fn drop(&mut self) {
        unsafe { ffi::rst_dataset_destroy(self.h) };
    }
}
