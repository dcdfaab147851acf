//! Raw bindings of `include/rstorch_b200.h`, one declaration per entry point, in the
//! header's order.  A unit test of the Python package compares the names and argument
//! counts in this file with the header, so the two cannot drift apart unnoticed.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_double, c_int, c_uchar, c_void};

macro_rules! opaque {
    ($($name:ident),*) => { $(#[repr(C)] pub struct $name { _private: [u8; 0] })* };
}
opaque!(rst_ctx, rst_tensor, rst_sgd_plan, rst_stager, rst_comm, rst_graph, rst_timer, rst_dataset);

pub const RST_OK: c_int = 0;
pub const RST_ERR_INVALID_ARG: c_int = 1;
pub const RST_ERR_SHAPE: c_int = 2;
pub const RST_ERR_FOREIGN_HANDLE: c_int = 3;
pub const RST_ERR_OOM: c_int = 4;
pub const RST_ERR_CUDA: c_int = 5;
pub const RST_ERR_NCCL: c_int = 6;
pub const RST_ERR_DEVICE_TIMEOUT: c_int = 7;
pub const RST_ERR_NAN: c_int = 8;
pub const RST_ERR_UNSUPPORTED: c_int = 9;
pub const RST_ERR_STATE: c_int = 10;

pub const RST_BIAS_GRAD_NOALLOC_MAX_COLS: i64 = 262144;
pub const RST_COMM_ID_BYTES: usize = 128;

extern "C" {
    // library
    pub fn rst_version() -> c_int;
    pub fn rst_status_string(status: c_int) -> *const c_char;
    pub fn rst_last_error(ctx: *const rst_ctx) -> *const c_char;

    // context
    pub fn rst_ctx_create(device: c_int, out: *mut *mut rst_ctx) -> c_int;
    pub fn rst_ctx_destroy(ctx: *mut rst_ctx) -> c_int;
    pub fn rst_ctx_synchronize(ctx: *mut rst_ctx) -> c_int;
    pub fn rst_ctx_device(ctx: *const rst_ctx, device: *mut c_int) -> c_int;
    pub fn rst_ctx_stream(ctx: *const rst_ctx, stream: *mut *mut c_void) -> c_int;
    pub fn rst_ctx_check_device(ctx: *mut rst_ctx) -> c_int;
    pub fn rst_selftest_wait_expiry(ctx: *mut rst_ctx, limit_cycles: i64) -> c_int;
    pub fn rst_ctx_launch_count(ctx: *const rst_ctx, count: *mut u64) -> c_int;
    pub fn rst_ctx_memory_stats(ctx: *const rst_ctx, stats: *mut u64) -> c_int;
    pub fn rst_ctx_set_memory_limit(ctx: *mut rst_ctx, max_reserved_bytes: u64) -> c_int;
    pub fn rst_ctx_empty_cache(ctx: *mut rst_ctx) -> c_int;

    // tensors
    pub fn rst_tensor_alloc(ctx: *mut rst_ctx, rows: i64, cols: i64, out: *mut *mut rst_tensor) -> c_int;
    pub fn rst_tensor_slice(parent: *mut rst_tensor, elem_offset: i64, rows: i64, cols: i64,
                            out: *mut *mut rst_tensor) -> c_int;
    pub fn rst_tensor_free(t: *mut rst_tensor) -> c_int;
    pub fn rst_tensor_shape(t: *const rst_tensor, rows: *mut i64, cols: *mut i64) -> c_int;
    pub fn rst_tensor_data(t: *const rst_tensor, device_ptr: *mut *mut c_void) -> c_int;
    pub fn rst_tensor_upload(t: *mut rst_tensor, host: *const c_double) -> c_int;
    pub fn rst_tensor_download(t: *const rst_tensor, host: *mut c_double) -> c_int;
    pub fn rst_tensor_copy(dst: *mut rst_tensor, src: *const rst_tensor) -> c_int;
    pub fn rst_tensor_fill(t: *mut rst_tensor, value: c_double) -> c_int;
    pub fn rst_tensor_checksum(t: *const rst_tensor, digest: *mut u64) -> c_int;

    // Linear
    pub fn rst_linear_forward(ctx: *mut rst_ctx, x: *const rst_tensor, w: *const rst_tensor,
                              b: *const rst_tensor, relu: c_int, y: *mut rst_tensor) -> c_int;
    pub fn rst_linear_backward(ctx: *mut rst_ctx, dy: *const rst_tensor, x: *const rst_tensor,
                               w: *const rst_tensor, relu_mask_src: *const rst_tensor,
                               dw: *mut rst_tensor, db: *mut rst_tensor, dx: *mut rst_tensor) -> c_int;
    pub fn rst_linear_backward_chain(ctx: *mut rst_ctx, n: c_int, dy: *const rst_tensor,
                                     x: *const *const rst_tensor, w: *const *const rst_tensor,
                                     relu_mask: *const c_uchar, dw: *const *mut rst_tensor,
                                     db: *const *mut rst_tensor, dx: *const *mut rst_tensor) -> c_int;
    pub fn rst_linear_backward_t(ctx: *mut rst_ctx, dy: *const rst_tensor, dy_t: *const rst_tensor,
                                 x: *const rst_tensor, w: *const rst_tensor, relu_mask_src: *const rst_tensor,
                                 dw: *mut rst_tensor, db: *mut rst_tensor, dx: *mut rst_tensor,
                                 dx_t: *mut rst_tensor) -> c_int;
    pub fn rst_transpose(ctx: *mut rst_ctx, src: *const rst_tensor, dst: *mut rst_tensor) -> c_int;
    pub fn rst_bias_grad_noalloc(dy: *const c_double, rows: i64, cols: i64, db: *mut c_double,
                                 stream: *mut c_void) -> c_int;

    // ReLU, softmax
    pub fn rst_relu_forward(ctx: *mut rst_ctx, x: *const rst_tensor, y: *mut rst_tensor) -> c_int;
    pub fn rst_relu_backward(ctx: *mut rst_ctx, dy: *const rst_tensor, x_pre: *const rst_tensor,
                             dx: *mut rst_tensor) -> c_int;
    pub fn rst_softmax(ctx: *mut rst_ctx, x: *const rst_tensor, p: *mut rst_tensor) -> c_int;
    pub fn rst_softmax_axis0(ctx: *mut rst_ctx, x: *const rst_tensor, p: *mut rst_tensor) -> c_int;
    pub fn rst_softmax_backward(ctx: *mut rst_ctx, output: *const rst_tensor, gradient: *const rst_tensor,
                                dx: *mut rst_tensor) -> c_int;

    // CrossEntropyLoss, accuracy
    pub fn rst_xent_slots() -> c_int;
    pub fn rst_xent_forward_backward(ctx: *mut rst_ctx, logits: *const rst_tensor, truth: *const rst_tensor,
                                     dlogits: *mut rst_tensor, slot: c_int) -> c_int;
    pub fn rst_xent_result(ctx: *mut rst_ctx, slot: c_int, loss: *mut c_double, accuracy: *mut c_double) -> c_int;
    pub fn rst_accuracy(ctx: *mut rst_ctx, pred: *const rst_tensor, truth: *const rst_tensor,
                        acc: *mut c_double) -> c_int;
    pub fn rst_argmax(ctx: *mut rst_ctx, t: *const rst_tensor, idx: *mut i64) -> c_int;

    // SGD
    pub fn rst_sgd_plan_create(ctx: *mut rst_ctx, n: c_int, params: *const *mut rst_tensor,
                               grads: *const *mut rst_tensor, out: *mut *mut rst_sgd_plan) -> c_int;
    pub fn rst_sgd_plan_step(plan: *mut rst_sgd_plan, lr: c_double) -> c_int;
    pub fn rst_sgd_plan_destroy(plan: *mut rst_sgd_plan) -> c_int;
    pub fn rst_sgd_step(ctx: *mut rst_ctx, n: c_int, params: *const *mut rst_tensor,
                        grads: *const *mut rst_tensor, lr: c_double) -> c_int;

    // batch staging
    pub fn rst_stager_create(ctx: *mut rst_ctx, batch: i64, x_cols: i64, t_cols: i64, slots: c_int,
                             out: *mut *mut rst_stager) -> c_int;
    pub fn rst_stager_destroy(s: *mut rst_stager) -> c_int;
    pub fn rst_stager_host(s: *mut rst_stager, slot: c_int, x_host: *mut *mut c_double,
                           t_host: *mut *mut c_double) -> c_int;
    pub fn rst_stager_submit(s: *mut rst_stager, slot: c_int) -> c_int;
    pub fn rst_stager_acquire(s: *mut rst_stager, slot: c_int, x: *mut *mut rst_tensor,
                              t: *mut *mut rst_tensor) -> c_int;

    // device-resident dataset
    pub fn rst_dataset_create_u8(ctx: *mut rst_ctx, images: *const c_uchar, labels: *const c_uchar, n: i64,
                                 features: i64, classes: i64, out: *mut *mut rst_dataset) -> c_int;
    pub fn rst_dataset_destroy(d: *mut rst_dataset) -> c_int;
    pub fn rst_dataset_len(d: *const rst_dataset, n: *mut i64) -> c_int;
    pub fn rst_dataset_gather(d: *mut rst_dataset, indices: *const i64, batch: i64, x: *mut rst_tensor,
                              t: *mut rst_tensor) -> c_int;

    pub fn rst_dataset_index_stage(d: *mut rst_dataset, batch: i64, host_indices: *mut *mut i64) -> c_int;
    pub fn rst_dataset_gather_staged(d: *mut rst_dataset, batch: i64, x: *mut rst_tensor,
                                     t: *mut rst_tensor) -> c_int;
    pub fn rst_dataset_shuffle(d: *mut rst_dataset, seed: u64) -> c_int;
    pub fn rst_dataset_gather_epoch(d: *mut rst_dataset, first: i64, batch: i64, x: *mut rst_tensor,
                                    t: *mut rst_tensor) -> c_int;
    pub fn rst_dataset_epoch_order(d: *mut rst_dataset, host_out: *mut i64) -> c_int;

    // data-parallel gradient exchange
    pub fn rst_comm_get_id(id_bytes: *mut c_void) -> c_int;
    pub fn rst_comm_create(ctx: *mut rst_ctx, id_bytes: *const c_void, rank: c_int, world: c_int,
                           out: *mut *mut rst_comm) -> c_int;
    pub fn rst_comm_destroy(comm: *mut rst_comm) -> c_int;
    pub fn rst_allreduce_avg(comm: *mut rst_comm, n: c_int, tensors: *const *mut rst_tensor) -> c_int;
    pub fn rst_comm_join(comm: *mut rst_comm) -> c_int;
    pub fn rst_comm_share_gradients(comm: *mut rst_comm, on: c_int) -> c_int;

    // whole-step replay
    pub fn rst_graph_capture_begin(ctx: *mut rst_ctx) -> c_int;
    pub fn rst_graph_capture_end(ctx: *mut rst_ctx, out: *mut *mut rst_graph) -> c_int;
    pub fn rst_graph_launch(g: *mut rst_graph) -> c_int;
    pub fn rst_graph_destroy(g: *mut rst_graph) -> c_int;

    // synthetic input streams
    pub fn rst_synth_uniform(key: u64, n: u64, offset: u64, out: *mut c_double) -> c_int;
    pub fn rst_synth_normal(key: u64, n: u64, offset: u64, mean: c_double, stddev: c_double,
                            out: *mut c_double) -> c_int;

    // timing and probes
    pub fn rst_timer_create(ctx: *mut rst_ctx, out: *mut *mut rst_timer) -> c_int;
    pub fn rst_timer_start(t: *mut rst_timer) -> c_int;
    pub fn rst_timer_stop(t: *mut rst_timer) -> c_int;
    pub fn rst_timer_elapsed_ms(t: *mut rst_timer, ms: *mut c_double) -> c_int;
    pub fn rst_timer_destroy(t: *mut rst_timer) -> c_int;
    pub fn rst_profile_begin(ctx: *mut rst_ctx) -> c_int;
    pub fn rst_profile_end(ctx: *mut rst_ctx, report: *mut c_char, capacity: usize) -> c_int;
    pub fn rst_probe_fp64_peak(ctx: *mut rst_ctx, kind: c_int, iters: c_int, tflops: *mut c_double) -> c_int;
    pub fn rst_probe_hbm_copy(ctx: *mut rst_ctx, bytes: u64, iters: c_int, gbs: *mut c_double) -> c_int;
    pub fn rst_flush_l2(ctx: *mut rst_ctx, bytes: u64) -> c_int;
}

/// Turns a non-zero status into a panic carrying the library's message: the reference
/// panics in the same situations (a missing cache `unwrap()`, src/module/linear.rs:61; a
/// shape mismatch inside `dot`; a NaN logit, src/module/activation/softmax.rs:38).
#[track_caller]
pub fn check(ctx: *const rst_ctx, status: c_int) {
    if status != RST_OK {
        let msg = unsafe {
            let p = rst_last_error(ctx);
            if p.is_null() { String::new() } else { std::ffi::CStr::from_ptr(p).to_string_lossy().into_owned() }
        };
        panic!("rstorch_b200 status {status}: {msg}");
    }
}
