/*
 * rstorch_b200.h — C ABI of the B200 (sm_100a) training-step library.
 *
 * The library re-implements, on one or more B200 GPUs, the f64 training step of
 * the `rstorch` crate: Sequential forward/backward through Linear and ReLU, the
 * CrossEntropyLoss softmax-cross-entropy forward/backward, SGD::step and the
 * batch assembly that feeds them.  The reference crate has no FFI of its own
 * (it is pure Rust over ndarray), so each entry point below names the Rust
 * function of the reference that a façade crate would route through it
 * (paths are relative to the reference repository root).
 *
 * Conventions
 *   - every tensor is a dense row-major matrix of f64 (the reference's
 *     `Array2<f64>`, src/module/mod.rs:42-49), addressed by an opaque handle;
 *   - every call returns an `rst_status`; 0 is success.  The reference panics
 *     where this library returns an error (missing cache `unwrap()`,
 *     src/module/linear.rs:61; shape mismatch inside `dot`); a façade maps a
 *     non-zero status back to `panic!`;
 *   - compute entry points are asynchronous on the context's compute stream;
 *     the calls that hand a value to the host (`rst_tensor_download`,
 *     `rst_xent_result`, `rst_accuracy`, `rst_argmax`, `rst_timer_elapsed_ms`)
 *     block until it is ready;
 *   - one context per GPU, used from one host thread at a time;
 *   - there is no CPU fall-back anywhere: without a CUDA device every compute
 *     entry point fails with RST_ERR_CUDA.
 */
#ifndef RSTORCH_B200_H
#define RSTORCH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct rst_ctx rst_ctx;         /* one GPU: streams, allocator, result ring   */
typedef struct rst_tensor rst_tensor;   /* device matrix (rows, cols), f64, row-major */
typedef struct rst_sgd_plan rst_sgd_plan; /* pointer table of one parameter set        */
typedef struct rst_stager rst_stager;   /* pinned-host batch ring + copy stream       */
typedef struct rst_comm rst_comm;       /* NCCL communicator bound to a context       */
typedef struct rst_graph rst_graph;     /* captured CUDA graph of a step              */
typedef struct rst_timer rst_timer;     /* pair of CUDA events on the compute stream  */

typedef enum rst_status {
    RST_OK = 0,
    RST_ERR_INVALID_ARG = 1,    /* null pointer, negative size, bad flag             */
    RST_ERR_SHAPE = 2,          /* operand shapes do not agree (ndarray would panic) */
    RST_ERR_FOREIGN_HANDLE = 3, /* handle belongs to another context or is stale     */
    RST_ERR_OOM = 4,            /* device allocation failed or the set limit is hit  */
    RST_ERR_CUDA = 5,           /* a CUDA runtime/driver call failed                 */
    RST_ERR_NCCL = 6,           /* NCCL missing or a collective failed               */
    RST_ERR_DEVICE_TIMEOUT = 7, /* a bounded device-side wait gave up                */
    RST_ERR_NAN = 8,            /* NaN logit: the reference panics in softmax `max`  */
    RST_ERR_UNSUPPORTED = 9,    /* size beyond a documented maximum                  */
    RST_ERR_STATE = 10          /* call out of order (e.g. result slot never written)*/
} rst_status;

/* ---- library ------------------------------------------------------------ */
int rst_version(void);                       /* (major<<16)|(minor<<8)|patch */
const char* rst_status_string(int status);
/* Message of the last failing call made through `ctx` (or through a handle it
 * owns).  With ctx == NULL: the last failure of a call that had no context. */
const char* rst_last_error(const rst_ctx* ctx);

/* ---- context ------------------------------------------------------------ */
/* Creates the per-GPU state every other call needs: compute, copy and
 * communication streams, the caching allocator that stands in for the
 * reference's implicit `Array2` allocations (src/module/linear.rs:44,63,66,68;
 * src/module/activation/relu.rs:20; src/optim/sgd.rs:23), and a ring of pinned
 * result slots for the loss/accuracy read-back. */
int rst_ctx_create(int device, rst_ctx** out);
int rst_ctx_destroy(rst_ctx* ctx);
int rst_ctx_synchronize(rst_ctx* ctx);
int rst_ctx_device(const rst_ctx* ctx, int* device);
/* Raw `cudaStream_t` of the compute stream (for callers that time or order
 * their own work against it). */
int rst_ctx_stream(const rst_ctx* ctx, void** stream);
/* Reads and clears the device-side status word written by kernels whose
 * bounded waits ran out; returns RST_ERR_DEVICE_TIMEOUT if it was set. */
int rst_ctx_check_device(rst_ctx* ctx);
/* Self-test of that path (no counterpart in the reference).  Launches one small GEMM whose
 * producer copies nothing, so every consumer wait runs out after `limit_cycles` SM cycles
 * (1..1e8); the kernel sets the status word, stores nothing and returns with no copy in
 * flight.  The call itself succeeds; the next rst_ctx_check_device returns
 * RST_ERR_DEVICE_TIMEOUT and clears the word, after which the context works as before. */
int rst_selftest_wait_expiry(rst_ctx* ctx, int64_t limit_cycles);
/* Number of kernels this library has launched through `ctx` so far. */
int rst_ctx_launch_count(const rst_ctx* ctx, uint64_t* count);

/* Caching allocator controls.  stats[0..5] = bytes in use, bytes reserved from
 * the driver, peak bytes in use, allocation requests, requests served from the
 * cache, driver allocations. */
int rst_ctx_memory_stats(const rst_ctx* ctx, uint64_t stats[6]);
int rst_ctx_set_memory_limit(rst_ctx* ctx, uint64_t max_reserved_bytes); /* 0 = none */
int rst_ctx_empty_cache(rst_ctx* ctx);

/* ---- tensors -------------------------------------------------------------
 * Stand-ins for `Array2<f64>` values that live in HBM.  A façade converts with
 * upload/download at the edges of the step (`Array2::as_standard_layout` on
 * the way in). */
int rst_tensor_alloc(rst_ctx* ctx, int64_t rows, int64_t cols, rst_tensor** out);
/* Non-owning window of `numel = rows*cols` elements starting `elem_offset`
 * elements into `parent` (used to carve parameters and gradients out of one
 * arena so that SGD and the gradient all-reduce see contiguous memory). */
int rst_tensor_slice(rst_tensor* parent, int64_t elem_offset, int64_t rows, int64_t cols,
                     rst_tensor** out);
int rst_tensor_free(rst_tensor* t);
int rst_tensor_shape(const rst_tensor* t, int64_t* rows, int64_t* cols);
int rst_tensor_data(const rst_tensor* t, void** device_ptr);
int rst_tensor_upload(rst_tensor* t, const double* host);     /* blocking */
int rst_tensor_download(const rst_tensor* t, double* host);   /* blocking */
int rst_tensor_copy(rst_tensor* dst, const rst_tensor* src);  /* device to device */
int rst_tensor_fill(rst_tensor* t, double value);
/* 64-bit digest of the tensor's bit patterns in element order, computed on the device
 * (no counterpart in the reference; blocking).  Equal digests mean bit-identical tensors up
 * to a 2^-64 collision chance: the ranks of a data-parallel run compare the digests of
 * their weights instead of moving the weights through the host. */
int rst_tensor_checksum(const rst_tensor* t, uint64_t* digest);

/* ---- Linear (src/module/linear.rs:41-79) ---------------------------------
 * forward:  Y[B,out] = X[B,in] · W[out,in]ᵀ + b[1,out]   (linear.rs:44-53);
 *           with relu != 0 the following ReLU::forward (relu.rs:21) is applied
 *           in the same kernel: Y = max(Y, 0).  b may be NULL (bias-less).
 * backward: n = rows(X);  dW[out,in] = dYᵀ·X / n  (linear.rs:62-63);
 *           db[1,out] = Σ_rows dY / n              (linear.rs:65-67);
 *           dX[B,in]  = dY · W, unscaled            (linear.rs:68).
 *           If relu_mask_src is given (shape of dX) the ReLU::backward of the
 *           layer in front (relu.rs:26) is fused in: dX *= (relu_mask_src > 0).
 *           The post-ReLU output of that layer (= this layer's cached X) is a
 *           valid mask source because max(x,0) > 0 ⇔ x > 0.
 *           db and dX may be NULL to skip them (dX of the first layer is
 *           discarded by the reference's training loop, README.md:72).
 */
int rst_linear_forward(rst_ctx* ctx, const rst_tensor* X, const rst_tensor* W,
                       const rst_tensor* b, int relu, rst_tensor* Y);
int rst_linear_backward(rst_ctx* ctx, const rst_tensor* dY, const rst_tensor* X,
                        const rst_tensor* W, const rst_tensor* relu_mask_src,
                        rst_tensor* dW, rst_tensor* db, rst_tensor* dX);

/* `Sequential::backward` (src/module/sequential.rs:88-94) over a run of n Linear
 * layers, listed in forward order, with nothing or a ReLU between consecutive ones.
 * Layer l maps its cached input X[l] (B, in_l) through W[l] (out_l, in_l); dY is the
 * gradient at the last layer's output.  From l = n-1 down to 0, with g = dY for the
 * last layer and g = dX[l+1] otherwise, the call computes exactly what n calls of
 * rst_linear_backward would:
 *   dX[l] = g · W[l], times (X[l] > 0) where relu_mask[l] != 0 (the ReLU in front of
 *           layer l, whose output X[l] is);  dW[l] = gᵀ·X[l] / B;  db[l] = Σ_rows g / B.
 * dX[0] may be NULL (the gradient of the network input is not needed); relu_mask and
 * db may be NULL (no masks / no bias gradients).  The dX products depend on one
 * another and run first; the dW/db products of layers too small to fill the GPU one
 * at a time then share one launch.  Meant for chains of small layers: every dX[l]
 * stays alive until the call's work has run. */
int rst_linear_backward_chain(rst_ctx* ctx, int n, const rst_tensor* dY, const rst_tensor* const* X,
                              const rst_tensor* const* W, const unsigned char* relu_mask,
                              rst_tensor* const* dW, rst_tensor* const* db, rst_tensor* const* dX);

/* rst_linear_backward for a caller that keeps a transposed companion of each gradient
 * (no counterpart in the reference; a layout optimisation).  dX = dY · W runs fastest
 * when both operands are stored with the reduction index outermost: W (out, in) is;
 * dY (B, out) is not, but dY_t (out, B) is.  dY_t may be NULL (then this is
 * rst_linear_backward).  dX_t (in, B), if given, receives dXᵀ, written by the same
 * kernel as dX where the shapes allow and by a transpose kernel otherwise, so that the
 * layer below can be called the same way.  rst_transpose makes the first companion
 * (of the loss gradient): dst (cols, rows) = srcᵀ. */
int rst_linear_backward_t(rst_ctx* ctx, const rst_tensor* dY, const rst_tensor* dY_t,
                          const rst_tensor* X, const rst_tensor* W, const rst_tensor* relu_mask_src,
                          rst_tensor* dW, rst_tensor* db, rst_tensor* dX, rst_tensor* dX_t);
int rst_transpose(rst_ctx* ctx, const rst_tensor* src, rst_tensor* dst);

/* Bias gradient without any allocation: db[c] = (Σ_r dY[r,c]) / rows, the same
 * value rst_linear_backward writes to db.  This entry point has no counterpart in
 * the reference.  It is for hosts that may not call cudaMalloc at the point where
 * they need the result: a serving process or framework whose own allocator has
 * claimed the whole device and hands this library raw pointers only (a cudaMalloc
 * from a second party would fail there, or eat into a budget it does not own), and
 * a step function with a hard latency bound (cudaMalloc and cudaFree can
 * synchronise the whole device, and the regular path grows its column-sum scratch
 * from the driver whenever a wider layer comes along).
 *   - dY and db are raw device pointers of the GPU that is current on the calling
 *     thread; `stream` is a cudaStream_t of that GPU (NULL = default stream).
 *   - No context, no tensor handles, no cudaMalloc/cudaFree and no allocating
 *     library call: the partial column sums go to a fixed 2 MiB array inside the
 *     library's device image, which every GPU that loads the library holds until
 *     the process exits.
 *   - cols may be at most RST_BIAS_GRAD_NOALLOC_MAX_COLS; larger requests fail
 *     with RST_ERR_UNSUPPORTED and a message naming the limit.
 *   - The first call on each device looks up the array's device address (once per
 *     device, with that device current); let that first call come before any
 *     stream capture.
 *   - All calls share the one array and it keeps the previous call's contents
 *     (the kernels overwrite every entry they later read, so nothing needs
 *     clearing).  Two calls whose kernels overlap on the GPU (different streams)
 *     race on it: order them on one stream or with events. */
#define RST_BIAS_GRAD_NOALLOC_MAX_COLS 262144
int rst_bias_grad_noalloc(const double* dY, int64_t rows, int64_t cols, double* db, void* stream);

/* ---- ReLU, unfused (src/module/activation/relu.rs:17-32) ----------------- */
int rst_relu_forward(rst_ctx* ctx, const rst_tensor* X, rst_tensor* Y);
/* dX = dY * (X_pre > 0 ? 1 : 0); X_pre is the tensor ReLU::forward cached. */
int rst_relu_backward(rst_ctx* ctx, const rst_tensor* dY, const rst_tensor* X_pre,
                      rst_tensor* dX);

/* ---- softmax free function (src/module/activation/softmax.rs:36-53) ------ */
int rst_softmax(rst_ctx* ctx, const rst_tensor* X, rst_tensor* P);

/* ---- Softmax module (src/module/activation/softmax.rs:5-34, 55-78) ---------
 * Forward over axis 1 is rst_softmax; rst_softmax_axis0 normalises every column
 * (Softmax::with_axis(0)).  rst_softmax_backward reproduces the reference's
 * backward as written: jacobian = -(outputᵀ·output) taken over the whole batch,
 * diagonal replaced by s(1-s) with s = Σ_b output[b][j]² (softmax.rs:66-70),
 * dX = gradient · jacobian (softmax.rs:72).  `output` is what forward returned. */
int rst_softmax_axis0(rst_ctx* ctx, const rst_tensor* X, rst_tensor* P);
int rst_softmax_backward(rst_ctx* ctx, const rst_tensor* output, const rst_tensor* gradient,
                         rst_tensor* dX);

/* ---- CrossEntropyLoss (src/loss/cross_entropy.rs:32-48) + accuracy --------
 * One pass over the rows computes
 *   p = softmax(logits, axis 1)                      (cross_entropy.rs:37)
 *   loss = -(Σ_ij truth_ij · ln p_ij) / B            (cross_entropy.rs:38)
 *   dlogits = p - truth, no 1/B                      (cross_entropy.rs:45-47)
 *   correct = #{rows: argmax(logits) == argmax(truth)}, first maximum wins
 *                                                    (src/utils.rs:44-65)
 * and queues the three scalars into pinned result slot `slot`
 * (0 <= slot < rst_xent_slots()).  dlogits may be NULL (loss only).
 * rst_xent_result blocks until the slot is written and returns the loss and
 * the accuracy (= correct / B).  It returns RST_ERR_NAN if a logit was NaN,
 * the case in which the reference's softmax panics (softmax.rs:38). */
int rst_xent_slots(void);
int rst_xent_forward_backward(rst_ctx* ctx, const rst_tensor* logits, const rst_tensor* truth,
                              rst_tensor* dlogits, int slot);
int rst_xent_result(rst_ctx* ctx, int slot, double* loss, double* accuracy);

/* Stand-alone `accuracy(pred, truth)` and row-wise `argmax` (src/utils.rs:44-65);
 * blocking.  `idx` receives `rows` indices. */
int rst_accuracy(rst_ctx* ctx, const rst_tensor* pred, const rst_tensor* truth, double* acc);
int rst_argmax(rst_ctx* ctx, const rst_tensor* t, int64_t* idx);

/* ---- SGD::step (src/optim/sgd.rs:18-25) -----------------------------------
 * For every (param, grad) pair: param = param - (lr · grad), product rounded
 * then difference rounded exactly as the reference's two ndarray operations do.
 * A plan holds the device-side table of one parameter set so that a step is a
 * single kernel launch whatever the number of tensors. */
int rst_sgd_plan_create(rst_ctx* ctx, int n, rst_tensor* const* params,
                        rst_tensor* const* grads, rst_sgd_plan** out);
int rst_sgd_plan_step(rst_sgd_plan* plan, double lr);
int rst_sgd_plan_destroy(rst_sgd_plan* plan);
/* Convenience: builds (and caches on the context) the plan for this exact list. */
int rst_sgd_step(rst_ctx* ctx, int n, rst_tensor* const* params, rst_tensor* const* grads,
                 double lr);

/* ---- batch staging (src/data/data_loader.rs:180-208) ----------------------
 * `ArrayDataLoaderIter::next` appends `batch` samples into two fresh arrays.
 * Here the loader writes the samples straight into a pinned host slot
 * (rst_stager_host), rst_stager_submit starts the host→device copies on the
 * copy stream, and rst_stager_acquire makes the compute stream wait for them
 * and hands out the device tensors of that slot.  A slot may be rewritten once
 * work that reads its device tensors has been queued and a later submit of
 * the same slot is ordered after it (the library inserts that dependency). */
int rst_stager_create(rst_ctx* ctx, int64_t batch, int64_t x_cols, int64_t t_cols, int slots,
                      rst_stager** out);
int rst_stager_destroy(rst_stager* s);
int rst_stager_host(rst_stager* s, int slot, double** x_host, double** t_host);
int rst_stager_submit(rst_stager* s, int slot);
int rst_stager_acquire(rst_stager* s, int slot, rst_tensor** X, rst_tensor** T);

/* ---- device-resident dataset and fused batch transform ------------------------
 * The u8 samples and labels of a dataset (the reference's MNIST item type,
 * src/data/dataset/hub/mnist.rs:181-194) are placed in HBM once.
 * rst_dataset_gather builds the batch of the given sample indices in one kernel:
 * per sample `flatten(normalize_zero_one(x))` (src/utils.rs:5-18, 30-35: min-max
 * to [0,1] by the sample's own min and max, 0/0 = NaN for a constant sample) into
 * row b of X (batch, features), and `one_hot(y, classes)` (src/utils.rs:38-42)
 * into row b of T (batch, classes) -- the transform of README.md:44 applied by
 * `ArrayDataLoaderIter::next` (src/data/data_loader.rs:192-207).  `indices` is a
 * host array (sampler order, shuffled or not); an index outside the dataset is
 * rejected, as is a label >= classes at creation (the reference panics on it). */
typedef struct rst_dataset rst_dataset;
int rst_dataset_create_u8(rst_ctx* ctx, const unsigned char* images, const unsigned char* labels,
                          int64_t n, int64_t features, int64_t classes, rst_dataset** out);
int rst_dataset_destroy(rst_dataset* d);
int rst_dataset_len(const rst_dataset* d, int64_t* n);
int rst_dataset_gather(rst_dataset* d, const int64_t* indices, int64_t batch, rst_tensor* X,
                       rst_tensor* T);
/* The same batch transform for a step that is replayed as a CUDA graph.
 * rst_dataset_index_stage hands out a pinned host buffer of at least `batch` indices
 * that belongs to the dataset (the same buffer on every call until a larger batch is
 * asked for; ask for it before capturing).  rst_dataset_gather_staged queues the copy
 * of its first `batch` entries to the device and the gather kernel; it reads no index
 * on the host, so it may be captured, and every replay gathers whatever the buffer
 * holds at that time.  The caller writes the next batch's indices only after the
 * previous replay has consumed them (e.g. after rst_xent_result of that step).  The
 * kernel checks the indices itself: a row whose index is outside the dataset is
 * filled with NaN, and the next rst_ctx_check_device returns RST_ERR_INVALID_ARG. */
int rst_dataset_index_stage(rst_dataset* d, int64_t batch, int64_t** host_indices);
int rst_dataset_gather_staged(rst_dataset* d, int64_t batch, rst_tensor* X, rst_tensor* T);
/* Shuffling on the device (`Shuffler::new` / `Shuffler::shuffle`,
 * src/data/dataset/shuffler.rs:15-25, called by `DataLoader::iter_array` before every
 * epoch, src/data/data_loader.rs:88-92).  The reference shuffles 0..len with an unseedable
 * thread generator; rst_dataset_shuffle draws the epoch's order from `seed` with a kernel:
 * position i maps to sample perm(i), a keyed bijection of [0, len) (four-round Feistel
 * network over the smallest even bit width covering len, cycle-walked below len; round
 * function splitmix64(seed + round·φ64 + right half)).  rst_dataset_gather_epoch builds the
 * batch of epoch positions [first, first + batch) (`Shuffler::get`, shuffler.rs:31-33) with
 * the same transform as rst_dataset_gather; positions beyond the dataset are rejected.
 * rst_dataset_epoch_order downloads the current order (len entries; blocking). */
int rst_dataset_shuffle(rst_dataset* d, uint64_t seed);
int rst_dataset_gather_epoch(rst_dataset* d, int64_t first, int64_t batch, rst_tensor* X, rst_tensor* T);
int rst_dataset_epoch_order(rst_dataset* d, int64_t* host_out);

/* ---- data-parallel gradient exchange (no counterpart in the reference, which
 * is single-threaded; required to shard the batch over the GPUs of one box) --
 * One rank per process/GPU.  Rank 0 obtains an id, the caller ships the
 * RST_COMM_ID_BYTES bytes to the other ranks by any means, every rank calls
 * rst_comm_create.  rst_allreduce_avg averages each tensor over the ranks
 * (with equal shards, the average of the per-rank dW = dYᵀX/(B/G) is the
 * full-batch dW = dYᵀX/B of linear.rs:63).  It runs on the communication
 * stream, ordered after the compute work queued so far; rst_comm_join makes
 * the compute stream wait for all exchanges queued so far. */
#define RST_COMM_ID_BYTES 128
int rst_comm_get_id(void* id_bytes);
int rst_comm_create(rst_ctx* ctx, const void* id_bytes, int rank, int world, rst_comm** out);
int rst_comm_destroy(rst_comm* comm);
int rst_allreduce_avg(rst_comm* comm, int n, rst_tensor* const* tensors);
int rst_comm_join(rst_comm* comm);
/* Optional: exchange shares instead of averages.  With `on`, rst_linear_backward (and the
 * chain and companion variants) on the communicator's context divide dW and db by
 * rows(X)·world, so that every rank holds its share of the global-batch gradient
 * dYᵀX / B, and rst_allreduce_avg adds the shares up with a plain sum, which NCCL may hand to
 * the NVSwitch's in-network reduction (an average cannot go there: every rank's input would
 * have to be scaled first).  After the exchange the tensors hold the same average as
 * without the option: bit for bit when world is a power of two, to the last place otherwise.
 * Between backward and exchange they hold 1/world of what linear.rs:63,66 computes. */
int rst_comm_share_gradients(rst_comm* comm, int on);

/* ---- whole-step replay (no counterpart in the reference) ----------------------
 * Captures everything queued on the compute stream between begin and end into
 * a CUDA graph (configs whose step is a dozen short kernels are launch-bound).
 * Calls that block are not allowed in between, and nothing is allocated from the
 * driver while recording: rst_tensor_alloc is served from the allocator's cache
 * or fails with RST_ERR_STATE, so run the same step once, unrecorded, directly
 * before every capture.  Every block the recorded kernels address (allocated or
 * freed between begin and end) belongs to the graph from rst_graph_capture_end
 * on: it stays out of the allocator, also after its tensor handle is freed,
 * until rst_graph_destroy, so no later tensor is handed memory that a replay
 * overwrites.  Tensors made before the capture (weights, inputs) must outlive
 * the graph. */
int rst_graph_capture_begin(rst_ctx* ctx);
int rst_graph_capture_end(rst_ctx* ctx, rst_graph** out);
int rst_graph_launch(rst_graph* g);
int rst_graph_destroy(rst_graph* g);

/* ---- synthetic input streams (host only; no counterpart in the reference,
 * whose initialiser draws from an unseedable thread generator,
 * src/module/init/he.rs:13) -------------------------------------------------
 * Word i of stream `key` is splitmix64(key + i·φ64); any slice of a stream can
 * be produced independently.  rst_synth_uniform writes n values of U[0,1)
 * starting at element `offset`; rst_synth_normal writes N(mean, stddev) by
 * Box-Muller (element i uses words 2i and 2i+1). */
int rst_synth_uniform(uint64_t key, uint64_t n, uint64_t offset, double* out);
int rst_synth_normal(uint64_t key, uint64_t n, uint64_t offset, double mean, double stddev,
                     double* out);

/* ---- timing and roofline probes ------------------------------------------- */
int rst_timer_create(rst_ctx* ctx, rst_timer** out);
int rst_timer_start(rst_timer* t);   /* records on the compute stream */
int rst_timer_stop(rst_timer* t);
int rst_timer_elapsed_ms(rst_timer* t, double* ms);  /* blocking */
int rst_timer_destroy(rst_timer* t);
/* Per-kernel-class device time.  Between begin and end every launch group of
 * the library (gemm_fwd, gemm_dW, gemm_dX, colsum, xent, sgd, relu_fwd, relu_bwd)
 * is bracketed by CUDA events on the compute stream; end blocks and writes
 * lines "name launches milliseconds" into `report`.  The extra events perturb
 * short kernels, so timed benchmark regions run with profiling off. */
int rst_profile_begin(rst_ctx* ctx);
int rst_profile_end(rst_ctx* ctx, char* report, size_t capacity);
/* Register-resident issue-rate probe of the f64 tensor instruction the GEMM
 * kernels use (kind 0: mma.sync m16n8k8 f64, 1: m8n8k4, 2: m16n8k16,
 * 3: plain DFMA); returns TFLOP/s over the whole GPU.  This is the measured
 * denominator of the GEMM roofline. */
int rst_probe_fp64_peak(rst_ctx* ctx, int kind, int iters, double* tflops);
/* Device-to-device streaming copy of `bytes` (read + write counted), GB/s. */
int rst_probe_hbm_copy(rst_ctx* ctx, uint64_t bytes, int iters, double* gbs);
/* Writes `bytes` of a scratch buffer (pass > L2 size to flush L2 between timed
 * iterations). */
int rst_flush_l2(rst_ctx* ctx, uint64_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* RSTORCH_B200_H */
