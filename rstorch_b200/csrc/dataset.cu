// Device-resident u8 dataset and the fused per-batch transform.
//
// The reference's training loop builds a batch on the CPU by calling, for each
// of `batch_size` sampler indices, `dataset.get(index)` (one 28x28 u8 image and
// its u8 label, src/data/dataset/hub/mnist.rs:181-194), the user transform
// `(flatten(normalize_zero_one(x)), one_hot(y, 10))` (README.md:44;
// src/utils.rs:5-18, 30-42) and `append` onto the batch arrays
// (src/data/data_loader.rs:192-207).  Here the raw u8 samples live in HBM and one
// kernel gathers the rows of a batch, normalises each sample to [0,1] with its own
// min and max, and writes the f64 batch and the one-hot targets:
//   x = (f64(v) - f64(min)) / (f64(max) - f64(min))      (utils.rs:13-17; 0/0 = NaN
//                                                          for a constant sample)
//   t = 1.0 at column `label`, 0.0 elsewhere              (utils.rs:38-42)
// Per sample the kernel reads F bytes and writes 8*(F + classes) bytes.
#include "common.h"

using namespace rst;

namespace {

constexpr int kGatherThreads = 256;
constexpr int kIndexSlots = 4;

__global__ void __launch_bounds__(kGatherThreads)
gather_normalize_onehot_kernel(const unsigned char* __restrict__ images, const unsigned char* __restrict__ labels,
                               const long long* __restrict__ indices, long long batch, int features, int classes,
                               double* __restrict__ X, double* __restrict__ T, long long n_samples,
                               int* __restrict__ status) {
    __shared__ double value_table[kGatherThreads / 32][256];       // per warp: the normalised value of every u8
    grid_dependency_release();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const long long warp_global = (long long)blockIdx.x * (kGatherThreads / 32) + (threadIdx.x >> 5);
    const long long warp_stride = (long long)gridDim.x * (kGatherThreads / 32);
    for (long long b = warp_global; b < batch; b += warp_stride) {
        const long long idx = indices[b];
        if (idx < 0 || idx >= n_samples) {
            // Indices of a replayed graph cannot be checked on the host: flag the batch row,
            // make it unmistakable, touch nothing outside the dataset.
            if (lane == 0) {
                atomicExch(status, kDevBadIndex);
                atomicExch(status + 1, (int)b);
            }
            for (int e = lane; e < features; e += 32) X[b * features + e] = __longlong_as_double(0x7ff8000000000000LL);
            for (int c = lane; c < classes; c += 32) T[b * classes + c] = 0.0;
            continue;
        }
        const unsigned char* src = images + idx * features;
        // pass 1: min and max of the sample by the ordering of u8 (utils.rs:11-12); four values
        // per load where the row allows it
        unsigned int lo = 255u, hi = 0u;
        const bool words = (features % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 3u) == 0);
        if (words) {
            const unsigned int* src4 = reinterpret_cast<const unsigned int*>(src);
            for (int w = lane; w < features / 4; w += 32) {
                const unsigned int q = src4[w];
                const unsigned int b0 = q & 0xffu, b1 = (q >> 8) & 0xffu, b2 = (q >> 16) & 0xffu, b3 = q >> 24;
                lo = min(min(lo, min(b0, b1)), min(b2, b3));
                hi = max(max(hi, max(b0, b1)), max(b2, b3));
            }
        } else {
            for (int e = lane; e < features; e += 32) {
                const unsigned int v = src[e];
                lo = min(lo, v);
                hi = max(hi, v);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        const double dmin = (double)lo;
        const double range = (double)hi - dmin;                     // max - min in f64 (utils.rs:14)
        // A sample holds at most 256 distinct values, so its `(f64(v) - min) / (max - min)` are
        // computed once per value (the same subtraction and the same correctly rounded division
        // as per element) and the elements are looked up: 256 divisions a sample instead of one
        // per element, which is what bounded this kernel.
        double* table = value_table[threadIdx.x >> 5];
        __syncwarp();                                               // the previous sample's look-ups are done
#pragma unroll
        for (int j = 0; j < 8; ++j) table[lane + 32 * j] = ((double)(lane + 32 * j) - dmin) / range;
        __syncwarp();
        // pass 2: normalise; lanes write consecutive doubles
        double* dst = X + b * features;
        if (words && ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0)) {
            const unsigned int* src4 = reinterpret_cast<const unsigned int*>(src);
            for (int w = lane; w < features / 4; w += 32) {
                const unsigned int q = src4[w];
                double v[4] = {table[q & 0xffu], table[(q >> 8) & 0xffu], table[(q >> 16) & 0xffu], table[q >> 24]};
                asm volatile("st.global.v4.f64 [%0], {%1,%2,%3,%4};" ::"l"(dst + 4 * w), "d"(v[0]), "d"(v[1]), "d"(v[2]),
                             "d"(v[3]) : "memory");
            }
        } else {
            for (int e = lane; e < features; e += 32) dst[e] = table[src[e]];
        }
        const int label = labels[idx];
        double* trow = T + b * classes;
        for (int c = lane; c < classes; c += 32) trow[c] = (c == label) ? 1.0 : 0.0;
    }
}

// Epoch permutation drawn on the device (Shuffler::new / Shuffler::shuffle,
// src/data/dataset/shuffler.rs:15-25, which shuffle 0..len with an unseedable thread
// generator).  Here position i of the epoch maps to sample perm(i), where perm is a keyed
// bijection of [0, n): a four-round Feistel network over the smallest even number of bits
// that covers n, walked until the value falls below n (cycle walking keeps it a bijection).
// Every position is computed independently, so no sort and no host round trip is needed,
// and a host mirror of these few lines reproduces it bit for bit.
__host__ __device__ __forceinline__ unsigned long long perm_mix(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__host__ __device__ __forceinline__ long long epoch_permute(unsigned long long seed, int half_bits,
                                                            unsigned long long n, unsigned long long i) {
    const unsigned long long mask = (1ull << half_bits) - 1ull;
    unsigned long long v = i;
    do {
        unsigned long long l = v >> half_bits, r = v & mask;
#pragma unroll
        for (int round = 0; round < 4; ++round) {
            const unsigned long long f = perm_mix(seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(round + 1) + r) & mask;
            const unsigned long long nl = r;
            r = l ^ f;
            l = nl;
        }
        v = (l << half_bits) | r;
    } while (v >= n);
    return (long long)v;
}

__global__ void __launch_bounds__(kGatherThreads)
epoch_permutation_kernel(unsigned long long seed, int half_bits, long long n, long long* __restrict__ perm) {
    grid_dependency_release();
    grid_dependency_wait();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        perm[i] = epoch_permute(seed, half_bits, (unsigned long long)n, (unsigned long long)i);
}

int feistel_half_bits(long long n) {
    int bits = 2;
    while (bits < 62 && (1ll << bits) < n) bits += 2;
    return bits / 2;
}

}  // namespace

struct rst_dataset {
    rst_ctx* ctx;
    long long n;
    int features, classes;
    unsigned char* d_images;
    unsigned char* d_labels;
    long long* h_idx[kIndexSlots];       // pinned
    long long* d_idx[kIndexSlots];
    cudaEvent_t idx_free[kIndexSlots];   // the gather that read the slot has finished
    long long idx_cap;
    int next_slot;
    bool slot_used[kIndexSlots];
    // one more pair of index buffers that the caller fills itself (rst_dataset_index_stage)
    long long* h_stage;
    long long* d_stage;
    long long stage_cap;
    // the current epoch's order of the samples (rst_dataset_shuffle); identity until then
    long long* d_perm;
    bool shuffled;
};

extern "C" int rst_dataset_destroy(rst_dataset* d);

extern "C" int rst_dataset_create_u8(rst_ctx* c, const unsigned char* images, const unsigned char* labels,
                                     int64_t n, int64_t features, int64_t classes, rst_dataset** out) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!out || !images || !labels || n <= 0 || features <= 0 || classes <= 0 || classes > 256 ||
        features > 0x7fffffff)
        return fail(c, RST_ERR_INVALID_ARG, "bad dataset arguments");
    *out = nullptr;
    if (c->capturing) return fail(c, RST_ERR_STATE, "dataset creation during graph capture");
    // one_hot(label, classes) panics in the reference for label >= classes (utils.rs:40)
    for (int64_t i = 0; i < n; ++i)
        if (labels[i] >= classes)
            return fail(c, RST_ERR_INVALID_ARG, "label %d of sample %lld is outside [0,%lld)", (int)labels[i],
                        (long long)i, (long long)classes);
    rst_dataset* d = new rst_dataset();
    d->ctx = c; d->n = n; d->features = (int)features; d->classes = (int)classes;
    d->d_images = nullptr; d->d_labels = nullptr; d->idx_cap = 0; d->next_slot = 0;
    d->h_stage = nullptr; d->d_stage = nullptr; d->stage_cap = 0;
    d->d_perm = nullptr; d->shuffled = false;
    for (int s = 0; s < kIndexSlots; ++s) { d->h_idx[s] = nullptr; d->d_idx[s] = nullptr; d->idx_free[s] = nullptr; d->slot_used[s] = false; }
    bool okay = cudaMalloc((void**)&d->d_images, (size_t)n * features) == cudaSuccess &&
                cudaMalloc((void**)&d->d_labels, (size_t)n) == cudaSuccess &&
                cudaMemcpy(d->d_images, images, (size_t)n * features, cudaMemcpyHostToDevice) == cudaSuccess &&
                cudaMemcpy(d->d_labels, labels, (size_t)n, cudaMemcpyHostToDevice) == cudaSuccess;
    for (int s = 0; okay && s < kIndexSlots; ++s)
        okay = cudaEventCreateWithFlags(&d->idx_free[s], cudaEventDisableTiming) == cudaSuccess;
    if (!okay) {
        cudaGetLastError();
        rst_dataset_destroy(d);
        return fail(c, RST_ERR_OOM, "cannot place the dataset (%lld x %lld bytes) on the device", (long long)n,
                    (long long)features);
    }
    *out = d;
    return RST_OK;
}

extern "C" int rst_dataset_destroy(rst_dataset* d) {
    if (!d) return RST_OK;
    if (valid(d->ctx)) cudaStreamSynchronize(d->ctx->compute);
    if (d->d_images) cudaFree(d->d_images);
    if (d->d_labels) cudaFree(d->d_labels);
    for (int s = 0; s < kIndexSlots; ++s) {
        if (d->h_idx[s]) cudaFreeHost(d->h_idx[s]);
        if (d->d_idx[s]) cudaFree(d->d_idx[s]);
        if (d->idx_free[s]) cudaEventDestroy(d->idx_free[s]);
    }
    if (d->h_stage) cudaFreeHost(d->h_stage);
    if (d->d_stage) cudaFree(d->d_stage);
    if (d->d_perm) cudaFree(d->d_perm);
    cudaGetLastError();
    delete d;
    return RST_OK;
}

namespace {

int check_batch_tensors(rst_dataset* d, int64_t batch, rst_tensor* X, rst_tensor* T) {
    rst_ctx* c = d->ctx;
    RST_TRY(check_tensor(c, X, "X"));
    RST_TRY(check_tensor(c, T, "T"));
    if (batch <= 0) return fail(c, RST_ERR_INVALID_ARG, "empty batch");
    if (X->rows != batch || X->cols != d->features || T->rows != batch || T->cols != d->classes)
        return fail(c, RST_ERR_SHAPE, "gather of %lld samples into X (%lld,%lld), T (%lld,%lld); dataset has %d features, %d classes",
                    (long long)batch, (long long)X->rows, (long long)X->cols, (long long)T->rows, (long long)T->cols,
                    d->features, d->classes);
    return RST_OK;
}

int launch_gather(rst_dataset* d, const long long* d_indices, int64_t batch, rst_tensor* X, rst_tensor* T) {
    rst_ctx* c = d->ctx;
    ProfScope prof(c, "gather");
    long long blocks = (batch + kGatherThreads / 32 - 1) / (kGatherThreads / 32);
    long long cap = (long long)c->num_sms * 8;
    if (blocks > cap) blocks = cap;
    launch_step_kernel(c, c->compute, gather_normalize_onehot_kernel, dim3((unsigned)blocks), dim3(kGatherThreads), 0,
                       d->d_images, d->d_labels, d_indices, (long long)batch, d->features, d->classes, X->data,
                       T->data, d->n, c->d_status);
    return after_launch(c, "gather_normalize_onehot_kernel");
}

}  // namespace

extern "C" int rst_dataset_len(const rst_dataset* d, int64_t* n) {
    if (!d || !n) return fail(nullptr, RST_ERR_INVALID_ARG, "bad argument");
    *n = d->n;
    return RST_OK;
}

extern "C" int rst_dataset_gather(rst_dataset* d, const int64_t* indices, int64_t batch, rst_tensor* X,
                                  rst_tensor* T) {
    if (!d || !valid(d->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad dataset");
    rst_ctx* c = d->ctx;
    if (!indices) return fail(c, RST_ERR_INVALID_ARG, "empty batch");
    RST_TRY(check_batch_tensors(d, batch, X, T));
    if (c->capturing) return fail(c, RST_ERR_STATE, "gather during graph capture");
    // `dataset.get(index)?` ends the reference's epoch on a missing sample (data_loader.rs:197)
    for (int64_t i = 0; i < batch; ++i)
        if (indices[i] < 0 || indices[i] >= d->n)
            return fail(c, RST_ERR_INVALID_ARG, "index %lld outside the dataset of %lld samples", (long long)indices[i],
                        (long long)d->n);
    if (batch > d->idx_cap) {
        RST_CUDA(c, cudaStreamSynchronize(c->compute));
        for (int s = 0; s < kIndexSlots; ++s) {
            if (d->h_idx[s]) cudaFreeHost(d->h_idx[s]);
            if (d->d_idx[s]) cudaFree(d->d_idx[s]);
            d->h_idx[s] = nullptr; d->d_idx[s] = nullptr; d->slot_used[s] = false;
            if (cudaMallocHost((void**)&d->h_idx[s], (size_t)batch * sizeof(long long)) != cudaSuccess ||
                cudaMalloc((void**)&d->d_idx[s], (size_t)batch * sizeof(long long)) != cudaSuccess) {
                cudaGetLastError();
                d->idx_cap = 0;
                return fail(c, RST_ERR_OOM, "cannot allocate index staging for %lld samples", (long long)batch);
            }
        }
        d->idx_cap = batch;
    }
    const int s = d->next_slot;
    d->next_slot = (s + 1) % kIndexSlots;
    if (d->slot_used[s]) RST_CUDA(c, cudaEventSynchronize(d->idx_free[s]));   // its previous gather has run
    for (int64_t i = 0; i < batch; ++i) d->h_idx[s][i] = indices[i];
    RST_CUDA(c, cudaMemcpyAsync(d->d_idx[s], d->h_idx[s], (size_t)batch * sizeof(long long), cudaMemcpyHostToDevice,
                                c->compute));
    RST_TRY(launch_gather(d, d->d_idx[s], batch, X, T));
    RST_CUDA(c, cudaEventRecord(d->idx_free[s], c->compute));
    d->slot_used[s] = true;
    return RST_OK;
}

// The caller-filled variant: the indices live in a pinned buffer that belongs to the dataset
// and that the caller writes directly.  Nothing here looks at their values on the host, so
// the copy and the kernel can be captured into a CUDA graph and replayed with other
// indices in the buffer; the kernel checks every index against the dataset size itself.
extern "C" int rst_dataset_index_stage(rst_dataset* d, int64_t batch, int64_t** host_indices) {
    if (!d || !valid(d->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad dataset");
    rst_ctx* c = d->ctx;
    if (batch <= 0 || !host_indices) return fail(c, RST_ERR_INVALID_ARG, "bad index stage arguments");
    if (batch > d->stage_cap) {
        if (c->capturing) return fail(c, RST_ERR_STATE, "the index stage cannot grow during graph capture");
        RST_CUDA(c, cudaStreamSynchronize(c->compute));
        if (d->h_stage) cudaFreeHost(d->h_stage);
        if (d->d_stage) cudaFree(d->d_stage);
        d->h_stage = nullptr; d->d_stage = nullptr; d->stage_cap = 0;
        if (cudaMallocHost((void**)&d->h_stage, (size_t)batch * sizeof(long long)) != cudaSuccess ||
            cudaMalloc((void**)&d->d_stage, (size_t)batch * sizeof(long long)) != cudaSuccess) {
            cudaGetLastError();
            return fail(c, RST_ERR_OOM, "cannot allocate the index stage for %lld samples", (long long)batch);
        }
        d->stage_cap = batch;
    }
    *host_indices = reinterpret_cast<int64_t*>(d->h_stage);
    return RST_OK;
}

extern "C" int rst_dataset_gather_staged(rst_dataset* d, int64_t batch, rst_tensor* X, rst_tensor* T) {
    if (!d || !valid(d->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad dataset");
    rst_ctx* c = d->ctx;
    RST_TRY(check_batch_tensors(d, batch, X, T));
    if (batch > d->stage_cap)
        return fail(c, RST_ERR_STATE, "gather of %lld staged indices, but the index stage holds %lld",
                    (long long)batch, (long long)d->stage_cap);
    RST_CUDA(c, cudaMemcpyAsync(d->d_stage, d->h_stage, (size_t)batch * sizeof(long long), cudaMemcpyHostToDevice,
                                c->compute));
    return launch_gather(d, d->d_stage, batch, X, T);
}

// ---- seeded epoch order on the device ------------------------------------------------
// rst_dataset_shuffle draws the order of the next epoch (Shuffler::shuffle, called by
// DataLoader::iter_array before every epoch, src/data/data_loader.rs:88-92);
// rst_dataset_gather_epoch builds the batch of epoch positions [first, first + batch),
// i.e. of samples perm[first .. first + batch), what ArrayDataLoaderIter::next does through
// Shuffler::get (shuffler.rs:31-33).  No sample index crosses the host bus.
extern "C" int rst_dataset_shuffle(rst_dataset* d, uint64_t seed) {
    if (!d || !valid(d->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad dataset");
    rst_ctx* c = d->ctx;
    if (!d->d_perm) {
        if (c->capturing) return fail(c, RST_ERR_STATE, "the first shuffle allocates; call it before capturing");
        if (cudaMalloc((void**)&d->d_perm, (size_t)d->n * sizeof(long long)) != cudaSuccess) {
            cudaGetLastError();
            return fail(c, RST_ERR_OOM, "cannot allocate the epoch order of %lld samples", d->n);
        }
    }
    long long blocks = (d->n + kGatherThreads - 1) / kGatherThreads;
    const long long cap = (long long)c->num_sms * 8;
    if (blocks > cap) blocks = cap;
    launch_step_kernel(c, c->compute, epoch_permutation_kernel, dim3((unsigned)blocks), dim3(kGatherThreads), 0,
                       (unsigned long long)seed, feistel_half_bits(d->n), d->n, d->d_perm);
    RST_TRY(after_launch(c, "epoch_permutation_kernel"));
    d->shuffled = true;
    return RST_OK;
}

extern "C" int rst_dataset_epoch_order(rst_dataset* d, int64_t* host_out) {
    if (!d || !valid(d->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad dataset");
    rst_ctx* c = d->ctx;
    if (!host_out) return fail(c, RST_ERR_INVALID_ARG, "host_out is NULL");
    if (c->capturing) return fail(c, RST_ERR_STATE, "blocking call during graph capture");
    if (!d->shuffled) {
        for (long long i = 0; i < d->n; ++i) host_out[i] = i;       // never shuffled: sampler order
        return RST_OK;
    }
    RST_CUDA(c, cudaMemcpyAsync(host_out, d->d_perm, (size_t)d->n * sizeof(long long), cudaMemcpyDeviceToHost,
                                c->compute));
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    return RST_OK;
}

extern "C" int rst_dataset_gather_epoch(rst_dataset* d, int64_t first, int64_t batch, rst_tensor* X, rst_tensor* T) {
    if (!d || !valid(d->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad dataset");
    rst_ctx* c = d->ctx;
    RST_TRY(check_batch_tensors(d, batch, X, T));
    if (!d->shuffled) return fail(c, RST_ERR_STATE, "rst_dataset_gather_epoch before rst_dataset_shuffle");
    // `dataset.get(index)?` ends the reference's epoch on a missing sample (data_loader.rs:197)
    if (first < 0 || first + batch > d->n)
        return fail(c, RST_ERR_INVALID_ARG, "epoch positions [%lld, %lld) outside the dataset of %lld samples",
                    (long long)first, (long long)(first + batch), d->n);
    return launch_gather(d, d->d_perm + first, batch, X, T);
}
