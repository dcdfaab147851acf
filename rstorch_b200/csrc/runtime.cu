// Host runtime: context, caching allocator, device tensors, timers, graph capture.
#include <cudaTypedefs.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cstring>

#include "common.h"

namespace rst {

static thread_local std::string g_noctx_error;

int fail(const rst_ctx* ctx, int status, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx && ctx->magic == kCtxMagic)
        const_cast<rst_ctx*>(ctx)->last_error = buf;
    else
        g_noctx_error = buf;
    return status;
}

bool valid(const rst_ctx* ctx) { return ctx && ctx->magic == kCtxMagic; }
bool valid(const rst_tensor* t) { return t && t->magic == kTensorMagic && valid(t->ctx); }

int check_tensor(const rst_ctx* ctx, const rst_tensor* t, const char* name) {
    if (!t) return fail(ctx, RST_ERR_INVALID_ARG, "%s is NULL", name);
    if (t->magic != kTensorMagic)
        return fail(ctx, RST_ERR_FOREIGN_HANDLE, "%s is not a live tensor handle", name);
    if (t->ctx != ctx)
        return fail(ctx, RST_ERR_FOREIGN_HANDLE, "%s belongs to another context", name);
    return RST_OK;
}

int after_launch(rst_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(ctx, RST_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return RST_OK;
}

int ensure_scratch(rst_ctx* ctx, void** buf, size_t* cap, size_t need, const char* what) {
    if (*cap >= need) return RST_OK;
    if (ctx->capturing)
        return fail(ctx, RST_ERR_STATE,
                    "%s scratch must grow to %zu bytes during graph capture; run the step once "
                    "before capturing", what, need);
    // Work queued earlier may still read the old buffer.
    RST_CUDA(ctx, cudaStreamSynchronize(ctx->compute));
    if (*buf) RST_CUDA(ctx, cudaFree(*buf));
    *buf = nullptr;
    *cap = 0;
    size_t grown = std::max(need, (size_t)1 << 20);
    cudaError_t e = cudaMalloc(buf, grown);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, RST_ERR_OOM, "cannot allocate %zu bytes of %s scratch: %s", grown, what,
                    cudaGetErrorString(e));
    }
    *cap = grown;
    return RST_OK;
}

// ------------------------------ profiling scopes -----------------------------
static cudaEvent_t prof_event(rst_ctx* ctx) {
    if (!ctx->prof_event_pool.empty()) {
        cudaEvent_t e = ctx->prof_event_pool.back();
        ctx->prof_event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

// Every launch group also opens an NVTX range named after its kernel class (gemm_fwd,
// gemm_dW, gemm_dX, colsum, xent, sgd, ...), so a timeline tool shows the step's phases.
// Without a tool attached the NVTX calls are no-ops of a few nanoseconds.
ProfScope::ProfScope(rst_ctx* ctx, const char* name) : ctx_(ctx), index_(-1) {
    nvtxRangePushA(name);
    if (!ctx->profiling || ctx->capturing) return;
    rst_ctx::ProfRecord r{name, prof_event(ctx), prof_event(ctx)};
    if (!r.start || !r.stop) return;
    cudaEventRecord(r.start, ctx->compute);
    index_ = (int)ctx->prof_records.size();
    ctx->prof_records.push_back(r);
}

ProfScope::~ProfScope() {
    if (index_ >= 0) cudaEventRecord(ctx_->prof_records[(size_t)index_].stop, ctx_->compute);
    nvtxRangePop();
}

// ------------------------------ allocator -----------------------------------
size_t CachingAllocator::bucket_size(size_t bytes) {
    if (bytes == 0) bytes = 1;
    const size_t kSmall = (size_t)1 << 20;
    if (bytes <= 4096) return (bytes + 511) & ~(size_t)511;
    if (bytes <= kSmall) {
        // quarter-octave steps: 1, 1.25, 1.5, 1.75 × 2^k
        size_t p = 4096;
        while ((p << 1) < bytes) p <<= 1;   // p < bytes <= 2p
        size_t step = p >> 2;
        return ((bytes + step - 1) / step) * step;
    }
    const size_t g = (size_t)2 << 20;
    return ((bytes + g - 1) / g) * g;
}

void* CachingAllocator::allocate(size_t bytes, size_t* granted, int* err, bool may_call_driver) {
    size_t want = bucket_size(bytes);
    requests++;
    auto it = free_.lower_bound(want);
    // exact bucket, or (for large blocks) one that wastes at most 1/8
    if (it != free_.end() && (it->first == want || (want >= ((size_t)1 << 20) && it->first <= want + want / 8))) {
        void* p = it->second;
        *granted = it->first;
        free_.erase(it);
        hits++;
        in_use += *granted;
        peak = std::max(peak, in_use);
        if (recording_) recorded_[p] = *granted;
        return p;
    }
    if (!may_call_driver) { *err = -2; return nullptr; }
    if (limit_ && reserved + want > limit_) {
        empty_cache();
        if (reserved + want > limit_) { *err = -1; return nullptr; }
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        empty_cache();
        e = cudaMalloc(&p, want);
        if (e != cudaSuccess) { cudaGetLastError(); *err = (int)e; return nullptr; }
    }
    driver_allocs++;
    reserved += want;
    in_use += want;
    peak = std::max(peak, in_use);
    *granted = want;
    return p;
}

void CachingAllocator::release(void* ptr, size_t granted) {
    if (!ptr) return;
    in_use -= granted;
    free_.emplace(granted, ptr);
    // recorded kernels may read or write a block that is handed back while recording
    if (recording_) recorded_[ptr] = granted;
}

void CachingAllocator::begin_recording() {
    recording_ = true;
    recorded_.clear();
}

void CachingAllocator::end_recording(std::vector<std::pair<void*, size_t>>* cached, std::vector<void*>* live) {
    recording_ = false;
    for (const auto& rec : recorded_) {
        bool in_cache = false;
        auto range = free_.equal_range(rec.second);
        for (auto it = range.first; it != range.second; ++it)
            if (it->second == rec.first) {
                free_.erase(it);
                in_cache = true;
                break;
            }
        if (in_cache) {
            if (cached) cached->emplace_back(rec.first, rec.second);
            else free_.emplace(rec.second, rec.first);        // capture failed: nothing pins it
        } else if (live) {
            live->push_back(rec.first);
        }
    }
    recorded_.clear();
}

void CachingAllocator::empty_cache() {
    for (auto& kv : free_) {
        cudaFree(kv.second);
        reserved -= kv.first;
    }
    free_.clear();
}

}  // namespace rst

using namespace rst;

// ------------------------------ library --------------------------------------
extern "C" int rst_version(void) { return (0 << 16) | (1 << 8) | 0; }

extern "C" const char* rst_status_string(int s) {
    switch (s) {
        case RST_OK: return "ok";
        case RST_ERR_INVALID_ARG: return "invalid argument";
        case RST_ERR_SHAPE: return "shape mismatch";
        case RST_ERR_FOREIGN_HANDLE: return "foreign or stale handle";
        case RST_ERR_OOM: return "out of device memory";
        case RST_ERR_CUDA: return "CUDA error";
        case RST_ERR_NCCL: return "NCCL error";
        case RST_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
        case RST_ERR_NAN: return "NaN in logits";
        case RST_ERR_UNSUPPORTED: return "unsupported size";
        case RST_ERR_STATE: return "call out of order";
        default: return "unknown status";
    }
}

extern "C" const char* rst_last_error(const rst_ctx* ctx) {
    if (valid(ctx)) return ctx->last_error.c_str();
    return g_noctx_error.c_str();
}

// ------------------------------ context ---------------------------------------
extern "C" int rst_ctx_create(int device, rst_ctx** out) {
    if (!out) return fail(nullptr, RST_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(nullptr, RST_ERR_CUDA,
                    "no CUDA device is available (%s); this library has no CPU path",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    if (device < 0 || device >= count)
        return fail(nullptr, RST_ERR_INVALID_ARG, "device %d out of range [0,%d)", device, count);
    RST_CUDA(nullptr, cudaSetDevice(device));
    cudaDeviceProp prop;
    RST_CUDA(nullptr, cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(nullptr, RST_ERR_CUDA,
                    "device %d is sm_%d%d; the kernels of this library are built for sm_100a only",
                    device, prop.major, prop.minor);

    rst_ctx* c = new rst_ctx();
    c->magic = kCtxMagic;
    c->device = device;
    c->num_sms = prop.multiProcessorCount > 0 ? prop.multiProcessorCount : kNumSMsFallback;
    c->launches = 0;
    c->capturing = false;
    {
        // RSTORCH_B200_OVERLAP_LAUNCHES=0 restores fully serialised launches (for A/B timing)
        const char* v = std::getenv("RSTORCH_B200_OVERLAP_LAUNCHES");
        c->overlap_launches = !(v && v[0] == '0');
    }
    {
        // RSTORCH_B200_STREAM_TAIL=0: every CTA of a large GEMM computes whole tiles (for A/B timing)
        const char* v = std::getenv("RSTORCH_B200_STREAM_TAIL");
        c->stream_tail = !(v && v[0] == '0');
    }
    c->grad_rows_scale = 1.0;
    c->profiling = false;
    c->xent_partials = nullptr; c->xent_partials_cap = 0; c->xent_counter = nullptr;
    c->splitk_ws = nullptr; c->splitk_ws_bytes = 0;
    c->colsum_ws = nullptr; c->colsum_ws_bytes = 0;
    c->flush_buf = nullptr; c->flush_bytes = 0;
    c->encode_tiled = nullptr;
    c->d_status = nullptr; c->h_status = nullptr; c->d_results = nullptr; c->h_results = nullptr;
    c->compute = c->copy = c->comm = nullptr;
    for (int i = 0; i < kXentSlots; ++i) { c->result_event[i] = nullptr; c->result_pending[i] = false; c->result_in_graph[i] = false; }

#define CTX_CUDA(call)                                                                   \
    do {                                                                                 \
        cudaError_t e__ = (call);                                                        \
        if (e__ != cudaSuccess) {                                                        \
            int s__ = fail(nullptr, RST_ERR_CUDA, "%s failed: %s", #call,                \
                           cudaGetErrorString(e__));                                     \
            rst_ctx_destroy(c);                                                          \
            return s__;                                                                  \
        }                                                                                \
    } while (0)

    CTX_CUDA(cudaStreamCreateWithFlags(&c->compute, cudaStreamNonBlocking));
    {
        // The collective's few CTAs must get an SM as soon as one frees up, ahead of the
        // thousands of queued CTAs of the GEMM it overlaps with: highest stream priority.
        int least = 0, greatest = 0;
        CTX_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        CTX_CUDA(cudaStreamCreateWithPriority(&c->comm, cudaStreamNonBlocking, greatest));
        CTX_CUDA(cudaStreamCreateWithPriority(&c->copy, cudaStreamNonBlocking, greatest));
    }
    // words 0-3: device status; words 4-5: the 64-bit accumulator of rst_tensor_checksum
    CTX_CUDA(cudaMalloc((void**)&c->d_status, 8 * sizeof(int)));
    CTX_CUDA(cudaMemset(c->d_status, 0, 8 * sizeof(int)));
    CTX_CUDA(cudaMallocHost((void**)&c->h_status, 4 * sizeof(int)));
    CTX_CUDA(cudaMalloc((void**)&c->d_results, kXentSlots * sizeof(ResultSlot)));
    CTX_CUDA(cudaMemset(c->d_results, 0, kXentSlots * sizeof(ResultSlot)));
    CTX_CUDA(cudaMallocHost((void**)&c->h_results, kXentSlots * sizeof(ResultSlot)));
    CTX_CUDA(cudaMalloc((void**)&c->xent_counter, 4 * sizeof(unsigned int)));
    CTX_CUDA(cudaMemset(c->xent_counter, 0, 4 * sizeof(unsigned int)));
    for (int i = 0; i < kXentSlots; ++i)
        CTX_CUDA(cudaEventCreateWithFlags(&c->result_event[i], cudaEventDisableTiming));

    cudaDriverEntryPointQueryResult qres;
    void* fn = nullptr;
    CTX_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || !fn) {
        int s = fail(nullptr, RST_ERR_CUDA, "driver does not export cuTensorMapEncodeTiled");
        rst_ctx_destroy(c);
        return s;
    }
    c->encode_tiled = fn;
#undef CTX_CUDA
    *out = c;
    return RST_OK;
}

extern "C" int rst_sgd_plan_destroy(rst_sgd_plan* plan);

extern "C" int rst_ctx_destroy(rst_ctx* c) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (auto& kv : c->plan_cache) rst_sgd_plan_destroy(kv.second);
    c->plan_cache.clear();
    c->alloc.empty_cache();
    for (int i = 0; i < kXentSlots; ++i)
        if (c->result_event[i]) cudaEventDestroy(c->result_event[i]);
    for (auto& r : c->prof_records) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
    for (cudaEvent_t e : c->prof_event_pool) cudaEventDestroy(e);
    if (c->d_status) cudaFree(c->d_status);
    if (c->h_status) cudaFreeHost(c->h_status);
    if (c->d_results) cudaFree(c->d_results);
    if (c->h_results) cudaFreeHost(c->h_results);
    if (c->xent_counter) cudaFree(c->xent_counter);
    if (c->xent_partials) cudaFree(c->xent_partials);
    if (c->splitk_ws) cudaFree(c->splitk_ws);
    if (c->colsum_ws) cudaFree(c->colsum_ws);
    if (c->flush_buf) cudaFree(c->flush_buf);
    if (c->compute) cudaStreamDestroy(c->compute);
    if (c->copy) cudaStreamDestroy(c->copy);
    if (c->comm) cudaStreamDestroy(c->comm);
    cudaGetLastError();
    c->magic = kDeadMagic;
    delete c;
    return RST_OK;
}

extern "C" int rst_ctx_synchronize(rst_ctx* c) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    RST_CUDA(c, cudaStreamSynchronize(c->copy));
    RST_CUDA(c, cudaStreamSynchronize(c->comm));
    return RST_OK;
}

extern "C" int rst_ctx_device(const rst_ctx* c, int* device) {
    if (!valid(c) || !device) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    *device = c->device;
    return RST_OK;
}

extern "C" int rst_ctx_stream(const rst_ctx* c, void** stream) {
    if (!valid(c) || !stream) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    *stream = (void*)c->compute;
    return RST_OK;
}

extern "C" int rst_ctx_check_device(rst_ctx* c) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    RST_CUDA(c, cudaMemcpyAsync(c->h_status, c->d_status, 4 * sizeof(int), cudaMemcpyDeviceToHost,
                                c->compute));
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    if (c->h_status[0] != kDevOk) {
        int code = c->h_status[0], where = c->h_status[1];
        RST_CUDA(c, cudaMemsetAsync(c->d_status, 0, 4 * sizeof(int), c->compute));
        // a kernel that gave up may have left the election counter half-counted
        RST_CUDA(c, cudaMemsetAsync(c->xent_counter, 0, 4 * sizeof(unsigned int), c->compute));
        if (code == kDevBadIndex)
            return fail(c, RST_ERR_INVALID_ARG,
                        "a staged gather read a sample index outside the dataset (batch row %d); that row "
                        "of the batch is NaN", where);
        return fail(c, RST_ERR_DEVICE_TIMEOUT,
                    "a kernel gave up a bounded wait (code %d, site %d); its output is invalid",
                    code, where);
    }
    return RST_OK;
}

extern "C" int rst_ctx_launch_count(const rst_ctx* c, uint64_t* count) {
    if (!valid(c) || !count) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    *count = c->launches;
    return RST_OK;
}

extern "C" int rst_ctx_memory_stats(const rst_ctx* c, uint64_t stats[6]) {
    if (!valid(c) || !stats) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    stats[0] = c->alloc.in_use; stats[1] = c->alloc.reserved; stats[2] = c->alloc.peak;
    stats[3] = c->alloc.requests; stats[4] = c->alloc.hits; stats[5] = c->alloc.driver_allocs;
    return RST_OK;
}

extern "C" int rst_ctx_set_memory_limit(rst_ctx* c, uint64_t max_reserved) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    c->alloc.set_limit(max_reserved);
    return RST_OK;
}

extern "C" int rst_ctx_empty_cache(rst_ctx* c) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    c->alloc.empty_cache();
    return RST_OK;
}

// ------------------------------ tensors ----------------------------------------
static void graph_adopt_block(rst_graph* g, void* ptr, size_t granted);

extern "C" int rst_tensor_alloc(rst_ctx* c, int64_t rows, int64_t cols, rst_tensor** out) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!out) return fail(c, RST_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (rows < 0 || cols < 0) return fail(c, RST_ERR_INVALID_ARG, "negative shape (%lld,%lld)",
                                          (long long)rows, (long long)cols);
    if (cols != 0 && rows > (int64_t)((1ull << 40) / (uint64_t)cols))
        return fail(c, RST_ERR_UNSUPPORTED, "tensor of %lld x %lld elements is too large",
                    (long long)rows, (long long)cols);
    size_t bytes = (size_t)rows * (size_t)cols * sizeof(double);
    size_t granted = 0;
    int err = 0;
    RST_CUDA(c, cudaSetDevice(c->device));
    void* p = c->alloc.allocate(bytes, &granted, &err, !c->capturing);
    if (!p) {
        if (err == -1)
            return fail(c, RST_ERR_OOM, "allocation of %zu bytes exceeds the memory limit", bytes);
        if (err == -2)
            return fail(c, RST_ERR_STATE, "allocation of %zu bytes misses the cache during graph capture "
                        "(no driver allocation is made while recording); run the same step once, "
                        "unrecorded, directly before every capture", bytes);
        return fail(c, RST_ERR_OOM, "cudaMalloc of %zu bytes failed: %s", bytes,
                    cudaGetErrorString((cudaError_t)err));
    }
    rst_tensor* t = new rst_tensor{kTensorMagic, c, (double*)p, rows, cols, granted, true};
    *out = t;
    return RST_OK;
}

extern "C" int rst_tensor_slice(rst_tensor* parent, int64_t off, int64_t rows, int64_t cols,
                                rst_tensor** out) {
    if (!valid(parent)) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "parent is not a live tensor");
    rst_ctx* c = parent->ctx;
    if (!out) return fail(c, RST_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    if (off < 0 || rows < 0 || cols < 0 || off + rows * cols > parent->rows * parent->cols)
        return fail(c, RST_ERR_SHAPE, "slice [%lld, +%lld x %lld) exceeds parent of %lld elements",
                    (long long)off, (long long)rows, (long long)cols,
                    (long long)(parent->rows * parent->cols));
    *out = new rst_tensor{kTensorMagic, c, parent->data + off, rows, cols, 0, false};
    return RST_OK;
}

extern "C" int rst_tensor_free(rst_tensor* t) {
    if (!t) return RST_OK;
    if (!valid(t)) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    if (t->owns) {
        rst_ctx* c = t->ctx;
        auto pin = c->graph_pinned.find(t->data);
        if (pin != c->graph_pinned.end()) {
            // a live graph writes or reads this block on every replay: it goes to the
            // graph, which returns it to the cache when it is destroyed
            graph_adopt_block(pin->second, t->data, t->granted);
            c->graph_pinned.erase(pin);
        } else {
            c->alloc.release(t->data, t->granted);
        }
    }
    t->magic = kDeadMagic;
    delete t;
    return RST_OK;
}

extern "C" int rst_tensor_shape(const rst_tensor* t, int64_t* rows, int64_t* cols) {
    if (!valid(t)) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    if (rows) *rows = t->rows;
    if (cols) *cols = t->cols;
    return RST_OK;
}

extern "C" int rst_tensor_data(const rst_tensor* t, void** p) {
    if (!valid(t) || !p) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    *p = t->data;
    return RST_OK;
}

extern "C" int rst_tensor_upload(rst_tensor* t, const double* host) {
    if (!valid(t)) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    rst_ctx* c = t->ctx;
    if (c->capturing) return fail(c, RST_ERR_STATE, "upload is not allowed during graph capture");
    size_t bytes = (size_t)(t->rows * t->cols) * sizeof(double);
    if (bytes == 0) return RST_OK;
    if (!host) return fail(c, RST_ERR_INVALID_ARG, "host pointer is NULL");
    RST_CUDA(c, cudaMemcpyAsync(t->data, host, bytes, cudaMemcpyHostToDevice, c->compute));
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    return RST_OK;
}

extern "C" int rst_tensor_download(const rst_tensor* t, double* host) {
    if (!valid(t)) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    rst_ctx* c = t->ctx;
    if (c->capturing) return fail(c, RST_ERR_STATE, "download is not allowed during graph capture");
    size_t bytes = (size_t)(t->rows * t->cols) * sizeof(double);
    if (bytes == 0) return RST_OK;
    if (!host) return fail(c, RST_ERR_INVALID_ARG, "host pointer is NULL");
    RST_CUDA(c, cudaMemcpyAsync(host, t->data, bytes, cudaMemcpyDeviceToHost, c->compute));
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    return RST_OK;
}

extern "C" int rst_tensor_copy(rst_tensor* dst, const rst_tensor* src) {
    if (!valid(dst) || !valid(src))
        return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    rst_ctx* c = dst->ctx;
    RST_TRY(check_tensor(c, src, "src"));
    if (dst->rows != src->rows || dst->cols != src->cols)
        return fail(c, RST_ERR_SHAPE, "copy (%lld,%lld) <- (%lld,%lld)", (long long)dst->rows,
                    (long long)dst->cols, (long long)src->rows, (long long)src->cols);
    size_t bytes = (size_t)(dst->rows * dst->cols) * sizeof(double);
    if (bytes)
        RST_CUDA(c, cudaMemcpyAsync(dst->data, src->data, bytes, cudaMemcpyDeviceToDevice,
                                    c->compute));
    return RST_OK;
}

// 64-bit digest of the tensor's bit patterns, computed on the device: two tensors have the
// same digest exactly when (up to a 2^-64 collision chance) they hold the same bits in the
// same order.  Data-parallel replicas compare digests instead of moving weights to the host.
extern "C" int rst_tensor_checksum(const rst_tensor* t, uint64_t* out) {
    if (!valid(t)) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    rst_ctx* c = t->ctx;
    if (!out) return fail(c, RST_ERR_INVALID_ARG, "out is NULL");
    if (c->capturing) return fail(c, RST_ERR_STATE, "blocking call during graph capture");
    unsigned long long* d_word = reinterpret_cast<unsigned long long*>(c->d_status + 4);
    RST_CUDA(c, cudaMemsetAsync(d_word, 0, sizeof(unsigned long long), c->compute));
    RST_TRY(launch_checksum(c, t->data, t->rows * t->cols, d_word));
    unsigned long long host = 0;
    RST_CUDA(c, cudaMemcpyAsync(&host, d_word, sizeof host, cudaMemcpyDeviceToHost, c->compute));
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    *out = host;
    return RST_OK;
}

extern "C" int rst_tensor_fill(rst_tensor* t, double v) {
    if (!valid(t)) return fail(nullptr, RST_ERR_FOREIGN_HANDLE, "not a live tensor handle");
    return launch_fill(t->ctx, t->data, v, t->rows * t->cols);
}

// ------------------------------ timers -------------------------------------------
struct rst_timer {
    rst_ctx* ctx;
    cudaEvent_t start, stop;
};

extern "C" int rst_timer_create(rst_ctx* c, rst_timer** out) {
    if (!valid(c) || !out) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    rst_timer* t = new rst_timer{c, nullptr, nullptr};
    cudaError_t e1 = cudaEventCreate(&t->start), e2 = cudaEventCreate(&t->stop);
    if (e1 != cudaSuccess || e2 != cudaSuccess) {
        delete t;
        return fail(c, RST_ERR_CUDA, "cudaEventCreate failed");
    }
    *out = t;
    return RST_OK;
}
extern "C" int rst_timer_start(rst_timer* t) {
    if (!t || !valid(t->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad timer");
    RST_CUDA(t->ctx, cudaEventRecord(t->start, t->ctx->compute));
    return RST_OK;
}
extern "C" int rst_timer_stop(rst_timer* t) {
    if (!t || !valid(t->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad timer");
    RST_CUDA(t->ctx, cudaEventRecord(t->stop, t->ctx->compute));
    return RST_OK;
}
extern "C" int rst_timer_elapsed_ms(rst_timer* t, double* ms) {
    if (!t || !valid(t->ctx) || !ms) return fail(nullptr, RST_ERR_INVALID_ARG, "bad timer");
    RST_CUDA(t->ctx, cudaEventSynchronize(t->stop));
    float f = 0.f;
    RST_CUDA(t->ctx, cudaEventElapsedTime(&f, t->start, t->stop));
    *ms = f;
    return RST_OK;
}
extern "C" int rst_timer_destroy(rst_timer* t) {
    if (!t) return RST_OK;
    cudaEventDestroy(t->start);
    cudaEventDestroy(t->stop);
    delete t;
    return RST_OK;
}

// ------------------------------ per-class kernel timing -------------------------------
extern "C" int rst_profile_begin(rst_ctx* c) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (c->capturing) return fail(c, RST_ERR_STATE, "profiling during graph capture");
    for (auto& r : c->prof_records) { c->prof_event_pool.push_back(r.start); c->prof_event_pool.push_back(r.stop); }
    c->prof_records.clear();
    c->profiling = true;
    return RST_OK;
}

extern "C" int rst_profile_end(rst_ctx* c, char* report, size_t capacity) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!report || capacity == 0) return fail(c, RST_ERR_INVALID_ARG, "bad report buffer");
    c->profiling = false;
    RST_CUDA(c, cudaStreamSynchronize(c->compute));
    std::map<std::string, std::pair<int, double>> by_name;
    for (auto& r : c->prof_records) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.start, r.stop) == cudaSuccess) {
            auto& slot = by_name[r.name];
            slot.first += 1;
            slot.second += ms;
        }
        c->prof_event_pool.push_back(r.start);
        c->prof_event_pool.push_back(r.stop);
    }
    cudaGetLastError();
    c->prof_records.clear();
    std::string out;
    char line[160];
    for (auto& kv : by_name) {
        snprintf(line, sizeof line, "%s %d %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
        out += line;
    }
    if (out.size() + 1 > capacity) return fail(c, RST_ERR_INVALID_ARG, "report buffer too small");
    std::memcpy(report, out.c_str(), out.size() + 1);
    return RST_OK;
}

// ------------------------------ graph capture --------------------------------------
struct rst_graph {
    rst_ctx* ctx;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    uint64_t launches_per_replay;
    // Blocks the recorded kernels address and no tensor holds any more.  They stay out of
    // the cache while the graph lives, so that no later allocation is handed memory that a
    // replay overwrites.
    std::vector<std::pair<void*, size_t>> blocks;
};

static void graph_adopt_block(rst_graph* g, void* ptr, size_t granted) {
    g->blocks.emplace_back(ptr, granted);      // stays counted as in use until the graph goes
}

static thread_local uint64_t g_capture_launch_base = 0;

extern "C" int rst_graph_capture_begin(rst_ctx* c) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (c->capturing) return fail(c, RST_ERR_STATE, "capture already in progress");
    RST_CUDA(c, cudaStreamBeginCapture(c->compute, cudaStreamCaptureModeRelaxed));
    c->capturing = true;
    c->alloc.begin_recording();
    g_capture_launch_base = c->launches;
    return RST_OK;
}

extern "C" int rst_graph_capture_end(rst_ctx* c, rst_graph** out) {
    if (!valid(c) || !out) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    if (!c->capturing) return fail(c, RST_ERR_STATE, "no capture in progress");
    c->capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(c->compute, &g);
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        c->alloc.end_recording(nullptr, nullptr);
        return fail(c, RST_ERR_CUDA, "cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
    }
    cudaGraphExec_t ex = nullptr;
    e = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        cudaGetLastError();
        c->alloc.end_recording(nullptr, nullptr);
        return fail(c, RST_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    }
    uint64_t per = c->launches - g_capture_launch_base;
    c->launches = g_capture_launch_base;   // captured launches have not run yet
    rst_graph* graph = new rst_graph{c, g, ex, per, {}};
    std::vector<void*> live;
    c->alloc.end_recording(&graph->blocks, &live);
    for (const auto& b : graph->blocks) c->alloc.adopt(b.second);
    for (void* p : live) c->graph_pinned[p] = graph;     // a later graph that records it takes over
    *out = graph;
    return RST_OK;
}

extern "C" int rst_graph_launch(rst_graph* g) {
    if (!g || !valid(g->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad graph");
    RST_CUDA(g->ctx, cudaGraphLaunch(g->exec, g->ctx->compute));
    g->ctx->launches += g->launches_per_replay;
    return RST_OK;
}

extern "C" int rst_graph_destroy(rst_graph* g) {
    if (!g) return RST_OK;
    // Wait for replays in flight, unless the stream is recording another graph (a
    // synchronisation would invalidate that capture; cudaGraphExecDestroy itself defers
    // the release of an executable graph that is still running).
    if (valid(g->ctx) && !g->ctx->capturing) cudaStreamSynchronize(g->ctx->compute);
    cudaGraphExecDestroy(g->exec);
    cudaGraphDestroy(g->graph);
    if (valid(g->ctx)) {
        rst_ctx* c = g->ctx;
        for (const auto& b : g->blocks) c->alloc.release(b.first, b.second);
        for (auto it = c->graph_pinned.begin(); it != c->graph_pinned.end();)
            it = (it->second == g) ? c->graph_pinned.erase(it) : std::next(it);
    }
    delete g;
    return RST_OK;
}
