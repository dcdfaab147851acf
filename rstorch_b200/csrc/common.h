// Internal declarations shared by the translation units of librstorch_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "../../include/rstorch_b200.h"

namespace rst {

constexpr uint32_t kCtxMagic = 0x52535443u;     // 'RSTC'
constexpr uint32_t kTensorMagic = 0x52535454u;  // 'RSTT'
constexpr uint32_t kDeadMagic = 0xDEADBEEFu;
constexpr int kXentSlots = 64;
constexpr int kNumSMsFallback = 148;

// Device status word indices (written by kernels, read by rst_ctx_check_device).
enum DeviceStatus : int { kDevOk = 0, kDevBarrierTimeout = 1, kDevBadIndex = 2 };

// ---------------------------------------------------------------------------
// Caching allocator: size-bucketed free lists over cudaMalloc.  All tensors of
// a context are used in the order of its compute stream, so a block handed back
// by rst_tensor_free can be reused by the next request without an event.
// ---------------------------------------------------------------------------
class CachingAllocator {
public:
    // Rounds a request to its bucket size: 512 B granules below 1 MiB (in
    // quarter-octave steps above 4 KiB), 2 MiB granules above.
    static size_t bucket_size(size_t bytes);

    // Returns nullptr and sets *err on failure (cudaError value or -1 = limit).
    void* allocate(size_t bytes, size_t* granted, int* err, bool may_call_driver);
    void release(void* ptr, size_t granted);
    void empty_cache();
    void set_limit(uint64_t max_reserved) { limit_ = max_reserved; }

    // Graph capture.  Between begin_recording and end_recording every block that is
    // handed out or handed back is remembered: the recorded kernels have its address
    // baked in.  end_recording takes the remembered blocks that sit in the cache out of
    // it (*cached: the graph owns them until it is destroyed) and lists the ones a
    // tensor still holds (*live: they go to the graph when that tensor is freed).
    void begin_recording();
    void end_recording(std::vector<std::pair<void*, size_t>>* cached, std::vector<void*>* live);
    // A block that a graph took out of the cache counts as in use until the graph returns it.
    void adopt(size_t granted) { in_use += granted; peak = peak > in_use ? peak : in_use; }

    uint64_t in_use = 0, reserved = 0, peak = 0, requests = 0, hits = 0, driver_allocs = 0;

private:
    std::multimap<size_t, void*> free_;
    uint64_t limit_ = 0;
    bool recording_ = false;
    std::map<void*, size_t> recorded_;
};

struct ResultSlot {  // written by the xent kernel, copied to pinned host memory
    double loss_sum;    // Σ_ij t_ij · ln p_ij  (sign and 1/B applied on the host)
    double correct;     // rows whose argmax(logits) == argmax(truth)
    double rows;        // B
    double nan_rows;    // rows holding a NaN logit
};

}  // namespace rst

struct rst_tensor {
    uint32_t magic;
    rst_ctx* ctx;
    double* data;
    int64_t rows, cols;
    size_t granted;      // bytes obtained from the allocator (0 for views)
    bool owns;
};

struct rst_ctx {
    uint32_t magic;
    int device;
    int num_sms;
    cudaStream_t compute, copy, comm;
    rst::CachingAllocator alloc;
    std::string last_error;
    uint64_t launches;
    bool capturing;
    bool overlap_launches;    // programmatic dependent launch for the step's kernels
    bool stream_tail;         // large GEMMs hand the last, partly filled wave out in equal k runs
    double grad_rows_scale;   // Linear::backward divides dW and db by rows(X) times this (1, or the world
                              // size of a communicator that sums gradient shares instead of averaging)

    int* d_status;            // device status words (kernels report bounded-wait expiry)
    int* h_status;            // pinned mirror

    // loss / accuracy read-back ring
    rst::ResultSlot* d_results;
    rst::ResultSlot* h_results;   // pinned
    cudaEvent_t result_event[rst::kXentSlots];
    bool result_pending[rst::kXentSlots];
    bool result_in_graph[rst::kXentSlots];   // written by a captured graph: no event to wait on

    // scratch owned by the context and grown on demand
    double* xent_partials;  size_t xent_partials_cap;   // per-block partial sums
    unsigned int* xent_counter;                          // last-block election
    double* splitk_ws;      size_t splitk_ws_bytes;     // split-K partial tiles
    double* colsum_ws;      size_t colsum_ws_bytes;     // two-pass column sums
    char* flush_buf;        size_t flush_bytes;

    void* encode_tiled;     // PFN_cuTensorMapEncodeTiled, resolved at creation

    // per-kernel-class timing (rst_profile_begin/end): event pairs around launches
    bool profiling;
    struct ProfRecord { const char* name; cudaEvent_t start, stop; };
    std::vector<ProfRecord> prof_records;
    std::vector<cudaEvent_t> prof_event_pool;
    std::map<std::string, rst_sgd_plan*> plan_cache;

    // Blocks that a live graph has recorded while a tensor still holds them: freeing the
    // tensor hands the block to that graph instead of the cache.
    std::map<void*, rst_graph*> graph_pinned;
    // Kernels whose dynamic shared-memory limit has been raised on this context's device.
    std::set<const void*> smem_attr_done;
};

namespace rst {

int fail(const rst_ctx* ctx, int status, const char* fmt, ...);
bool valid(const rst_ctx* ctx);
bool valid(const rst_tensor* t);
int check_tensor(const rst_ctx* ctx, const rst_tensor* t, const char* name);
// Grows a context-owned scratch buffer (never during graph capture).
int ensure_scratch(rst_ctx* ctx, void** buf, size_t* cap, size_t need, const char* what);
int after_launch(rst_ctx* ctx, const char* what);

// Brackets the launches of one kernel class with CUDA events while profiling is on.
class ProfScope {
public:
    ProfScope(rst_ctx* ctx, const char* name);
    ~ProfScope();
private:
    rst_ctx* ctx_;
    int index_;
};

#define RST_CUDA(ctx, call)                                                            \
    do {                                                                               \
        cudaError_t e__ = (call);                                                      \
        if (e__ != cudaSuccess)                                                        \
            return rst::fail((ctx), RST_ERR_CUDA, "%s failed: %s (%s:%d)", #call,      \
                             cudaGetErrorString(e__), __FILE__, __LINE__);             \
    } while (0)

// Launches a kernel of the step.  With ctx->overlap_launches the launch carries the
// programmatic-stream-serialization attribute: the grid may start while the grid queued
// before it on the same stream is still draining, so its prologue (barrier set-up,
// descriptor prefetch, index arithmetic) hides the launch gap.  Only kernels that call
// grid_dependency_wait() before their first global access may be launched through
// here; launched without the attribute that call returns at once.
template <typename... Params, typename... Args>
inline void launch_step_kernel(rst_ctx* ctx, cudaStream_t stream, void (*kernel)(Params...), dim3 grid,
                               dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->overlap_launches ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, Params(std::forward<Args>(args))...);   // error read by after_launch
}

#ifdef __CUDACC__
// Blocks until every grid this one depends on has completed and its writes are visible.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Lets the next grid on the stream start launching once every CTA of this grid got here.
__device__ __forceinline__ void grid_dependency_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif

#define RST_TRY(call)                      \
    do {                                   \
        int s__ = (call);                  \
        if (s__ != RST_OK) return s__;     \
    } while (0)

// ---- kernel launchers implemented in the .cu files -------------------------
enum GemmEpilogue : int { kEpiNone = 0, kEpiBias = 1, kEpiBiasRelu = 2, kEpiDivN = 3, kEpiMask = 4 };

struct GemmArgs {
    // C[M,N] = op(A)·op(B); A is K-major ([M][K] in memory) or M-major ([K][M]);
    // B is K-major ([N][K]) or N-major ([K][N]).
    const double* A; const double* B; double* C;
    int64_t M, N, K;
    bool a_kmajor, b_kmajor;
    int epilogue;
    const double* bias;       // [N]          (kEpiBias, kEpiBiasRelu)
    const double* mask_src;   // [M,N]        (kEpiMask)
    double divisor;           // n            (kEpiDivN)
    double* colsum_out;       // optional [M]: Σ_k A(m,k) / divisor when A is M-major (db)
    double* C_transposed;     // optional [N,M]: a second, transposed copy of C (M-major A with N-major B
                              // and large tiles only; the caller checks gemm_writes_transposed)
    long long wait_limit_cycles;  // 0 = the default bound of a barrier wait (about two seconds)
    bool starve_producer;     // self-test only: no tile is ever copied, every consumer wait runs out
};
// Whether launch_gemm would honour C_transposed for this product.
bool gemm_writes_transposed(const rst_ctx* ctx, const GemmArgs& a);
// *colsum_done (optional) tells whether colsum_out was produced by the GEMM kernel itself.
int launch_gemm(rst_ctx* ctx, const GemmArgs& a, bool* colsum_done = nullptr);
// Up to four dW-type products (M-major A, N-major B, 1/n epilogue, column sums) in one
// launch when together they fit one wave of small tiles; *grouped = false means nothing
// was launched.
int launch_gemm_group(rst_ctx* ctx, const GemmArgs* args, int n, bool* grouped);

int launch_colsum_div(rst_ctx* ctx, const double* dY, int64_t rows, int64_t cols, double n,
                      double* out);
int launch_relu_forward(rst_ctx* ctx, const double* x, double* y, int64_t n);
int launch_relu_backward(rst_ctx* ctx, const double* dy, const double* xpre, double* dx,
                         int64_t n);
int launch_fill(rst_ctx* ctx, double* x, double v, int64_t n);
// Adds the digest of x[0..n) to *d_out (a zeroed device word).
int launch_checksum(rst_ctx* ctx, const double* x, int64_t n, unsigned long long* d_out);
int launch_transpose(rst_ctx* ctx, const double* src, int64_t rows, int64_t cols, double* dst);
int launch_softmax_axis0(rst_ctx* ctx, const double* x, double* p, int64_t rows, int64_t cols);
int launch_softmax_jacobian_diag(rst_ctx* ctx, double* J, int64_t n);
int launch_softmax(rst_ctx* ctx, const double* x, double* p, int64_t rows, int64_t cols);
int launch_xent(rst_ctx* ctx, const double* logits, const double* truth, double* dlogits,
                int64_t rows, int64_t cols, ResultSlot* d_slot);
int launch_argmax(rst_ctx* ctx, const double* x, int64_t rows, int64_t cols, long long* d_idx);

}  // namespace rst
