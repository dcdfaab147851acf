// Unfused ReLU forward/backward, fill, and the two-pass column sum behind db.
// All of them are HBM-streaming kernels: 16-byte vector accesses on the aligned
// body, grids sized in multiples of the SM count.
#include "common.h"

namespace rst {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ double relu1(double v) { return fmax(v, 0.0); }  // NaN -> 0 like f64::max
__device__ __forceinline__ double gate1(double dy, double x) { return dy * (x > 0.0 ? 1.0 : 0.0); }

// y = max(x, 0)                                   (src/module/activation/relu.rs:21)
__global__ void __launch_bounds__(kThreads) relu_forward_kernel(const double* __restrict__ x,
                                                                double* __restrict__ y, int64_t n,
                                                                int vec_ok) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec_ok) {
        int64_t n2 = n >> 1;
        const double2* x2 = reinterpret_cast<const double2*>(x);
        double2* y2 = reinterpret_cast<double2*>(y);
        for (int64_t i = tid; i < n2; i += stride) {
            double2 v = x2[i];
            v.x = relu1(v.x); v.y = relu1(v.y);
            y2[i] = v;
        }
        if (tid == 0 && (n & 1)) y[n - 1] = relu1(x[n - 1]);
    } else {
        for (int64_t i = tid; i < n; i += stride) y[i] = relu1(x[i]);
    }
}

// dx = dy * (x_pre > 0 ? 1 : 0)                   (src/module/activation/relu.rs:26)
__global__ void __launch_bounds__(kThreads) relu_backward_kernel(const double* __restrict__ dy,
                                                                 const double* __restrict__ xpre,
                                                                 double* __restrict__ dx, int64_t n,
                                                                 int vec_ok) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec_ok) {
        int64_t n2 = n >> 1;
        const double2* g2 = reinterpret_cast<const double2*>(dy);
        const double2* x2 = reinterpret_cast<const double2*>(xpre);
        double2* o2 = reinterpret_cast<double2*>(dx);
        for (int64_t i = tid; i < n2; i += stride) {
            double2 g = g2[i], v = x2[i];
            g.x = gate1(g.x, v.x); g.y = gate1(g.y, v.y);
            o2[i] = g;
        }
        if (tid == 0 && (n & 1)) dx[n - 1] = gate1(dy[n - 1], xpre[n - 1]);
    } else {
        for (int64_t i = tid; i < n; i += stride) dx[i] = gate1(dy[i], xpre[i]);
    }
}

// Softmax over axis 0 (every column sums to one; Softmax::with_axis(0),
// src/module/activation/softmax.rs:21-27,45-53).  One thread per column, so a warp
// reads consecutive elements of a row; the maximum is folded from f64::MIN.
__global__ void __launch_bounds__(kThreads) softmax_axis0_kernel(const double* __restrict__ x,
                                                                 double* __restrict__ p, int64_t rows,
                                                                 int64_t cols) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    double m = -1.7976931348623157e308;
    for (int64_t r = 0; r < rows; ++r) {
        const double v = x[r * cols + c];
        m = v > m ? v : m;
    }
    double s = 0.0;
    for (int64_t r = 0; r < rows; ++r) s += exp(x[r * cols + c] - m);
    for (int64_t r = 0; r < rows; ++r) p[r * cols + c] = exp(x[r * cols + c] - m) / s;
}

// Diagonal of the Softmax module's Jacobian: J holds -OᵀO; each diagonal element becomes
// s(1 - s) with s = -J[j][j]                        (src/module/activation/softmax.rs:67-70)
__global__ void __launch_bounds__(kThreads) softmax_jacobian_diag_kernel(double* __restrict__ J, int64_t n) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    double el = J[j * n + j];
    el = -el;
    el = el * (1.0 - el);
    J[j * n + j] = el;
}

// dst[c][r] = src[r][c] through a padded 32x32 shared tile: reads and writes are both
// contiguous along their own rows.  256 threads = 32 columns x 8 rows, four row steps.
__global__ void __launch_bounds__(kThreads) transpose_kernel(const double* __restrict__ src,
                                                             double* __restrict__ dst, int64_t rows, int64_t cols) {
    __shared__ double tile[32][33];
    const int64_t tiles_c = (cols + 31) / 32;
    const int64_t r0 = (blockIdx.x / tiles_c) * 32, c0 = (blockIdx.x % tiles_c) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t r = r0 + ty + 8 * j, c = c0 + tx;
        if (r < rows && c < cols) tile[ty + 8 * j][tx] = src[r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t c = c0 + ty + 8 * j, r = r0 + tx;
        if (r < rows && c < cols) dst[c * rows + r] = tile[tx][ty + 8 * j];
    }
}

__global__ void __launch_bounds__(kThreads) fill_kernel(double* __restrict__ x, double v, int64_t n) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) x[i] = v;
}

// Column sums of dY[rows, cols] in two deterministic passes.
// Pass 1: block (bx, by) sums rows [by*rows_per, ...) of columns [bx*128, +128) into
// ws[by][col].  Pass 2: sums the `parts` partial rows in index order and divides by n.
constexpr int kColsPerBlock = 128;
constexpr int kRowLanes = 2;   // 256 threads = 128 columns x 2 row lanes

__global__ void __launch_bounds__(kThreads) colsum_pass1(const double* __restrict__ dY, int64_t rows,
                                                         int64_t cols, int64_t rows_per,
                                                         double* __restrict__ ws) {
    __shared__ double sh[kRowLanes][kColsPerBlock];
    int c_local = threadIdx.x % kColsPerBlock;
    int lane_r = threadIdx.x / kColsPerBlock;
    int64_t col = (int64_t)blockIdx.x * kColsPerBlock + c_local;
    int64_t r0 = (int64_t)blockIdx.y * rows_per;
    int64_t r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
    double acc = 0.0;
    if (col < cols) {
        // four independent partial sums keep several loads in flight per thread
        double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
        int64_t r = r0 + lane_r;
        for (; r + 3 * kRowLanes < r1; r += 4 * kRowLanes) {
            a0 += dY[r * cols + col];
            a1 += dY[(r + kRowLanes) * cols + col];
            a2 += dY[(r + 2 * kRowLanes) * cols + col];
            a3 += dY[(r + 3 * kRowLanes) * cols + col];
        }
        for (; r < r1; r += kRowLanes) a0 += dY[r * cols + col];
        acc = (a0 + a1) + (a2 + a3);
    }
    sh[lane_r][c_local] = acc;
    __syncthreads();
    if (lane_r == 0 && col < cols) ws[(int64_t)blockIdx.y * cols + col] = sh[0][c_local] + sh[1][c_local];
}

// db = (Σ_rows dY) / n                              (src/module/linear.rs:65-67)
__global__ void __launch_bounds__(kThreads) colsum_pass2(const double* __restrict__ ws, int parts,
                                                         int64_t cols, double n,
                                                         double* __restrict__ out) {
    int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= cols) return;
    double acc = 0.0;
    for (int p = 0; p < parts; ++p) acc += ws[(int64_t)p * cols + col];
    out[col] = acc / n;
}

// Order-sensitive 64-bit digest of a tensor's bit patterns: Σ_i mix(bits_i + (i+1)·φ64)
// in wrapping arithmetic.  Integer addition commutes, so the result does not depend on the
// grid or on the order in which blocks finish.
__global__ void __launch_bounds__(kThreads) checksum_kernel(const double* __restrict__ x, int64_t n,
                                                            unsigned long long* __restrict__ out) {
    unsigned long long acc = 0ull;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        unsigned long long z = (unsigned long long)__double_as_longlong(x[i]) + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        acc += z ^ (z >> 31);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0 && acc) atomicAdd(out, acc);
}

inline int grid_for(const rst_ctx* ctx, int64_t work_items, int per_sm) {
    int64_t blocks = (work_items + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)ctx->num_sms * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace

int launch_relu_forward(rst_ctx* ctx, const double* x, double* y, int64_t n) {
    if (n == 0) return RST_OK;
    int vec = aligned16(x) && aligned16(y);
    relu_forward_kernel<<<grid_for(ctx, vec ? n / 2 + 1 : n, 8), kThreads, 0, ctx->compute>>>(x, y, n, vec);
    return after_launch(ctx, "relu_forward_kernel");
}

int launch_relu_backward(rst_ctx* ctx, const double* dy, const double* xpre, double* dx, int64_t n) {
    if (n == 0) return RST_OK;
    int vec = aligned16(dy) && aligned16(xpre) && aligned16(dx);
    relu_backward_kernel<<<grid_for(ctx, vec ? n / 2 + 1 : n, 8), kThreads, 0, ctx->compute>>>(dy, xpre, dx, n, vec);
    return after_launch(ctx, "relu_backward_kernel");
}

int launch_softmax_axis0(rst_ctx* ctx, const double* x, double* p, int64_t rows, int64_t cols) {
    if (rows == 0 || cols == 0) return RST_OK;
    softmax_axis0_kernel<<<(unsigned)((cols + kThreads - 1) / kThreads), kThreads, 0, ctx->compute>>>(x, p, rows, cols);
    return after_launch(ctx, "softmax_axis0_kernel");
}

int launch_softmax_jacobian_diag(rst_ctx* ctx, double* J, int64_t n) {
    if (n == 0) return RST_OK;
    softmax_jacobian_diag_kernel<<<(unsigned)((n + kThreads - 1) / kThreads), kThreads, 0, ctx->compute>>>(J, n);
    return after_launch(ctx, "softmax_jacobian_diag_kernel");
}

int launch_transpose(rst_ctx* ctx, const double* src, int64_t rows, int64_t cols, double* dst) {
    if (rows == 0 || cols == 0) return RST_OK;
    const int64_t tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
    if (tiles > 0x7fffffffLL) return fail(ctx, RST_ERR_UNSUPPORTED, "matrix too large to transpose in one launch");
    transpose_kernel<<<(unsigned)tiles, kThreads, 0, ctx->compute>>>(src, dst, rows, cols);
    return after_launch(ctx, "transpose_kernel");
}

int launch_checksum(rst_ctx* ctx, const double* x, int64_t n, unsigned long long* d_out) {
    if (n == 0) return RST_OK;
    checksum_kernel<<<grid_for(ctx, n, 8), kThreads, 0, ctx->compute>>>(x, n, d_out);
    return after_launch(ctx, "checksum_kernel");
}

int launch_fill(rst_ctx* ctx, double* x, double v, int64_t n) {
    if (n == 0) return RST_OK;
    fill_kernel<<<grid_for(ctx, n, 8), kThreads, 0, ctx->compute>>>(x, v, n);
    return after_launch(ctx, "fill_kernel");
}

int launch_colsum_div(rst_ctx* ctx, const double* dY, int64_t rows, int64_t cols, double n,
                      double* out) {
    if (cols == 0) return RST_OK;
    int64_t col_blocks = (cols + kColsPerBlock - 1) / kColsPerBlock;
    // enough row parts to fill the GPU about four times over, at least 64 rows each
    int64_t want_parts = ((int64_t)ctx->num_sms * 4 + col_blocks - 1) / col_blocks;
    int64_t max_parts = (rows + 63) / 64;
    int64_t parts = want_parts < max_parts ? want_parts : max_parts;
    if (parts < 1) parts = 1;
    if (parts > 65535) parts = 65535;
    int64_t rows_per = (rows + parts - 1) / parts;
    if (rows_per < 1) rows_per = 1;
    parts = rows == 0 ? 1 : (rows + rows_per - 1) / rows_per;
    size_t need = (size_t)parts * (size_t)cols * sizeof(double);
    RST_TRY(ensure_scratch(ctx, (void**)&ctx->colsum_ws, &ctx->colsum_ws_bytes, need, "column-sum"));
    dim3 g1((unsigned)col_blocks, (unsigned)parts);
    colsum_pass1<<<g1, kThreads, 0, ctx->compute>>>(dY, rows, cols, rows_per, ctx->colsum_ws);
    RST_TRY(after_launch(ctx, "colsum_pass1"));
    int g2 = (int)((cols + kThreads - 1) / kThreads);
    colsum_pass2<<<g2, kThreads, 0, ctx->compute>>>(ctx->colsum_ws, (int)parts, cols, n, out);
    return after_launch(ctx, "colsum_pass2");
}

}  // namespace rst

// ---------------------------------------------------------------------------
// Bias gradient for callers that must not allocate.
//
// Some hosts of this library may not call cudaMalloc at the point where they need db: a
// process whose device memory is wholly claimed by another allocator and handed out as raw
// pointers (a second party's cudaMalloc fails there or takes memory it was never given), and
// a step function with a hard latency bound (cudaMalloc and cudaFree may synchronise the
// whole device).  The regular path grows its column-sum scratch from the driver on demand;
// this entry point uses a fixed array that lives in the library's device image instead, so
// every GPU that loads the library holds kNoAllocScratchDoubles * 8 bytes (2 MiB) until exit.
// ---------------------------------------------------------------------------
namespace rst {
namespace {

constexpr int64_t kNoAllocScratchDoubles = (int64_t)1 << 18;   // 2 MiB of partial column sums
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) double g_noalloc_colsum_scratch[kNoAllocScratchDoubles];

// Host code cannot use the array's name as a device address (it names a host-side
// shadow symbol); the device address is looked up once per device.
std::mutex g_noalloc_mutex;
double* g_noalloc_scratch_ptr[kNoAllocMaxDevices] = {nullptr};
int g_noalloc_sm_count[kNoAllocMaxDevices] = {0};

int noalloc_scratch_for_current_device(double** out, int* sm_count) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return fail(nullptr, RST_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kNoAllocMaxDevices)
        return fail(nullptr, RST_ERR_UNSUPPORTED, "device ordinal %d beyond %d", dev, kNoAllocMaxDevices);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_scratch_ptr[dev]) {
        double* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_colsum_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(nullptr, RST_ERR_CUDA, "cudaGetSymbolAddress of the static scratch failed on device %d: %s",
                        dev, cudaGetErrorString(e));
        }
        int sms = 0;      // an attribute query; it allocates nothing
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
            cudaGetLastError();
            sms = kNumSMsFallback;
        }
        g_noalloc_sm_count[dev] = sms;
        g_noalloc_scratch_ptr[dev] = p;
    }
    *out = g_noalloc_scratch_ptr[dev];
    *sm_count = g_noalloc_sm_count[dev];
    return RST_OK;
}

}  // namespace
}  // namespace rst

extern "C" int rst_bias_grad_noalloc(const double* dY, int64_t rows, int64_t cols, double* db, void* stream) {
    using namespace rst;
    if (rows < 0 || cols < 0) return fail(nullptr, RST_ERR_INVALID_ARG, "negative shape (%lld,%lld)",
                                          (long long)rows, (long long)cols);
    if (cols == 0) return RST_OK;
    if (!db || (rows > 0 && !dY)) return fail(nullptr, RST_ERR_INVALID_ARG, "dY or db is NULL");
    if (cols > kNoAllocScratchDoubles)
        return fail(nullptr, RST_ERR_UNSUPPORTED,
                    "rst_bias_grad_noalloc: %lld columns exceed the static scratch of %lld columns; "
                    "use rst_linear_backward, which may allocate",
                    (long long)cols, (long long)kNoAllocScratchDoubles);
    double* scratch = nullptr;
    int sm_count = 0;
    RST_TRY(noalloc_scratch_for_current_device(&scratch, &sm_count));
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

    // as many row parts as fit the fixed scratch, up to about four waves of blocks
    const int64_t col_blocks = (cols + kColsPerBlock - 1) / kColsPerBlock;
    int64_t parts = ((int64_t)sm_count * 4 + col_blocks - 1) / col_blocks;
    const int64_t fit = kNoAllocScratchDoubles / cols;          // >= 1 by the check above
    if (parts > fit) parts = fit;
    const int64_t by_rows = (rows + 63) / 64;
    if (parts > by_rows) parts = by_rows;
    if (parts < 1) parts = 1;
    if (parts > 65535) parts = 65535;
    int64_t rows_per = (rows + parts - 1) / parts;
    if (rows_per < 1) rows_per = 1;
    parts = rows == 0 ? 1 : (rows + rows_per - 1) / rows_per;

    // pass 1 writes every scratch entry that pass 2 reads, so nothing has to be
    // cleared between calls
    dim3 g1((unsigned)col_blocks, (unsigned)parts);
    colsum_pass1<<<g1, kThreads, 0, st>>>(dY, rows, cols, rows_per, scratch);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(nullptr, RST_ERR_CUDA, "launch of colsum_pass1 failed: %s", cudaGetErrorString(e));
    const int g2 = (int)((cols + kThreads - 1) / kThreads);
    colsum_pass2<<<g2, kThreads, 0, st>>>(scratch, (int)parts, cols, (double)rows, db);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(nullptr, RST_ERR_CUDA, "launch of colsum_pass2 failed: %s", cudaGetErrorString(e));
    return RST_OK;
}
