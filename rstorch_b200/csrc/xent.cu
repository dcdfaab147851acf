// Softmax + cross-entropy + gradient + accuracy in one pass over the rows, the
// softmax free function, and row-wise argmax.
//
// Reference semantics kept (paths relative to the reference repository):
//   - row maximum folded from f64::MIN              src/module/activation/softmax.rs:36-49
//   - e = exp(x - max), p = e / Σe                  src/module/activation/softmax.rs:50-52
//   - loss = -(Σ_ij t_ij · ln p_ij) / B over the whole matrix, every class
//     term evaluated (0 · ln 0 = NaN is preserved)  src/loss/cross_entropy.rs:38
//   - gradient = p - t, no 1/B                      src/loss/cross_entropy.rs:45-47
//   - argmax: first maximum wins, a later element replaces the running one only
//     on strict `>`, so a NaN never replaces        src/utils.rs:44-53
//
// A row is owned by LPR lanes of one warp; each lane keeps EPL elements of the
// row in registers (column = lane_in_row + j*LPR, so a warp reads contiguous
// memory), reductions are warp shuffles.  Loss and correct-count are reduced
// per block, written as one partial per block, and the last block to finish
// adds the partials in index order, so the result does not depend on block
// scheduling.  Algorithmic traffic: 24 B per logit (read x, read t, write g).
#include <algorithm>
#include <cfloat>

#include "common.h"

namespace rst {
namespace {

constexpr int kXentThreads = 256;
constexpr int kWarps = kXentThreads / 32;
constexpr unsigned kFull = 0xffffffffu;

struct ArgMax {
    double v;
    int i;
};

// Combine two candidates of one row.  Values of NaN elements at columns > 0 are
// mapped to -inf by the caller (they can never replace the running maximum), and
// ties go to the smaller column, which reproduces the left-to-right fold.
__device__ __forceinline__ ArgMax pick(ArgMax a, ArgMax b) {
    bool take_b = (b.v > a.v) || (b.v == a.v && b.i < a.i);
    return take_b ? b : a;
}

template <int LPR>
__device__ __forceinline__ double group_sum(double v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}
template <int LPR>
__device__ __forceinline__ double group_max(double v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
        double w = __shfl_xor_sync(kFull, v, o);
        v = w > v ? w : v;
    }
    return v;
}
template <int LPR>
__device__ __forceinline__ ArgMax group_argmax(ArgMax a) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(kFull, a.v, o);
        b.i = __shfl_xor_sync(kFull, a.i, o);
        a = pick(a, b);
    }
    return a;
}
template <int LPR>
__device__ __forceinline__ int group_or(int v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v |= __shfl_xor_sync(kFull, v, o);
    return v;
}

// Row-wise argmax with the reference's fold semantics over values held as
// v[j] <-> column lane + j*LPR.
template <int LPR, int EPL>
__device__ __forceinline__ int row_argmax(const double (&v)[EPL], int lane, int cols) {
    ArgMax best{-INFINITY, 0x7fffffff};
    int first_is_nan = 0;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        int col = lane + j * LPR;
        if (col < cols) {
            double x = v[j];
            if (x != x) {
                if (col == 0) first_is_nan = 1;
                x = -INFINITY;
            }
            best = pick(best, ArgMax{x, col});
        }
    }
    best = group_argmax<LPR>(best);
    first_is_nan = group_or<LPR>(first_is_nan);
    return first_is_nan ? 0 : best.i;
}

// t * ln(p), the summand of cross_entropy.rs:38.  The f64 logarithm is the most
// expensive part of the kernel and, with one-hot targets, all but one term per row are
// 0 * ln(p) with p > 0, i.e. a signed zero that leaves the sum unchanged; those skip the
// logarithm.  p == 0 (0 * -inf = NaN), NaN and non-zero targets take the full expression,
// so the value of the loss is the reference's in every case.
__device__ __forceinline__ double loss_term(double t, double p) {
    return (t == 0.0 && p > 0.0) ? 0.0 : t * log(p);
}

struct BlockPartial {
    double loss;      // Σ t · ln p over the block's rows
    double correct;
    double nan_rows;
    double pad;
};

// Block-level reduction of three per-thread values followed by the last-block
// final sum.  `partials` holds gridDim.x entries; `counter` is zero on entry
// and is reset to zero by the last block.
__device__ __forceinline__ void finish_block(double loss, double correct, double nan_rows,
                                             BlockPartial* partials, unsigned int* counter,
                                             ResultSlot* slot, double rows_total) {
    __shared__ double sh[3][kWarps];
    __shared__ bool is_last;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    loss = group_sum<32>(loss);
    correct = group_sum<32>(correct);
    nan_rows = group_sum<32>(nan_rows);
    if (lane == 0) { sh[0][warp] = loss; sh[1][warp] = correct; sh[2][warp] = nan_rows; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double a = 0.0, b = 0.0, c = 0.0;
        for (int w = 0; w < kWarps; ++w) { a += sh[0][w]; b += sh[1][w]; c += sh[2][w]; }
        partials[blockIdx.x] = BlockPartial{a, b, c, 0.0};
        __threadfence();
        unsigned int done = atomicAdd(counter, 1u);
        is_last = (done == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // fixed-order final sum: thread t adds partials t, t+256, ... then a fixed tree
    double a = 0.0, b = 0.0, c = 0.0;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += kXentThreads) {
        BlockPartial p = partials[i];
        a += p.loss; b += p.correct; c += p.nan_rows;
    }
    a = group_sum<32>(a); b = group_sum<32>(b); c = group_sum<32>(c);
    __syncthreads();
    if (lane == 0) { sh[0][warp] = a; sh[1][warp] = b; sh[2][warp] = c; }
    __syncthreads();
    if (threadIdx.x == 0) {
        a = b = c = 0.0;
        for (int w = 0; w < kWarps; ++w) { a += sh[0][w]; b += sh[1][w]; c += sh[2][w]; }
        slot->loss_sum = a;
        slot->correct = b;
        slot->rows = rows_total;
        slot->nan_rows = c;
        *counter = 0u;
    }
}

// MODE 0: loss + gradient + accuracy.  MODE 1: softmax only (writes p to `out`).
template <int LPR, int EPL, int MODE>
__global__ void __launch_bounds__(kXentThreads)
xent_rows_kernel(const double* __restrict__ logits, const double* __restrict__ truth,
                 double* __restrict__ out, int64_t rows, int cols, BlockPartial* partials,
                 unsigned int* counter, ResultSlot* slot) {
    grid_dependency_release();
    grid_dependency_wait();
    constexpr int kRowsPerWarp = 32 / LPR;
    const int lane_in_warp = threadIdx.x & 31;
    const int lane = lane_in_warp % LPR;
    const int sub = lane_in_warp / LPR;
    const int64_t warp_global = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int64_t warp_stride = (int64_t)gridDim.x * kWarps;

    double loss_acc = 0.0, correct_acc = 0.0, nan_acc = 0.0;

    for (int64_t row0 = warp_global * kRowsPerWarp; row0 < rows; row0 += warp_stride * kRowsPerWarp) {
        const int64_t row = row0 + sub;
        const bool live = row < rows;          // whole LPR-lane group shares this
        const double* xr = logits + row * cols;
        double x[EPL], t[EPL];
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            int col = lane + j * LPR;
            bool in = live && col < cols;
            x[j] = in ? xr[col] : 0.0;
            if (MODE == 0) t[j] = in ? truth[row * cols + col] : 0.0;
        }
        // row maximum, folded from the most negative finite value like the reference
        double m = -DBL_MAX;
        int has_nan = 0;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            int col = lane + j * LPR;
            if (col < cols) {
                if (x[j] != x[j]) has_nan = 1;
                m = x[j] > m ? x[j] : m;
            }
        }
        m = group_max<LPR>(m);
        has_nan = group_or<LPR>(has_nan);

        int pred_arg = 0, truth_arg = 0;
        if (MODE == 0) {
            pred_arg = row_argmax<LPR, EPL>(x, lane, cols);
            truth_arg = row_argmax<LPR, EPL>(t, lane, cols);
        }

        double s = 0.0;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            int col = lane + j * LPR;
            if (col < cols) {
                x[j] = exp(x[j] - m);
                s += x[j];
            }
        }
        s = group_sum<LPR>(s);

        double row_loss = 0.0;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            int col = lane + j * LPR;
            if (live && col < cols) {
                double p = x[j] / s;
                if (MODE == 0) {
                    row_loss += loss_term(t[j], p);
                    if (out) out[row * cols + col] = p - t[j];
                } else {
                    out[row * cols + col] = p;
                }
            }
        }
        if (MODE == 0) {
            row_loss = group_sum<LPR>(row_loss);
            if (live && lane == 0) {
                loss_acc += row_loss;
                correct_acc += (pred_arg == truth_arg) ? 1.0 : 0.0;
                nan_acc += has_nan ? 1.0 : 0.0;
            }
        }
    }
    if (MODE == 0) finish_block(loss_acc, correct_acc, nan_acc, partials, counter, slot, (double)rows);
}

// Rows of 129 to 2048 columns: one CTA per row, EPT elements per thread (column =
// thread + j*256).  A warp per row would need 32 to 64 doubles per lane for x and as many
// for t, which leaves one CTA of 8 warps per SM at over 200 registers, far too few warps
// to cover the latency of the f64 exp and division chains (measured: 19 % of the HBM
// bandwidth on 16384 x 1000).  Here a thread holds at most 2 x 8 doubles, eight CTAs fit an
// SM, and a row costs two block-wide reductions: (max, NaN flag, both arg-maxima) and the
// sum of the exponentials.  The loss terms stay per thread across all rows of the CTA and
// are reduced once, in a fixed order, at the end.
template <int EPT, int MODE>
__global__ void __launch_bounds__(kXentThreads)
xent_block_kernel(const double* __restrict__ logits, const double* __restrict__ truth,
                  double* __restrict__ out, int64_t rows, int cols, BlockPartial* partials,
                  unsigned int* counter, ResultSlot* slot) {
    grid_dependency_release();
    grid_dependency_wait();
    __shared__ double sh_max[kWarps], sh_sum[kWarps];
    __shared__ double sh_xv[kWarps], sh_tv[kWarps];
    __shared__ int sh_xi[kWarps], sh_ti[kWarps], sh_flags[kWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    double loss_acc = 0.0, correct_acc = 0.0, nan_acc = 0.0;

    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const double* xr = logits + row * cols;
        const double* tr = MODE == 0 ? truth + row * cols : nullptr;
        double x[EPT], t[EPT];
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int col = tid + j * kXentThreads;
            x[j] = col < cols ? xr[col] : 0.0;
            t[j] = (MODE == 0 && col < cols) ? tr[col] : 0.0;
        }
        // first block-wide reduction: maximum (folded from the most negative finite value like
        // the reference), NaN flag, arg-maxima of x and t with the fold's tie and NaN rules
        double m = -DBL_MAX;
        int flags = 0;                       // 1: a NaN logit, 2: x[0] is NaN, 4: t[0] is NaN
        ArgMax bx{-INFINITY, 0x7fffffff}, bt{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int col = tid + j * kXentThreads;
            if (col < cols) {
                const double v = x[j];
                if (v != v) flags |= (col == 0) ? 3 : 1;
                m = v > m ? v : m;
                if (MODE == 0) {
                    bx = pick(bx, ArgMax{v != v ? -INFINITY : v, col});
                    const double w = t[j];
                    if (w != w && col == 0) flags |= 4;
                    bt = pick(bt, ArgMax{w != w ? -INFINITY : w, col});
                }
            }
        }
        m = group_max<32>(m);
        flags = group_or<32>(flags);
        if (MODE == 0) { bx = group_argmax<32>(bx); bt = group_argmax<32>(bt); }
        if (lane == 0) {
            sh_max[warp] = m; sh_flags[warp] = flags;
            sh_xv[warp] = bx.v; sh_xi[warp] = bx.i; sh_tv[warp] = bt.v; sh_ti[warp] = bt.i;
        }
        __syncthreads();
        m = sh_max[0]; flags = sh_flags[0];
        bx = ArgMax{sh_xv[0], sh_xi[0]}; bt = ArgMax{sh_tv[0], sh_ti[0]};
#pragma unroll
        for (int w = 1; w < kWarps; ++w) {
            m = sh_max[w] > m ? sh_max[w] : m;
            flags |= sh_flags[w];
            if (MODE == 0) {
                bx = pick(bx, ArgMax{sh_xv[w], sh_xi[w]});
                bt = pick(bt, ArgMax{sh_tv[w], sh_ti[w]});
            }
        }
        // second: sum of the exponentials, added in warp order by every thread alike
        double s = 0.0;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int col = tid + j * kXentThreads;
            if (col < cols) {
                x[j] = exp(x[j] - m);
                s += x[j];
            }
        }
        s = group_sum<32>(s);
        if (lane == 0) sh_sum[warp] = s;
        __syncthreads();
        s = sh_sum[0];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) s += sh_sum[w];

#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const int col = tid + j * kXentThreads;
            if (col < cols) {
                const double p = x[j] / s;
                if (MODE == 0) {
                    loss_acc += loss_term(t[j], p);
                    if (out) out[row * cols + col] = p - t[j];
                } else {
                    out[row * cols + col] = p;
                }
            }
        }
        if (MODE == 0 && tid == 0) {
            const int pred_arg = (flags & 2) ? 0 : bx.i, truth_arg = (flags & 4) ? 0 : bt.i;
            correct_acc += (pred_arg == truth_arg) ? 1.0 : 0.0;
            nan_acc += (flags & 1) ? 1.0 : 0.0;
        }
        // No barrier needed before the next row: a warp can overwrite sh_max and its
        // companions only after the second barrier of this row, which every thread reaches
        // after its reads of them, and sh_sum only after the first barrier of the next row.
    }
    if (MODE == 0) finish_block(loss_acc, correct_acc, nan_acc, partials, counter, slot, (double)rows);
}

// Rows wider than 2048 columns: one warp per row, three sweeps over the row
// (it stays in L1/L2 between them).
template <int MODE>
__global__ void __launch_bounds__(kXentThreads)
xent_wide_kernel(const double* __restrict__ logits, const double* __restrict__ truth,
                 double* __restrict__ out, int64_t rows, int cols, BlockPartial* partials,
                 unsigned int* counter, ResultSlot* slot) {
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int64_t warp_stride = (int64_t)gridDim.x * kWarps;
    double loss_acc = 0.0, correct_acc = 0.0, nan_acc = 0.0;
    for (int64_t row = warp_global; row < rows; row += warp_stride) {
        const double* xr = logits + row * cols;
        const double* tr = truth ? truth + row * cols : nullptr;
        double m = -DBL_MAX;
        int has_nan = 0, x0_nan = 0, t0_nan = 0;
        ArgMax bx{-INFINITY, 0x7fffffff}, bt{-INFINITY, 0x7fffffff};
        for (int col = lane; col < cols; col += 32) {
            double x = xr[col];
            if (x != x) { has_nan = 1; if (col == 0) x0_nan = 1; }
            m = x > m ? x : m;
            if (MODE == 0) {
                bx = pick(bx, ArgMax{x != x ? -INFINITY : x, col});
                double t = tr[col];
                if (t != t && col == 0) t0_nan = 1;
                bt = pick(bt, ArgMax{t != t ? -INFINITY : t, col});
            }
        }
        m = group_max<32>(m);
        has_nan = group_or<32>(has_nan);
        int pred_arg = 0, truth_arg = 0;
        if (MODE == 0) {
            bx = group_argmax<32>(bx); bt = group_argmax<32>(bt);
            x0_nan = group_or<32>(x0_nan); t0_nan = group_or<32>(t0_nan);
            pred_arg = x0_nan ? 0 : bx.i;
            truth_arg = t0_nan ? 0 : bt.i;
        }
        double s = 0.0;
        for (int col = lane; col < cols; col += 32) s += exp(xr[col] - m);
        s = group_sum<32>(s);
        double row_loss = 0.0;
        for (int col = lane; col < cols; col += 32) {
            double p = exp(xr[col] - m) / s;
            if (MODE == 0) {
                double t = tr[col];
                row_loss += loss_term(t, p);
                if (out) out[row * cols + col] = p - t;
            } else {
                out[row * cols + col] = p;
            }
        }
        if (MODE == 0) {
            row_loss = group_sum<32>(row_loss);
            if (lane == 0) {
                loss_acc += row_loss;
                correct_acc += (pred_arg == truth_arg) ? 1.0 : 0.0;
                nan_acc += has_nan ? 1.0 : 0.0;
            }
        }
    }
    if (MODE == 0) finish_block(loss_acc, correct_acc, nan_acc, partials, counter, slot, (double)rows);
}

template <int LPR, int EPL>
__global__ void __launch_bounds__(kXentThreads)
argmax_rows_kernel(const double* __restrict__ x, int64_t rows, int cols, long long* __restrict__ idx) {
    constexpr int kRowsPerWarp = 32 / LPR;
    const int lane_in_warp = threadIdx.x & 31;
    const int lane = lane_in_warp % LPR;
    const int sub = lane_in_warp / LPR;
    const int64_t warp_global = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int64_t warp_stride = (int64_t)gridDim.x * kWarps;
    for (int64_t row0 = warp_global * kRowsPerWarp; row0 < rows; row0 += warp_stride * kRowsPerWarp) {
        const int64_t row = row0 + sub;
        const bool live = row < rows;
        double v[EPL];
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            int col = lane + j * LPR;
            v[j] = (live && col < cols) ? x[row * cols + col] : 0.0;
        }
        int a = row_argmax<LPR, EPL>(v, lane, cols);
        if (live && lane == 0) idx[row] = a;
    }
}

__global__ void __launch_bounds__(kXentThreads)
argmax_wide_kernel(const double* __restrict__ x, int64_t rows, int cols, long long* __restrict__ idx) {
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int64_t warp_stride = (int64_t)gridDim.x * kWarps;
    for (int64_t row = warp_global; row < rows; row += warp_stride) {
        ArgMax b{-INFINITY, 0x7fffffff};
        int x0_nan = 0;
        for (int col = lane; col < cols; col += 32) {
            double v = x[row * cols + col];
            if (v != v && col == 0) x0_nan = 1;
            b = pick(b, ArgMax{v != v ? -INFINITY : v, col});
        }
        b = group_argmax<32>(b);
        x0_nan = group_or<32>(x0_nan);
        if (lane == 0) idx[row] = x0_nan ? 0 : b.i;
    }
}

inline int xent_grid(const rst_ctx* ctx, int64_t rows, int rows_per_warp) {
    int64_t warps = (rows + rows_per_warp - 1) / rows_per_warp;
    int64_t blocks = (warps + kWarps - 1) / kWarps;
    int64_t cap = (int64_t)ctx->num_sms * 8;   // 8 blocks of 256 threads fill an SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

template <int MODE>
int dispatch_rows(rst_ctx* ctx, const double* logits, const double* truth, double* out,
                  int64_t rows, int64_t cols, ResultSlot* d_slot) {
    BlockPartial* partials = nullptr;
    int max_grid = ctx->num_sms * 8;
    if (MODE == 0) {
        RST_TRY(ensure_scratch(ctx, (void**)&ctx->xent_partials, &ctx->xent_partials_cap,
                               (size_t)max_grid * sizeof(BlockPartial), "loss-reduction"));
        partials = reinterpret_cast<BlockPartial*>(ctx->xent_partials);
    }
    unsigned int* counter = ctx->xent_counter;
    cudaStream_t st = ctx->compute;
    int c = (int)cols;
#define XENT_CASE(LPR, EPL)                                                                    \
    launch_step_kernel(ctx, st, xent_rows_kernel<LPR, EPL, MODE>,                              \
                       dim3((unsigned)xent_grid(ctx, rows, 32 / LPR)), dim3(kXentThreads), 0, \
                       logits, truth, out, rows, c, partials, counter, d_slot)
#define XENT_BLOCK_CASE(EPT)                                                                          \
    launch_step_kernel(ctx, st, xent_block_kernel<EPT, MODE>,                                         \
                       dim3((unsigned)std::max<int64_t>(1, std::min<int64_t>(rows, max_grid))), dim3(kXentThreads), 0, \
                       logits, truth, out, rows, c, partials, counter, d_slot)
    if (cols <= 16) XENT_CASE(4, 4);
    else if (cols <= 32) XENT_CASE(8, 4);
    else if (cols <= 128) XENT_CASE(32, 4);
    else if (cols <= 512) XENT_BLOCK_CASE(2);
    else if (cols <= 1024) XENT_BLOCK_CASE(4);
    else if (cols <= 2048) XENT_BLOCK_CASE(8);
    else
        xent_wide_kernel<MODE><<<xent_grid(ctx, rows, 1), kXentThreads, 0, st>>>(
            logits, truth, out, rows, c, partials, counter, d_slot);
#undef XENT_CASE
#undef XENT_BLOCK_CASE
    return after_launch(ctx, MODE == 0 ? "xent_rows_kernel" : "softmax_rows_kernel");
}

}  // namespace

int launch_xent(rst_ctx* ctx, const double* logits, const double* truth, double* dlogits,
                int64_t rows, int64_t cols, ResultSlot* d_slot) {
    return dispatch_rows<0>(ctx, logits, truth, dlogits, rows, cols, d_slot);
}

int launch_softmax(rst_ctx* ctx, const double* x, double* p, int64_t rows, int64_t cols) {
    if (rows == 0 || cols == 0) return RST_OK;
    return dispatch_rows<1>(ctx, x, nullptr, p, rows, cols, nullptr);
}

int launch_argmax(rst_ctx* ctx, const double* x, int64_t rows, int64_t cols, long long* d_idx) {
    if (rows == 0) return RST_OK;
    cudaStream_t st = ctx->compute;
    int c = (int)cols;
#define ARG_CASE(LPR, EPL) \
    argmax_rows_kernel<LPR, EPL><<<xent_grid(ctx, rows, 32 / LPR), kXentThreads, 0, st>>>(x, rows, c, d_idx)
    if (cols <= 16) ARG_CASE(4, 4);
    else if (cols <= 32) ARG_CASE(8, 4);
    else if (cols <= 128) ARG_CASE(32, 4);
    else if (cols <= 512) ARG_CASE(32, 16);
    else if (cols <= 1024) ARG_CASE(32, 32);
    else argmax_wide_kernel<<<xent_grid(ctx, rows, 1), kXentThreads, 0, st>>>(x, rows, c, d_idx);
#undef ARG_CASE
    return after_launch(ctx, "argmax_rows_kernel");
}

}  // namespace rst
