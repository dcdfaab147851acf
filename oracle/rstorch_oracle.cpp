// TEST INFRASTRUCTURE — CPU restatement of the reference's training step.
//
// This file restates, in plain f64 C++, what the `rstorch` crate computes on the
// path Sequential -> Linear/ReLU -> CrossEntropyLoss -> SGD.  It is the checker
// for the CUDA library and the timed CPU baseline; it is never linked into or
// called from the product path.  Only tests/, the smoke entry and the benchmark's
// CPU-baseline leg load it.
//
// The reference cannot be built here (no Rust toolchain) and delegates its
// arithmetic to the un-vendored crate ndarray 0.15.x (Cargo.toml:17), whose GEMM
// summation order is hardware dependent; this restatement therefore pins:
//   - the reference's own known-answer tests (tests/golden/reference_kat.json:
//     linear.rs:97-131, relu.rs:38-57, identity.rs:35-51, softmax.rs:85-113),
//     checked by tests/test_oracle.py;
//   - formulas, not bit patterns, for the GEMMs: agreement is judged at relative
//     1e-9, and `orc_gemm_precise` (long-double accumulation) bounds both sides.
// For CrossEntropyLoss, SGD::step, argmax/accuracy and the whole step the
// reference has no asserting test: parity there is pinned by this restatement
// alone ("parity unpinned" by reference vectors).
//
// Build: oracle/Makefile (g++ -O3 -march=x86-64-v3 -fopenmp -ffp-contract=off for
// the element-wise part; the GEMM part allows FMA contraction like the
// reference's matrixmultiply kernels do on FMA hardware).
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Implemented in oracle_gemm.cpp: C[M,N] = A[M,K]·B[K,N], all row-major.
void orc_gemm_nn(int64_t M, int64_t N, int64_t K, const double* A, const double* B, double* C);
// The same with strided operands: A(i,p) at A[i*sai + p*sak], B(p,j) at B[p*sbk + j*sbn].
void orc_gemm_strided(int64_t M, int64_t N, int64_t K, const double* A, int64_t sai, int64_t sak, const double* B,
                      int64_t sbk, int64_t sbn, double* C);
// Same product with long-double accumulation, single thread (error bound for tests).
void orc_gemm_precise(int64_t M, int64_t N, int64_t K, const double* A, const double* B, double* C);

static void transpose(const double* src, int64_t rows, int64_t cols, double* dst) {
    const int64_t T = 32;
#pragma omp parallel for schedule(static)
    for (int64_t r0 = 0; r0 < rows; r0 += T)
        for (int64_t c0 = 0; c0 < cols; c0 += T)
            for (int64_t r = r0; r < r0 + T && r < rows; ++r)
                for (int64_t c = c0; c < c0 + T && c < cols; ++c) dst[c * rows + r] = src[r * cols + c];
}

// Linear::forward — src/module/linear.rs:43-57
//   x = input.dot(&weight.t())      (:44)     Y[B,out] = X[B,in] · W[out,in]ᵀ
//   x += bias                        (:51-53)  broadcast of (1,out) over rows
void orc_linear_forward(const double* X, const double* W, const double* b, int64_t B, int64_t in,
                        int64_t out, double* Y, int precise) {
    if (precise) {
        std::vector<double> WT((size_t)in * out);
        transpose(W, out, in, WT.data());
        orc_gemm_precise(B, out, in, X, WT.data(), Y);
    } else {
        orc_gemm_strided(B, out, in, X, in, 1, W, 1, in, Y);          // weight.t() read in place
    }
    if (b) {
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < B; ++r)
            for (int64_t c = 0; c < out; ++c) Y[r * out + c] += b[c];
    }
}

// Linear::backward — src/module/linear.rs:60-69
//   n = prev_input.nrows()                                  (:62)
//   grad_weight = gradient.t().dot(&prev_input) / n         (:63)
//   grad_bias   = gradient.sum_axis(Axis(0)) / n            (:66)
//   returns gradient.dot(&weight)                           (:68)  (not scaled)
void orc_linear_backward(const double* dY, const double* X, const double* W, int64_t B, int64_t in,
                         int64_t out, double* dW, double* db, double* dX, int precise) {
    const double n = (double)B;
    {
        if (precise) {
            std::vector<double> dYT((size_t)B * out);
            transpose(dY, B, out, dYT.data());
            orc_gemm_precise(out, in, B, dYT.data(), X, dW);
        } else {
            orc_gemm_strided(out, in, B, dY, 1, out, X, in, 1, dW);       // gradient.t() read in place
        }
        const int64_t total = out * in;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < total; ++i) dW[i] = dW[i] / n;
    }
    if (db) {
        // every column summed over the rows in ascending order; threads take blocks of columns
#pragma omp parallel for schedule(static)
        for (int64_t c0 = 0; c0 < out; c0 += 512) {
            const int64_t c1 = c0 + 512 < out ? c0 + 512 : out;
            for (int64_t c = c0; c < c1; ++c) db[c] = 0.0;
            for (int64_t r = 0; r < B; ++r)
                for (int64_t c = c0; c < c1; ++c) db[c] += dY[r * out + c];
            for (int64_t c = c0; c < c1; ++c) db[c] = db[c] / n;
        }
    }
    if (dX) {
        if (precise) orc_gemm_precise(B, in, out, dY, W, dX);
        else orc_gemm_nn(B, in, out, dY, W, dX);
    }
}

// ReLU::forward — src/module/activation/relu.rs:19-22: x.max(0.0); f64::max
// returns the non-NaN operand, so NaN maps to 0.
void orc_relu_forward(const double* x, int64_t n, double* y) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        double v = x[i];
        y[i] = (v != v) ? 0.0 : (v > 0.0 ? v : 0.0);
    }
}

// ReLU::backward — relu.rs:25-27: gradient * f64::from(prev_input > 0.0)
void orc_relu_backward(const double* dy, const double* xpre, int64_t n, double* dx) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) dx[i] = dy[i] * (xpre[i] > 0.0 ? 1.0 : 0.0);
}

// softmax free function — src/module/activation/softmax.rs:36-53
//   max folded from f64::MIN with partial_cmp().unwrap() (:36-49): a NaN panics;
//   exp = (input - max).mapv(f64::exp) (:50); sum over the axis (:51); exp / sum (:52)
// Returns the number of rows holding a NaN (the reference would have panicked).
int64_t orc_softmax(const double* x, int64_t rows, int64_t cols, double* p) {
    int64_t nan_rows = 0;
#pragma omp parallel for schedule(static) reduction(+ : nan_rows)
    for (int64_t r = 0; r < rows; ++r) {
        const double* xr = x + r * cols;
        double* pr = p + r * cols;
        double m = -DBL_MAX;   // f64::MIN
        bool has_nan = false;
        for (int64_t c = 0; c < cols; ++c) {
            if (xr[c] != xr[c]) has_nan = true;
            // Ordering::Less => b, otherwise a
            if (m < xr[c]) m = xr[c];
        }
        double s = 0.0;
        for (int64_t c = 0; c < cols; ++c) {
            pr[c] = std::exp(xr[c] - m);
            s += pr[c];
        }
        for (int64_t c = 0; c < cols; ++c) pr[c] = pr[c] / s;
        if (has_nan) nan_rows += 1;
    }
    return nan_rows;
}

// CrossEntropyLoss::forward — src/loss/cross_entropy.rs:34-42
//   pred = softmax(pred, Axis(1))                               (:37)
//   loss = -(&truth * pred.mapv(f64::ln)).sum() / batch_size     (:38)
// Every class term is evaluated, so 0 * ln(0) = NaN propagates as in the reference.
// p_out receives the cached softmax output.
double orc_xent_forward(const double* pred, const double* truth, int64_t rows, int64_t cols, double* p_out,
                        int64_t* nan_rows) {
    int64_t nr = orc_softmax(pred, rows, cols, p_out);
    if (nan_rows) *nan_rows = nr;
    double total = 0.0;
    for (int64_t r = 0; r < rows; ++r) {
        double row = 0.0;
        for (int64_t c = 0; c < cols; ++c) row += truth[r * cols + c] * std::log(p_out[r * cols + c]);
        total += row;
    }
    return -total / (double)rows;
}

// CrossEntropyLoss::backward — cross_entropy.rs:45-47: -(truth - pred), no 1/B
void orc_xent_backward(const double* p, const double* truth, int64_t n, double* g) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) g[i] = -(truth[i] - p[i]);
}

// SGD::step — src/optim/sgd.rs:19-24: parm - (lr * grad): the product is rounded,
// then the difference (this file is compiled without FMA contraction).
void orc_sgd_step(double* p, const double* g, int64_t n, double lr) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        volatile double prod = lr * g[i];
        p[i] = p[i] - prod;
    }
}

// argmax — src/utils.rs:44-53: per row, reduce(|acc, e| if e.1 > acc.1 { e } else { acc })
void orc_argmax(const double* x, int64_t rows, int64_t cols, int64_t* idx) {
    for (int64_t r = 0; r < rows; ++r) {
        int64_t best = 0;
        double bv = x[r * cols];
        for (int64_t c = 1; c < cols; ++c) {
            double v = x[r * cols + c];
            if (v > bv) { bv = v; best = c; }
        }
        idx[r] = best;
    }
}

// accuracy — src/utils.rs:55-65
double orc_accuracy(const double* pred, const double* truth, int64_t rows, int64_t cols) {
    std::vector<int64_t> a((size_t)rows), b((size_t)rows);
    orc_argmax(pred, rows, cols, a.data());
    orc_argmax(truth, rows, cols, b.data());
    int64_t hit = 0;
    for (int64_t r = 0; r < rows; ++r) hit += (a[r] == b[r]);
    return (double)hit / (double)rows;
}

// Seeded input streams: an independent restatement of the generator that produces the
// benchmark's synthetic weights and batches, so that the CPU arm of the benchmark needs
// nothing from the library it is compared with.  Word i of stream `key` is
// splitmix64(key + (i+1)·0x9E3779B97F4A7C15); a uniform takes the top 53 bits; a normal is
// Box-Muller over words 2i and 2i+1.  tests/test_oracle.py checks both against the
// library's generator bit for bit.
static inline uint64_t synth_word(uint64_t key, uint64_t index) {
    uint64_t z = key + index * 0x9E3779B97F4A7C15ull + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline double synth_unit(uint64_t w) { return (double)(w >> 11) * (1.0 / 9007199254740992.0); }

void orc_synth_uniform(uint64_t key, uint64_t n, uint64_t offset, double* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = synth_unit(synth_word(key, offset + (uint64_t)i));
}

void orc_synth_normal(uint64_t key, uint64_t n, uint64_t offset, double mean, double stddev, double* out) {
    const double two_pi = 6.283185307179586476925286766559;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        const uint64_t e = offset + (uint64_t)i;
        const double u1 = 1.0 - synth_unit(synth_word(key, 2 * e));       // (0, 1]
        const double u2 = synth_unit(synth_word(key, 2 * e + 1));
        const double radius = std::sqrt(-2.0 * std::log(u1));
        const double v = radius * std::cos(two_pi * u2);
        const double scaled = stddev * v;
        out[i] = mean + scaled;
    }
}

// Whole training steps of an MLP `Linear, ReLU, Linear, ReLU, ..., Linear` in the
// order of BasicModel::step (src/model.rs:19-27) / the README loop
// (README.md:64-73): forward, loss.forward, accuracy, loss.backward, backward,
// optim.step.  A leading Identity (README.md:49) changes nothing and is omitted.
//   dims[0..L]   layer widths;  W[l] is (dims[l+1], dims[l]), b[l] is (dims[l+1]); updated in place
//   X [steps*B, dims[0]], T [steps*B, dims[L]]
//   skip_first_dx: do not form dX of the first Linear (its value is discarded by the loop)
//   grads_out (nullable): after the last step dW0, db0, dW1, db1, ... back to back
void orc_mlp_train(int L, const int64_t* dims, double* const* W, double* const* b, const double* X,
                   const double* T, int64_t B, int64_t steps, double lr, int skip_first_dx, double* losses,
                   double* accs, double* grads_out) {
    const int64_t C = dims[L];
    std::vector<std::vector<double>> act((size_t)L + 1), pre((size_t)L);
    std::vector<std::vector<double>> dW((size_t)L), db((size_t)L);
    for (int l = 0; l < L; ++l) {
        pre[l].resize((size_t)B * dims[l + 1]);
        act[l + 1].resize((size_t)B * dims[l + 1]);
        dW[l].resize((size_t)dims[l + 1] * dims[l]);
        db[l].resize((size_t)dims[l + 1]);
    }
    std::vector<double> p((size_t)B * C), g, gnext;
    for (int64_t s = 0; s < steps; ++s) {
        const double* x0 = X + s * B * dims[0];
        const double* t = T + s * B * C;
        // forward
        for (int l = 0; l < L; ++l) {
            const double* in = l == 0 ? x0 : act[l].data();
            orc_linear_forward(in, W[l], b[l], B, dims[l], dims[l + 1], pre[l].data(), 0);
            if (l + 1 < L) orc_relu_forward(pre[l].data(), B * dims[l + 1], act[l + 1].data());
        }
        const double* logits = pre[L - 1].data();
        double loss = orc_xent_forward(logits, t, B, C, p.data(), nullptr);
        if (losses) losses[s] = loss;
        if (accs) accs[s] = orc_accuracy(logits, t, B, C);
        // backward
        g.resize((size_t)B * C);
        orc_xent_backward(p.data(), t, B * C, g.data());
        for (int l = L - 1; l >= 0; --l) {
            const double* in = l == 0 ? x0 : act[l].data();
            const bool want_dx = !(l == 0 && skip_first_dx);
            gnext.resize(want_dx ? (size_t)B * dims[l] : 0);
            orc_linear_backward(g.data(), in, W[l], B, dims[l], dims[l + 1], dW[l].data(), db[l].data(),
                                want_dx ? gnext.data() : nullptr, 0);
            if (l > 0) {
                g.resize((size_t)B * dims[l]);
                orc_relu_backward(gnext.data(), pre[l - 1].data(), B * dims[l], g.data());
            }
        }
        // optimiser
        for (int l = 0; l < L; ++l) {
            orc_sgd_step(W[l], dW[l].data(), dims[l + 1] * dims[l], lr);
            orc_sgd_step(b[l], db[l].data(), dims[l + 1], lr);
        }
    }
    if (grads_out) {
        double* o = grads_out;
        for (int l = 0; l < L; ++l) {
            std::memcpy(o, dW[l].data(), dW[l].size() * sizeof(double)); o += dW[l].size();
            std::memcpy(o, db[l].data(), db[l].size() * sizeof(double)); o += db[l].size();
        }
    }
}

}  // extern "C"
