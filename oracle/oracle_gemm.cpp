// TEST INFRASTRUCTURE — the GEMM of the CPU restatement (see rstorch_oracle.cpp).
//
// The reference calls ndarray's `dot` (src/module/linear.rs:44,63,68), which
// forwards to the matrixmultiply crate's blocked dgemm; its summation order and
// FMA use depend on the CPU.  This file is a plain blocked row-major GEMM with
// each C element accumulated over k in ascending order, threaded over row blocks
// with OpenMP; `orc_gemm_precise` is the same product accumulated in long double
// and serves as the error yard-stick in the tests.
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

// C[M,N] = A[M,K]·B[K,N]; row-major, dense.
void orc_gemm_nn(int64_t M, int64_t N, int64_t K, const double* A, const double* B, double* C) {
    const int64_t NC = 512, KC = 256, MR = 4;
    const int64_t total = M * N;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total; ++i) C[i] = 0.0;
    for (int64_t jc = 0; jc < N; jc += NC) {
        const int64_t nb = (N - jc < NC) ? N - jc : NC;
        for (int64_t pc = 0; pc < K; pc += KC) {
            const int64_t kb = (K - pc < KC) ? K - pc : KC;
#pragma omp parallel for schedule(dynamic, 4)
            for (int64_t ic = 0; ic < M; ic += MR) {
                const int64_t mb = (M - ic < MR) ? M - ic : MR;
                if (mb == MR) {
                    double* c0 = C + (ic + 0) * N + jc;
                    double* c1 = C + (ic + 1) * N + jc;
                    double* c2 = C + (ic + 2) * N + jc;
                    double* c3 = C + (ic + 3) * N + jc;
                    for (int64_t p = 0; p < kb; ++p) {
                        const double a0 = A[(ic + 0) * K + pc + p], a1 = A[(ic + 1) * K + pc + p];
                        const double a2 = A[(ic + 2) * K + pc + p], a3 = A[(ic + 3) * K + pc + p];
                        const double* brow = B + (pc + p) * N + jc;
#pragma omp simd
                        for (int64_t j = 0; j < nb; ++j) {
                            const double bv = brow[j];
                            c0[j] += a0 * bv;
                            c1[j] += a1 * bv;
                            c2[j] += a2 * bv;
                            c3[j] += a3 * bv;
                        }
                    }
                } else {
                    for (int64_t r = 0; r < mb; ++r) {
                        double* c = C + (ic + r) * N + jc;
                        for (int64_t p = 0; p < kb; ++p) {
                            const double a = A[(ic + r) * K + pc + p];
                            const double* brow = B + (pc + p) * N + jc;
#pragma omp simd
                            for (int64_t j = 0; j < nb; ++j) c[j] += a * brow[j];
                        }
                    }
                }
            }
        }
    }
}

void orc_gemm_precise(int64_t M, int64_t N, int64_t K, const double* A, const double* B, double* C) {
    std::vector<long double> acc((size_t)N);
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) acc[j] = 0.0L;
        for (int64_t p = 0; p < K; ++p) {
            const long double a = A[i * K + p];
            const double* brow = B + p * N;
            for (int64_t j = 0; j < N; ++j) acc[j] += a * (long double)brow[j];
        }
        for (int64_t j = 0; j < N; ++j) C[i * N + j] = (double)acc[j];
    }
}

}  // extern "C"
