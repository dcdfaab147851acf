// TEST INFRASTRUCTURE — the GEMM of the CPU restatement (see rstorch_oracle.cpp).
//
// The reference calls ndarray's `dot` (src/module/linear.rs:44,63,68), which
// forwards to the matrixmultiply crate's blocked dgemm; its summation order and
// FMA use depend on the CPU.  This file is a blocked, packed row-major GEMM of the same
// kind (k ascending within a block, blocks added in ascending order), threaded with
// OpenMP; `orc_gemm_precise` is the same product accumulated in long double and serves
// as the error yard-stick in the tests.
#include <cstdint>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// C[M,N] = A[M,K]·B[K,N]; row-major, dense.
//
// Blocked like the dgemm of the matrixmultiply crate the reference calls through ndarray:
// a KC x NC panel of B is packed once, every thread packs its own MC x KC block of A, and a
// register-tiled micro-kernel (6 rows x 8 columns, fused multiply-add where the CPU has it)
// walks k in ascending order.  A C element is therefore the sum, in ascending order, of its
// KC-long partial sums.  Work is split over (row block, column chunk) pairs so that a product
// with few rows (the forward pass at a small batch) still feeds every thread.
namespace {

typedef double v4d __attribute__((vector_size(32), aligned(8)));

constexpr int64_t MR = 6, NR = 8, KC = 256, MC = 96, NC = 2048, NCT = 256;

inline v4d splat(double a) { return (v4d){a, a, a, a}; }

// C[0:mr, 0:nr] += Ap(kc x MR panel) · Bp(kc x NR panel)
inline void micro_kernel(int64_t kc, const double* __restrict__ Ap, const double* __restrict__ Bp, double* C,
                         int64_t ldc, int64_t mr, int64_t nr) {
    v4d c00 = splat(0), c01 = splat(0), c10 = splat(0), c11 = splat(0), c20 = splat(0), c21 = splat(0);
    v4d c30 = splat(0), c31 = splat(0), c40 = splat(0), c41 = splat(0), c50 = splat(0), c51 = splat(0);
    for (int64_t p = 0; p < kc; ++p) {
        const v4d b0 = *(const v4d*)(Bp + p * NR), b1 = *(const v4d*)(Bp + p * NR + 4);
        const double* a = Ap + p * MR;
        v4d av;
        av = splat(a[0]); c00 += av * b0; c01 += av * b1;
        av = splat(a[1]); c10 += av * b0; c11 += av * b1;
        av = splat(a[2]); c20 += av * b0; c21 += av * b1;
        av = splat(a[3]); c30 += av * b0; c31 += av * b1;
        av = splat(a[4]); c40 += av * b0; c41 += av * b1;
        av = splat(a[5]); c50 += av * b0; c51 += av * b1;
    }
    const v4d acc[MR][2] = {{c00, c01}, {c10, c11}, {c20, c21}, {c30, c31}, {c40, c41}, {c50, c51}};
    if (mr == MR && nr == NR) {
        for (int64_t i = 0; i < MR; ++i) {
            v4d* row = (v4d*)(C + i * ldc);
            row[0] += acc[i][0];
            row[1] += acc[i][1];
        }
    } else {
        for (int64_t i = 0; i < mr; ++i)
            for (int64_t j = 0; j < nr; ++j) C[i * ldc + j] += acc[i][j / 4][j % 4];
    }
}

// rows [i0, i0+mc) x k [p0, p0+kc) of A into MR-row panels: panel q holds Ap[q][p][i].
// Element (i, p) of A lives at A[i*sai + p*sak].
inline void pack_a(const double* A, int64_t sai, int64_t sak, int64_t i0, int64_t mc, int64_t p0, int64_t kc,
                   double* out) {
    for (int64_t q = 0; q < mc; q += MR) {
        const int64_t mr = (mc - q < MR) ? mc - q : MR;
        if (sak == 1) {                       // rows are contiguous in k: walk each row
            for (int64_t i = 0; i < mr; ++i) {
                const double* src = A + (i0 + q + i) * sai + p0;
                for (int64_t p = 0; p < kc; ++p) out[p * MR + i] = src[p];
            }
            for (int64_t i = mr; i < MR; ++i)
                for (int64_t p = 0; p < kc; ++p) out[p * MR + i] = 0.0;
        } else {
            for (int64_t p = 0; p < kc; ++p) {
                const double* src = A + (p0 + p) * sak + (i0 + q) * sai;
                for (int64_t i = 0; i < mr; ++i) out[p * MR + i] = src[i * sai];
                for (int64_t i = mr; i < MR; ++i) out[p * MR + i] = 0.0;
            }
        }
        out += kc * MR;
    }
}

// k [p0, p0+kc) x columns [j0, j0+nr) of B into one NR-column panel: Bp[p][j].
// Element (p, j) of B lives at B[p*sbk + j*sbn].
inline void pack_b_panel(const double* B, int64_t sbk, int64_t sbn, int64_t p0, int64_t kc, int64_t j0, int64_t nr,
                         double* out) {
    if (sbk == 1) {                           // columns are contiguous in k: walk each column
        for (int64_t j = 0; j < nr; ++j) {
            const double* src = B + (j0 + j) * sbn + p0;
            for (int64_t p = 0; p < kc; ++p) out[p * NR + j] = src[p];
        }
        for (int64_t j = nr; j < NR; ++j)
            for (int64_t p = 0; p < kc; ++p) out[p * NR + j] = 0.0;
    } else {
        for (int64_t p = 0; p < kc; ++p) {
            const double* src = B + (p0 + p) * sbk + j0 * sbn;
            for (int64_t j = 0; j < nr; ++j) out[p * NR + j] = src[j * sbn];
            for (int64_t j = nr; j < NR; ++j) out[p * NR + j] = 0.0;
        }
    }
}

}  // namespace

void orc_gemm_strided(int64_t M, int64_t N, int64_t K, const double* A, int64_t sai, int64_t sak, const double* B,
                      int64_t sbk, int64_t sbn, double* C);

void orc_gemm_nn(int64_t M, int64_t N, int64_t K, const double* A, const double* B, double* C) {
    orc_gemm_strided(M, N, K, A, K, 1, B, N, 1, C);
}

// C[M,N] (row-major, dense) = A·B with A(i,p) at A[i*sai + p*sak] and B(p,j) at B[p*sbk + j*sbn]:
// the transposed operands of Linear::forward and Linear::backward are read in place.
void orc_gemm_strided(int64_t M, int64_t N, int64_t K, const double* A, int64_t sai, int64_t sak, const double* B,
                      int64_t sbk, int64_t sbn, double* C) {
    const int64_t total = M * N;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total; ++i) C[i] = 0.0;
    if (M == 0 || N == 0 || K == 0) return;
    // Packing buffers live across calls (one caller thread at a time): a fresh allocation of
    // this size per call is an mmap plus its page faults, which costs more than the packing.
    static std::vector<double> bpack, apack_all;
    int threads = 1;
#ifdef _OPENMP
    threads = omp_get_max_threads();
#endif
    const size_t apack_size = (size_t)((MC + MR) * KC);
    if (bpack.size() < (size_t)(KC * (NC + NR))) bpack.resize((size_t)(KC * (NC + NR)));
    if (apack_all.size() < apack_size * (size_t)threads) apack_all.resize(apack_size * (size_t)threads);
    for (int64_t jc = 0; jc < N; jc += NC) {
        const int64_t nc = (N - jc < NC) ? N - jc : NC;
        const int64_t panels = (nc + NR - 1) / NR;
        for (int64_t pc = 0; pc < K; pc += KC) {
            const int64_t kc = (K - pc < KC) ? K - pc : KC;
#pragma omp parallel for schedule(static)
            for (int64_t q = 0; q < panels; ++q) {
                const int64_t j0 = q * NR;
                pack_b_panel(B, sbk, sbn, pc, kc, jc + j0, (nc - j0 < NR) ? nc - j0 : NR, bpack.data() + q * kc * NR);
            }
            const int64_t row_blocks = (M + MC - 1) / MC, col_chunks = (nc + NCT - 1) / NCT;
#pragma omp parallel
            {
                int me = 0;
#ifdef _OPENMP
                me = omp_get_thread_num();
#endif
                double* apack = apack_all.data() + apack_size * (size_t)me;
                int64_t packed_block = -1;
#pragma omp for collapse(2) schedule(dynamic, 1)
                for (int64_t rb = 0; rb < row_blocks; ++rb)
                    for (int64_t cc = 0; cc < col_chunks; ++cc) {
                        const int64_t i0 = rb * MC, mc = (M - i0 < MC) ? M - i0 : MC;
                        if (packed_block != rb) {
                            pack_a(A, sai, sak, i0, mc, pc, kc, apack);
                            packed_block = rb;
                        }
                        const int64_t jt = cc * NCT, jt_end = (jt + NCT < nc) ? jt + NCT : nc;
                        for (int64_t jr = jt; jr < jt_end; jr += NR) {
                            const int64_t nr = (nc - jr < NR) ? nc - jr : NR;
                            const double* bp = bpack.data() + (jr / NR) * kc * NR;
                            for (int64_t ir = 0; ir < mc; ir += MR)
                                micro_kernel(kc, apack + (ir / MR) * kc * MR, bp, C + (i0 + ir) * N + jc + jr, N,
                                             (mc - ir < MR) ? mc - ir : MR, nr);
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
