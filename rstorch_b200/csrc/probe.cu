// Roofline probes: the issue rate of the f64 tensor instruction (the GEMM
// denominator), a streaming copy (the HBM denominator) and an L2 flush.
#include "common.h"
#include "mma_f64.cuh"

namespace rst {
namespace {

constexpr int kProbeThreads = 256;
constexpr int kChains = 8;   // independent accumulator tiles per warp

// Every warp keeps kChains independent 16x8 accumulators and feeds them from
// register operands only, so the loop measures the DMMA pipe, not memory.
template <int KIND>
__global__ void __launch_bounds__(kProbeThreads) fp64_issue_kernel(int iters, double* sink) {
    double acc[kChains][4];
    double a[4], b[2];
    const double seed = 1.0 + 1e-9 * (double)(threadIdx.x & 31);
#pragma unroll
    for (int c = 0; c < kChains; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[c][e] = 0.0;
#pragma unroll
    for (int e = 0; e < 4; ++e) a[e] = seed + e;
    b[0] = 1e-3 * seed; b[1] = -1e-3 * seed;

    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int c = 0; c < kChains; ++c) {
            if (KIND == 0) {
                asm volatile(
                    "mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                    : "+d"(acc[c][0]), "+d"(acc[c][1]), "+d"(acc[c][2]), "+d"(acc[c][3])
                    : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
            } else if (KIND == 1) {
                // four m8n8k4 = the flops of one m16n8k8
                asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                             : "+d"(acc[c][0]), "+d"(acc[c][1]) : "d"(a[0]), "d"(b[0]));
                asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                             : "+d"(acc[c][2]), "+d"(acc[c][3]) : "d"(a[1]), "d"(b[0]));
                asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                             : "+d"(acc[c][0]), "+d"(acc[c][1]) : "d"(a[2]), "d"(b[1]));
                asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                             : "+d"(acc[c][2]), "+d"(acc[c][3]) : "d"(a[3]), "d"(b[1]));
            } else if (KIND == 2) {
                // one m16n8k16 = two m16n8k8; counted as such by the host
                asm volatile(
                    "mma.sync.aligned.m16n8k16.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, "
                    "{%4,%5,%6,%7,%4,%5,%6,%7}, {%8,%9,%8,%9}, {%0,%1,%2,%3};"
                    : "+d"(acc[c][0]), "+d"(acc[c][1]), "+d"(acc[c][2]), "+d"(acc[c][3])
                    : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
            } else {
                // plain DFMA: 16x8x8 multiply-adds per warp = 32 per thread
#pragma unroll
                for (int r = 0; r < 8; ++r) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[c][e] = fma(a[e], b[r & 1], acc[c][e]);
                }
            }
        }
    }
    double s = 0.0;
#pragma unroll
    for (int c = 0; c < kChains; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) s += acc[c][e];
    if (s == 12345.678) sink[0] = s;   // keeps the loop alive without a store in practice
}

__global__ void __launch_bounds__(256) copy_kernel(const double2* __restrict__ src, double2* __restrict__ dst,
                                                  long long n2) {
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += stride) dst[i] = src[i];
}

__global__ void __launch_bounds__(256) flush_kernel(double2* __restrict__ dst, long long n2) {
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += stride)
        dst[i] = make_double2(0.0, 0.0);
}

}  // namespace
}  // namespace rst

using namespace rst;

extern "C" int rst_probe_fp64_peak(rst_ctx* c, int kind, int iters, double* tflops) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!tflops || iters <= 0 || kind < 0 || kind > 3) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    if (c->capturing) return fail(c, RST_ERR_STATE, "probe during graph capture");
    const int blocks = c->num_sms * 4;   // 32 warps per SM
    cudaEvent_t e0, e1;
    RST_CUDA(c, cudaEventCreate(&e0));
    RST_CUDA(c, cudaEventCreate(&e1));
    double* sink = reinterpret_cast<double*>(c->d_results);   // never written (see kernel)
    float best = 1e30f;
    for (int rep = 0; rep < 4; ++rep) {   // first repetition warms up
        RST_CUDA(c, cudaEventRecord(e0, c->compute));
        switch (kind) {
            case 0: fp64_issue_kernel<0><<<blocks, kProbeThreads, 0, c->compute>>>(iters, sink); break;
            case 1: fp64_issue_kernel<1><<<blocks, kProbeThreads, 0, c->compute>>>(iters, sink); break;
            case 2: fp64_issue_kernel<2><<<blocks, kProbeThreads, 0, c->compute>>>(iters, sink); break;
            default: fp64_issue_kernel<3><<<blocks, kProbeThreads, 0, c->compute>>>(iters, sink); break;
        }
        RST_TRY(after_launch(c, "fp64_issue_kernel"));
        RST_CUDA(c, cudaEventRecord(e1, c->compute));
        RST_CUDA(c, cudaEventSynchronize(e1));
        float ms = 0.f;
        RST_CUDA(c, cudaEventElapsedTime(&ms, e0, e1));
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    // flops per chain step: 16*8*8*2 = 2048 (kind 2 issues twice that)
    const double per_step = (kind == 2 ? 2.0 : 1.0) * 2048.0;
    const double warps = (double)blocks * (kProbeThreads / 32);
    const double flops = per_step * kChains * (double)iters * warps;
    *tflops = flops / ((double)best * 1e-3) / 1e12;
    return RST_OK;
}

extern "C" int rst_probe_hbm_copy(rst_ctx* c, uint64_t bytes, int iters, double* gbs) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!gbs || iters <= 0 || bytes < 32) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    if (c->capturing) return fail(c, RST_ERR_STATE, "probe during graph capture");
    rst_tensor *a = nullptr, *b = nullptr;
    const int64_t n = (int64_t)(bytes / 16) * 2;
    RST_TRY(rst_tensor_alloc(c, 1, n, &a));
    int s = rst_tensor_alloc(c, 1, n, &b);
    if (s != RST_OK) { rst_tensor_free(a); return s; }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaMemsetAsync(a->data, 0, (size_t)n * 8, c->compute);
    float best = 1e30f;
    const int blocks = c->num_sms * 16;
    for (int rep = 0; rep < iters + 1; ++rep) {
        cudaEventRecord(e0, c->compute);
        copy_kernel<<<blocks, 256, 0, c->compute>>>(reinterpret_cast<const double2*>(a->data),
                                                    reinterpret_cast<double2*>(b->data), n / 2);
        c->launches++;
        cudaEventRecord(e1, c->compute);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    rst_tensor_free(a);
    rst_tensor_free(b);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(c, RST_ERR_CUDA, "copy probe failed: %s", cudaGetErrorString(e));
    *gbs = 2.0 * (double)n * 8.0 / ((double)best * 1e-3) / 1e9;
    return RST_OK;
}

extern "C" int rst_flush_l2(rst_ctx* c, uint64_t bytes) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (bytes < 32) return RST_OK;
    RST_TRY(ensure_scratch(c, (void**)&c->flush_buf, &c->flush_bytes, bytes, "L2-flush"));
    flush_kernel<<<c->num_sms * 8, 256, 0, c->compute>>>(reinterpret_cast<double2*>(c->flush_buf),
                                                         (long long)(bytes / 16));
    return after_launch(c, "flush_kernel");
}
