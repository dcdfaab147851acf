// SGD::step over every parameter tensor in one launch (src/optim/sgd.rs:18-25).
//
// The reference evaluates `parm.clone() - (lr * grad.clone())` per tensor: the
// product is rounded to f64, then the difference is rounded.  The kernel keeps
// both roundings (__dmul_rn, __dsub_rn: no FMA contraction), so given the same
// inputs the update is bit-identical to the reference's.
//
// Work is cut into chunks of kChunk elements; a device table maps a chunk id to
// (tensor, offset) by binary search over per-tensor first-chunk indices, so one
// persistent grid streams all tensors whatever their number or sizes.
// Algorithmic traffic: 24 B per parameter (read p, read g, write p).
#include <algorithm>
#include <string>

#include "common.h"

namespace rst {

struct SgdEntry {
    double* p;
    const double* g;
    long long numel;
    long long first_chunk;
};

namespace {

constexpr int kSgdThreads = 256;
constexpr int kVec = 4;                                   // doubles per 32-byte access
constexpr int kUnroll = 4;                                // accesses in flight per thread and array
constexpr int kChunk = kSgdThreads * kVec * kUnroll;      // 4096 elements = 32 KiB per array

struct __align__(32) double4a { double x, y, z, w; };

__device__ __forceinline__ double4a ld256(const double* p) {
    double4a v;
    asm volatile("ld.global.v4.f64 {%0,%1,%2,%3}, [%4];"
                 : "=d"(v.x), "=d"(v.y), "=d"(v.z), "=d"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ double4a ld256_stream(const double* p) {
    double4a v;
    asm volatile("ld.global.L1::no_allocate.v4.f64 {%0,%1,%2,%3}, [%4];"
                 : "=d"(v.x), "=d"(v.y), "=d"(v.z), "=d"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st256(double* p, const double4a& v) {
    asm volatile("st.global.v4.f64 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "d"(v.x), "d"(v.y), "d"(v.z), "d"(v.w) : "memory");
}

__device__ __forceinline__ double sgd1(double p, double g, double lr) {
    return __dsub_rn(p, __dmul_rn(lr, g));
}

__global__ void __launch_bounds__(kSgdThreads)
sgd_multi_tensor_kernel(const SgdEntry* __restrict__ table, int n_tensors, long long total_chunks,
                        double lr) {
    grid_dependency_release();
    grid_dependency_wait();
    for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        // largest t with table[t].first_chunk <= chunk
        int lo = 0, hi = n_tensors - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (table[mid].first_chunk <= chunk) lo = mid; else hi = mid - 1;
        }
        const SgdEntry e = table[lo];
        long long base = (chunk - e.first_chunk) * (long long)kChunk;
        long long left = e.numel - base;
        double* p = e.p + base;
        const double* g = e.g + base;
        bool vec = (((uintptr_t)p | (uintptr_t)g) & 31u) == 0;
        if (vec && left >= kChunk) {
            double4a pv[kUnroll], gv[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                int off = (u * kSgdThreads + threadIdx.x) * kVec;
                pv[u] = ld256(p + off);
                gv[u] = ld256_stream(g + off);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                int off = (u * kSgdThreads + threadIdx.x) * kVec;
                double4a r;
                r.x = sgd1(pv[u].x, gv[u].x, lr);
                r.y = sgd1(pv[u].y, gv[u].y, lr);
                r.z = sgd1(pv[u].z, gv[u].z, lr);
                r.w = sgd1(pv[u].w, gv[u].w, lr);
                st256(p + off, r);
            }
        } else {
            long long lim = left < kChunk ? left : kChunk;
            for (long long i = threadIdx.x; i < lim; i += kSgdThreads) p[i] = sgd1(p[i], g[i], lr);
        }
    }
}

}  // namespace
}  // namespace rst

using namespace rst;

struct rst_sgd_plan {
    rst_ctx* ctx;
    SgdEntry* d_table;
    int n;
    long long total_chunks;
    long long total_numel;
};

extern "C" int rst_sgd_plan_create(rst_ctx* c, int n, rst_tensor* const* params,
                                   rst_tensor* const* grads, rst_sgd_plan** out) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!out || n < 0 || (n > 0 && (!params || !grads)))
        return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    *out = nullptr;
    std::vector<SgdEntry> table;
    long long chunks = 0, numel = 0;
    for (int i = 0; i < n; ++i) {
        RST_TRY(check_tensor(c, params[i], "params[i]"));
        RST_TRY(check_tensor(c, grads[i], "grads[i]"));
        if (params[i]->rows != grads[i]->rows || params[i]->cols != grads[i]->cols)
            return fail(c, RST_ERR_SHAPE, "parameter %d is (%lld,%lld) but its gradient is (%lld,%lld)",
                        i, (long long)params[i]->rows, (long long)params[i]->cols,
                        (long long)grads[i]->rows, (long long)grads[i]->cols);
        long long ne = params[i]->rows * params[i]->cols;
        if (ne == 0) continue;
        table.push_back(SgdEntry{params[i]->data, grads[i]->data, ne, chunks});
        chunks += (ne + kChunk - 1) / kChunk;
        numel += ne;
    }
    rst_sgd_plan* p = new rst_sgd_plan{c, nullptr, (int)table.size(), chunks, numel};
    if (!table.empty()) {
        cudaError_t e = cudaMalloc((void**)&p->d_table, table.size() * sizeof(SgdEntry));
        if (e != cudaSuccess) {
            cudaGetLastError();
            delete p;
            return fail(c, RST_ERR_OOM, "cannot allocate the SGD table: %s", cudaGetErrorString(e));
        }
        e = cudaMemcpy(p->d_table, table.data(), table.size() * sizeof(SgdEntry), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            cudaFree(p->d_table);
            delete p;
            return fail(c, RST_ERR_CUDA, "cannot upload the SGD table: %s", cudaGetErrorString(e));
        }
    }
    *out = p;
    return RST_OK;
}

extern "C" int rst_sgd_plan_step(rst_sgd_plan* plan, double lr) {
    if (!plan || !valid(plan->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad plan");
    rst_ctx* c = plan->ctx;
    if (plan->total_chunks == 0) return RST_OK;
    long long cap = (long long)c->num_sms * 8;
    int grid = (int)std::min(plan->total_chunks, cap);
    ProfScope prof(c, "sgd");
    launch_step_kernel(c, c->compute, sgd_multi_tensor_kernel, dim3((unsigned)grid), dim3(kSgdThreads), 0,
                       plan->d_table, plan->n, plan->total_chunks, lr);
    return after_launch(c, "sgd_multi_tensor_kernel");
}

extern "C" int rst_sgd_plan_destroy(rst_sgd_plan* plan) {
    if (!plan) return RST_OK;
    if (valid(plan->ctx)) cudaStreamSynchronize(plan->ctx->compute);
    if (plan->d_table) cudaFree(plan->d_table);
    delete plan;
    return RST_OK;
}

extern "C" int rst_sgd_step(rst_ctx* c, int n, rst_tensor* const* params, rst_tensor* const* grads,
                            double lr) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (n < 0 || (n > 0 && (!params || !grads))) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    // The plan is keyed by the device addresses and sizes of the list, so a
    // parameter set that was re-allocated gets a fresh table.
    std::string key;
    key.reserve((size_t)n * 24);
    for (int i = 0; i < n; ++i) {
        RST_TRY(check_tensor(c, params[i], "params[i]"));
        RST_TRY(check_tensor(c, grads[i], "grads[i]"));
        const void* a = params[i]->data; const void* b = grads[i]->data;
        long long ne = params[i]->rows * params[i]->cols;
        key.append((const char*)&a, sizeof a);
        key.append((const char*)&b, sizeof b);
        key.append((const char*)&ne, sizeof ne);
    }
    auto it = c->plan_cache.find(key);
    if (it == c->plan_cache.end()) {
        if (c->plan_cache.size() >= 64) {   // bound the cache; plans are cheap to rebuild
            for (auto& kv : c->plan_cache) rst_sgd_plan_destroy(kv.second);
            c->plan_cache.clear();
        }
        rst_sgd_plan* p = nullptr;
        RST_TRY(rst_sgd_plan_create(c, n, params, grads, &p));
        it = c->plan_cache.emplace(key, p).first;
    }
    return rst_sgd_plan_step(it->second, lr);
}
