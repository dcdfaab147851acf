// Data-parallel gradient exchange over NCCL (NVLink 5 / NVSwitch inside a box).
// The reference is single-threaded and has no counterpart; sharding the batch
// over G GPUs needs one exchange per step: the average over ranks of every
// dW/db, because Linear::backward divides by the local row count
// (src/module/linear.rs:62-66) and avg_g(dY_gᵀX_g / (B/G)) = dYᵀX / B.
//
// NCCL is resolved at run time (dlopen) so the library loads on hosts without
// it and shares whichever libnccl the process already has.
#include <dlfcn.h>
#include <nvtx3/nvToolsExt.h>

#include <cstring>

#include "common.h"

namespace {

// Minimal mirror of the NCCL C API (stable since 2.10, the release that added
// the averaging reduction).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat64 = 8 };
enum { ncclSum = 0, ncclAvg = 4 };

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(ncclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*GetVersion)(int*) = nullptr;
    std::string error;
};

NcclApi& nccl() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle) break;
    }
    if (!api.handle) {
        api.error = std::string("cannot load libnccl.so.2: ") + (dlerror() ? dlerror() : "unknown");
        return api;
    }
#define LOAD(field, sym)                                                         \
    *(void**)(&api.field) = dlsym(api.handle, sym);                              \
    if (!api.field) { api.error = std::string("libnccl lacks ") + sym; api.handle = nullptr; return api; }
    LOAD(GetUniqueId, "ncclGetUniqueId")
    LOAD(CommInitRank, "ncclCommInitRank")
    LOAD(CommDestroy, "ncclCommDestroy")
    LOAD(AllReduce, "ncclAllReduce")
    LOAD(GroupStart, "ncclGroupStart")
    LOAD(GroupEnd, "ncclGroupEnd")
    LOAD(GetErrorString, "ncclGetErrorString")
    LOAD(GetVersion, "ncclGetVersion")
#undef LOAD
    return api;
}

}  // namespace

using namespace rst;

struct rst_comm {
    rst_ctx* ctx;
    ncclComm_t comm;
    int rank, world;
    cudaEvent_t ready;   // compute -> comm
    cudaEvent_t done;    // comm -> compute
    bool pending;
    bool shares;         // gradients arrive divided by the global batch: the exchange sums them
};

static_assert(RST_COMM_ID_BYTES == sizeof(ncclUniqueId), "id size");

extern "C" int rst_comm_get_id(void* id_bytes) {
    if (!id_bytes) return fail(nullptr, RST_ERR_INVALID_ARG, "id_bytes is NULL");
    NcclApi& api = nccl();
    if (!api.handle) return fail(nullptr, RST_ERR_NCCL, "%s", api.error.c_str());
    ncclUniqueId id;
    int r = api.GetUniqueId(&id);
    if (r != ncclSuccess) return fail(nullptr, RST_ERR_NCCL, "ncclGetUniqueId: %s", api.GetErrorString(r));
    std::memcpy(id_bytes, &id, sizeof id);
    return RST_OK;
}

extern "C" int rst_comm_create(rst_ctx* c, const void* id_bytes, int rank, int world, rst_comm** out) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!out || !id_bytes || world < 1 || rank < 0 || rank >= world)
        return fail(c, RST_ERR_INVALID_ARG, "bad communicator arguments (rank %d of %d)", rank, world);
    *out = nullptr;
    NcclApi& api = nccl();
    if (!api.handle) return fail(c, RST_ERR_NCCL, "%s", api.error.c_str());
    RST_CUDA(c, cudaSetDevice(c->device));
    ncclUniqueId id;
    std::memcpy(&id, id_bytes, sizeof id);
    ncclComm_t comm = nullptr;
    int r = api.CommInitRank(&comm, world, id, rank);
    if (r != ncclSuccess) return fail(c, RST_ERR_NCCL, "ncclCommInitRank: %s", api.GetErrorString(r));
    rst_comm* m = new rst_comm{c, comm, rank, world, nullptr, nullptr, false, false};
    if (cudaEventCreateWithFlags(&m->ready, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->done, cudaEventDisableTiming) != cudaSuccess) {
        api.CommDestroy(comm);
        delete m;
        return fail(c, RST_ERR_CUDA, "cannot create communicator events");
    }
    *out = m;
    return RST_OK;
}

// With `on`, Linear::backward of the communicator's context divides dW and db by
// rows(X) * world instead of rows(X): every rank then holds its share of the global-batch
// gradient, and rst_allreduce_avg adds the shares up (a plain sum, which NCCL can hand to
// the switch's in-network reduction; an average cannot go there because every rank's input
// would have to be scaled first).  The result is the same average, bit for bit when the world
// size is a power of two (dividing by 2^k commutes with rounding), to the last place otherwise.
extern "C" int rst_comm_share_gradients(rst_comm* m, int on) {
    if (!m || !valid(m->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad communicator");
    if (m->ctx->capturing) return fail(m->ctx, RST_ERR_STATE, "mode change during graph capture");
    m->shares = on != 0;
    m->ctx->grad_rows_scale = m->shares ? (double)m->world : 1.0;
    return RST_OK;
}

extern "C" int rst_comm_destroy(rst_comm* m) {
    if (!m) return RST_OK;
    if (valid(m->ctx) && m->shares) m->ctx->grad_rows_scale = 1.0;
    if (valid(m->ctx)) {
        cudaStreamSynchronize(m->ctx->comm);
        cudaStreamSynchronize(m->ctx->compute);
    }
    NcclApi& api = nccl();
    if (api.handle && m->comm) api.CommDestroy(m->comm);
    if (m->ready) cudaEventDestroy(m->ready);
    if (m->done) cudaEventDestroy(m->done);
    delete m;
    return RST_OK;
}

extern "C" int rst_allreduce_avg(rst_comm* m, int n, rst_tensor* const* tensors) {
    if (!m || !valid(m->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad communicator");
    rst_ctx* c = m->ctx;
    if (n < 0 || (n > 0 && !tensors)) return fail(c, RST_ERR_INVALID_ARG, "bad argument");
    for (int i = 0; i < n; ++i) RST_TRY(check_tensor(c, tensors[i], "tensors[i]"));
    if (n == 0) return RST_OK;
    NcclApi& api = nccl();
    struct Range { Range() { nvtxRangePushA("allreduce_avg"); } ~Range() { nvtxRangePop(); } } range;
    // the exchange starts once the gradients queued so far on the compute stream exist
    RST_CUDA(c, cudaEventRecord(m->ready, c->compute));
    RST_CUDA(c, cudaStreamWaitEvent(c->comm, m->ready, 0));
    int r = api.GroupStart();
    if (r != ncclSuccess) return fail(c, RST_ERR_NCCL, "ncclGroupStart: %s", api.GetErrorString(r));
    for (int i = 0; i < n; ++i) {
        size_t count = (size_t)(tensors[i]->rows * tensors[i]->cols);
        if (count == 0) continue;
        r = api.AllReduce(tensors[i]->data, tensors[i]->data, count, ncclFloat64, m->shares ? ncclSum : ncclAvg, m->comm,
                          c->comm);
        if (r != ncclSuccess) {
            api.GroupEnd();
            return fail(c, RST_ERR_NCCL, "ncclAllReduce: %s", api.GetErrorString(r));
        }
    }
    r = api.GroupEnd();
    if (r != ncclSuccess) return fail(c, RST_ERR_NCCL, "ncclGroupEnd: %s", api.GetErrorString(r));
    RST_CUDA(c, cudaEventRecord(m->done, c->comm));
    m->pending = true;
    return RST_OK;
}

extern "C" int rst_comm_join(rst_comm* m) {
    if (!m || !valid(m->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad communicator");
    if (m->pending) {
        RST_CUDA(m->ctx, cudaStreamWaitEvent(m->ctx->compute, m->done, 0));
        m->pending = false;
    }
    return RST_OK;
}
