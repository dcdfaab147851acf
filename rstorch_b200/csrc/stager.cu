// Pinned-host batch staging on a side stream: the device-side counterpart of
// ArrayDataLoaderIter::next (src/data/data_loader.rs:180-208), which assembles
// `batch` samples into one (batch, features) and one (batch, classes) array.
// Here the loader writes the rows into a pinned slot, the copy stream moves the
// slot to HBM while the compute stream works on the previous batch.
#include "common.h"

using namespace rst;

struct rst_stager {
    rst_ctx* ctx;
    int64_t batch, x_cols, t_cols;
    int slots;
    std::vector<double*> hx, ht;           // pinned
    std::vector<rst_tensor*> dx, dt;       // device
    std::vector<cudaEvent_t> copied;       // H2D of the slot finished
    std::vector<cudaEvent_t> consumed;     // compute work that reads the slot was queued up to here
    std::vector<char> submitted, acquired, consumed_marked;
};

extern "C" int rst_stager_destroy(rst_stager* s);

extern "C" int rst_stager_create(rst_ctx* c, int64_t batch, int64_t x_cols, int64_t t_cols, int slots,
                                 rst_stager** out) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    if (!out || batch <= 0 || x_cols <= 0 || t_cols <= 0 || slots < 1 || slots > 16)
        return fail(c, RST_ERR_INVALID_ARG, "bad stager geometry");
    *out = nullptr;
    if (c->capturing) return fail(c, RST_ERR_STATE, "stager creation during graph capture");
    rst_stager* s = new rst_stager{c, batch, x_cols, t_cols, slots};
    for (int i = 0; i < slots; ++i) {
        double *hx = nullptr, *ht = nullptr;
        rst_tensor *dx = nullptr, *dt = nullptr;
        cudaEvent_t e1 = nullptr, e2 = nullptr;
        bool okay = cudaMallocHost((void**)&hx, (size_t)batch * x_cols * sizeof(double)) == cudaSuccess;
        s->hx.push_back(hx);
        okay = okay && cudaMallocHost((void**)&ht, (size_t)batch * t_cols * sizeof(double)) == cudaSuccess;
        s->ht.push_back(ht);
        okay = okay && rst_tensor_alloc(c, batch, x_cols, &dx) == RST_OK;
        s->dx.push_back(dx);
        okay = okay && rst_tensor_alloc(c, batch, t_cols, &dt) == RST_OK;
        s->dt.push_back(dt);
        okay = okay && cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) == cudaSuccess;
        s->copied.push_back(e1);
        okay = okay && cudaEventCreateWithFlags(&e2, cudaEventDisableTiming) == cudaSuccess;
        s->consumed.push_back(e2);
        s->submitted.push_back(0);
        s->acquired.push_back(0);
        s->consumed_marked.push_back(0);
        if (!okay) {
            cudaGetLastError();
            std::string why = c->last_error;
            rst_stager_destroy(s);
            return fail(c, RST_ERR_OOM, "cannot allocate staging slot %d (%s)", i, why.c_str());
        }
    }
    *out = s;
    return RST_OK;
}

extern "C" int rst_stager_destroy(rst_stager* s) {
    if (!s) return RST_OK;
    if (valid(s->ctx)) {
        cudaStreamSynchronize(s->ctx->copy);
        cudaStreamSynchronize(s->ctx->compute);
    }
    for (double* p : s->hx) if (p) cudaFreeHost(p);
    for (double* p : s->ht) if (p) cudaFreeHost(p);
    for (rst_tensor* t : s->dx) if (t) rst_tensor_free(t);
    for (rst_tensor* t : s->dt) if (t) rst_tensor_free(t);
    for (cudaEvent_t e : s->copied) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : s->consumed) if (e) cudaEventDestroy(e);
    delete s;
    return RST_OK;
}

extern "C" int rst_stager_host(rst_stager* s, int slot, double** x_host, double** t_host) {
    if (!s || !valid(s->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad stager");
    if (slot < 0 || slot >= s->slots) return fail(s->ctx, RST_ERR_INVALID_ARG, "slot %d out of range", slot);
    // The previous copy out of this pinned slot must have finished before the
    // loader overwrites it.
    if (s->submitted[slot]) RST_CUDA(s->ctx, cudaEventSynchronize(s->copied[slot]));
    if (x_host) *x_host = s->hx[slot];
    if (t_host) *t_host = s->ht[slot];
    return RST_OK;
}

extern "C" int rst_stager_submit(rst_stager* s, int slot) {
    if (!s || !valid(s->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad stager");
    rst_ctx* c = s->ctx;
    if (slot < 0 || slot >= s->slots) return fail(c, RST_ERR_INVALID_ARG, "slot %d out of range", slot);
    // Do not overwrite the device tensors while compute work queued after the
    // last acquire of this slot may still read them.
    // The mark is normally recorded when the next slot is acquired; with a
    // single slot (or a slot resubmitted straight away) it is recorded here.
    if (s->acquired[slot]) {
        if (!s->consumed_marked[slot]) RST_CUDA(c, cudaEventRecord(s->consumed[slot], c->compute));
        RST_CUDA(c, cudaStreamWaitEvent(c->copy, s->consumed[slot], 0));
    }
    RST_CUDA(c, cudaMemcpyAsync(s->dx[slot]->data, s->hx[slot], (size_t)s->batch * s->x_cols * sizeof(double),
                                cudaMemcpyHostToDevice, c->copy));
    RST_CUDA(c, cudaMemcpyAsync(s->dt[slot]->data, s->ht[slot], (size_t)s->batch * s->t_cols * sizeof(double),
                                cudaMemcpyHostToDevice, c->copy));
    RST_CUDA(c, cudaEventRecord(s->copied[slot], c->copy));
    s->submitted[slot] = 1;
    s->acquired[slot] = 0;
    s->consumed_marked[slot] = 0;
    return RST_OK;
}

extern "C" int rst_stager_acquire(rst_stager* s, int slot, rst_tensor** X, rst_tensor** T) {
    if (!s || !valid(s->ctx)) return fail(nullptr, RST_ERR_INVALID_ARG, "bad stager");
    rst_ctx* c = s->ctx;
    if (slot < 0 || slot >= s->slots) return fail(c, RST_ERR_INVALID_ARG, "slot %d out of range", slot);
    if (!s->submitted[slot]) return fail(c, RST_ERR_STATE, "slot %d was not submitted", slot);
    if (c->capturing) return fail(c, RST_ERR_STATE, "acquire during graph capture");
    // Mark how far compute had been queued for the slot handed out before this
    // one: every other acquired slot's readers are in the stream by now.
    for (int i = 0; i < s->slots; ++i)
        if (i != slot && s->acquired[i] && !s->consumed_marked[i]) {
            RST_CUDA(c, cudaEventRecord(s->consumed[i], c->compute));
            s->consumed_marked[i] = 1;
        }
    RST_CUDA(c, cudaStreamWaitEvent(c->compute, s->copied[slot], 0));
    s->acquired[slot] = 1;
    if (X) *X = s->dx[slot];
    if (T) *T = s->dt[slot];
    return RST_OK;
}
