// C-ABI entry points of the training-step operators: argument checks, shape
// rules of the reference, and dispatch to the kernels.
#include "common.h"

using namespace rst;

namespace {

int need_ctx(const rst_ctx* c) {
    if (!valid(c)) return fail(nullptr, RST_ERR_INVALID_ARG, "not a live context");
    return RST_OK;
}

int same_shape(const rst_ctx* c, const rst_tensor* a, const rst_tensor* b, const char* what) {
    if (a->rows != b->rows || a->cols != b->cols)
        return fail(c, RST_ERR_SHAPE, "%s: (%lld,%lld) vs (%lld,%lld)", what, (long long)a->rows,
                    (long long)a->cols, (long long)b->rows, (long long)b->cols);
    return RST_OK;
}

}  // namespace

// Y = X · Wᵀ + b, optional fused ReLU          (src/module/linear.rs:43-57, relu.rs:21)
extern "C" int rst_linear_forward(rst_ctx* c, const rst_tensor* X, const rst_tensor* W,
                                  const rst_tensor* b, int relu, rst_tensor* Y) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, X, "X"));
    RST_TRY(check_tensor(c, W, "W"));
    RST_TRY(check_tensor(c, Y, "Y"));
    if (b) RST_TRY(check_tensor(c, b, "b"));
    const int64_t B = X->rows, in = X->cols, out = W->rows;
    if (W->cols != in)
        return fail(c, RST_ERR_SHAPE, "Linear::forward: input (%lld,%lld) against weight (%lld,%lld)",
                    (long long)B, (long long)in, (long long)out, (long long)W->cols);
    if (b && b->rows * b->cols != out)
        return fail(c, RST_ERR_SHAPE, "Linear::forward: bias has %lld elements, expected %lld",
                    (long long)(b->rows * b->cols), (long long)out);
    if (Y->rows != B || Y->cols != out)
        return fail(c, RST_ERR_SHAPE, "Linear::forward: output is (%lld,%lld), expected (%lld,%lld)",
                    (long long)Y->rows, (long long)Y->cols, (long long)B, (long long)out);
    if (Y->data == X->data || Y->data == W->data)
        return fail(c, RST_ERR_INVALID_ARG, "Linear::forward: output aliases an input");
    GemmArgs g{};
    g.A = X->data; g.B = W->data; g.C = Y->data;
    g.M = B; g.N = out; g.K = in;
    g.a_kmajor = true; g.b_kmajor = true;
    g.bias = b ? b->data : nullptr;
    g.epilogue = b ? (relu ? kEpiBiasRelu : kEpiBias) : kEpiNone;
    g.divisor = 1.0;
    {
        ProfScope prof(c, "gemm_fwd");
        RST_TRY(launch_gemm(c, g));
    }
    if (!b && relu) return launch_relu_forward(c, Y->data, Y->data, B * out);
    return RST_OK;
}

// dW = dYᵀ·X / n, db = Σ_rows dY / n, dX = dY·W [* relu mask]   (src/module/linear.rs:60-69, relu.rs:26)
namespace {

int check_linear_backward(rst_ctx* c, const rst_tensor* dY, const rst_tensor* X, const rst_tensor* W,
                          const rst_tensor* mask, rst_tensor* dW, rst_tensor* db, rst_tensor* dX) {
    RST_TRY(check_tensor(c, dY, "dY"));
    RST_TRY(check_tensor(c, X, "X"));
    RST_TRY(check_tensor(c, W, "W"));
    RST_TRY(check_tensor(c, dW, "dW"));
    if (db) RST_TRY(check_tensor(c, db, "db"));
    if (dX) RST_TRY(check_tensor(c, dX, "dX"));
    if (mask) RST_TRY(check_tensor(c, mask, "relu_mask_src"));
    const int64_t B = X->rows, in = X->cols, out = W->rows;
    if (W->cols != in || dY->rows != B || dY->cols != out)
        return fail(c, RST_ERR_SHAPE,
                    "Linear::backward: gradient (%lld,%lld), cached input (%lld,%lld), weight (%lld,%lld)",
                    (long long)dY->rows, (long long)dY->cols, (long long)B, (long long)in,
                    (long long)out, (long long)W->cols);
    RST_TRY(same_shape(c, dW, W, "Linear::backward: dW against W"));
    if (db && db->rows * db->cols != out)
        return fail(c, RST_ERR_SHAPE, "Linear::backward: db has %lld elements, expected %lld",
                    (long long)(db->rows * db->cols), (long long)out);
    if (dX) RST_TRY(same_shape(c, dX, X, "Linear::backward: dX against X"));
    if (mask && !dX) return fail(c, RST_ERR_INVALID_ARG, "relu_mask_src given without dX");
    if (mask) RST_TRY(same_shape(c, mask, X, "Linear::backward: relu_mask_src against X"));
    if (dX && (dX->data == dY->data || dX->data == W->data))
        return fail(c, RST_ERR_INVALID_ARG, "Linear::backward: dX aliases an input");
    return RST_OK;
}

GemmArgs weight_grad_args(const rst_tensor* dY, const rst_tensor* X, rst_tensor* dW, rst_tensor* db) {
    GemmArgs gw{};
    gw.A = dY->data; gw.B = X->data; gw.C = dW->data;
    gw.M = dY->cols; gw.N = X->cols; gw.K = X->rows;
    gw.a_kmajor = false; gw.b_kmajor = false;
    // n = rows(X) (linear.rs:62); times the world size when the ranks of a data-parallel run
    // exchange shares of the global-batch gradient (rst_comm_share_gradients)
    gw.epilogue = kEpiDivN; gw.divisor = (double)X->rows * X->ctx->grad_rows_scale;
    gw.colsum_out = db ? db->data : nullptr;
    return gw;
}

int weight_grad(rst_ctx* c, const rst_tensor* dY, const rst_tensor* X, rst_tensor* dW, rst_tensor* db) {
    const GemmArgs gw = weight_grad_args(dY, X, dW, db);
    bool db_done = false;
    {
        ProfScope prof(c, "gemm_dW");
        RST_TRY(launch_gemm(c, gw, &db_done));
    }
    if (db && !db_done) {
        ProfScope prof(c, "colsum");
        RST_TRY(launch_colsum_div(c, dY->data, X->rows, dY->cols, gw.divisor, db->data));
    }
    return RST_OK;
}

int input_grad(rst_ctx* c, const rst_tensor* dY, const rst_tensor* W, const rst_tensor* mask, rst_tensor* dX) {
    GemmArgs gx{};
    gx.A = dY->data; gx.B = W->data; gx.C = dX->data;
    gx.M = dY->rows; gx.N = W->cols; gx.K = W->rows;
    gx.a_kmajor = true; gx.b_kmajor = false;
    gx.epilogue = mask ? kEpiMask : kEpiNone;
    gx.mask_src = mask ? mask->data : nullptr;
    gx.divisor = 1.0;
    ProfScope prof(c, "gemm_dX");
    return launch_gemm(c, gx);
}

}  // namespace

extern "C" int rst_linear_backward(rst_ctx* c, const rst_tensor* dY, const rst_tensor* X,
                                   const rst_tensor* W, const rst_tensor* mask, rst_tensor* dW,
                                   rst_tensor* db, rst_tensor* dX) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_linear_backward(c, dY, X, W, mask, dW, db, dX));
    RST_TRY(weight_grad(c, dY, X, dW, db));
    if (dX) RST_TRY(input_grad(c, dY, W, mask, dX));
    return RST_OK;
}

extern "C" int rst_transpose(rst_ctx* c, const rst_tensor* src, rst_tensor* dst) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, src, "src"));
    RST_TRY(check_tensor(c, dst, "dst"));
    if (dst->rows != src->cols || dst->cols != src->rows)
        return fail(c, RST_ERR_SHAPE, "transpose of (%lld,%lld) into (%lld,%lld)", (long long)src->rows,
                    (long long)src->cols, (long long)dst->rows, (long long)dst->cols);
    if (dst->data == src->data) return fail(c, RST_ERR_INVALID_ARG, "transpose in place");
    return launch_transpose(c, src->data, src->rows, src->cols, dst->data);
}

// Linear::backward with transposed companions of the gradients.  The dX product is fastest
// when both of its operands are stored with the reduction index outermost: W [out][in] is,
// dY [B][out] is not, its transpose [out][B] is.  A caller that holds dYᵀ passes it, and
// asks for dXᵀ next to dX so that the layer below can do the same.
extern "C" int rst_linear_backward_t(rst_ctx* c, const rst_tensor* dY, const rst_tensor* dY_t,
                                     const rst_tensor* X, const rst_tensor* W, const rst_tensor* mask,
                                     rst_tensor* dW, rst_tensor* db, rst_tensor* dX, rst_tensor* dX_t) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_linear_backward(c, dY, X, W, mask, dW, db, dX));
    if (dY_t) {
        RST_TRY(check_tensor(c, dY_t, "dY_t"));
        if (dY_t->rows != dY->cols || dY_t->cols != dY->rows)
            return fail(c, RST_ERR_SHAPE, "Linear::backward: dY_t is (%lld,%lld), expected (%lld,%lld)",
                        (long long)dY_t->rows, (long long)dY_t->cols, (long long)dY->cols, (long long)dY->rows);
    }
    if (dX_t) {
        if (!dX) return fail(c, RST_ERR_INVALID_ARG, "dX_t given without dX");
        RST_TRY(check_tensor(c, dX_t, "dX_t"));
        if (dX_t->rows != dX->cols || dX_t->cols != dX->rows)
            return fail(c, RST_ERR_SHAPE, "Linear::backward: dX_t is (%lld,%lld), expected (%lld,%lld)",
                        (long long)dX_t->rows, (long long)dX_t->cols, (long long)dX->cols, (long long)dX->rows);
        if (dX_t->data == dX->data || dX_t->data == dY->data || dX_t->data == W->data)
            return fail(c, RST_ERR_INVALID_ARG, "Linear::backward: dX_t aliases another operand");
    }
    RST_TRY(weight_grad(c, dY, X, dW, db));
    if (!dX) return RST_OK;
    if (!dY_t) {
        RST_TRY(input_grad(c, dY, W, mask, dX));
    } else {
        GemmArgs gx{};
        gx.A = dY_t->data; gx.B = W->data; gx.C = dX->data;         // dX[B,in] = (dYᵀ)ᵀ · W
        gx.M = dY->rows; gx.N = W->cols; gx.K = W->rows;
        gx.a_kmajor = false; gx.b_kmajor = false;
        gx.epilogue = mask ? kEpiMask : kEpiNone;
        gx.mask_src = mask ? mask->data : nullptr;
        gx.divisor = 1.0;
        gx.C_transposed = dX_t ? dX_t->data : nullptr;
        const bool fused_copy = dX_t && gemm_writes_transposed(c, gx);
        if (!fused_copy) gx.C_transposed = nullptr;
        {
            ProfScope prof(c, "gemm_dX");
            RST_TRY(launch_gemm(c, gx));
        }
        if (!dX_t || fused_copy) return RST_OK;
    }
    if (dX_t) RST_TRY(launch_transpose(c, dX->data, dX->rows, dX->cols, dX_t->data));
    return RST_OK;
}

// Sequential::backward over n Linear layers (src/module/sequential.rs:88-94 folding
// linear.rs:60-69, with relu.rs:26 for the ReLUs in between).  The dX products form a
// dependent chain and run first; the dW/db products only read that chain's tensors and
// go out together.
extern "C" int rst_linear_backward_chain(rst_ctx* c, int n, const rst_tensor* dY, const rst_tensor* const* X,
                                         const rst_tensor* const* W, const unsigned char* relu_mask,
                                         rst_tensor* const* dW, rst_tensor* const* db,
                                         rst_tensor* const* dX) {
    RST_TRY(need_ctx(c));
    if (n < 1 || !X || !W || !dW || !dX) return fail(c, RST_ERR_INVALID_ARG, "Linear backward chain: bad arguments");
    for (int l = n - 1; l >= 0; --l) {
        if (l > 0 && !dX[l])
            return fail(c, RST_ERR_INVALID_ARG, "Linear backward chain: dX[%d] is needed by layer %d", l, l - 1);
        const rst_tensor* g = (l == n - 1) ? dY : dX[l + 1];
        const rst_tensor* mask = (relu_mask && relu_mask[l] && dX[l]) ? X[l] : nullptr;
        RST_TRY(check_linear_backward(c, g, X[l], W[l], mask, dW[l], db ? db[l] : nullptr, dX[l]));
    }
    for (int l = n - 1; l >= 0; --l) {
        if (!dX[l]) continue;
        const rst_tensor* g = (l == n - 1) ? dY : dX[l + 1];
        RST_TRY(input_grad(c, g, W[l], (relu_mask && relu_mask[l]) ? X[l] : nullptr, dX[l]));
    }
    constexpr int kChunk = 4;
    for (int hi = n - 1; hi >= 0; hi -= kChunk) {
        const int lo = hi - kChunk + 1 > 0 ? hi - kChunk + 1 : 0;
        GemmArgs group[kChunk];
        int m = 0;
        for (int l = hi; l >= lo; --l) {
            const rst_tensor* g = (l == n - 1) ? dY : dX[l + 1];
            rst_tensor* dbl = db ? db[l] : nullptr;
            if (!dbl) { m = 0; break; }             // the grouped kernel always produces db
            group[m++] = weight_grad_args(g, X[l], dW[l], dbl);
        }
        bool grouped = false;
        if (m >= 2) {
            ProfScope prof(c, "gemm_dW");
            RST_TRY(launch_gemm_group(c, group, m, &grouped));
        }
        if (!grouped)
            for (int l = hi; l >= lo; --l)
                RST_TRY(weight_grad(c, (l == n - 1) ? dY : dX[l + 1], X[l], dW[l], db ? db[l] : nullptr));
    }
    return RST_OK;
}

// Self-test of the bounded device-side waits.  One small product (64x64x64) is launched
// with its producer disabled, so no tile is ever copied: every consumer warp's wait on the
// first stage runs out after `limit_cycles`, the kernel writes the device status word,
// stores nothing and returns with no copy in flight.  The next rst_ctx_check_device then
// reports RST_ERR_DEVICE_TIMEOUT and clears the word; the context stays usable.
extern "C" int rst_selftest_wait_expiry(rst_ctx* c, int64_t limit_cycles) {
    RST_TRY(need_ctx(c));
    if (limit_cycles < 1 || limit_cycles > 100000000LL)
        return fail(c, RST_ERR_INVALID_ARG, "limit_cycles must be in [1, 1e8] (at most a twentieth of a second)");
    if (c->capturing) return fail(c, RST_ERR_STATE, "self-test during graph capture");
    rst_tensor *A = nullptr, *B = nullptr, *C = nullptr;
    int s = rst_tensor_alloc(c, 64, 64, &A);
    if (s == RST_OK) s = rst_tensor_alloc(c, 64, 64, &B);
    if (s == RST_OK) s = rst_tensor_alloc(c, 64, 64, &C);
    if (s == RST_OK) {
        GemmArgs g{};
        g.A = A->data; g.B = B->data; g.C = C->data;
        g.M = 64; g.N = 64; g.K = 64;
        g.a_kmajor = true; g.b_kmajor = true;
        g.epilogue = kEpiNone; g.divisor = 1.0;
        g.wait_limit_cycles = limit_cycles;
        g.starve_producer = true;
        s = launch_gemm(c, g);
    }
    rst_tensor_free(A); rst_tensor_free(B); rst_tensor_free(C);   // stream-ordered reuse
    return s;
}

extern "C" int rst_relu_forward(rst_ctx* c, const rst_tensor* X, rst_tensor* Y) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, X, "X"));
    RST_TRY(check_tensor(c, Y, "Y"));
    RST_TRY(same_shape(c, X, Y, "ReLU::forward"));
    ProfScope prof(c, "relu_fwd");
    return launch_relu_forward(c, X->data, Y->data, X->rows * X->cols);
}

extern "C" int rst_relu_backward(rst_ctx* c, const rst_tensor* dY, const rst_tensor* Xpre,
                                 rst_tensor* dX) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, dY, "dY"));
    RST_TRY(check_tensor(c, Xpre, "X_pre"));
    RST_TRY(check_tensor(c, dX, "dX"));
    RST_TRY(same_shape(c, dY, Xpre, "ReLU::backward: gradient against cached input"));
    RST_TRY(same_shape(c, dY, dX, "ReLU::backward: output"));
    ProfScope prof(c, "relu_bwd");
    return launch_relu_backward(c, dY->data, Xpre->data, dX->data, dY->rows * dY->cols);
}

extern "C" int rst_softmax(rst_ctx* c, const rst_tensor* X, rst_tensor* P) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, X, "X"));
    RST_TRY(check_tensor(c, P, "P"));
    RST_TRY(same_shape(c, X, P, "softmax"));
    if (X->cols > 0x7fffffff) return fail(c, RST_ERR_UNSUPPORTED, "more than 2^31 columns");
    return launch_softmax(c, X->data, P->data, X->rows, X->cols);
}

// Softmax module, forward over axis 0 (src/module/activation/softmax.rs:21-27,45-53).
extern "C" int rst_softmax_axis0(rst_ctx* c, const rst_tensor* X, rst_tensor* P) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, X, "X"));
    RST_TRY(check_tensor(c, P, "P"));
    RST_TRY(same_shape(c, X, P, "softmax"));
    return launch_softmax_axis0(c, X->data, P->data, X->rows, X->cols);
}

// Softmax::backward (src/module/activation/softmax.rs:62-75), kept exactly as the
// reference computes it: jacobian = -(outputᵀ·output) over the whole batch, its diagonal
// replaced by s(1-s) with s = Σ_b output[b][j]², result = gradient · jacobian.
extern "C" int rst_softmax_backward(rst_ctx* c, const rst_tensor* output, const rst_tensor* gradient,
                                    rst_tensor* dX) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, output, "output"));
    RST_TRY(check_tensor(c, gradient, "gradient"));
    RST_TRY(check_tensor(c, dX, "dX"));
    const int64_t B = output->rows, C = output->cols;
    if (gradient->cols != C)
        return fail(c, RST_ERR_SHAPE, "Softmax::backward: gradient (%lld,%lld) against output (%lld,%lld)",
                    (long long)gradient->rows, (long long)gradient->cols, (long long)B, (long long)C);
    if (dX->rows != gradient->rows || dX->cols != C)
        return fail(c, RST_ERR_SHAPE, "Softmax::backward: result must be (%lld,%lld)", (long long)gradient->rows,
                    (long long)C);
    rst_tensor* J = nullptr;
    RST_TRY(rst_tensor_alloc(c, C, C, &J));
    GemmArgs gj{};                                   // -(Oᵀ·O): both operands are `output`, reduced over the batch
    gj.A = output->data; gj.B = output->data; gj.C = J->data;
    gj.M = C; gj.N = C; gj.K = B;
    gj.a_kmajor = false; gj.b_kmajor = false;
    gj.epilogue = kEpiDivN; gj.divisor = -1.0;
    int s = launch_gemm(c, gj);
    if (s == RST_OK) s = launch_softmax_jacobian_diag(c, J->data, C);
    if (s == RST_OK) {
        GemmArgs gx{};                               // gradient · jacobian
        gx.A = gradient->data; gx.B = J->data; gx.C = dX->data;
        gx.M = gradient->rows; gx.N = C; gx.K = C;
        gx.a_kmajor = true; gx.b_kmajor = false;
        gx.epilogue = kEpiNone; gx.divisor = 1.0;
        s = launch_gemm(c, gx);
    }
    rst_tensor_free(J);      // stream-ordered: the block is reused only by later launches
    return s;
}

extern "C" int rst_xent_slots(void) { return kXentSlots; }

extern "C" int rst_xent_forward_backward(rst_ctx* c, const rst_tensor* logits, const rst_tensor* truth,
                                         rst_tensor* dlogits, int slot) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, logits, "logits"));
    RST_TRY(check_tensor(c, truth, "truth"));
    if (dlogits) RST_TRY(check_tensor(c, dlogits, "dlogits"));
    if (slot < 0 || slot >= kXentSlots)
        return fail(c, RST_ERR_INVALID_ARG, "slot %d out of range [0,%d)", slot, kXentSlots);
    RST_TRY(same_shape(c, logits, truth, "CrossEntropyLoss::forward: pred against truth"));
    if (dlogits) RST_TRY(same_shape(c, logits, dlogits, "CrossEntropyLoss::backward: output"));
    if (logits->cols == 0) return fail(c, RST_ERR_SHAPE, "CrossEntropyLoss: zero classes");
    if (logits->cols > 0x7fffffff) return fail(c, RST_ERR_UNSUPPORTED, "more than 2^31 columns");
    {
        ProfScope prof(c, "xent");
        RST_TRY(launch_xent(c, logits->data, truth->data, dlogits ? dlogits->data : nullptr, logits->rows,
                            logits->cols, c->d_results + slot));
    }
    RST_CUDA(c, cudaMemcpyAsync(c->h_results + slot, c->d_results + slot, sizeof(ResultSlot),
                                cudaMemcpyDeviceToHost, c->compute));
    if (c->capturing) {
        c->result_pending[slot] = true;   // replayed by a graph: read after a stream sync
        c->result_in_graph[slot] = true;
    } else {
        RST_CUDA(c, cudaEventRecord(c->result_event[slot], c->compute));
        c->result_pending[slot] = true;
        c->result_in_graph[slot] = false;
    }
    return RST_OK;
}

extern "C" int rst_xent_result(rst_ctx* c, int slot, double* loss, double* accuracy) {
    RST_TRY(need_ctx(c));
    if (slot < 0 || slot >= kXentSlots)
        return fail(c, RST_ERR_INVALID_ARG, "slot %d out of range [0,%d)", slot, kXentSlots);
    if (!c->result_pending[slot])
        return fail(c, RST_ERR_STATE, "result slot %d was never written (forward not called)", slot);
    if (c->capturing) return fail(c, RST_ERR_STATE, "blocking read during graph capture");
    if (c->result_in_graph[slot]) RST_CUDA(c, cudaStreamSynchronize(c->compute));
    else RST_CUDA(c, cudaEventSynchronize(c->result_event[slot]));
    const ResultSlot r = c->h_results[slot];
    // loss = -(Σ t·ln p) / B                               (src/loss/cross_entropy.rs:38)
    if (loss) *loss = -r.loss_sum / r.rows;
    // accuracy = correct / rows                             (src/utils.rs:59-64)
    if (accuracy) *accuracy = r.correct / r.rows;
    if (r.nan_rows > 0.0)
        return fail(c, RST_ERR_NAN, "%lld row(s) of the logits hold NaN; the reference panics in softmax",
                    (long long)r.nan_rows);
    return RST_OK;
}

extern "C" int rst_argmax(rst_ctx* c, const rst_tensor* t, int64_t* idx) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, t, "t"));
    if (c->capturing) return fail(c, RST_ERR_STATE, "blocking call during graph capture");
    if (t->rows == 0) return RST_OK;
    if (!idx) return fail(c, RST_ERR_INVALID_ARG, "idx is NULL");
    if (t->cols == 0) return fail(c, RST_ERR_SHAPE, "argmax of rows with zero columns");
    if (t->cols > 0x7fffffff) return fail(c, RST_ERR_UNSUPPORTED, "more than 2^31 columns");
    rst_tensor* tmp = nullptr;   // rows int64 values fit a (rows,1) f64 block
    RST_TRY(rst_tensor_alloc(c, t->rows, 1, &tmp));
    int s = launch_argmax(c, t->data, t->rows, t->cols, reinterpret_cast<long long*>(tmp->data));
    if (s == RST_OK) {
        cudaError_t e = cudaMemcpyAsync(idx, tmp->data, (size_t)t->rows * sizeof(int64_t),
                                        cudaMemcpyDeviceToHost, c->compute);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->compute);
        if (e != cudaSuccess) s = fail(c, RST_ERR_CUDA, "argmax read-back failed: %s", cudaGetErrorString(e));
    }
    rst_tensor_free(tmp);
    return s;
}

extern "C" int rst_accuracy(rst_ctx* c, const rst_tensor* pred, const rst_tensor* truth, double* acc) {
    RST_TRY(need_ctx(c));
    RST_TRY(check_tensor(c, pred, "pred"));
    RST_TRY(check_tensor(c, truth, "truth"));
    if (!acc) return fail(c, RST_ERR_INVALID_ARG, "acc is NULL");
    if (pred->rows != truth->rows)
        return fail(c, RST_ERR_SHAPE, "accuracy: %lld predictions against %lld targets",
                    (long long)pred->rows, (long long)truth->rows);
    std::vector<int64_t> a((size_t)pred->rows), b((size_t)truth->rows);
    RST_TRY(rst_argmax(c, pred, a.data()));
    RST_TRY(rst_argmax(c, truth, b.data()));
    int64_t hit = 0;
    for (size_t i = 0; i < a.size(); ++i) hit += (a[i] == b[i]);
    *acc = (double)hit / (double)pred->rows;
    return RST_OK;
}
