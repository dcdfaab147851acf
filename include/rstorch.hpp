// rstorch.hpp — C++17 host-side façade over the C ABI of librstorch_b200.so.
//
// Mirrors the public API of the `rstorch` crate for its training step, with the
// same names, argument meaning and failure behaviour (where the crate panics,
// these classes throw rstorch::Panic):
//   Module / Parameter / Parameters   src/module/mod.rs:16-56
//   Linear, InitParameters, KaimingNormal
//                                     src/module/linear.rs, src/module/init/{mod,he}.rs
//   ReLU, Identity                    src/module/activation/{relu,identity}.rs
//   Sequential, sequential(...)       src/module/sequential.rs
//   Loss, CrossEntropyLoss            src/loss/{mod,cross_entropy}.rs
//   Optimizer, SGD                    src/optim/{mod,sgd}.rs
//   accuracy, argmax, one_hot         src/utils.rs:38-65
//   DataLoader::iter_array            src/data/data_loader.rs:42-93,180-208
// Tensors are device matrices; `Tensor` is a shared handle (a move in the Rust API
// becomes a cheap copy of the handle here).  Header only; link with -lrstorch_b200.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <typeinfo>
#include <utility>
#include <vector>

#include "rstorch_b200.h"

namespace rstorch {

struct Panic : std::runtime_error {
    int status;
    Panic(int s, const std::string& m) : std::runtime_error(m), status(s) {}
};

inline void check(const rst_ctx* ctx, int status) {
    if (status != RST_OK) {
        const char* m = rst_last_error(ctx);
        throw Panic(status, std::string(rst_status_string(status)) + ": " + (m ? m : ""));
    }
}

class Context {
public:
    explicit Context(int device = 0) { check(nullptr, rst_ctx_create(device, &h_)); }
    ~Context() { if (h_) rst_ctx_destroy(h_); }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
    rst_ctx* handle() const { return h_; }
    void synchronize() { check(h_, rst_ctx_synchronize(h_)); }
    void check_device() { check(h_, rst_ctx_check_device(h_)); }
private:
    rst_ctx* h_ = nullptr;
};

// Device `Array2<f64>`: rows x cols, row-major.
class Tensor {
public:
    Tensor() = default;
    Tensor(Context& ctx, int64_t rows, int64_t cols) : ctx_(ctx.handle()), rows_(rows), cols_(cols) {
        rst_tensor* t = nullptr;
        check(ctx_, rst_tensor_alloc(ctx_, rows, cols, &t));
        h_ = std::shared_ptr<rst_tensor>(t, [](rst_tensor* p) { rst_tensor_free(p); });
    }
    Tensor(Context& ctx, int64_t rows, int64_t cols, const std::vector<double>& host) : Tensor(ctx, rows, cols) {
        if ((int64_t)host.size() != rows * cols) throw Panic(RST_ERR_SHAPE, "host buffer does not match the shape");
        check(ctx_, rst_tensor_upload(h_.get(), host.data()));
    }
    // Borrowed handle that something else owns (e.g. a staging slot).
    static Tensor borrowed(rst_ctx* ctx, rst_tensor* t) {
        Tensor out;
        out.ctx_ = ctx;
        out.h_ = std::shared_ptr<rst_tensor>(t, [](rst_tensor*) {});
        check(ctx, rst_tensor_shape(t, &out.rows_, &out.cols_));
        return out;
    }
    static Tensor like(const Tensor& o, int64_t rows, int64_t cols) {
        Tensor out;
        out.ctx_ = o.ctx_; out.rows_ = rows; out.cols_ = cols;
        rst_tensor* t = nullptr;
        check(o.ctx_, rst_tensor_alloc(o.ctx_, rows, cols, &t));
        out.h_ = std::shared_ptr<rst_tensor>(t, [](rst_tensor* p) { rst_tensor_free(p); });
        return out;
    }
    std::vector<double> to_host() const {
        std::vector<double> v((size_t)(rows_ * cols_));
        check(ctx_, rst_tensor_download(h_.get(), v.data()));
        return v;
    }
    explicit operator bool() const { return (bool)h_; }
    rst_tensor* handle() const { return h_.get(); }
    rst_ctx* ctx() const { return ctx_; }
    int64_t nrows() const { return rows_; }
    int64_t ncols() const { return cols_; }
private:
    std::shared_ptr<rst_tensor> h_;
    rst_ctx* ctx_ = nullptr;
    int64_t rows_ = 0, cols_ = 0;
};

struct Parameter {   // module/mod.rs:16-19
    Tensor parm;
    Tensor grad;
};
using Parameters = std::vector<Parameter>;

class Module {       // module/mod.rs:42-56
public:
    virtual ~Module() = default;
    virtual Tensor forward(Tensor input) = 0;       // (batch, in)  -> (batch, out)
    virtual Tensor backward(Tensor gradient) = 0;   // (batch, out) -> (batch, in)
    virtual Parameters parameters() { return {}; }
    virtual void train() {}
    virtual void eval() {}
};

// module/init/mod.rs:11-18: weight is (output_size, input_size) row-major, bias (1, output_size).
class InitParameters {
public:
    virtual ~InitParameters() = default;
    virtual std::vector<double> weight(size_t input_size, size_t output_size) const = 0;
    virtual std::vector<double> bias(size_t, size_t output_size) const { return std::vector<double>(output_size, 0.0); }
};

// module/init/he.rs:9-15: N(0, 1/sqrt(input_size)); the stream is the library's seeded generator.
class KaimingNormal : public InitParameters {
public:
    explicit KaimingNormal(uint64_t key = 0x9E3779B97F4A7C15ull) : key_(key) {}
    std::vector<double> weight(size_t input_size, size_t output_size) const override {
        std::vector<double> w(input_size * output_size);
        check(nullptr, rst_synth_normal(key_ + calls_++, w.size(), 0, 0.0, 1.0 / std::sqrt((double)input_size), w.data()));
        return w;
    }
private:
    uint64_t key_;
    mutable uint64_t calls_ = 0;
};

// The initialiser of a Linear built without one: a single shared instance whose stream
// index advances with every weight matrix it hands out, so that successive layers draw
// independent weights as they do from the reference's thread generator (he.rs:13).
inline const KaimingNormal& default_init() {
    static const KaimingNormal shared;
    return shared;
}

class Identity : public Module {   // activation/identity.rs:15-29
public:
    Tensor forward(Tensor input) override { return input; }
    Tensor backward(Tensor gradient) override { return gradient; }
};

class ReLU : public Module {       // activation/relu.rs:17-32
public:
    Tensor forward(Tensor input) override {
        Tensor out = Tensor::like(input, input.nrows(), input.ncols());
        check(input.ctx(), rst_relu_forward(input.ctx(), input.handle(), out.handle()));
        prev_input = input;
        return out;
    }
    Tensor backward(Tensor gradient) override {
        Tensor prev = take();
        Tensor out = Tensor::like(gradient, gradient.nrows(), gradient.ncols());
        check(gradient.ctx(), rst_relu_backward(gradient.ctx(), gradient.handle(), prev.handle(), out.handle()));
        return out;
    }
    Tensor take() {
        if (!prev_input) throw Panic(RST_ERR_STATE, "ReLU::backward without a preceding forward (relu.rs:26 unwrap)");
        Tensor p = prev_input;
        prev_input = Tensor();
        return p;
    }
    Tensor prev_input;   // any tensor with the sign pattern of the pre-activation
};

// Softmax as a layer (activation/softmax.rs:5-34, 55-78).  The backward is the reference's, kept
// as written: Jacobian -(Oᵀ·O) over the whole batch with the diagonal replaced by s(1-s),
// applied as gradient · jacobian.
class Softmax : public Module {
public:
    explicit Softmax(size_t axis = 1) : axis_(axis) {
        if (axis > 1) throw Panic(RST_ERR_INVALID_ARG, "axis out of range for a 2-D array");
    }
    static Softmax with_axis(size_t axis) { return Softmax(axis); }
    Tensor forward(Tensor input) override {
        Tensor out = Tensor::like(input, input.nrows(), input.ncols());
        check(input.ctx(), axis_ == 1 ? rst_softmax(input.ctx(), input.handle(), out.handle())
                                      : rst_softmax_axis0(input.ctx(), input.handle(), out.handle()));
        output_ = out;
        return out;
    }
    Tensor backward(Tensor gradient) override {
        if (!output_) throw Panic(RST_ERR_STATE, "Softmax::backward without a preceding forward (softmax.rs:63 unwrap)");
        Tensor output = output_;
        output_ = Tensor();
        Tensor dx = Tensor::like(gradient, gradient.nrows(), output.ncols());
        check(gradient.ctx(), rst_softmax_backward(gradient.ctx(), output.handle(), gradient.handle(), dx.handle()));
        return dx;
    }
private:
    size_t axis_;
    Tensor output_;
};

class Linear : public Module {     // module/linear.rs
public:
    Linear(Context& ctx, size_t input_size, size_t output_size, const InitParameters& init = default_init(),
           bool with_bias = true)
        : in_(input_size), out_(output_size),
          weight(ctx, (int64_t)output_size, (int64_t)input_size, init.weight(input_size, output_size)) {
        if (with_bias) bias = Tensor(ctx, 1, (int64_t)output_size, init.bias(input_size, output_size));
    }
    static Linear new_with_kernel(Context& ctx, size_t input_size, size_t output_size, const InitParameters& init) {
        return Linear(ctx, input_size, output_size, init);
    }
    // A layer whose `bias` is None: the reference's struct holds `Option<Array2<f64>>` and
    // branches on it (linear.rs:51-53, 65-67, 74-77) although its public constructors always
    // fill it (:27).  y = x·Wᵀ, no db, one parameter pair.
    static Linear without_bias(Context& ctx, size_t input_size, size_t output_size,
                               const InitParameters& init = default_init()) {
        return Linear(ctx, input_size, output_size, init, false);
    }
    Tensor forward(Tensor input) override { return forward_fused(std::move(input), false); }
    Tensor forward_fused(Tensor input, bool relu) {      // linear.rs:43-57 (+ relu.rs:21 in the epilogue)
        Tensor y = Tensor::like(input, input.nrows(), (int64_t)out_);
        check(input.ctx(), rst_linear_forward(input.ctx(), input.handle(), weight.handle(),
                                              bias ? bias.handle() : nullptr, relu ? 1 : 0, y.handle()));
        prev_input = input;
        return y;
    }
    Tensor backward(Tensor gradient) override { return backward_fused(std::move(gradient), false, true); }
    Tensor backward_fused(Tensor gradient, bool relu_mask, bool need_input_grad) {   // linear.rs:60-69
        if (!prev_input) throw Panic(RST_ERR_STATE, "Linear::backward without a preceding forward (linear.rs:61 unwrap)");
        Tensor x = prev_input;
        prev_input = Tensor();
        if (!grad_weight) {
            grad_weight = Tensor::like(x, (int64_t)out_, (int64_t)in_);
            if (bias) grad_bias = Tensor::like(x, 1, (int64_t)out_);          // linear.rs:65
        }
        Tensor dx = need_input_grad ? Tensor::like(x, x.nrows(), x.ncols()) : Tensor();
        check(x.ctx(), rst_linear_backward(x.ctx(), gradient.handle(), x.handle(), weight.handle(),
                                           (relu_mask && dx) ? x.handle() : nullptr, grad_weight.handle(),
                                           bias ? grad_bias.handle() : nullptr, dx ? dx.handle() : nullptr));
        return dx;
    }
    Parameters parameters() override {                   // linear.rs:71-78
        if (!grad_weight) throw Panic(RST_ERR_STATE, "Linear::parameters before any backward (linear.rs:72 unwrap)");
        if (!bias) return {{weight, grad_weight}};
        return {{weight, grad_weight}, {bias, grad_bias}};
    }
    size_t in_, out_;
    Tensor weight, bias, prev_input, grad_weight, grad_bias;
};

class Sequential : public Module {   // module/sequential.rs:11-110
public:
    Sequential() = default;
    explicit Sequential(std::vector<std::unique_ptr<Module>> layers) : layers_(std::move(layers)) {}
    void push(std::unique_ptr<Module> layer) { layers_.push_back(std::move(layer)); }
    void insert(size_t index, std::unique_ptr<Module> layer) {
        if (index > layers_.size()) throw Panic(RST_ERR_INVALID_ARG, "insertion index out of range");
        layers_.insert(layers_.begin() + (std::ptrdiff_t)index, std::move(layer));
    }
    std::unique_ptr<Module> remove(size_t index) {      // None when out of range (sequential.rs:43-48)
        if (index >= layers_.size()) return nullptr;
        auto l = std::move(layers_[index]);
        layers_.erase(layers_.begin() + (std::ptrdiff_t)index);
        return l;
    }
    size_t len() const { return layers_.size(); }
    bool is_empty() const { return layers_.empty(); }
    Module& layer(size_t i) { return *layers_[i]; }

    // Peephole fusion over adjacent plain layers; results are unchanged.
    Tensor forward(Tensor input) override {
        Tensor x = std::move(input);
        for (size_t i = 0; i < layers_.size(); ++i) {
            Linear* lin = plain<Linear>(i);
            ReLU* next = i + 1 < layers_.size() ? plain<ReLU>(i + 1) : nullptr;
            if (lin && next) {
                x = lin->forward_fused(x, true);
                next->prev_input = x;
                ++i;
            } else {
                x = layers_[i]->forward(x);
            }
        }
        return x;
    }
    Tensor backward(Tensor gradient) override { return backward(std::move(gradient), true); }
    // need_input_grad = false skips dX of the first Linear (discarded by the loop of README.md:72).
    Tensor backward(Tensor gradient, bool need_input_grad) {
        Tensor g = std::move(gradient);
        size_t first = 0;
        while (first < layers_.size() && plain<Identity>(first)) ++first;
        if (small_linear_chain(first)) return backward_chain(first, g, need_input_grad);
        for (size_t k = layers_.size(); k-- > 0;) {
            if (Linear* lin = plain<Linear>(k)) {
                ReLU* before = k > 0 ? plain<ReLU>(k - 1) : nullptr;
                g = lin->backward_fused(g, before != nullptr, need_input_grad || k != first);
                if (before) { before->take(); --k; }
                if (!g) return g;
            } else {
                g = layers_[k]->backward(g);
            }
        }
        return g;
    }
    void train() override { for (auto& l : layers_) l->train(); }
    void eval() override { for (auto& l : layers_) l->eval(); }
    Parameters parameters() override {                   // flat_map in layer order (sequential.rs:102-109)
        Parameters all;
        for (auto& l : layers_) for (auto& p : l->parameters()) all.push_back(p);
        return all;
    }
private:
    template <class T> T* plain(size_t i) {              // exact type only: subclasses may override behaviour
        Module* m = layers_[i].get();
        return typeid(*m) == typeid(T) ? static_cast<T*>(m) : nullptr;
    }
    // `Linear, (ReLU, Linear)*` of plain small layers from `first` to the end: the whole
    // backward is one library call (dX chain first, then every dW/db in one launch).
    static constexpr size_t kChainMaxWeightElems = size_t(1) << 20;
    bool small_linear_chain(size_t first) {
        const size_t n = layers_.size() - first;
        if (n < 3 || n % 2 == 0) return false;
        for (size_t k = 0; k < n; ++k) {
            if (k % 2 == 0) {
                Linear* lin = plain<Linear>(first + k);
                if (!lin || !lin->bias || lin->in_ * lin->out_ > kChainMaxWeightElems) return false;
            } else if (!plain<ReLU>(first + k)) {
                return false;
            }
        }
        return true;
    }
    Tensor backward_chain(size_t first, const Tensor& gradient, bool need_input_grad) {
        std::vector<Linear*> lins;
        for (size_t k = first; k < layers_.size(); k += 2) lins.push_back(plain<Linear>(k));
        const int n = (int)lins.size();
        std::vector<Tensor> xs(n), dxs(n);
        for (int l = 0; l < n; ++l) {
            if (!lins[l]->prev_input)
                throw Panic(RST_ERR_STATE, "Linear::backward without a preceding forward (linear.rs:61 unwrap)");
            xs[l] = lins[l]->prev_input;
        }
        std::vector<const rst_tensor*> hx(n), hw(n);
        std::vector<rst_tensor*> hdw(n), hdb(n), hdx(n);
        std::vector<unsigned char> mask(n);
        for (int l = 0; l < n; ++l) {
            Linear* lin = lins[l];
            lin->prev_input = Tensor();
            if (l > 0) plain<ReLU>(first + 2 * (size_t)l - 1)->take();
            if (!lin->grad_weight) {
                lin->grad_weight = Tensor::like(xs[l], (int64_t)lin->out_, (int64_t)lin->in_);
                lin->grad_bias = Tensor::like(xs[l], 1, (int64_t)lin->out_);
            }
            if (l > 0 || need_input_grad) dxs[l] = Tensor::like(xs[l], xs[l].nrows(), xs[l].ncols());
            hx[l] = xs[l].handle();
            hw[l] = lin->weight.handle();
            hdw[l] = lin->grad_weight.handle();
            hdb[l] = lin->grad_bias.handle();
            hdx[l] = dxs[l] ? dxs[l].handle() : nullptr;
            mask[l] = l > 0 ? 1 : 0;
        }
        check(gradient.ctx(), rst_linear_backward_chain(gradient.ctx(), n, gradient.handle(), hx.data(), hw.data(),
                                                        mask.data(), hdw.data(), hdb.data(), hdx.data()));
        return dxs[0];
    }
    std::vector<std::unique_ptr<Module>> layers_;
};

// sequential!(Identity(), Linear(784, 100), ReLU(), ...) (sequential.rs:62-74)
template <class... Layers>
Sequential sequential(Layers&&... layers) {
    std::vector<std::unique_ptr<Module>> v;
    (v.push_back(std::make_unique<std::decay_t<Layers>>(std::forward<Layers>(layers))), ...);
    return Sequential(std::move(v));
}

class Loss {           // loss/mod.rs:6-11
public:
    virtual ~Loss() = default;
    virtual double forward(Tensor pred, Tensor truth) = 0;
    virtual Tensor backward() = 0;
};

class CrossEntropyLoss : public Loss {   // loss/cross_entropy.rs:32-48
public:
    double forward(Tensor pred, Tensor truth) override {
        Tensor g = Tensor::like(pred, pred.nrows(), pred.ncols());
        check(pred.ctx(), rst_xent_forward_backward(pred.ctx(), pred.handle(), truth.handle(), g.handle(), 0));
        double loss = 0.0;
        check(pred.ctx(), rst_xent_result(pred.ctx(), 0, &loss, &last_accuracy));   // blocks, like `-> f64`
        grad_ = g;
        return loss;
    }
    Tensor backward() override {
        if (!grad_) throw Panic(RST_ERR_STATE, "CrossEntropyLoss::backward without a preceding forward (cross_entropy.rs:46 unwrap)");
        Tensor g = grad_;
        grad_ = Tensor();
        return g;
    }
    double last_accuracy = 0.0;   // accuracy(pred, truth) of the last forward, from the same kernel
private:
    Tensor grad_;
};

class Optimizer {      // optim/mod.rs:6-8
public:
    virtual ~Optimizer() = default;
    virtual void step(Module& module) = 0;
};

class SGD : public Optimizer {   // optim/sgd.rs
public:
    explicit SGD(double lr) : lr_(lr) {}
    void step(Module& module) override {
        Parameters ps = module.parameters();
        if (ps.empty()) return;
        std::vector<rst_tensor*> p, g;
        for (auto& q : ps) { p.push_back(q.parm.handle()); g.push_back(q.grad.handle()); }
        check(ps[0].parm.ctx(), rst_sgd_step(ps[0].parm.ctx(), (int)p.size(), p.data(), g.data(), lr_));
    }
private:
    double lr_;
};

// BasicModel (model.rs:4-32): the reference's own statement of the training step and of
// inference over a module, a loss and an optimiser.
template <class M, class L, class O>
class BasicModel {
public:
    BasicModel(M module, L loss, O optim) : module(std::move(module)), loss(std::move(loss)), optim(std::move(optim)) {}
    void step(Tensor input, Tensor truth) {              // model.rs:19-27
        Tensor pred = module.forward(std::move(input));
        loss.forward(pred, std::move(truth));
        Tensor gradient = loss.backward();
        module.backward(std::move(gradient));
        optim.step(module);
    }
    Tensor predict(Tensor input) { return module.forward(std::move(input)); }   // model.rs:29-31
    M module;
    L loss;
    O optim;
};

inline double accuracy(const Tensor& pred, const Tensor& truth) {   // utils.rs:55-65
    double a = 0.0;
    check(pred.ctx(), rst_accuracy(pred.ctx(), pred.handle(), truth.handle(), &a));
    return a;
}

inline std::vector<int64_t> argmax(const Tensor& t) {               // utils.rs:44-53
    std::vector<int64_t> idx((size_t)t.nrows());
    check(t.ctx(), rst_argmax(t.ctx(), t.handle(), idx.data()));
    return idx;
}

inline std::vector<double> one_hot(size_t x, size_t n) {            // utils.rs:38-42
    if (x >= n) throw Panic(RST_ERR_INVALID_ARG, "one_hot index out of bounds");
    std::vector<double> v(n, 0.0);
    v[x] = 1.0;
    return v;
}

// DataLoader::new(dataset, batch_size, shuffle = false, SequentialSampler) over host rows;
// iter_array visits the full batches in order and drops the remainder (data_loader.rs:69-71,192-207).
class DataLoader {
public:
    DataLoader(Context& ctx, const std::vector<double>& samples, const std::vector<double>& targets, int64_t n,
               int64_t features, int64_t classes, int64_t batch_size, int slots = 2)
        : ctx_(ctx.handle()), samples_(samples), targets_(targets), n_(n), f_(features), c_(classes), b_(batch_size),
          slots_(slots) {
        check(ctx_, rst_stager_create(ctx_, b_, f_, c_, slots_, &stager_));
    }
    ~DataLoader() { if (stager_) rst_stager_destroy(stager_); }
    DataLoader(const DataLoader&) = delete;
    size_t len() const { return (size_t)(n_ / b_); }
    bool is_empty() const { return n_ < b_; }
    void iter_array(const std::function<void(Tensor, Tensor)>& body) {
        const int64_t batches = n_ / b_;
        auto fill = [&](int64_t k) {
            double *x = nullptr, *t = nullptr;
            const int slot = (int)(k % slots_);
            check(ctx_, rst_stager_host(stager_, slot, &x, &t));
            std::copy(samples_.begin() + k * b_ * f_, samples_.begin() + (k + 1) * b_ * f_, x);
            std::copy(targets_.begin() + k * b_ * c_, targets_.begin() + (k + 1) * b_ * c_, t);
            check(ctx_, rst_stager_submit(stager_, slot));
        };
        const int64_t ahead = std::min<int64_t>(slots_ > 1 ? slots_ - 1 : 0, batches);
        for (int64_t k = 0; k < ahead; ++k) fill(k);
        for (int64_t k = 0; k < batches; ++k) {
            if (slots_ == 1) fill(k);
            rst_tensor *X = nullptr, *T = nullptr;
            check(ctx_, rst_stager_acquire(stager_, (int)(k % slots_), &X, &T));
            body(Tensor::borrowed(ctx_, X), Tensor::borrowed(ctx_, T));
            if (slots_ > 1 && k + ahead < batches) fill(k + ahead);
        }
    }
private:
    rst_ctx* ctx_;
    const std::vector<double>& samples_;
    const std::vector<double>& targets_;
    int64_t n_, f_, c_, b_;
    int slots_;
    rst_stager* stager_ = nullptr;
};

// A u8 dataset resident in HBM (the MNIST item type, data/dataset/hub/mnist.rs:181-194) with
// the README transform `(flatten(normalize_zero_one(x)), one_hot(y, classes))` applied by the
// kernel that builds a batch (README.md:44, utils.rs:5-42, data_loader.rs:192-207).
class DeviceDataset {
public:
    DeviceDataset(Context& ctx, const std::vector<unsigned char>& images, const std::vector<unsigned char>& labels,
                  int64_t features, int64_t classes)
        : ctx_(ctx.handle()), n_((int64_t)labels.size()), f_(features), c_(classes) {
        if ((int64_t)images.size() != n_ * f_) throw Panic(RST_ERR_SHAPE, "images and labels differ in length");
        check(ctx_, rst_dataset_create_u8(ctx_, images.data(), labels.data(), n_, f_, c_, &h_));
    }
    ~DeviceDataset() { if (h_) rst_dataset_destroy(h_); }
    DeviceDataset(const DeviceDataset&) = delete;
    size_t len() const { return (size_t)n_; }
    // The batch of the given sample indices: X (n, features), T (n, classes).
    std::pair<Tensor, Tensor> gather(Context& ctx, const std::vector<int64_t>& indices) {
        Tensor x(ctx, (int64_t)indices.size(), f_), t(ctx, (int64_t)indices.size(), c_);
        check(ctx_, rst_dataset_gather(h_, indices.data(), (int64_t)indices.size(), x.handle(), t.handle()));
        return {x, t};
    }
    // The pinned index buffer a replayed step reads its sample indices from.
    int64_t* index_stage(int64_t batch) {
        int64_t* p = nullptr;
        check(ctx_, rst_dataset_index_stage(h_, batch, &p));
        return p;
    }
    // Builds the batch of the staged indices into x, t; reads no index on the host (capturable).
    void gather_staged(int64_t batch, Tensor& x, Tensor& t) {
        check(ctx_, rst_dataset_gather_staged(h_, batch, x.handle(), t.handle()));
    }
private:
    rst_ctx* ctx_;
    int64_t n_, f_, c_;
    rst_dataset* h_ = nullptr;
};

// Everything queued between the constructor and end() becomes a CUDA graph; launch() replays it.
class Graph {
public:
    explicit Graph(Context& ctx) : ctx_(ctx.handle()) { check(ctx_, rst_graph_capture_begin(ctx_)); }
    ~Graph() { if (h_) rst_graph_destroy(h_); }
    Graph(const Graph&) = delete;
    void end() { check(ctx_, rst_graph_capture_end(ctx_, &h_)); }
    void launch() { check(ctx_, rst_graph_launch(h_)); }
private:
    rst_ctx* ctx_;
    rst_graph* h_ = nullptr;
};

}  // namespace rstorch
