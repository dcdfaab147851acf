// Exercises include/rstorch.hpp the way the reference's own unit tests and README
// loop exercise the crate.  Part 1 re-states the unit tests of the reference
// (src/module/linear.rs:97-131, activation/relu.rs:38-57, activation/identity.rs:35-51,
// optim/sgd.rs:34-43, module/sequential.rs:119-172) against the device path.  Part 2
// runs the README training loop (README.md:39-80) on the inputs found in the file
// given as argv[1] and writes per-step loss/accuracy and the final parameters to
// argv[2]; the Python test compares that file with the CPU restatement.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>

#include "rstorch.hpp"

using namespace rstorch;

static int failures = 0;
#define EXPECT(cond)                                                              \
    do {                                                                          \
        if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); ++failures; } \
    } while (0)

static bool close_to(const std::vector<double>& a, const std::vector<double>& b, double tol = 1e-6) {
    if (a.size() != b.size()) return false;                       // assert_array_eq!: shape, then |a-b| <= tol
    for (size_t i = 0; i < a.size(); ++i) if (std::fabs(a[i] - b[i]) > tol) return false;
    return true;
}

struct FixedInit : InitParameters {                                // linear.rs:85-95
    std::vector<double> weight(size_t, size_t) const override { return {1.0, 0.5}; }
    std::vector<double> bias(size_t, size_t) const override { return {10.0}; }
};

struct FileInit : InitParameters {
    std::vector<double> w, b;
    std::vector<double> weight(size_t, size_t) const override { return w; }
    std::vector<double> bias(size_t, size_t) const override { return b; }
};

static void unit_tests(Context& ctx) {
    {   // linear.rs:97-105
        Linear m = Linear::new_with_kernel(ctx, 2, 1, FixedInit());
        Tensor result = m.forward(Tensor(ctx, 3, 2, {1.0, 2.0, 3.0, -4.0, -5.0, -6.0}));
        EXPECT(result.nrows() == 3 && result.ncols() == 1);
        EXPECT(close_to(result.to_host(), {12.0, 11.0, 2.0}));
    }
    {   // linear.rs:107-131
        Linear m = Linear::new_with_kernel(ctx, 2, 1, FixedInit());
        m.forward(Tensor(ctx, 4, 2, {1.0, 2.0, 3.0, -4.0, -5.0, -6.0, -7.0, 8.0}));
        Tensor result = m.backward(Tensor(ctx, 4, 1, {1.0, 1.0, 1.0, 1.0}));
        EXPECT(m.grad_weight.nrows() == m.weight.nrows() && m.grad_weight.ncols() == m.weight.ncols());
        EXPECT(m.grad_bias.nrows() == m.bias.nrows() && m.grad_bias.ncols() == m.bias.ncols());
        EXPECT(close_to(m.grad_weight.to_host(), {-2.0, 0.0}));
        EXPECT(close_to(m.grad_bias.to_host(), {1.0}));
        EXPECT(close_to(result.to_host(), {1.0, 0.5, 1.0, 0.5, 1.0, 0.5, 1.0, 0.5}));
    }
    {   // relu.rs:38-57
        ReLU m;
        Tensor data(ctx, 3, 2, {1.0, 2.0, 3.0, -4.0, -5.0, -6.0});
        EXPECT(close_to(m.forward(data).to_host(), {1.0, 2.0, 3.0, 0.0, 0.0, 0.0}));
        m.forward(data);
        EXPECT(close_to(m.backward(Tensor(ctx, 3, 2, std::vector<double>(6, 1.0))).to_host(), {1.0, 1.0, 1.0, 0.0, 0.0, 0.0}));
    }
    {   // identity.rs:35-51
        Identity m;
        Tensor data(ctx, 3, 2, {1.0, 2.0, 3.0, 4.0, 5.0, 6.0});
        EXPECT(close_to(m.forward(data).to_host(), data.to_host()));
        EXPECT(close_to(m.backward(data).to_host(), data.to_host()));
    }
    {   // sgd.rs:34-43: zero input, zero gradient, one step leaves the weights alone
        SGD optim(0.1);
        Linear linear(ctx, 2, 2);
        std::vector<double> before = linear.weight.to_host();
        linear.forward(Tensor(ctx, 2, 2, std::vector<double>(4, 0.0)));
        linear.backward(Tensor(ctx, 2, 2, std::vector<double>(4, 0.0)));
        optim.step(linear);
        EXPECT(linear.weight.to_host() == before);
    }
    {   // sequential.rs:119-172 (macro expansion, forward and backward smoke tests; Softmax layer left out)
        Sequential module = sequential(Linear(ctx, 3, 10), ReLU(), Linear(ctx, 10, 100), ReLU(), Linear(ctx, 100, 2));
        EXPECT(module.len() == 5 && !module.is_empty());
        Tensor out = module.forward(Tensor(ctx, 2, 3, {1.0, 2.0, 3.0, -4.0, -5.0, -6.0}));
        EXPECT(out.nrows() == 2 && out.ncols() == 2);
        Tensor dx = module.backward(Tensor(ctx, 2, 2, std::vector<double>(4, 1.0)));
        EXPECT(dx.nrows() == 2 && dx.ncols() == 3);
        EXPECT(module.parameters().size() == 6);
        EXPECT(module.remove(99) == nullptr);
        EXPECT(module.remove(4) != nullptr && module.len() == 4);
    }
    {   // default initialiser: every layer draws its own stream (he.rs:13 draws from the thread generator)
        Linear a(ctx, 100, 100), b(ctx, 100, 100);
        EXPECT(a.weight.to_host() != b.weight.to_host());
    }
    {   // bias: None (linear.rs:51-53, 65-67, 74-77): y = x·Wᵀ, no db, one parameter pair
        Linear m = Linear::without_bias(ctx, 2, 1, FixedInit());
        Tensor y = m.forward(Tensor(ctx, 3, 2, {1.0, 2.0, 3.0, -4.0, -5.0, -6.0}));
        EXPECT(close_to(y.to_host(), {2.0, 1.0, -8.0}));
        Tensor dx = m.backward(Tensor(ctx, 3, 1, {1.0, 1.0, 1.0}));
        EXPECT(close_to(dx.to_host(), {1.0, 0.5, 1.0, 0.5, 1.0, 0.5}));
        EXPECT(m.parameters().size() == 1 && !m.grad_bias);
        EXPECT(close_to(m.grad_weight.to_host(), {-1.0 / 3.0, -8.0 / 3.0}));
    }
    {   // BasicModel::step / predict (model.rs:19-31)
        BasicModel<Sequential, CrossEntropyLoss, SGD> model(
            sequential(Linear(ctx, 3, 8), ReLU(), Linear(ctx, 8, 2)), CrossEntropyLoss(), SGD(0.1));
        Tensor x(ctx, 2, 3, {1.0, 2.0, 3.0, -4.0, -5.0, -6.0}), t(ctx, 2, 2, {1.0, 0.0, 0.0, 1.0});
        std::vector<double> before = model.predict(x).to_host();
        model.step(x, t);
        std::vector<double> after = model.predict(x).to_host();
        EXPECT(before.size() == 4 && after.size() == 4 && before != after);
    }
    {   // the reference's unwrap() panics
        bool threw = false;
        try { Linear(ctx, 2, 2).backward(Tensor(ctx, 1, 2, {0.0, 0.0})); } catch (const Panic&) { threw = true; }
        EXPECT(threw);
        threw = false;
        try { Linear(ctx, 2, 2).parameters(); } catch (const Panic&) { threw = true; }
        EXPECT(threw);
        threw = false;
        try { CrossEntropyLoss().backward(); } catch (const Panic&) { threw = true; }
        EXPECT(threw);
        threw = false;
        try { Linear(ctx, 4, 3).forward(Tensor(ctx, 2, 5, std::vector<double>(10, 0.0))); } catch (const Panic& p) { threw = p.status == RST_ERR_SHAPE; }
        EXPECT(threw);
        EXPECT(one_hot(3, 5) == (std::vector<double>{0, 0, 0, 1, 0}));
    }
    {   // softmax.rs:85-113: rows (axis 1) and columns (axis 0) sum to one; backward known answer
        Softmax rows;
        std::vector<double> p = rows.forward(Tensor(ctx, 3, 2, {1.0, 10.0, -3.0, 4.0, 5.0, 6.0})).to_host();
        for (int r = 0; r < 3; ++r) EXPECT(std::fabs(p[2 * r] + p[2 * r + 1] - 1.0) <= 1e-6);
        Softmax cols = Softmax::with_axis(0);
        Tensor data(ctx, 3, 2, {1.0, 2.0, 3.0, 4.0, 5.0, 6.0});
        std::vector<double> q = cols.forward(data).to_host();
        EXPECT(std::fabs(q[0] + q[2] + q[4] - 1.0) <= 1e-6 && std::fabs(q[1] + q[3] + q[5] - 1.0) <= 1e-6);
        Softmax m;
        m.forward(data);
        std::vector<double> g = m.backward(Tensor(ctx, 3, 2, std::vector<double>(6, 1.0))).to_host();
        EXPECT(close_to(g, {-0.41, -1.55, -0.41, -1.55, -0.41, -1.55}, 0.01));
        bool threw = false;
        try { Softmax().backward(data); } catch (const Panic&) { threw = true; }
        EXPECT(threw);
    }
    {   // device-resident u8 dataset: README transform in the gather kernel, eager and replayed
        const int64_t n = 40, f = 6, c = 4, b = 8;
        std::vector<unsigned char> images((size_t)(n * f)), labels((size_t)n);
        for (int64_t i = 0; i < n; ++i) {
            labels[(size_t)i] = (unsigned char)(i % c);
            for (int64_t e = 0; e < f; ++e) images[(size_t)(i * f + e)] = (unsigned char)((i * 37 + e * 11) % 251);
        }
        DeviceDataset ds(ctx, images, labels, f, c);
        EXPECT(ds.len() == 40);
        auto expect_batch = [&](const std::vector<int64_t>& idx, const std::vector<double>& x, const std::vector<double>& t) {
            for (size_t r = 0; r < idx.size(); ++r) {
                const unsigned char* s = &images[(size_t)(idx[r] * f)];
                double lo = 255, hi = 0;
                for (int64_t e = 0; e < f; ++e) { lo = std::min<double>(lo, s[e]); hi = std::max<double>(hi, s[e]); }
                for (int64_t e = 0; e < f; ++e) EXPECT(x[r * (size_t)f + (size_t)e] == (s[e] - lo) / (hi - lo));
                for (int64_t k = 0; k < c; ++k) EXPECT(t[r * (size_t)c + (size_t)k] == (k == labels[(size_t)idx[r]] ? 1.0 : 0.0));
            }
        };
        std::vector<int64_t> idx = {3, 39, 0, 17, 17, 8, 21, 30};
        auto [x, t] = ds.gather(ctx, idx);
        expect_batch(idx, x.to_host(), t.to_host());
        Tensor xs(ctx, b, f), ts(ctx, b, c);
        int64_t* stage = ds.index_stage(b);
        std::copy(idx.begin(), idx.end(), stage);
        ds.gather_staged(b, xs, ts);
        expect_batch(idx, xs.to_host(), ts.to_host());
        Graph g(ctx);
        ds.gather_staged(b, xs, ts);
        g.end();
        std::vector<int64_t> idx2 = {1, 2, 3, 4, 5, 6, 7, 38};
        std::copy(idx2.begin(), idx2.end(), stage);
        g.launch();
        expect_batch(idx2, xs.to_host(), ts.to_host());
        ctx.check_device();
    }
}

template <class T> static void read_vec(std::ifstream& f, std::vector<T>& v, size_t n) {
    v.resize(n);
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)(n * sizeof(T)));
}

static int training_loop(Context& ctx, const char* in_path, const char* out_path) {
    std::ifstream f(in_path, std::ios::binary);
    if (!f) { std::printf("cannot open %s\n", in_path); return 1; }
    std::vector<int64_t> head;
    read_vec(f, head, 3);
    const int64_t L = head[0], batch = head[1], steps = head[2];
    std::vector<int64_t> dims;
    read_vec(f, dims, (size_t)L + 1);
    std::vector<double> lr;
    read_vec(f, lr, 1);
    Sequential model;
    model.push(std::make_unique<Identity>());                         // README.md:49
    for (int64_t l = 0; l < L; ++l) {
        FileInit init;
        read_vec(f, init.w, (size_t)(dims[l] * dims[l + 1]));
        read_vec(f, init.b, (size_t)dims[l + 1]);
        model.push(std::make_unique<Linear>(ctx, (size_t)dims[l], (size_t)dims[l + 1], init));
        if (l + 1 < L) model.push(std::make_unique<ReLU>());
    }
    std::vector<double> X, T;
    read_vec(f, X, (size_t)(steps * batch * dims[0]));
    read_vec(f, T, (size_t)(steps * batch * dims[L]));
    if (!f) { std::printf("short input file\n"); return 1; }

    DataLoader data_loader(ctx, X, T, steps * batch, dims[0], dims[L], batch);
    CrossEntropyLoss loss;
    SGD optim(lr[0]);
    std::vector<double> out;
    data_loader.iter_array([&](Tensor x, Tensor y) {                  // README.md:64-73
        Tensor pred = model.forward(x);
        double l = loss.forward(pred, y);
        double acc = accuracy(pred, y);
        out.push_back(l);
        out.push_back(acc);
        model.backward(loss.backward());
        optim.step(model);
    });
    ctx.check_device();
    for (auto& p : model.parameters()) {
        std::vector<double> v = p.parm.to_host();
        out.insert(out.end(), v.begin(), v.end());
    }
    std::ofstream o(out_path, std::ios::binary);
    o.write(reinterpret_cast<const char*>(out.data()), (std::streamsize)(out.size() * sizeof(double)));
    return o ? 0 : 1;
}

int main(int argc, char** argv) {
    try {
        Context ctx(0);
        unit_tests(ctx);
        if (argc >= 3 && training_loop(ctx, argv[1], argv[2]) != 0) ++failures;
        ctx.check_device();
    } catch (const Panic& p) {
        std::printf("unexpected Panic: %s\n", p.what());
        return 2;
    }
    std::printf(failures ? "FAILED (%d)\n" : "OK\n", failures);
    return failures ? 1 : 0;
}
