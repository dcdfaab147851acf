//! The reference's known-answer unit tests (src/module/linear.rs:97-131,
//! src/module/activation/relu.rs:38-57, src/data/data_loader.rs:289-324) and its README
//! training loop (README.md:59-79), run through the façade on a GPU.  Needs a B200 and
//! `RSTORCH_B200_LIB_DIR`; run with `cargo test -- --test-threads 1`.
use rstorch_b200::data::Basic;
use rstorch_b200::prelude::*;
use rstorch_b200::utils::accuracy;
use rstorch_b200::{CrossEntropyLoss, Identity, Linear, ReLU, Sequential, SGD};

fn assert_close(a: &Array2<f64>, b: &Array2<f64>, tol: f64) {
    assert_eq!(a.shape(), b.shape(), "incompatible shapes");
    for (x, y) in a.iter().zip(b) {
        assert!((x - y).abs() <= tol, "not equal with tolerance {tol}\n a = {a}\n b = {b}");
    }
}

struct FixedInit;

impl InitParameters for FixedInit {
    fn weight(&self, _input_size: usize, _output_size: usize) -> Array2<f64> {
        array![[1.0, 0.5]]
    }
    fn bias(&self, _input_size: usize, _output_size: usize) -> Array2<f64> {
        array![[10.0]]
    }
}

#[test]
fn linear_forward_known_answer() {
    let mut layer = Linear::new_with_kernel(2, 1, FixedInit);
    let input = array![[1.0, 2.0], [3.0, -4.0], [-5.0, -6.0]];
    let out = layer.forward(Tensor::from(input)).to_array();
    assert_close(&out, &array![[12.0], [11.0], [2.0]], 1e-6);
}

#[test]
fn linear_backward_known_answer() {
    let mut layer = Linear::new_with_kernel(2, 1, FixedInit);
    let input = array![[1.0, 2.0], [3.0, -4.0], [-5.0, -6.0], [-7.0, 8.0]];
    let _ = layer.forward(Tensor::from(input));
    let dx = layer.backward(Tensor::from(array![[1.0], [1.0], [1.0], [1.0]])).to_array();
    assert_close(&layer.grad_weight().unwrap().to_array(), &array![[-2.0, 0.0]], 1e-6);
    assert_close(&layer.grad_bias().unwrap().to_array(), &array![[1.0]], 1e-6);
    assert_close(&dx, &array![[1.0, 0.5], [1.0, 0.5], [1.0, 0.5], [1.0, 0.5]], 1e-6);
}

#[test]
#[should_panic]
fn linear_backward_without_forward_panics() {
    let mut layer = Linear::new(2, 1);
    layer.backward(Tensor::from(array![[1.0]]));
}

#[test]
fn relu_known_answers() {
    let mut layer = ReLU::new();
    let input = array![[1.0, 2.0], [3.0, -4.0], [-5.0, -6.0]];
    let out = layer.forward(Tensor::from(input)).to_array();
    assert_close(&out, &array![[1.0, 2.0], [3.0, 0.0], [0.0, 0.0]], 0.0);
    let grad = layer.backward(Tensor::from(Array2::<f64>::ones((3, 2)))).to_array();
    assert_close(&grad, &array![[1.0, 1.0], [1.0, 0.0], [0.0, 0.0]], 0.0);
}

#[test]
fn fused_and_unfused_layers_agree() {
    // the same weights through `Sequential` (fused epilogues) and layer by layer (unfused)
    rstorch_b200::module::init::set_seed(7);
    let mut fused = sequential!(Linear(5, 4), ReLU(), Linear(4, 3));
    rstorch_b200::module::init::set_seed(7);
    let (mut l1, mut r, mut l2) = (Linear::new(5, 4), ReLU::new(), Linear::new(4, 3));
    let x = Array2::from_shape_fn((6, 5), |(i, j)| (i as f64 - 2.5) * 0.3 + (j as f64) * 0.1 - 0.2);
    let g = Array2::from_shape_fn((6, 3), |(i, j)| 0.05 * (i as f64) - 0.1 * (j as f64));

    let y_fused = fused.forward(Tensor::from(&x)).to_array();
    let y_plain = l2.forward(r.forward(l1.forward(Tensor::from(&x)))).to_array();
    assert_close(&y_fused, &y_plain, 1e-12);

    let dx_fused = fused.backward(Tensor::from(&g)).to_array();
    let dx_plain = l1.backward(r.backward(l2.backward(Tensor::from(&g)))).to_array();
    assert_close(&dx_fused, &dx_plain, 1e-12);
    let fused_grads: Vec<_> = fused.parameters().iter().map(|p| p.grad.to_array()).collect();
    assert_close(&fused_grads[0], &l1.grad_weight().unwrap().to_array(), 1e-12);
    assert_close(&fused_grads[3], &l2.grad_bias().unwrap().to_array(), 1e-12);
}

#[test]
fn data_loader_first_batch_and_len() {
    let items: Vec<_> = (0..100)
        .map(|i| (Array2::from_elem((4, 4), i as f64), Array1::from_elem(4, i as f64)))
        .collect();
    let sampler = SequentialSampler::new(items.len());
    let mut loader = DataLoader::new(Basic::new(items), 32, false, sampler);
    assert_eq!(loader.len(), 3);
    let batches: Vec<_> = loader.iter_array().map(|(x, t)| (x.to_array(), t.to_array())).collect();
    assert_eq!(batches.len(), 3); // the last 4 samples do not fill a batch
    let (x, t) = &batches[0];
    assert_eq!((x.shape(), t.shape()), (&[32usize, 16][..], &[32usize, 4][..]));
    for i in 0..32 {
        assert!(x.row(i).iter().all(|v| *v == i as f64));
        assert!(t.row(i).iter().all(|v| *v == i as f64));
    }
}

#[test]
fn readme_loop_reduces_the_loss() {
    // 784-100-100-10 on a seeded stand-in for the README's data set: 81 % zeros, the rest
    // in (0, 1], labels uniform over ten classes
    let mut state = 1u64;
    let mut next = move || {
        state = state.wrapping_mul(6364136223846793005).wrapping_add(1442695040888963407);
        (state >> 11) as f64 / (1u64 << 53) as f64
    };
    let items: Vec<_> = (0..256)
        .map(|_| {
            let x = Array1::from_shape_fn(784, |_| if next() < 0.81 { 0.0 } else { 1.0 - next() });
            let mut y = Array1::zeros(10);
            y[(next() * 10.0) as usize] = 1.0;
            (x, y)
        })
        .collect();
    let sampler = SequentialSampler::new(items.len());
    let mut data_loader = DataLoader::new(Basic::new(items), 32, true, sampler);

    let mut model: Sequential =
        sequential!(Identity(), Linear(784, 100), ReLU(), Linear(100, 100), ReLU(), Linear(100, 10));
    let mut loss = CrossEntropyLoss::new();
    let mut optim = SGD::new(0.01);

    let mut epoch_loss = Vec::new();
    for _ in 0..5 {
        let n = data_loader.len() as f64;
        let (mut total_loss, mut total_acc) = (0.0, 0.0);
        for (x, y) in data_loader.iter_array() {
            let pred = model.forward(x);
            let l = loss.forward(pred.clone(), y.clone());
            let acc = accuracy(pred, y);
            assert_eq!(acc, loss.last_accuracy());
            total_loss += l;
            total_acc += acc;
            model.backward(loss.backward());
            optim.step(&mut model);
        }
        assert!((0.0..=1.0).contains(&(total_acc / n)));
        epoch_loss.push(total_loss / n);
    }
    assert!(epoch_loss.iter().all(|l| l.is_finite()));
    assert!(epoch_loss[4] < epoch_loss[0], "loss did not go down: {epoch_loss:?}");
}
