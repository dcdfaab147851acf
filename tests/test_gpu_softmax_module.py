"""The Softmax layer and the Xavier/Normal initialisers (the rest of the crate's
`module/` surface): the reference's own tests for the layer, and parity of its
batch-mixed backward with the numpy restatement."""
import numpy as np
import pytest

import rstorch_b200 as rt
from conftest import REL_TOL, rel_err
from oracle import oracle_np as on

pytestmark = pytest.mark.gpu


def A(x):
    return np.array(x, dtype=np.float64)


def test_reference_tests_of_the_softmax_layer(ctx, kat):
    f = kat["softmax_rows_sum_to_one"]                       # softmax.rs:85-93
    out = rt.Softmax().forward(ctx.tensor(A(f["input"]))).numpy()
    assert np.max(np.abs(out.sum(axis=1) - 1.0)) <= kat["tolerance"] and abs(out.sum() - 3.0) < 1e-15
    g = kat["softmax_axis0_columns_sum_to_one"]              # softmax.rs:95-103
    out0 = rt.Softmax.with_axis(0).forward(ctx.tensor(A(g["input"]))).numpy()
    assert np.max(np.abs(out0.sum(axis=0) - 1.0)) <= kat["tolerance"] and abs(out0.sum() - 2.0) < 1e-15
    b = kat["softmax_module_backward"]                       # softmax.rs:105-113
    m = rt.Softmax()
    m.forward(ctx.tensor(A(b["input"])))
    got = m.backward(ctx.tensor(A(b["gradient"]))).numpy()
    assert np.max(np.abs(got - A(b["expected"]))) <= b["tolerance"]
    with pytest.raises(RuntimeError, match="without a preceding forward"):
        m.backward(ctx.tensor(A(b["gradient"])))


@pytest.mark.parametrize("rows,cols,axis", [(3, 2, 1), (64, 10, 1), (257, 100, 1), (128, 1000, 1), (33, 6, 0), (500, 70, 0)])
def test_softmax_layer_parity(ctx, rows, cols, axis):
    rng = np.random.default_rng(rows + cols)
    x, g = rng.standard_normal((rows, cols)) * 3, rng.standard_normal((rows, cols))
    m = rt.Softmax.with_axis(axis)
    out = m.forward(ctx.tensor(x)).numpy()
    want = on.softmax_axis(x, axis)
    assert rel_err(out, want) < REL_TOL
    dx = m.backward(ctx.tensor(g)).numpy()
    assert rel_err(dx, on.softmax_module_backward(want, g)) < REL_TOL


def test_model_ending_in_softmax_trains_one_step(ctx):
    """sequential!(Linear, ReLU, Linear, Softmax) as in the reference's macro test
    (sequential.rs:119-138): forward, backward and parameters against the restatement."""
    rng = np.random.default_rng(3)
    W1, b1 = rng.standard_normal((10, 3)), rng.standard_normal((1, 10))
    W2, b2 = rng.standard_normal((2, 10)), rng.standard_normal((1, 2))

    class Fixed(rt.InitParameters):
        def __init__(self, w, b):
            self.w, self.b = w, b

        def weight(self, i, o):
            return self.w

        def bias(self, i, o):
            return self.b

    model = rt.sequential(rt.Linear.new_with_kernel(3, 10, Fixed(W1, b1), ctx), rt.ReLU(),
                          rt.Linear.new_with_kernel(10, 2, Fixed(W2, b2), ctx), rt.Softmax())
    x = A([[1.0, 2.0, 3.0], [-4.0, -5.0, -6.0]])
    out = model.forward(ctx.tensor(x)).numpy()
    z1 = on.linear_forward(x, W1, b1)
    h = on.relu_forward(z1)
    z2 = on.linear_forward(h, W2, b2)
    want = on.softmax_axis(z2, 1)
    assert rel_err(out, want) < REL_TOL
    dx = model.backward(ctx.tensor(np.ones((2, 2)))).numpy()
    g2 = on.softmax_module_backward(want, np.ones((2, 2)))
    dW2, db2, dh = on.linear_backward(g2, h, W2)
    dW1, db1, dX = on.linear_backward(on.relu_backward(dh, z1), x, W1)
    assert rel_err(dx, dX) < REL_TOL
    got = [p.grad.numpy() for p in model.parameters()]
    for a, b in zip(got, [dW1, db1, dW2, db2]):
        assert np.max(np.abs(a - b)) <= REL_TOL * max(1.0, np.max(np.abs(b)))

