"""Regenerates tests/golden/mlp_small_steps.npz from the numpy restatement.

    python tests/golden/make_golden.py

The fixture holds the inputs (weights, batches) and the per-step outputs (loss,
accuracy, every dW/db, every updated W/b, logits) of four training steps of a
20-16-12-5 MLP at batch 8, lr 0.05, computed by oracle/oracle_np.py.  It is a
regression anchor for the oracle and the CUDA path; it does not come from the
reference itself, which cannot be built in this environment (the vectors that
do come from the reference's tests are in reference_kat.json).
Inputs are stored, not regenerated, so the fixture does not depend on the libm
of the machine that reads it.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle_np as on  # noqa: E402
from rstorch_b200 import synth  # noqa: E402

DIMS = [20, 16, 12, 5]
BATCH, STEPS, LR, SEED = 8, 4, 0.05, 7


def main() -> None:
    weights = synth.mlp_weights(SEED, DIMS)
    X, T = synth.mnist_like(SEED, 0, BATCH * STEPS, features=DIMS[0], classes=DIMS[-1], zero_fraction=0.5)
    out = {"dims": np.array(DIMS), "batch": BATCH, "steps": STEPS, "lr": LR, "X": X, "T": T}
    for l, (W, b) in enumerate(weights):
        out[f"W0_{l}"], out[f"b0_{l}"] = W, b
    for s in range(STEPS):
        xb, tb = X[s * BATCH:(s + 1) * BATCH], T[s * BATCH:(s + 1) * BATCH]
        loss, acc, grads, weights, logits = on.mlp_step(weights, xb, tb, LR)
        out[f"loss_{s}"], out[f"acc_{s}"], out[f"logits_{s}"] = loss, acc, logits
        for l, ((dW, db), (W, b)) in enumerate(zip(grads, weights)):
            out[f"dW_{s}_{l}"], out[f"db_{s}_{l}"], out[f"W_{s}_{l}"], out[f"b_{s}_{l}"] = dW, db, W, b
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mlp_small_steps.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
