"""TEST INFRASTRUCTURE: CPU restatement of the reference's training step.

Only tests/, the smoke entry point and the benchmark's CPU-baseline leg import
this package; the product (rstorch_b200) never does.
"""
