"""CPU oracle for the sparse-convolution hot path.

TEST INFRASTRUCTURE ONLY.  This package restates, on the CPU, the algorithm of
the reference's rulebook generation, gather-GEMM (forward / input-gradient /
weight-gradient) and sparse pooling.  It exists to check the CUDA kernels and
to be timed as the CPU baseline; nothing in the product package imports it and
no product code path may route through it.

Parity is pinned: ``tests/golden/*.npz`` were produced by executing the
reference itself (its Triton kernels under Triton's CPU interpreter) and by
extracting the reference's own frozen golden cases; ``tests/test_oracle_*``
check every function here against those vectors.
"""
