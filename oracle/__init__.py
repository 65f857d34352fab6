"""TEST INFRASTRUCTURE: CPU oracle for the transformer-forward op set.

`msl_ref` wraps oracle/msl_ref.c (a C restatement of the reference's Metal kernel math);
`torch_ref` holds PyTorch-CPU-eager models (the reference's own correctness oracle and benchmark
baseline: python/tests/test_cpp_backend.py:121-133, python/tests/bench_comparison.py:23-50).
Nothing in the product path imports this package.
"""
