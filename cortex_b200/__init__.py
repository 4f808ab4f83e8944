"""cortex_b200 -- B200 (sm_100a) backend for cortex's dense-inference hot path.

Layout (mirrors the reference's namespaces for this path):
  dimensions   cortex.tensor.dimensions   shape / stride / index descriptors
  tensor       cortex.tensor              gemm!, binary-op!, unary-op!, unary-reduce!, assign!, softmax!, conv
  tensor_math  cortex.tensor.math         TensorMath protocol -> C ABI marshalling
  driver       cortex.compute.driver      driver / device / stream / buffer / event over the C ABI
  nn           cortex.compute.nn.*        linear / relu / softmax / convolution layer glue
  parallel     (no counterpart)           batch sharding across GPUs, column-sharded last layer
  csrc/        resources/*.cu + cuBLAS/cuDNN call sites, rewritten as sm_100a kernels

The CUDA shared library is loaded on first use of the driver; there is no CPU
fallback anywhere in this package.
"""
__all__ = ["dimensions", "tensor", "tensor_math", "driver", "nn", "parallel"]
