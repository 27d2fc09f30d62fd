"""B200-native (sm_100a) block-sparse operators behind the ``sparta`` API.

    import sparta_b200 as sparta
    op = sparta.nn.SparseLinear(dense_linear, weight_mask=mask)
    sparta.nn.tune(op, sample_inputs=[x])

The operators call hand-written CUDA kernels through the C-ABI library declared in
``include/sparta_b200.h``; there is no CPU or eager fallback.
"""
from sparta_b200 import nn, testing, tesa

__version__ = '0.1.0'
__env_ready__ = True
