from sparta_b200.specializer.kernels.kernel_base import KernelBase, PortConfig
from sparta_b200.specializer.kernels.matmul import (
    SparseMatMulKernel, SparTASparseMatMulKernel, OpenAISparseMatMulKernel,
)
from sparta_b200.specializer.kernels.softmax import (
    SparseSoftmaxForwardKernel, SparTASparseSoftmaxForwardKernel,
    SparseSoftmaxBackwardKernel, SparTASparseSoftmaxBackwardKernel,
)
