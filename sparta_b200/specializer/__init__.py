from sparta_b200.specializer.operators import (
    OperatorBase, SparseLinear, SparseBatchMatMul, SparseSoftmax, SparseAttention,
)
