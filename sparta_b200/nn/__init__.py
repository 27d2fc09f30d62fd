from sparta_b200.specializer import OperatorBase, SparseLinear, SparseBatchMatMul, SparseSoftmax, SparseAttention
from sparta_b200.nn.module_tuner import tune_combined_module as tune, build_combined_module as build
from sparta_b200.nn.host_stream import HostStreamedRows
