from sparta_b200.testing.mask import block_mask, band_global_random_mask
from sparta_b200.testing.utils import check, profile
from sparta_b200.testing.math import (
    sparse_softmax_forward_reference,
    sparse_softmax_backward_reference,
    sparse_multi_head_attention_reference,
)
