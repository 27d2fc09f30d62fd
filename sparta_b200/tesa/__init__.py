from sparta_b200.tesa.tesa_base import TeSAIndexes, TeSAFunctionContext
from sparta_b200.tesa.block_compressed import (
    get_bcs_function, BCSIndexes, BCSRIndexes, BCSCIndexes, BCSRCIndexes, BCSFunctionContext,
)
