"""HostStreamedRows: chunked, overlapped host -> device -> host application of a row-sharded operator
gives the same rows as one call on the whole input."""
import pytest
import torch

import sparta_b200 as sparta
from oracle import oracle

pytestmark = pytest.mark.gpu


def _linear(rows, K, N, mask, dense):
    op = sparta.nn.SparseLinear(dense, weight_mask=mask)
    op.build({'forward:C': {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 128, 'BLOCK_SIZE_K_VALUE': 32,
                            'BLOCK_SIZE_N_VALUE': 32}},
             sample_inputs=[torch.zeros((rows, K), dtype=torch.float16, device='cuda')])
    return op


@pytest.mark.parametrize('chunks,depth', [(1, 1), (4, 2), (8, 3)])
def test_streamed_rows_match_single_call(chunks, depth):
    rows, K, N = 1024, 256, 384
    g = torch.Generator().manual_seed(7)
    x = torch.randn((rows, K), generator=g).half()
    mask = oracle.block_mask((N, K), (32, 32), 0.6, generator=g).cuda()
    dense = torch.nn.Linear(K, N, device='cuda', dtype=torch.float16)
    whole = _linear(rows, K, N, mask, dense)(x.cuda()).cpu()
    chunk_op = _linear(rows // chunks, K, N, mask, dense)
    streamed = sparta.nn.HostStreamedRows(chunk_op, rows // chunks, depth=depth)
    x_host, y_host = x.pin_memory(), torch.empty((rows, N), dtype=torch.float16).pin_memory()
    for _ in range(2):  # the second call reuses the buffers and streams
        y_host.zero_()
        streamed(x_host, y_host)
        torch.cuda.synchronize()
        assert torch.equal(y_host, whole)


def test_streamed_rows_replayed_from_a_graph():
    """graph=True: the second and later calls replay the captured sequence; new host buffers capture anew."""
    rows, K, N, chunks = 1024, 256, 384, 4
    g = torch.Generator().manual_seed(8)
    mask = oracle.block_mask((N, K), (32, 32), 0.6, generator=g).cuda()
    dense = torch.nn.Linear(K, N, device='cuda', dtype=torch.float16)
    whole_op = _linear(rows, K, N, mask, dense)
    streamed = sparta.nn.HostStreamedRows(_linear(rows // chunks, K, N, mask, dense), rows // chunks, graph=True)
    for trial in range(2):  # two different pairs of host buffers
        x = torch.randn((rows, K), generator=g).half()
        x_host, y_host = x.pin_memory(), torch.empty((rows, N), dtype=torch.float16).pin_memory()
        for call in range(3):
            if call == 2:  # new contents in the same buffers: the graph reads them at replay time
                x_host.copy_(torch.randn((rows, K), generator=g).half())
            y_host.zero_()
            streamed(x_host, y_host)
            torch.cuda.synchronize()
            assert torch.equal(y_host, whole_op(x_host.cuda()).cpu())
        assert streamed._graph is not None


def test_streamed_rows_rejects_bad_inputs():
    streamed = sparta.nn.HostStreamedRows(lambda t: t, 128)
    x = torch.zeros((256, 8)).pin_memory()
    with pytest.raises(AssertionError):
        streamed(torch.zeros((256, 8)), x)          # not pinned
    with pytest.raises(AssertionError):
        streamed(torch.zeros((200, 8)).pin_memory(), torch.zeros((200, 8)).pin_memory())  # not a multiple
