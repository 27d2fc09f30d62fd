"""Row-sharded operators on host-resident data.

The block-sparse operators shard by token rows with no exchange between shards.  When the
activations live in pinned host memory, that lets the copy of the next rows in, the kernel on the
current rows and the copy of the previous results out run at the same time (PCIe is full duplex and
the GPU has separate copy engines per direction), instead of in-copy, kernel, out-copy back to back.
"""
from typing import Callable, List, Optional

import torch


class HostStreamedRows(object):
    """Apply ``op`` (built for ``chunk_rows`` input rows) to a pinned host tensor, chunk by chunk.

    Args:
        op: callable taking one device tensor ``[chunk_rows, ...]`` and returning ``[chunk_rows, ...]``,
            e.g. a ``SparseLinear`` built with a ``chunk_rows``-row sample input.
        chunk_rows: rows per chunk; the host tensor's row count must be a multiple of it.
        depth: device input buffers kept in flight.
        graph: capture the whole sequence (copies, kernels and their cross-stream dependencies) in a CUDA
            graph on the first call for a pair of host buffers and replay it afterwards: one launch instead
            of about a dozen host calls per chunk.  The host buffers' addresses are baked into the graph, so
            a different buffer (or shape) captures anew.  The operator must be capturable: no synchronisation
            and no host-side read of device data inside it (the prebuilt kernels of this package qualify; a
            failed capture raises, and PyTorch leaves the CUDA random generator unusable after one).

    ``__call__(x_host, y_host)`` enqueues everything relative to the current stream: work starts after
    what the current stream already holds and the current stream waits for the last copy out, so events
    or a synchronize on the current stream bracket the whole transfer + compute.
    """

    def __init__(self, op: Callable[[torch.Tensor], torch.Tensor], chunk_rows: int, depth: int = 2,
                 graph: bool = False):
        assert chunk_rows > 0 and depth >= 1
        self._op = op
        self._rows = chunk_rows
        self._depth = depth
        self._use_graph = graph
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_key = None
        self._bufs: Optional[List[torch.Tensor]] = None
        self._s_in: Optional[torch.cuda.Stream] = None
        self._s_out: Optional[torch.cuda.Stream] = None

    def _prepare(self, x_host: torch.Tensor, device: torch.device):
        shape = (self._rows,) + tuple(x_host.shape[1:])
        if self._bufs is None or self._bufs[0].shape != shape or self._bufs[0].dtype != x_host.dtype:
            self._bufs = [torch.empty(shape, dtype=x_host.dtype, device=device) for _ in range(self._depth)]
            self._s_in = torch.cuda.Stream(device)
            self._s_out = torch.cuda.Stream(device)

    def __call__(self, x_host: torch.Tensor, y_host: torch.Tensor, device: Optional[torch.device] = None):
        assert x_host.is_pinned() and y_host.is_pinned(), 'host buffers must be pinned for asynchronous copies'
        n = x_host.shape[0]
        assert n % self._rows == 0, f'{n} rows are not a multiple of the chunk size {self._rows}'
        assert y_host.shape[0] == n
        device = device or torch.device('cuda', torch.cuda.current_device())
        if not self._use_graph:
            return self._enqueue(x_host, y_host, device)
        key = (x_host.data_ptr(), y_host.data_ptr(), tuple(x_host.shape), tuple(y_host.shape), x_host.dtype, device)
        if self._graph is None or self._graph_key != key:
            self._enqueue(x_host, y_host, device)  # plain first pass: buffers, lazy initialisation in the operator
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            # thread-local capture mode: other threads of the process (a collective library's watchdog) may go on
            # making CUDA calls while this thread captures
            with torch.cuda.graph(graph, capture_error_mode='thread_local'):
                self._enqueue(x_host, y_host, device)
            self._graph, self._graph_key = graph, key
        self._graph.replay()
        return y_host

    def _enqueue(self, x_host: torch.Tensor, y_host: torch.Tensor, device: torch.device):
        n = x_host.shape[0]
        self._prepare(x_host, device)
        cur = torch.cuda.current_stream(device)
        start = torch.cuda.Event()
        start.record(cur)
        self._s_in.wait_event(start)
        self._s_out.wait_event(start)
        computed: List[torch.cuda.Event] = []
        for i in range(n // self._rows):
            rows = slice(i * self._rows, (i + 1) * self._rows)
            buf = self._bufs[i % self._depth]
            with torch.cuda.stream(self._s_in):
                if i >= self._depth:  # the kernel that read this buffer last has finished
                    self._s_in.wait_event(computed[i - self._depth])
                buf.copy_(x_host[rows], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self._s_in)
            cur.wait_event(arrived)
            y = self._op(buf)
            done = torch.cuda.Event()
            done.record(cur)
            computed.append(done)
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(done)
                y_host[rows].copy_(y, non_blocking=True)
                y.record_stream(self._s_out)
        finished = torch.cuda.Event()
        finished.record(self._s_out)
        cur.wait_event(finished)
        return y_host
