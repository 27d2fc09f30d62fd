"""Timing and checking helpers (API of sparta/testing/utils.py:9-73)."""
from typing import Callable, List, Optional

import torch


def check(func: Callable, inputs: List, target_outputs: List, atol: float = 1e-4, rtol: float = 1e-8):
    """Run ``func(*inputs)`` and compare with ``target_outputs`` (fp32 tolerance of the reference by
    default; pass atol=2e-2, rtol=1e-4 for half types)."""
    outputs = func(*inputs)
    if len(target_outputs) == 1:
        outputs = [outputs]
    assert len(outputs) == len(target_outputs), \
        f'expected {len(target_outputs)} outputs, got {len(outputs)}'
    for out, ref in zip(outputs, target_outputs):
        torch.testing.assert_close(out, ref.to(out.dtype), atol=atol, rtol=rtol)


def profile(func: Callable, inputs: List, target_outputs: Optional[List] = None, num_warmups: int = 10,
            num_iters: int = 10, cuda: bool = False, atol: float = 1e-4, rtol: float = 1e-8) -> float:
    """Latency of ``func(*inputs)`` in milliseconds, measured with CUDA events on the current stream.
    ``cuda=True`` (kernel-only time through the torch profiler in the reference) uses the same event
    timing here.  A failing call yields ``inf``; a failing check raises."""
    if target_outputs is not None:
        check(func, inputs, target_outputs, atol, rtol)
    try:
        torch.cuda.synchronize()
        for _ in range(num_warmups):
            func(*inputs)
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(num_iters):
            func(*inputs)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / max(num_iters, 1)
    except Exception:
        return float('inf')
