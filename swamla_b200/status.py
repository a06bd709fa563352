"""Host-side reading of the device status word without stalling the launch queue.

Every forward/backward of the path owns one int32 status word on the device.  Kernels write a non-zero code into it
when a bounded wait gives up (101-103) or when an expert-parallel shard receives more rows than its buffers hold
(201: the excess rows are dropped, the results of that step are wrong).  Reading the word with ``.item()`` would
synchronise the stream on every step, so the word is copied to pinned host memory behind the step's kernels and looked
at later: ``poll()`` inspects the copies that have already completed and raises for the first non-zero code;
``poll(block=True)`` waits for all of them first.  The layers call ``poll()`` at the start of every forward and in
``update_bias_from_last_forward()`` (once per training step), and expose the blocking form as ``check_status()``.
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from . import _cabi

_pending: List[Tuple[torch.cuda.Event, torch.Tensor, str]] = []
_free: List[torch.Tensor] = []


def post(status: torch.Tensor, label: str) -> None:
    """Queues an asynchronous copy of ``status`` (device int32[1]) behind the work already on the current stream."""
    if torch.cuda.is_current_stream_capturing():
        return                       # a captured step keeps its status word in a static buffer; nothing to queue
    host = _free.pop() if _free else torch.empty(1, dtype=torch.int32, pin_memory=True)
    host.copy_(status, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record()
    _pending.append((ev, host, label))


def poll(block: bool = False) -> None:
    """Raises ``LmoeError`` if a completed step reported a non-zero device status."""
    global _pending
    if not _pending or torch.cuda.is_current_stream_capturing():
        return
    keep, bad = [], None
    for ev, host, label in _pending:
        if block:
            ev.synchronize()
        if ev.query():
            code = int(host[0])
            _free.append(host)
            if code != 0 and bad is None:
                bad = (code, label)
        else:
            keep.append((ev, host, label))
    _pending = keep
    if bad is not None:
        code, label = bad
        raise _cabi.LmoeError(f"device status {code} in {label}: {_cabi.status_string(code)}")


def pending() -> int:
    return len(_pending)
