"""Hooks used by the parity tests only; the product path never sets them.

``SINK``       when set to a dict, the next forward/backward stores its intermediates there.
``FORCE_SEL``  an int [T, K] tensor that replaces the top-k selection of the next forward, so that the float path
               can be compared with a reference run whose near-tie selections differ (the gating weights are then
               recomputed with torch from the kernel's own logits).
"""
from __future__ import annotations

from typing import Optional

import torch

SINK: Optional[dict] = None
FORCE_SEL: Optional[torch.Tensor] = None


def capture(**tensors) -> None:
    if SINK is not None:
        SINK.update(tensors)


def capturing() -> bool:
    return SINK is not None


def forced_selection(logits: torch.Tensor):
    """(sel, weights) for the forced selection, or None."""
    if FORCE_SEL is None:
        return None
    forced = FORCE_SEL.to(device=logits.device, dtype=torch.int32).contiguous()
    aff = torch.sigmoid(logits).gather(1, forced.long())
    return forced, (aff / (aff.sum(-1, keepdim=True) + 1e-9)).contiguous()
