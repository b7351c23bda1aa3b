"""What a mixer asks of the cache, declared as data."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVNeed:
    """Keys and values of every cached position (``window`` None) or of the last
    ``window`` positions only.  ``value_plane`` False: one row per position and head instead of a key row
    and a value row (a compressed cache whose rows serve as both).  ``value_dim`` not None: value rows of that
    many lanes instead of ``head_dim``, in a pool of their own.  ``keep_first`` > 0 (with a window): the first
    ``keep_first`` positions of a sequence are kept for good beside the window."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_plane: bool = True
    value_dim: Optional[int] = None
    keep_first: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size tensor per sequence, zero when the sequence starts.  A mixer that keeps several of
    the same shape tells them apart by ``name``."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32
    name: str = ""
