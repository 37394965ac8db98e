"""What a mixer asks of the cache for one entry of the schedule."""
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class CacheNeed:
    """Per-token keys and values (n_kv_heads > 0), all of them or a window of the last ones,
    and/or a per-sequence state of fixed shape (float32, zeroed when a slot is handed out)."""
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
