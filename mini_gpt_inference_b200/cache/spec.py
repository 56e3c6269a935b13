"""What a layer keeps per request between steps.

The reference has one kind only: keys and values of every token, for every layer alike
(src/minigpt_infer/cache/paged.py:109-123).  Here a mixer states its need as data and
the cache manager groups layers with equal needs.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values in pages.  ``window``: only the last ``window`` positions are ever
    read again (None: all of them), so older pages can be given back early."""

    n_kv_head: int
    head_dim: int
    window: int | None = None
    # Page geometry of the group these layers form.  None: the cache manager's default page
    # size; and for the pool, the manager's default number of pages, or, with a window, as many as
    # every request slot can hold at once (a window's length plus the portion being written never
    # needs more), if that is fewer.
    page_tokens: int | None = None
    num_pages: int | None = None

    def __post_init__(self) -> None:
        if self.n_kv_head <= 0 or self.head_dim <= 0:
            raise ValueError("n_kv_head and head_dim must be positive")
        if self.window is not None and self.window <= 0:
            raise ValueError("window must be positive when given")
        if self.page_tokens is not None and self.page_tokens <= 0:
            raise ValueError("page_tokens must be positive when given")
        if self.num_pages is not None and self.num_pages <= 0:
            raise ValueError("num_pages must be positive when given")


@dataclass(frozen=True)
class FixedStateSpec:
    """A tensor of fixed shape per request, living in a slot of the state pool."""

    shape: tuple[int, ...]
    dtype: str = "float32"
