"""Device side of the cache: the pages and state tensors, and which run uses which.

:func:`plan_cache` reads a built model's run order and every mixer's declared need and says
which runs own pages (in which group), which read another run's pages and which keep a state
slot. :class:`CacheStorage` allocates accordingly: per owning run two tensors
``[num_pages, page_size, kv_heads, head_dim]`` (keys, values) in the model dtype, as the
reference lays out its per-layer cache (``src/turboserve/engine/core/kv_cache.py:375-379,
554-566``), and per stateful run one tensor ``[num_slots, *shape]``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import PagedKVNeed, StateNeed
from .manager import GroupSpec


@dataclass
class RunCache:
    """What one run of a layer gets to see of the cache."""

    kind: str  # "paged" (pages, and states if the mixer declares some too) or "state"
    group: int = 0
    writes: bool = True
    k_pages: torch.Tensor | None = None
    v_pages: torch.Tensor | None = None
    states: list[torch.Tensor] = field(default_factory=list)
    """One tensor ``[slots, *shape]`` per state the mixer declares, in its order."""

    @property
    def state(self) -> torch.Tensor | None:
        return self.states[0] if self.states else None


@dataclass(frozen=True)
class RunPlan:
    kind: str | None  # "paged", "state" or None
    owner: int  # run index whose storage is used (own index when it owns)
    group: int = 0
    need: PagedKVNeed | StateNeed | None = None
    """The pages the run needs (``kind == "paged"``), else its first state."""

    states: tuple[StateNeed, ...] = ()
    """Every fixed-size state the run keeps per request."""


def split_needs(need) -> tuple[PagedKVNeed | None, tuple[StateNeed, ...]]:
    """What a mixer declares (one need, a tuple of them, or nothing) as (pages, states)."""
    if need is None:
        return None, ()
    items = need if isinstance(need, (tuple, list)) else (need,)
    paged = [n for n in items if isinstance(n, PagedKVNeed)]
    states = tuple(n for n in items if isinstance(n, StateNeed))
    if len(paged) > 1 or len(paged) + len(states) != len(items):
        raise TypeError(f"a mixer declares at most one PagedKVNeed and any number of StateNeed, got {need!r}")
    return (paged[0] if paged else None), states


@dataclass
class CachePlan:
    runs: list[RunPlan]
    windows: list[int | None] = field(default_factory=list)
    """One entry per group: the window of that group (``None`` = keeps everything)."""

    def group_names(self) -> list[str]:
        return ["full" if w is None else f"window{w}" for w in self.windows]

    def bytes_per_page(self, page_size: int, itemsize: int) -> list[int]:
        """Bytes one page id of each group stands for, over all runs that own pages in it."""
        out = [0] * len(self.windows)
        for index, run in enumerate(self.runs):
            if run.kind == "paged" and run.owner == index:
                out[run.group] += page_size * run.need.num_kv_heads * (run.need.head_dim + run.need.v_dim) * itemsize
        return out

    def state_bytes_per_slot(self) -> int:
        total = 0
        for index, run in enumerate(self.runs):
            if run.owner != index:
                continue
            for need in run.states:
                count = 1
                for s in need.shape:
                    count *= s
                # a state in the activation type is counted at four bytes an element: never too little
                total += count * (4 if need.dtype is None else torch.empty((), dtype=need.dtype).element_size())
        return total


def plan_cache(needs: list[PagedKVNeed | StateNeed | None], cache_from: list[int | None]) -> CachePlan:
    """``needs[i]`` is what run ``i``'s mixer declares; ``cache_from[i]`` the run it reads instead."""
    windows: list[int | None] = []
    runs: list[RunPlan] = []
    for index, (declared, source) in enumerate(zip(needs, cache_from)):
        need, states = split_needs(declared)
        if source is not None:
            src = runs[source]
            if src.kind != "paged" or need is None or states:
                raise ValueError(f"run {index} can only read pages of keys and values from run {source}")
            if (need.num_kv_heads, need.head_dim, need.v_dim) != (src.need.num_kv_heads, src.need.head_dim, src.need.v_dim):
                raise ValueError(f"run {index} and run {source} disagree on kv heads or head size")
            if need.window != src.need.window:
                raise ValueError(f"run {index} reads the pages of run {source} but has another window")
            runs.append(RunPlan("paged", source, src.group, need))
        elif need is not None:
            if need.window not in windows:
                windows.append(need.window)
            runs.append(RunPlan("paged", index, windows.index(need.window), need, states))
        elif states:
            runs.append(RunPlan("state", index, 0, states[0], states))
        else:
            runs.append(RunPlan(None, index))
    if not windows:
        windows.append(None)  # a model without paged layers still gets one (unused) group
    return CachePlan(runs, windows)


class CacheStorage:
    def __init__(self, plan: CachePlan, groups: list[GroupSpec], num_state_slots: int, dtype: torch.dtype,
                 device: torch.device | str) -> None:
        if len(groups) != len(plan.windows):
            raise ValueError("one GroupSpec per cache group is needed")
        self.plan, self.groups, self.dtype, self.device = plan, groups, dtype, torch.device(device)
        self.num_state_slots = num_state_slots
        owned: dict[int, RunCache] = {}
        for index, run in enumerate(plan.runs):
            if run.owner != index:
                continue
            states = [torch.zeros((num_state_slots, *need.shape), dtype=need.dtype or dtype, device=self.device)
                      for need in run.states]
            if run.kind == "paged":
                g = groups[run.group]
                shape = (g.num_pages, g.page_size, run.need.num_kv_heads)
                owned[index] = RunCache(
                    "paged", group=run.group, writes=True,
                    k_pages=torch.zeros((*shape, run.need.head_dim), dtype=dtype, device=self.device),
                    v_pages=torch.zeros((*shape, run.need.v_dim), dtype=dtype, device=self.device),
                    states=states,
                )
            elif run.kind == "state":
                owned[index] = RunCache("state", states=states)
        self.run_caches: list[RunCache | None] = []
        for index, run in enumerate(plan.runs):
            if run.kind is None:
                self.run_caches.append(None)
            elif run.owner == index:
                self.run_caches.append(owned[index])
            else:
                src = owned[run.owner]
                self.run_caches.append(RunCache("paged", group=src.group, writes=False, k_pages=src.k_pages, v_pages=src.v_pages))

    def reset_state_slot(self, slot: int) -> None:
        """Zero a slot's state in every stateful run (at admission, and before a recompute)."""
        for cache in self.run_caches:
            if cache is not None and cache.writes:
                for state in cache.states:
                    state[slot].zero_()

    def nbytes(self) -> int:
        total = 0
        seen = set()
        for cache in self.run_caches:
            if cache is None:
                continue
            for t in (cache.k_pages, cache.v_pages, *cache.states):
                if t is not None and t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total
