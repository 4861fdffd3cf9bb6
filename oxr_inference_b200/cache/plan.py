"""What the model's schedule needs of the cache: which runs share a pool of pages, which keep fixed state."""

from __future__ import annotations

from dataclasses import dataclass

from oxr_inference_b200.parts.base import PagedKVNeed, StateNeed


@dataclass(frozen=True)
class GroupPlan:
    """Layers with the same need (KV heads, head size, window) share pages: one page id is valid in each of
    them, as in the reference one block id is valid in every layer (oxr_runtime/kv_cache.py:23). Layers with a
    different need get a pool and block tables of their own."""

    need: PagedKVNeed
    num_layers: int


@dataclass(frozen=True)
class EntryPlan:
    """Where one schedule entry keeps what it keeps."""

    group: int | None = None
    layer_in_group: int = 0
    store: bool = True
    state: int | None = None


@dataclass(frozen=True)
class CachePlan:
    groups: tuple[GroupPlan, ...]
    states: tuple[StateNeed, ...]
    entries: tuple[EntryPlan, ...]


def split_need(need, where: str = "") -> tuple[PagedKVNeed | None, StateNeed | None]:
    """A mixer's need as (paged part, state part): it may keep pages, a fixed-size state, both (given as a pair) or nothing."""
    paged = state = None
    for one in (need if isinstance(need, (tuple, list)) else (need,)):
        if one is None:
            continue
        if isinstance(one, PagedKVNeed) and paged is None:
            paged = one
        elif isinstance(one, StateNeed) and state is None:
            state = one
        else:
            raise TypeError(f"{where}unknown or repeated cache need {one!r}")
    return paged, state


def make_cache_plan(needs: list, cache_of: list[int | None]) -> CachePlan:
    """``needs[i]``: what schedule entry i's mixer keeps (a :class:`PagedKVNeed`, a :class:`StateNeed`, a pair of both, or None);
    ``cache_of[i]``: the entry whose cache it reads instead."""
    groups: list[list] = []  # [need, layer count]
    states: list[StateNeed] = []
    entries: list[EntryPlan | None] = [None] * len(needs)
    for i, (need, src) in enumerate(zip(needs, cache_of)):
        if src is not None:
            continue
        paged, fixed = split_need(need, f"schedule entry {i}: ")
        group = layer_in_group = state = None
        if paged is not None:
            for g, (have, count) in enumerate(groups):
                if have == paged:
                    group, layer_in_group = g, count
                    groups[g][1] += 1
                    break
            else:
                groups.append([paged, 1])
                group, layer_in_group = len(groups) - 1, 0
        if fixed is not None:
            states.append(fixed)
            state = len(states) - 1
        entries[i] = EntryPlan(group=group, layer_in_group=layer_in_group or 0, state=state)
    for i, src in enumerate(cache_of):
        if src is None:
            continue
        if not 0 <= src < len(needs) or cache_of[src] is not None:
            raise ValueError(f"schedule entry {i} reads the cache of entry {src}, which has none of its own")
        if src >= i:
            raise ValueError(f"schedule entry {i} reads the cache of a later entry ({src}); it would read stale keys")
        owner = entries[src]
        if owner.group is None:
            raise ValueError(f"schedule entry {i} reads the cache of entry {src}, which keeps no keys and values")
        if needs[i] != needs[src]:
            raise ValueError(f"schedule entry {i} needs {needs[i]} but reads the cache of entry {src} with {needs[src]}")
        entries[i] = EntryPlan(group=owner.group, layer_in_group=owner.layer_in_group, store=False)
    return CachePlan(tuple(GroupPlan(n, c) for n, c in groups), tuple(states), tuple(entries))
