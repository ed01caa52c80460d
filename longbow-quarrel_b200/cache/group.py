"""What a group of cache entries with one need looks like to the cache.

The cache knows slots and lengths; each group knows its own storage.  A mixer's need
(`parts.base.CacheNeed`) makes its group, so a mixer with storage of another shape
than the two kinds that live here (paged keys and values, fixed-size state) brings a
class derived from `CacheGroup` with it and no file of the cache changes.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class CacheSizing:
    """How large the cache is: `n_pages` pages of `page_size` tokens for all live sequences together,
    at most `pages_per_seq` of them for one sequence, `max_slots` live sequences."""
    n_pages: int
    page_size: int
    max_slots: int
    pages_per_seq: int
    max_context: int
    dtype: torch.dtype
    device: object


class CacheGroup:
    """Storage for the cache entries `entries`.  Every call below comes from the host, before a
    step's kernels are launched or after they are queued; none may wait for the device."""

    entries: list[int]

    def start(self, slot: int) -> None:
        """A sequence starts in `slot`: what the last sequence left there must not show."""

    def reserve(self, slot: int, old_len: int, new_len: int) -> None:
        """Room for positions [old_len, new_len) of the sequence in `slot`; raises CacheError if there is none
        (before anything of the step is launched)."""

    def commit(self, slot: int, length: int) -> None:
        """The step is queued; the sequence now holds `length` tokens.  What no later token needs may go back."""

    def reserve_one_each(self, slots, old_lens) -> None:
        """reserve(slot, old, old + 1) for many sequences at once (numpy arrays): the step of one token per
        sequence, which a group may do faster than one call per sequence."""
        for slot, old in zip(slots.tolist(), old_lens.tolist()):
            self.reserve(slot, old, old + 1)

    def commit_one_each(self, slots, new_lens) -> None:
        for slot, length in zip(slots.tolist(), new_lens.tolist()):
            self.commit(slot, length)

    def release(self, slot: int) -> None:
        """The sequence in `slot` has ended: everything it holds goes back."""

    def upload(self) -> None:
        """Bring the device's copy of the group's tables up to date (called once before a step's kernels)."""

    def view(self, entry: int):
        """What the mixer of cache entry `entry` is given as `cache_view`."""
        raise NotImplementedError

    def nbytes(self) -> int:
        return 0

    def pages_in_use(self) -> int:
        return 0


class SeveralGroups(CacheGroup):
    """The groups of a need that is several needs at once (`parts.base.SeveralNeeds`): every call goes to each of
    them in turn, and an entry's view is the tuple of their views."""

    def __init__(self, entries: list[int], groups: list):
        """groups: one for each of the needs; None for a side that keeps nothing (its view is None)."""
        self.entries, self.views_of = list(entries), list(groups)
        self.groups = [g for g in groups if g is not None]

    def start(self, slot: int) -> None:
        for g in self.groups:
            g.start(slot)

    def reserve(self, slot: int, old_len: int, new_len: int) -> None:
        for g in self.groups:
            g.reserve(slot, old_len, new_len)

    def commit(self, slot: int, length: int) -> None:
        for g in self.groups:
            g.commit(slot, length)

    def reserve_one_each(self, slots, old_lens) -> None:
        for g in self.groups:
            g.reserve_one_each(slots, old_lens)

    def commit_one_each(self, slots, new_lens) -> None:
        for g in self.groups:
            g.commit_one_each(slots, new_lens)

    def release(self, slot: int) -> None:
        for g in self.groups:
            g.release(slot)

    def upload(self) -> None:
        for g in self.groups:
            g.upload()

    def view(self, entry: int):
        return tuple(g.view(entry) if g is not None else None for g in self.views_of)

    def nbytes(self) -> int:
        return sum(g.nbytes() for g in self.groups)

    def pages_in_use(self) -> int:
        return sum(g.pages_in_use() for g in self.groups)

    def flat(self) -> list[CacheGroup]:
        out = []
        for g in self.groups:
            out += g.flat() if isinstance(g, SeveralGroups) else [g]
        return out
