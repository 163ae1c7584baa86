"""The cache manager: pages for every group, a slot per request, and the device storage.

Lifecycle of a request: ``admit`` (a slot), then before each step ``reserve`` (pages in
every group for the positions the step touches; all or nothing), after the step ``commit``
(the new length; window groups give passed pages back), at the end ``release`` (everything
back).  Host-side logic needs no GPU: with ``device=None`` no storage is allocated and only
the bookkeeping runs.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .groups import NO_PAGE, CacheGroup, CacheNeed, PagedKV, StateSlot, StateSlots
from .pages import OutOfPages
from .slots import OutOfSlots, SlotAllocator


class KVView:
    """What a mixer sees of its cache: its pages and the group whose block table indexes them."""

    def __init__(self, group_index: int, k_pages, v_pages, page_size: int):
        self.group_index = group_index
        self.k_pages, self.v_pages, self.page_size = k_pages, v_pages, page_size


class StateView:
    """A state-keeping mixer's tensor ``[num_slots, *shape]``; index it with the step's slot ids."""

    def __init__(self, state):
        self.state = state


class StateViews:
    """The tensors of a ``StateSlots`` need, in its order."""

    def __init__(self, views):
        self.views = list(views)

    def __getitem__(self, i: int) -> StateView:
        return self.views[i]

    def __len__(self) -> int:
        return len(self.views)


class CacheManager:
    def __init__(self, needs: Sequence[object], num_pages: int, page_size: int, max_requests: int,
                 max_positions: int, dtype: torch.dtype = torch.bfloat16, device=None,
                 pages_per_group: Optional[Dict[int, int]] = None, entry_states: Sequence[object] = ()):
        """``needs[c]`` is what cache ``c`` asks for: a ``PagedKV``, a ``StateSlot`` or None.  ``entry_states[i]`` is the
        state that entry i of the run order keeps for itself beside its cache (a ``StateSlot`` or None: the tail of a
        short convolution, say, which a layer has even when the keys it reads are another layer's); its view is
        ``state_views[i]``.

        ``num_pages`` is the number of usable pages of every group (one more, the null page,
        is added); ``pages_per_group`` overrides it by group index.
        """
        if page_size < 1:
            raise ValueError("page size must be positive")
        self.page_size = page_size
        self.max_positions = max_positions
        self.max_blocks = (max_positions + page_size - 1) // page_size
        self.dtype, self.device = dtype, device
        self.slots = SlotAllocator(max_requests)
        self.groups: List[CacheGroup] = []
        self.views: List[object] = [None] * len(needs)
        self.lengths: Dict[object, int] = {}
        self._state_tensors: List[torch.Tensor] = []
        self._slot_rows: Dict[int, List[torch.Tensor]] = {}      # slot -> its row of every state tensor
        # request -> positions that every group has pages for already (a step within them asks the groups nothing:
        # fifteen of sixteen decode steps with pages of 16)
        self._room: Dict[object, int] = {}

        # Needs with equal group keys share a group; a need without a key (per-request state) gets storage of its own.
        # What each kind of need provides is the need's own business (``CacheNeed`` in groups.py).
        by_key: Dict[object, List[int]] = {}
        for c, need in enumerate(needs):
            if need is not None and need.group_key() is not None:
                by_key.setdefault(need.group_key(), []).append(c)
        from ..kernels.host import max_cache_groups
        group_need = {key: needs[ids[0]] for key, ids in by_key.items()}
        if len(by_key) > max_cache_groups():
            # more kinds of cache than a step carries block tables for (many windows, say): caches that differ only in what
            # they may give back share a group that keeps pages for the widest of them; every layer still masks by its own
            merged: Dict[object, List[int]] = {}
            merged_need: Dict[object, object] = {}
            for key, ids in by_key.items():
                need = needs[ids[0]]
                coarse = next((k for k, other in merged_need.items()
                               if hasattr(other, "shared_with") and other.shared_with(need) is not None), None)
                if coarse is None:
                    merged[key], merged_need[key] = list(ids), need
                else:
                    merged[coarse].extend(ids)
                    merged_need[coarse] = merged_need[coarse].shared_with(need)
            by_key, group_need = merged, merged_need
            if len(by_key) > max_cache_groups():
                raise ValueError(f"the model's layers need {len(by_key)} kinds of paged cache; a step carries block tables for {max_cache_groups()}")
        for gi, (key, ids) in enumerate(by_key.items()):
            need = group_need[key]
            n = (pages_per_group or {}).get(gi, num_pages)
            self.groups.append(need.make_group(ids, n + 1, page_size, self.max_blocks))
            storage = need.make_storage(len(ids), n + 1, page_size, self.slots.num_slots, dtype, device)
            for i, c in enumerate(ids):
                self.views[c] = need.make_view(storage, i, gi, page_size)
        for c, need in enumerate(needs):
            if need is not None and need.group_key() is None:
                storage = need.make_storage(1, 0, page_size, self.slots.num_slots, dtype, device)
                self._keep_state(storage)
                self.views[c] = need.make_view(storage, 0, -1, page_size)

        self.state_views: List[object] = [None] * len(entry_states)
        for i, need in enumerate(entry_states):
            if need is not None:
                storage = need.make_storage(1, 0, page_size, self.slots.num_slots, dtype, device)
                self._keep_state(storage)
                self.state_views[i] = need.make_view(storage, 0, -1, page_size)

    def _keep_state(self, storage) -> None:
        """Remember per-request state tensors (one, or a list of them): a slot is cleared when a request takes it."""
        if storage is None:
            return
        for t in (storage if isinstance(storage, (list, tuple)) else [storage]):
            if hasattr(t, "zero_"):
                self._state_tensors.append(t)

    # ---- requests ------------------------------------------------------------------------
    def admit(self, req) -> int:
        slot = self.slots.acquire(req)         # raises OutOfSlots
        self.lengths[req] = 0
        self._clear_slot(slot)
        return slot

    def _clear_slot(self, slot: int) -> None:
        """Zeros in every state tensor's row of ``slot``: one launch for all of them where the device has one."""
        rows = self._slot_rows.get(slot)
        if rows is None:
            rows = self._slot_rows[slot] = [st[slot] for st in self._state_tensors]
        if rows and rows[0].is_cuda:
            torch._foreach_zero_(rows)
        else:
            for row in rows:
                row.zero_()

    def is_live(self, req) -> bool:
        return req in self.lengths

    def length(self, req) -> int:
        return self.lengths[req]

    def pages_needed(self, req, new_len: int) -> List[int]:
        if new_len <= self._room.get(req, 0):
            return [0] * len(self.groups)
        start = self.lengths.get(req, 0)
        return [g.pages_needed(req, start, new_len) for g in self.groups]

    def can_reserve(self, wants: Dict[object, int]) -> bool:
        """Would ``reserve`` succeed for all of ``{request: new_len}`` together?"""
        need = [0] * len(self.groups)
        room = self._room
        for req, new_len in wants.items():
            if new_len <= room.get(req, 0):
                continue
            for gi, n in enumerate(self.pages_needed(req, new_len)):
                need[gi] += n
        return all(n <= g.pool.available for n, g in zip(need, self.groups))

    def reserve(self, req, new_len: int) -> None:
        """Pages in every group for a step that takes ``req`` from its length to ``new_len``."""
        if req not in self.lengths:
            raise KeyError(f"request {req!r} was not admitted")
        if new_len > self.max_positions:
            raise ValueError(f"request {req!r}: {new_len} positions exceed the maximum of {self.max_positions}")
        if new_len <= self._room.get(req, 0):
            return
        start = self.lengths[req]
        done = []
        try:
            for g in self.groups:
                done.append((g, g.reserve(req, start, new_len)))
        except OutOfPages:
            for g, pages in done:
                g.give_back(req, pages)
            raise
        self._room[req] = min((len(g.tables[req]) for g in self.groups), default=0) * self.page_size if self.groups else self.max_positions

    def commit(self, req, new_len: int) -> None:
        self.lengths[req] = new_len
        for g in self.groups:
            g.trim(req, new_len)

    def truncate(self, req, new_len: int) -> None:
        """Go back to ``new_len`` cached positions (new_len <= the current length)."""
        if new_len > self.lengths[req]:
            raise ValueError(f"request {req!r} holds {self.lengths[req]} positions, cannot truncate to {new_len}")
        if new_len < self.lengths[req] and self._state_tensors:
            # state that is carried from token to token keeps no history: a request can go back to its start only
            if new_len != 0:
                raise ValueError(f"request {req!r}: a model with per-request state cannot go back to position {new_len} "
                                 f"of {self.lengths[req]}; start it again from 0")
            self._clear_slot(self.slots.slot_of(req))
        for g in self.groups:
            g.truncate(req, new_len)
        self.lengths[req] = new_len
        self._room[req] = min((len(g.tables.get(req, ())) for g in self.groups), default=0) * self.page_size if self.groups else self.max_positions

    def release(self, req) -> None:
        if req not in self.lengths:
            raise KeyError(f"request {req!r} is not live")
        for g in self.groups:
            g.release(req)
        self.slots.release(req)
        del self.lengths[req]
        self._room.pop(req, None)

    # ---- what a step uploads ----------------------------------------------------------------
    def block_table_rows(self, group_index: int, reqs: Sequence[object], out: np.ndarray) -> None:
        """Fill ``out[i, :]`` (int32, ``[len(reqs), max_blocks]``) with request i's pages."""
        g = self.groups[group_index]
        for i, r in enumerate(reqs):
            row = g.row(r)
            if row is None:
                out[i].fill(NO_PAGE)
            else:
                out[i] = row

    def slot_ids(self, reqs: Sequence[object]) -> List[int]:
        return [self.slots.slot_of(r) for r in reqs]

    # ---- accounting ------------------------------------------------------------------------
    def stats(self) -> dict:
        return {
            "live_requests": len(self.lengths),
            "groups": [{"name": g.name, "pages_in_use": g.pool.in_use, "pages_free": g.pool.available,
                        "high_water": g.pool.high_water} for g in self.groups],
        }

    def check_invariants(self) -> None:
        """No page lost, none held twice: every page is free or in exactly one table."""
        for g in self.groups:
            seen = {}
            for req, table in g.tables.items():
                for p in table:
                    if p == NO_PAGE:
                        continue
                    if p in seen:
                        raise AssertionError(f"{g.name}: page {p} held by {seen[p]!r} and {req!r}")
                    seen[p] = req
            held = set(g.pool.held_pages())
            if held != set(seen):
                raise AssertionError(f"{g.name}: pool says {sorted(held)} are out, tables hold {sorted(seen)}")
            if g.pool.in_use + g.pool.available != g.pool.capacity:
                raise AssertionError(f"{g.name}: a page is lost")
            for req, room in self._room.items():
                table = g.tables.get(req, [])
                last = (room + self.page_size - 1) // self.page_size
                first = max(g._first_needed_block(self.lengths.get(req, 0)), g.first_block.get(req, 0))
                if last > len(table) or any(p == NO_PAGE for p in table[first:last]):
                    raise AssertionError(f"{g.name}: {req!r} is said to have pages for {room} positions and has not")
            for req, table in g.tables.items():
                row = g.row(req)
                mirror = [] if row is None else row.tolist()
                if mirror[:len(table)] != table and any(p != NO_PAGE for p in table):
                    raise AssertionError(f"{g.name}: the row of {req!r} differs from its table")
                if any(p != NO_PAGE for p in mirror[len(table):]):
                    raise AssertionError(f"{g.name}: the row of {req!r} holds pages beyond its table")
