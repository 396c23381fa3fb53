"""The cache: a slot per sequence, storage per group of layers.

* A **slot** is one live sequence's record: its length and the pages it holds.
  Slots are handed out by :meth:`Cache.open_seq` and come back with
  :meth:`Cache.close_seq`; a closed slot's pages return to the pool and are used
  again by later sequences without being cleared (positions at or beyond a
  sequence's length are never read).
* Keys and values live in **pages** of 64 positions.  A sequence holds
  ``ceil(length / 64)`` pages, so the pool's size is the number of tokens (each
  sequence rounded up to 64) that live sequences may hold at once.
* Schedule entries (layers as they run) with equal needs form a **group** with
  storage of its own, of the class registered for the need's kind
  (:func:`register_storage`): ``paged_kv`` groups [entries, pages, 2, kv_heads,
  64, head_dim]; ``state`` groups [entries, slots, *shape], a record of fixed
  size per sequence that is zeroed when the sequence opens.  All paged groups
  share the page ids (page p of a sequence is page p in each group).  Another
  kind of storage (a ring of the last positions, say) is another registered
  class; nothing here changes for it.
* Page 0 and slot 0 are never handed out: padded batch entries point there.

The bookkeeping is host-side Python over :class:`IndexPool` and needs no GPU;
only the storage tensors live on the device.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..layout import PAGE
from ..parts.base import CacheNeed
from .pool import IndexPool, PoolError, PoolExhausted


class CacheFull(PoolExhausted):
    pass


@dataclasses.dataclass
class SeqRecord:
    """The fixed-size record of one sequence."""
    length: int = 0
    pages: List[int] = dataclasses.field(default_factory=list)
    reserved_tokens: int = 0


class CacheView:
    """What one schedule entry's mixer sees of the cache during a step: ``kv`` (this entry's
    keys and values), ``state`` with ``slots`` (this entry's records and the step's slot of
    each sequence), or whatever else a storage class of another kind hands out by keyword."""

    def __init__(self, kv=None, state=None, slots=None, **more):
        self.kv, self.state, self.slots = kv, state, slots
        for k, v in more.items():
            setattr(self, k, v)


class Storage:
    """The storage of one group of schedule entries with equal needs.

    A subclass is registered under the ``kind`` of the :class:`CacheNeed` it serves.  It
    is made with the need, the number of entries in the group, the cache's sizes (pages
    including the padding page 0, slots including the padding slot 0), the element type
    and the device; it allocates in :meth:`allocate`, hands one entry's part of itself to
    a mixer in :meth:`view`, prepares a slot for a new sequence in :meth:`open_seq`, and
    says how many bytes a step reads from it in :meth:`read_bytes`."""

    kind = ""

    def __init__(self, need: CacheNeed, n_entries: int, *, n_pages: int, n_slots: int, dtype: torch.dtype,
                 device: torch.device):
        self.need, self.n_entries, self.n_pages, self.n_slots = need, n_entries, n_pages, n_slots
        self.dtype, self.device = dtype, device
        self.tensor: Optional[torch.Tensor] = None

    def shape(self) -> Tuple[int, ...]:
        raise NotImplementedError

    def allocate(self) -> None:
        self.tensor = torch.zeros(self.shape(), dtype=self.dtype, device=self.device)

    def view(self, idx: int, batch) -> "CacheView":
        raise NotImplementedError

    def open_seq(self, slot: int) -> None:
        """A sequence starts in ``slot``."""

    def read_bytes(self, cached_tokens: int, n_seqs: int) -> int:
        """Bytes a decode step reads from this group for ``n_seqs`` sequences that hold
        ``cached_tokens`` positions between them."""
        return 0

    def element_size(self) -> int:
        return torch.empty((), dtype=self.dtype).element_size()


class PagedKV(Storage):
    """Keys and values of every position: [entries, pages, 2, kv_heads, 64, head_dim]."""
    kind = "paged_kv"

    def __init__(self, need, n_entries, **kw):
        super().__init__(need, n_entries, **kw)
        if need.window is not None:
            raise ValueError("paged key/value storage keeps every position; a window needs a storage kind of its own")

    def shape(self):
        n = self.need
        return (self.n_entries, self.n_pages, 2, n.kv_heads, PAGE, n.head_dim)

    def view(self, idx, batch):
        return CacheView(kv=self.tensor[idx])

    def bytes_per_token(self) -> int:
        return self.n_entries * 2 * self.need.kv_heads * self.need.head_dim * self.element_size()

    def read_bytes(self, cached_tokens, n_seqs):
        return cached_tokens * self.bytes_per_token()


class StateRecords(Storage):
    """A record of fixed shape per sequence: [entries, slots, *shape], zero when a sequence starts."""
    kind = "state"

    def shape(self):
        return (self.n_entries, self.n_slots) + tuple(self.need.shape)

    def view(self, idx, batch):
        return CacheView(state=self.tensor[idx], slots=None if batch is None else batch.slots)

    def open_seq(self, slot):
        if self.tensor is not None:
            self.tensor[:, slot].zero_()

    def read_bytes(self, cached_tokens, n_seqs):
        n = self.element_size()
        for d in self.need.shape:
            n *= d
        return n_seqs * self.n_entries * n


_STORAGE: Dict[str, type] = {}


def register_storage(kind: str, cls: type) -> type:
    _STORAGE[kind] = cls
    return cls


register_storage("paged_kv", PagedKV)
register_storage("state", StateRecords)


class _Group:
    def __init__(self, need: CacheNeed, dtype: torch.dtype):
        self.need = need
        self.dtype = need.dtype or dtype
        self.entries: List[int] = []
        self.store: Optional[Storage] = None

    @property
    def storage(self) -> Optional[torch.Tensor]:
        return None if self.store is None else self.store.tensor

    def key(self):
        n = self.need
        return (n.kind, n.kv_heads, n.head_dim, n.window, tuple(n.shape), self.dtype)


class Cache:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], *, max_tokens: int, dtype: torch.dtype,
                 device: torch.device | str, max_seqs: Optional[int] = None, max_position: Optional[int] = None,
                 allocate: bool = True):
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        self.max_tokens = (max_tokens + PAGE - 1) // PAGE * PAGE
        self.n_pages = self.max_tokens // PAGE + 1                 # + the pad page 0
        self.max_seqs = max_seqs if max_seqs is not None else self.n_pages - 1
        self.max_position = max_position
        self.device = torch.device(device)
        self.dtype = dtype
        self.pages = IndexPool(self.n_pages, reserved=(0,), what="page")
        self.slots = IndexPool(self.max_seqs + 1, reserved=(0,), what="slot")
        self.seqs: Dict[int, SeqRecord] = {}
        self.groups: List[_Group] = []
        self.entry_place: Dict[int, Tuple[_Group, int]] = {}
        by_key: Dict[tuple, _Group] = {}
        for i, need in enumerate(needs):
            if need is None:
                continue
            if need.kind not in _STORAGE:
                raise ValueError(f"unknown cache need {need.kind} (registered: {', '.join(sorted(_STORAGE))})")
            g = _Group(need, dtype)
            g = by_key.setdefault(g.key(), g)
            if not g.entries:
                self.groups.append(g)
            self.entry_place[i] = (g, len(g.entries))
            g.entries.append(i)
        for g in self.groups:
            g.store = _STORAGE[g.need.kind](g.need, len(g.entries), n_pages=self.n_pages, n_slots=self.max_seqs + 1,
                                            dtype=g.dtype, device=self.device)
            if allocate:
                g.store.allocate()

    # ---- sizes -------------------------------------------------------------
    def bytes_per_token(self) -> int:
        """Bytes of keys and values that one cached position takes in all paged groups."""
        return sum(g.store.bytes_per_token() for g in self.groups if isinstance(g.store, PagedKV))

    def read_bytes(self, cached_tokens: int, n_seqs: int) -> int:
        """Bytes one decode step reads from the cache: every group's share for ``n_seqs``
        sequences that hold ``cached_tokens`` positions between them."""
        return sum(g.store.read_bytes(cached_tokens, n_seqs) for g in self.groups)

    def storage_bytes(self) -> int:
        return sum(g.storage.numel() * g.storage.element_size() for g in self.groups if g.storage is not None)

    @property
    def free_tokens(self) -> int:
        return self.pages.n_free * PAGE

    # ---- sequences -----------------------------------------------------------
    def open_seq(self) -> int:
        slot = self.slots.alloc()
        self.seqs[slot] = SeqRecord()
        for g in self.groups:
            g.store.open_seq(slot)
        return slot

    def _rec(self, slot: int) -> SeqRecord:
        try:
            return self.seqs[slot]
        except KeyError:
            raise PoolError(f"slot {slot} is not open") from None

    def length(self, slot: int) -> int:
        return self._rec(slot).length

    def pages_of(self, slot: int) -> List[int]:
        return self._rec(slot).pages

    def reserve(self, slot: int, n_tokens: int) -> None:
        """Make sure the sequence holds pages for ``n_tokens`` positions."""
        rec = self._rec(slot)
        if self.max_position is not None and n_tokens > self.max_position:
            raise ValueError(f"context length exceeded: {n_tokens} tokens, the model takes {self.max_position}")
        need = (n_tokens + PAGE - 1) // PAGE - len(rec.pages)
        if need > 0:
            if need > self.pages.n_free:
                raise CacheFull(f"the cache is full: sequence needs {need} more pages of {PAGE} tokens, "
                                f"{self.pages.n_free} are free of {self.pages.capacity}")
            rec.pages.extend(self.pages.alloc_many(need))
        rec.reserved_tokens = max(rec.reserved_tokens, n_tokens)

    def advance(self, slot: int, n: int) -> None:
        rec = self._rec(slot)
        if rec.length + n > len(rec.pages) * PAGE:
            raise PoolError(f"slot {slot} advanced to {rec.length + n} tokens but holds {len(rec.pages)} pages")
        rec.length += n

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions from ``length`` on (pages beyond are given back)."""
        rec = self._rec(slot)
        if not 0 <= length <= rec.length:
            raise ValueError(f"cannot truncate slot {slot} of length {rec.length} to {length}")
        keep = (length + PAGE - 1) // PAGE
        for p in rec.pages[keep:]:
            self.pages.free(p)
        del rec.pages[keep:]
        rec.length = length

    def close_seq(self, slot: int) -> None:
        rec = self.seqs.pop(slot, None)
        if rec is None:
            raise PoolError(f"slot {slot} is closed but is not open (closed twice?)")
        for p in rec.pages:
            self.pages.free(p)
        self.slots.free(slot)

    def check(self) -> None:
        """Bookkeeping invariants: no page held by two sequences or by none."""
        self.pages.check()
        self.slots.check()
        seen = set()
        for slot, rec in self.seqs.items():
            if not self.slots.is_held(slot):
                raise PoolError(f"open slot {slot} is not held")
            for p in rec.pages:
                if p in seen:
                    raise PoolError(f"page {p} is held by two sequences")
                if not self.pages.is_held(p):
                    raise PoolError(f"page {p} of slot {slot} is not held")
                seen.add(p)
        if seen != self.pages.held():
            raise PoolError("a held page belongs to no sequence")
        if set(self.seqs) != self.slots.held():
            raise PoolError("a held slot has no record")

    # ---- views ---------------------------------------------------------------
    def view(self, entry: int, batch=None) -> Optional[CacheView]:
        place = self.entry_place.get(entry)
        if place is None:
            return None
        g, idx = place
        return g.store.view(idx, batch)
