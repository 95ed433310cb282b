"""The cache manager: pages of keys and values, block tables, state slots.

Reference (serve/kv_cache.py:30-135): per layer a K and a V pool
``[num_blocks, n_heads, block_size, head_dim]`` (one (page, head) slab is
contiguous; here the pools are ``[n_kv_heads, num_blocks, block_size, head_dim]``,
so that consecutive pages of one kv head are one contiguous run as well), ``tables: seq -> [page ids]``, ``lens: seq -> tokens stored``, a
LIFO free list; pages are claimed at admission (``allocate``) and one at a time
at page boundaries (``append_slot``, :64-73), lengths advance once per step
after all layers wrote (``set_len``, :85-88,107-108) and everything is given
back at ``free`` (:75-77).

Here the model's cache slots (one per layer call that owns a cache) are sorted
into groups by what they need.  Slots with the same ``PagedKV`` spec share one
page pool and one block table per request (a page id means the same page in
every member of the group, as one table serves all layers in the reference);
a group with a window gives pages back as soon as the window has passed them.
Slots with a ``FixedState`` spec share the request's state slot.

    reserve(req, n)  -> bool   pages for the next n tokens, all groups or none
    commit(req, n)             the n tokens are stored; windows release pages
    truncate(req, n)           only the first n tokens stay; whole pages past them go back
    free(req)                  everything back
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import CacheHandle, FixedState, PagedKV
from .page_pool import PagePool
from .state_slots import StateSlotPool


class CacheError(RuntimeError):
    pass


@dataclass
class PagedGroup:
    gid: int
    spec: PagedKV
    members: list                     # cache slot indices, in order
    pool: PagePool
    kv: torch.Tensor | None           # [members, 2, Hkv, pages, block, hd]
    table: np.ndarray                 # [max_requests, max_blocks] int32, -1 = none


@dataclass
class FixedGroup:
    gid: int
    spec: FixedState
    members: list
    state: torch.Tensor | None        # [members, max_requests, *shape]


@dataclass
class _Record:
    owner: object
    row: int                          # state slot id = row of the block tables
    length: int = 0                   # tokens stored (committed)
    n_pages: list = field(default_factory=list)     # per paged group: table length
    released: list = field(default_factory=list)    # per paged group: pages given back in front


class CacheManager:
    def __init__(self, specs: list, num_blocks: int, block_size: int,
                 max_requests: int, max_seq_len: int, device="cpu",
                 kv_dtype: torch.dtype = torch.float32, allocate: bool = True):
        self.block_size = int(block_size)
        self.num_blocks = int(num_blocks)
        self.max_requests = int(max_requests)
        self.max_blocks = (int(max_seq_len) + self.block_size - 1) // self.block_size
        self.device, self.kv_dtype = device, kv_dtype
        self.slots = StateSlotPool(self.max_requests)
        self.paged: list[PagedGroup] = []
        self.fixed: list[FixedGroup] = []
        self._records: dict = {}
        self._slot_home: list = []    # cache slot -> ("paged"|"fixed"|"none", gid, member)

        by_key: dict = {}
        for slot, spec in enumerate(specs):
            if spec is None:
                self._slot_home.append(("none", -1, -1))
                continue
            kind = "paged" if isinstance(spec, PagedKV) else "fixed"
            if kind == "fixed" and not isinstance(spec, FixedState):
                raise CacheError(f"cache slot {slot}: unknown cache spec {spec!r}")
            key = (kind, spec)
            if key not in by_key:
                if kind == "paged":
                    by_key[key] = PagedGroup(
                        len(self.paged), spec, [], PagePool(self.num_blocks), None,
                        np.full((self.max_requests, self.max_blocks), -1, np.int32))
                    self.paged.append(by_key[key])
                else:
                    by_key[key] = FixedGroup(len(self.fixed), spec, [], None)
                    self.fixed.append(by_key[key])
            grp = by_key[key]
            self._slot_home.append((kind, grp.gid, len(grp.members)))
            grp.members.append(slot)
        if allocate:
            for g in self.paged:
                g.kv = torch.zeros(
                    (len(g.members), 2, g.spec.n_kv_heads, self.num_blocks,
                     self.block_size, g.spec.head_dim),
                    device=device, dtype=kv_dtype)
            for g in self.fixed:
                g.state = torch.zeros(
                    (len(g.members), self.max_requests) + tuple(g.spec.shape),
                    device=device, dtype=g.spec.dtype)

    # ------------------------------------------------------------------ handles
    def handles(self) -> list:
        """One ``CacheHandle`` per cache slot, in slot order."""
        out = []
        for kind, gid, m in self._slot_home:
            if kind == "paged":
                g = self.paged[gid]
                out.append(CacheHandle(
                    kind="paged", group=gid,
                    k_pool=None if g.kv is None else g.kv[m, 0],
                    v_pool=None if g.kv is None else g.kv[m, 1],
                    window=g.spec.window))
            elif kind == "fixed":
                g = self.fixed[gid]
                out.append(CacheHandle(kind="fixed", group=gid,
                                       state=None if g.state is None else g.state[m]))
            else:
                out.append(CacheHandle())
        return out

    # --------------------------------------------------------------- accounting
    def pages_for(self, n_tokens: int) -> int:
        """``ceil(n / block_size)`` (serve/kv_cache.py:48-49)."""
        return (n_tokens + self.block_size - 1) // self.block_size

    def num_free_pages(self) -> int:
        """Free pages of the fullest group (all of them if nothing is paged)."""
        return min((g.pool.num_free for g in self.paged), default=self.num_blocks)

    def has(self, owner) -> bool:
        return owner in self._records

    def length(self, owner) -> int:
        return self._records[owner].length

    def row(self, owner) -> int:
        return self._records[owner].row

    def live(self) -> list:
        return list(self._records)

    def _most_pages(self, g: PagedGroup, n_tokens: int, portion: int | None) -> int:
        """Most pages of group ``g`` a request of ``n_tokens`` holds at one time
        when it is fed at most ``portion`` tokens a step (all at once if None)."""
        need = self.pages_for(n_tokens)
        w = g.spec.window
        if w is not None and portion is not None:
            # keys older than the window are given back after every step; one
            # page more because the live span need not start at a page's edge
            need = min(need, self.pages_for(w - 1 + portion) + 1)
        return need

    def can_hold(self, n_tokens: int, portion: int | None = None) -> bool:
        """Could a new request with ``n_tokens`` be admitted right now?

        The reference's admission test, ``can_allocate(len(tokens) + 1)``
        (serve/engine.py:195), asked of every group, plus a free state slot.
        """
        if self.slots.num_free == 0:
            return False
        return all(g.pool.num_free >= self._most_pages(g, n_tokens, portion)
                   for g in self.paged)

    def fits_at_all(self, n_tokens: int, portion: int | None = None) -> bool:
        """Could ``n_tokens`` ever be held, with every page free?"""
        if self.pages_for(n_tokens) > self.max_blocks:
            return False
        return all(self._most_pages(g, n_tokens, portion) <= self.num_blocks
                   for g in self.paged)

    def admit(self, owner) -> bool:
        """Open an empty record for ``owner``; False if no state slot is free."""
        if owner in self._records:
            raise CacheError(f"request {owner!r} is already in the cache")
        row = self.slots.claim(owner)
        if row is None:
            return False
        self._records[owner] = _Record(owner, row, 0,
                                       [0] * len(self.paged), [0] * len(self.paged))
        for g in self.fixed:
            if g.state is not None:
                g.state[:, row].zero_()
        return True

    def _pages_short(self, rec: _Record, n_more: int) -> list:
        total = self.pages_for(rec.length + n_more)
        if total > self.max_blocks:
            raise CacheError(
                f"request {rec.owner!r} would hold {rec.length + n_more} tokens, "
                f"more than the block table's {self.max_blocks * self.block_size}")
        return [max(0, total - rec.n_pages[g.gid]) for g in self.paged]

    def can_reserve(self, owner, n_more: int) -> bool:
        short = self._pages_short(self._records[owner], n_more)
        return all(g.pool.num_free >= s for g, s in zip(self.paged, short))

    def reserve(self, owner, n_more: int) -> bool:
        """Pages for the next ``n_more`` tokens in every group, or no change.

        A page is claimed only when a token crosses into it
        (serve/kv_cache.py:64-73).
        """
        rec = self._records[owner]
        short = self._pages_short(rec, n_more)
        if any(g.pool.num_free < s for g, s in zip(self.paged, short)):
            return False
        for g, s in zip(self.paged, short):
            pages = g.pool.take(s, owner)
            n0 = rec.n_pages[g.gid]
            g.table[rec.row, n0:n0 + s] = pages
            rec.n_pages[g.gid] = n0 + s
        return True

    def commit(self, owner, n_tokens: int) -> None:
        """``n_tokens`` more are stored; pages a window has passed go back."""
        rec = self._records[owner]
        rec.length += n_tokens
        for g in self.paged:
            if rec.length > rec.n_pages[g.gid] * self.block_size:
                raise CacheError(f"request {owner!r} stored tokens beyond its pages")
            w = g.spec.window
            if w is None:
                continue
            # the next query sits at position >= length and sees keys
            # j > position - w, so every key < length - w + 1 is never read again
            dead = max(0, rec.length - w + 1) // self.block_size
            dead = min(dead, rec.n_pages[g.gid])
            first = rec.released[g.gid]
            if dead > first:
                pages = [int(p) for p in g.table[rec.row, first:dead]]
                g.pool.give(list(reversed(pages)), owner)
                g.table[rec.row, first:dead] = -1
                rec.released[g.gid] = dead

    def truncate(self, owner, n_tokens: int) -> None:
        """Forget the tokens past the first ``n_tokens``; whole pages past them go back.

        (The reference never shortens a sequence; a caller that takes back tokens it
        had stored, e.g. after rejecting a guessed continuation, needs it.)  A window
        group that has released pages the shorter sequence would read again, and a
        fixed-size state, cannot go back: both are refused.
        """
        rec = self._records[owner]
        if not 0 <= n_tokens <= rec.length:
            raise CacheError(f"request {owner!r} holds {rec.length} tokens, not {n_tokens}")
        if n_tokens == rec.length:
            return
        if self.fixed:
            raise CacheError("a state of fixed size cannot be taken back to an earlier token")
        for g in self.paged:
            w = g.spec.window
            if w is not None and rec.released[g.gid] * self.block_size > max(0, n_tokens - w + 1):
                raise CacheError(
                    f"request {owner!r}: pages behind the window of {w} were given back; "
                    f"it cannot be cut to {n_tokens} tokens")
        keep = self.pages_for(n_tokens)
        for g in self.paged:
            n = rec.n_pages[g.gid]
            first = max(keep, rec.released[g.gid])
            if n > first:
                pages = [int(p) for p in g.table[rec.row, first:n]]
                g.pool.give(list(reversed(pages)), owner)
                g.table[rec.row, first:n] = -1
                rec.n_pages[g.gid] = first
        rec.length = n_tokens

    def free(self, owner) -> None:
        """Give back everything ``owner`` holds (serve/kv_cache.py:75-77)."""
        rec = self._records.pop(owner)
        for g in self.paged:
            first, n = rec.released[g.gid], rec.n_pages[g.gid]
            pages = [int(p) for p in g.table[rec.row, first:n]]
            g.pool.give(list(reversed(pages)), owner)
            g.table[rec.row, :n] = -1
        self.slots.release(rec.row, owner)

    def pages_of(self, owner, gid: int = 0) -> list:
        """Page ids by logical page index (-1 where a window released one)."""
        rec = self._records[owner]
        return [int(p) for p in self.paged[gid].table[rec.row, :rec.n_pages[gid]]]

    def check(self) -> None:
        """No page or slot lost, held twice or free twice; tables match owners."""
        self.slots.check()
        for g in self.paged:
            g.pool.check()
            held = 0
            for owner, rec in self._records.items():
                for i, p in enumerate(g.table[rec.row, :rec.n_pages[g.gid]]):
                    if i < rec.released[g.gid]:
                        if p != -1:
                            raise CacheError("a released table entry still names a page")
                        continue
                    if g.pool.owner_of(int(p)) != owner:
                        raise CacheError(f"page {int(p)} is in the table of "
                                         f"{owner!r} but owned by "
                                         f"{g.pool.owner_of(int(p))!r}")
                    held += 1
            if held != g.pool.num_held:
                raise CacheError(f"group {g.gid}: {g.pool.num_held} pages are held "
                                 f"but the tables name {held}")

    # -------------------------------------------------------------- step arrays
    def step_arrays(self, entries: list) -> dict:
        """Per paged group, the block-table rows and slot map of a step.

        ``entries`` is ``[(owner, n_tokens)]`` in batch order; pages for the
        tokens must have been reserved.  Returns ``{gid: (block_table [R,
        max_blocks] int32, slot_map [T] int32)}`` as numpy arrays.
        """
        out = {}
        bs = self.block_size
        recs = [self._records[o] for o, _ in entries]
        rows = [r.row for r in recs]
        if all(n == 1 for _, n in entries):
            # single decoded tokens: one gather instead of a loop over requests
            rows_a = np.asarray(rows)
            pos = np.fromiter((r.length for r in recs), dtype=np.int64, count=len(recs))
            for g in self.paged:
                pages = g.table[rows_a, pos // bs]
                if pages.size and pages.min() < 0:
                    raise CacheError("no page reserved for a token of this step")
                out[g.gid] = (g.table[rows_a],
                              (pages.astype(np.int64) * bs + pos % bs).astype(np.int32))
            return out
        for g in self.paged:
            table = g.table[rows]
            slot_parts = []
            for (owner, n), row in zip(entries, rows):
                rec = self._records[owner]
                pos = np.arange(rec.length, rec.length + n)
                pages = g.table[row, pos // bs]
                if n and pages.min() < 0:
                    raise CacheError(f"request {owner!r}: no page reserved for a "
                                     f"token of this step")
                slot_parts.append(pages.astype(np.int64) * bs + pos % bs)
            slot_map = (np.concatenate(slot_parts) if slot_parts
                        else np.zeros(0, np.int64)).astype(np.int32)
            out[g.gid] = (table, slot_map)
        return out

    # --------------------------------------------------------------- debug view
    def gather_contiguous(self, slot: int, owner, n: int | None = None):
        """K and V of one cache slot for ``owner`` as [Hkv, n, hd]
        (serve/kv_cache.py:124-135); positions a window released read as NaN."""
        kind, gid, m = self._slot_home[slot]
        if kind != "paged":
            raise CacheError("gather_contiguous needs a paged cache slot")
        g = self.paged[gid]
        rec = self._records[owner]
        n = rec.length if n is None else n
        bs = self.block_size
        ks, vs = [], []
        for i in range(self.pages_for(n)):
            take = min(bs, n - i * bs)
            p = int(g.table[rec.row, i])
            if p < 0:
                nan = torch.full((g.spec.n_kv_heads, take, g.spec.head_dim),
                                 float("nan"), device=g.kv.device, dtype=g.kv.dtype)
                ks.append(nan)
                vs.append(nan)
            else:
                ks.append(g.kv[m, 0, :, p, :take])
                vs.append(g.kv[m, 1, :, p, :take])
        return torch.cat(ks, dim=1), torch.cat(vs, dim=1)
