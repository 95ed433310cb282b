"""Turning a step's entries into the arrays the kernels read.

The reference builds its arrays inside each runner call: ``torch.tensor([tokens])``
for a prefill (serve/engine.py:81-83) and token list, positions, padded block
tables and context lengths for a decode step (serve/engine.py:121-127,
serve/kv_cache.py:112-122).  Here one builder handles every mix of prompt
portions and single decoded tokens: all arrays of a step are laid out in one
pinned int32 buffer and reach the device in a single copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import GroupView, StepContext


@dataclass
class Entry:
    """One request's share of a step: its next tokens and the wanted places.

    ``want`` indexes into ``tokens``; logits come back in the order of the
    entries and, inside an entry, of ``want``.
    """
    owner: object
    tokens: list
    want: list = field(default_factory=list)


class BatchError(ValueError):
    pass


@dataclass
class Prepared:
    """A step laid out in a pinned buffer, not yet on the device."""
    which: int
    size: int
    off: dict
    groups: dict
    t_total: int
    r_total: int
    n_out: int
    q_lens: list
    ctx_lens: list
    owners: list


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class BatchBuilder:
    def __init__(self, cache, device, vocab_size: int, max_positions: int):
        self.cache = cache
        self.device = torch.device(device)
        self.vocab_size, self.max_positions = int(vocab_size), int(max_positions)
        self._pinned = [None, None]
        self._events = [None, None]
        self._turn = 0
        self._dev = None
        self.generation = 0           # grows when the device buffer moves
        self.last_bytes = 0           # bytes of the last step's host-to-device copy

    def _staging(self, n: int):
        use_cuda = self.device.type == "cuda"
        i = self._turn
        self._turn ^= 1
        if self._pinned[i] is None or self._pinned[i].numel() < n:
            cap = max(n, 1 << 14)
            self._pinned[i] = torch.empty(cap, dtype=torch.int32, pin_memory=use_cuda)
        elif self._events[i] is not None:
            self._events[i].synchronize()      # the copy that last read this buffer is done
        if self._dev is None or self._dev.numel() < n:
            self._dev = torch.empty(max(n, 1 << 14), dtype=torch.int32, device=self.device)
            self.generation += 1
        return i, self._pinned[i]

    def build(self, entries: list) -> StepContext:
        """Arrays for ``entries``; their pages must already be reserved."""
        return self.submit(self.prepare(entries))

    def prepare(self, entries: list) -> "Prepared":
        """Lay the step's arrays out in a pinned buffer without sending them.

        Everything but the token ids depends only on lengths and pages, so a step
        of single decoded tokens can be prepared while the device still computes
        the tokens it will be fed (``submit`` then takes the ids).
        """
        if not entries:
            raise BatchError("a step needs at least one entry")
        cache = self.cache
        seen = set()
        q_lens, ctx_lens, rows = [], [], []
        for e in entries:
            if e.owner in seen:
                raise BatchError(f"request {e.owner!r} appears twice in one step")
            seen.add(e.owner)
            n = len(e.tokens)
            if n == 0:
                raise BatchError(f"request {e.owner!r} brings no tokens")
            have = cache.length(e.owner)
            if have + n > self.max_positions:
                raise BatchError(
                    f"request {e.owner!r} would reach {have + n} tokens; the model's "
                    f"positions end at {self.max_positions}")
            for w in e.want:
                if not (0 <= w < n):
                    raise BatchError(f"request {e.owner!r}: wanted place {w} is not "
                                     f"among its {n} tokens")
            q_lens.append(n)
            ctx_lens.append(have + n)
            rows.append(cache.row(e.owner))
        t_total, r_total = sum(q_lens), len(entries)
        n_out = sum(len(e.want) for e in entries)
        groups = cache.step_arrays([(e.owner, len(e.tokens)) for e in entries])

        # layout of the packed buffer (int32 elements)
        off = {}
        cur = 0
        for name, n in (("token_ids", t_total), ("positions", t_total),
                        ("req_of_token", t_total), ("cu_q", r_total + 1),
                        ("ctx_len", r_total + 1), ("state_slot", r_total),
                        ("out_rows", max(n_out, 1))):
            off[name] = (cur, n)
            cur += _align(n)
        for gid, (table, slot_map) in groups.items():
            off[f"slot_map{gid}"] = (cur, t_total)
            cur += _align(t_total)
            off[f"table{gid}"] = (cur, table.size)
            cur += _align(table.size)
        which, pinned = self._staging(cur)
        host = pinned.numpy()

        def view(name):
            b, n = off[name]
            return host[b:b + n]

        if t_total == r_total:
            tok = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=t_total)
        else:
            tok = np.fromiter((x for e in entries for x in e.tokens), dtype=np.int64,
                              count=t_total)
        if tok.size and (tok.min() < 0 or tok.max() >= self.vocab_size):
            raise BatchError(f"a token id lies outside the vocabulary of "
                             f"{self.vocab_size}")
        view("token_ids")[:] = tok
        cu = np.zeros(r_total + 1, np.int64)
        np.cumsum(q_lens, out=cu[1:])
        view("cu_q")[:] = cu
        view("ctx_len")[:r_total] = ctx_lens
        view("ctx_len")[r_total] = max(ctx_lens)     # one past the requests: the longest context
        view("state_slot")[:] = rows
        pos = view("positions")
        rot = view("req_of_token")
        outs = []
        if t_total == r_total:                       # single tokens: no loop over requests
            pos[:] = np.asarray(ctx_lens) - 1
            rot[:] = np.arange(r_total)
            outs = [r for r, e in enumerate(entries) if e.want]
        else:
            for r, e in enumerate(entries):
                b, n = int(cu[r]), q_lens[r]
                pos[b:b + n] = np.arange(ctx_lens[r] - n, ctx_lens[r])
                rot[b:b + n] = r
                outs.extend(b + w for w in e.want)
        if n_out:
            view("out_rows")[:] = outs
        else:
            view("out_rows")[:] = 0
        for gid, (table, slot_map) in groups.items():
            view(f"slot_map{gid}")[:] = slot_map
            view(f"table{gid}")[:] = table.reshape(-1)

        return Prepared(which=which, size=cur, off=off, groups={g: t.shape[1] for g, (t, _) in groups.items()},
                        t_total=t_total, r_total=r_total, n_out=n_out, q_lens=q_lens,
                        ctx_lens=ctx_lens, owners=[e.owner for e in entries])

    def submit(self, prep: "Prepared", token_ids=None) -> StepContext:
        """Send a prepared step to the device; ``token_ids`` replaces the ids it was
        prepared with (a step of single tokens whose ids were not yet known)."""
        pinned = self._pinned[prep.which]
        off, cur = prep.off, prep.size
        if token_ids is not None:
            tok = np.asarray(token_ids, dtype=np.int64)
            if tok.size != prep.t_total or (tok.size and (tok.min() < 0 or
                                                          tok.max() >= self.vocab_size)):
                raise BatchError("token ids do not fit the prepared step or the vocabulary")
            b, n = off["token_ids"]
            pinned.numpy()[b:b + n] = tok
        dev = self._dev
        self.last_bytes = cur * 4
        if self.device.type == "cuda":
            dev[:cur].copy_(pinned[:cur], non_blocking=True)
            ev = self._events[prep.which] or torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._events[prep.which] = ev
        else:
            dev[:cur].copy_(pinned[:cur])

        def dview(name):
            b, n = off[name]
            return dev[b:b + n]

        r_total, t_total, n_out = prep.r_total, prep.t_total, prep.n_out
        gviews = {}
        for gid, width in prep.groups.items():
            gviews[gid] = GroupView(
                block_table=dview(f"table{gid}").view(r_total, width),
                slot_map=dview(f"slot_map{gid}"),
                block_size=self.cache.block_size, max_blocks=width)
        return StepContext(
            n_tokens=t_total, n_requests=r_total,
            token_ids=dview("token_ids"), positions=dview("positions"),
            req_of_token=dview("req_of_token"), cu_q=dview("cu_q"),
            ctx_len=dview("ctx_len"), state_slot=dview("state_slot"),
            out_rows=dview("out_rows")[:n_out] if n_out else dview("out_rows")[:0],
            n_out=n_out, groups=gviews, q_lens=prep.q_lens, ctx_lens=prep.ctx_lens,
            max_q_len=max(prep.q_lens), max_ctx_len=max(prep.ctx_lens))
