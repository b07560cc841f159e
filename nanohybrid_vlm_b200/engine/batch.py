"""One step's batch: (request, its next tokens) for several requests, packed.

A :class:`StepItem` says: these are the next tokens of that request, ``start`` tokens of it
are already in the cache, and the logits at the places ``want`` among them are asked for.
Prompt portions and single decoded tokens sit side by side; the only difference between
them is the number of tokens.  (The reference builds two kinds of batch and never mixes
them, nanovllm/engine/model_runner.py:924-1146,2029-2033.)

:class:`BatchBuilder` turns items into the device arrays that kernels index: everything
is written into ONE pinned host buffer and crosses to the device in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepItem:
    req_id: object
    tokens: list[int]
    start: int                      # tokens of this request already in the cache = position of tokens[0]
    want: list[int] = field(default_factory=list)   # places among `tokens` whose logits are wanted
    # what the position encoding sees of these tokens, if it is not their index in the request: one number per
    # token, or one list per position axis of the model (``ModelSpec.position_axes``).  The cache is indexed by
    # ``start`` whatever stands here.
    positions: list | None = None


@dataclass
class GroupTables:
    block_tables: torch.Tensor      # [S, width] int32, -1 where there is no page
    slot_mapping: torch.Tensor      # [T] int32: page * page_size + offset of every token of the step


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    n_logit_rows: int
    token_ids: torch.Tensor         # [T] int32
    positions: torch.Tensor         # [T] int32, position of each token in its own request (axis 0 of position_axes)
    position_axes: torch.Tensor     # [P, T] int32: every position axis of the model (P = 1 unless the model says otherwise)
    cu_q: torch.Tensor              # [S+1] int32, where each request's tokens start in the packed arrays
    kv_len: torch.Tensor            # [S] int32, tokens of the request in the cache after this step
    q_start: torch.Tensor           # [S] int32, kv_len minus this step's tokens
    state_slots: torch.Tensor       # [S] int32, slot of fixed-size state (-1: none)
    logit_rows: torch.Tensor        # [R] int32, rows of the packed arrays whose logits are wanted
    groups: list[GroupTables]
    # the same facts on the host, for parts that plan their launches from them
    host_cu_q: list[int] = field(default_factory=list)
    host_kv_len: list[int] = field(default_factory=list)
    max_new_tokens: int = 0
    max_kv_len: int = 0
    decode_only: bool = False
    n_decode_seqs: int = 0          # requests that bring exactly one token
    n_prefill_seqs: int = 0         # requests that bring more
    n_prefill_tokens: int = 0
    # sampling inputs, one per wanted row (None if the caller only wants logits)
    temperatures: torch.Tensor | None = None    # [R] float32
    seeds: torch.Tensor | None = None           # [R] int64
    sample_positions: torch.Tensor | None = None  # [R] int32: the position of the token being chosen


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class BatchBuilder:
    def __init__(self, cache_manager, vocab_size: int, device, max_tokens: int, max_seqs: int, max_pages_per_seq: int,
                 position_axes: int = 1):
        self.cm = cache_manager
        self.n_axes = position_axes
        self.vocab = vocab_size
        self.device = torch.device(device)
        self.page_size = cache_manager.page_size
        self.n_groups = len(cache_manager.groups)
        self.max_tokens, self.max_seqs, self.max_pages = max_tokens, max_seqs, max_pages_per_seq
        self._layouts: dict = {}
        self._table_rows = None          # (layout, per row (request, table length)) of the last all-decode step
        self._windows = any(g.window is not None for g in cache_manager.groups)
        cap = self._layout(max_tokens, max_seqs, max_tokens, max_pages_per_seq)[1]
        self._host = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self._np = self._host.numpy()
        self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.bytes_last_copy = 0
        # the host buffer is written again at the next step: wait until the last copy has read it
        self._copied = torch.cuda.Event() if self.device.type == "cuda" else None

    def _layout(self, T: int, S: int, R: int, width: int):
        key = (T, S, R, width)
        cached = self._layouts.get(key)
        if cached is not None:
            return cached
        off, sections = 0, {}
        for name, n in (("seeds", 2 * R), ("temperatures", R), ("sample_positions", R), ("token_ids", T),
                        ("positions", self.n_axes * T), ("cu_q", S + 1), ("kv_len", S), ("q_start", S),
                        ("state_slots", S), ("logit_rows", R), ("feed_src", T)):
            sections[name] = (off, n)
            off += _align(n)
        for g in range(self.n_groups):
            sections[f"slots{g}"] = (off, T)
            off += _align(T)
            sections[f"tables{g}"] = (off, S * width)
            off += _align(S * width)
        self._layouts[key] = (sections, off)
        return sections, off

    def build(self, items: list[StepItem], table_width: int | None = None, sampling=None,
              pad_to: int | None = None, views: bool = True, feed: list[int] | None = None) -> StepBatch | None:
        """``sampling``: one (temperature, seed, position of the token being chosen) per wanted row.
        ``feed``: per item, the row of the step before whose chosen token is this item's (single) token, or -1; the
        arrays ``last_token_ids`` / ``last_feed_src`` then say on the device which tokens to take from there.
        ``pad_to``: for a batch of single tokens, fill up to this many requests with idle entries (one
        token that is stored nowhere and reads no page), so that the batch has a fixed shape.
        ``views`` False: only fill and copy the arrays (for the replay of a captured step) and return None."""
        n_real = len(items)
        pad = 0 if pad_to is None else pad_to - n_real
        if pad < 0 or (pad_to is not None and any(len(it.tokens) != 1 or it.want != [0] for it in items)):
            raise ValueError("only a batch of single tokens that all want their logits can be padded")
        S = n_real + pad
        T = sum(len(it.tokens) for it in items) + pad
        R = sum(len(it.want) for it in items) + pad
        if S == 0 or T == 0:
            raise ValueError("a step needs at least one request with at least one token")
        if S > self.max_seqs or T > self.max_tokens:
            raise ValueError(f"step of {S} requests / {T} tokens is beyond the limits {self.max_seqs} / {self.max_tokens}")
        ps = self.page_size
        width = table_width or max(1, max((-(-(it.start + len(it.tokens)) // ps) for it in items), default=1))
        if width > self.max_pages:
            raise ValueError(f"a request needs {width} pages, beyond the limit of {self.max_pages}")
        sec, total = self._layout(T, S, R, width)
        if self._copied is not None:
            self._copied.synchronize()
        buf = self._np

        def view(name):
            o, n = sec[name]
            return buf[o:o + n]

        tok, pos_axes = view("token_ids"), view("positions").reshape(self.n_axes, T)
        cu, kvl, qs, st, rows = view("cu_q"), view("kv_len"), view("q_start"), view("state_slots"), view("logit_rows")
        slot_views = [view(f"slots{g}") for g in range(self.n_groups)]
        table_views = [view(f"tables{g}").reshape(S, width) for g in range(self.n_groups)]
        # In a run of decode steps over the same requests the tables change only when a request gets a page.  The
        # host buffer still holds the last step's rows if the arrays lie where they lay then: a row is written
        # again only if its request or the length of its table differs (a group with a window rewrites always:
        # pages given back change entries without changing the length).
        layout_key = (T, S, R, width)
        decode_only = n_real > 0 and all(len(it.tokens) == 1 and it.want == [0] and it.positions is None for it in items)
        keep = decode_only and self._table_rows is not None and self._table_rows[0] == layout_key
        old_rows = self._table_rows[1] if keep else None
        self._table_rows = None          # a build that fails half-way leaves rows nobody has a record of
        new_rows = [None] * S if decode_only else None
        if not keep:
            for tv in table_views:
                tv.fill(-1)
        if sampling is not None:
            if len(sampling) != R - pad:
                raise ValueError("one (temperature, seed, position) per wanted row is needed")
            temps = view("temperatures").view(np.float32)
            seeds = view("seeds").view(np.int64)
            spos = view("sample_positions")
            temps[:], seeds[:], spos[:] = 0.0, 0, 0
            for i, (temp, seed, p) in enumerate(sampling):
                temps[i], seeds[i], spos[i] = temp, seed, p
        t = r = 0
        cu[0] = 0
        if decode_only:
            # a step of decoded tokens, each wanting its logits: the per-request numbers as whole arrays, the
            # tables row by row
            requests = self.cm._requests
            starts, slots_state, firsts = [], [], []
            for s, it in enumerate(items):
                req = requests[it.req_id]
                start = it.start
                if req.num_tokens <= start:
                    raise RuntimeError(f"request {it.req_id!r}: pages cover {req.num_tokens} tokens, the step needs {start + 1}")
                starts.append(start)
                firsts.append(it.tokens[0])
                slots_state.append(-1 if req.state_slot is None else req.state_slot)
                lp, off = divmod(start, ps)
                stamp = (req.serial, len(req.tables[0]))     # a request that was given up and came back is another record
                new_rows[s] = stamp
                same = keep and not self._windows and old_rows[s] == stamp
                for g in range(self.n_groups):
                    table = req.tables[g]
                    if not same:
                        k = len(table) if len(table) < width else width
                        table_views[g][s, :k] = table[:k]
                        table_views[g][s, k:] = -1
                    page = table[lp]
                    slot_views[g][s] = page * ps + off if page >= 0 else -1
            n = n_real
            tok[:n], qs[:n], st[:n] = firsts, starts, slots_state
            pos_axes[:, :n] = starts
            kvl[:n] = qs[:n] + 1
            cu[1:n + 1] = np.arange(1, n + 1, dtype=np.int32)
            rows[:n] = cu[:n]
            t = r = n
            items_loop = ()
        else:
            items_loop = items
        for s, it in enumerate(items_loop):
            n = len(it.tokens)
            if n == 0:
                raise ValueError(f"request {it.req_id!r} brings no token")
            end = it.start + n
            if self.cm.num_tokens(it.req_id) < end:
                raise RuntimeError(f"request {it.req_id!r}: pages cover {self.cm.num_tokens(it.req_id)} tokens, "
                                   f"the step needs {end}")
            cu[s + 1] = t + n
            kvl[s], qs[s] = end, it.start
            slot = self.cm.state_slot(it.req_id)
            st[s] = -1 if slot is None else slot
            for w in it.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {it.req_id!r}: wanted place {w} is not among its {n} tokens")
                rows[r] = t + w
                r += 1
            if it.positions is not None:
                given = np.asarray(it.positions, dtype=np.int64)
                if given.shape not in ((n,), (self.n_axes, n)) or given.min() < 0:
                    raise ValueError(f"request {it.req_id!r}: positions must be {n} numbers, or {self.n_axes} lists of "
                                     f"{n}, none negative")
                pos_axes[:, t:t + n] = given
            if n == 1:
                # a decoded token: scalars instead of arrays (this is the hot path of every decode step)
                tok[t] = it.tokens[0]
                if it.positions is None:
                    pos_axes[:, t] = it.start
                for g in range(self.n_groups):
                    table = self.cm.block_table(it.req_id, g)
                    k = min(len(table), width)
                    table_views[g][s, :k] = table[:k]
                    page = table[it.start // ps]
                    slot_views[g][t] = page * ps + it.start % ps if page >= 0 else -1
            else:
                tok[t:t + n] = it.tokens
                p = np.arange(it.start, end, dtype=np.int32)
                if it.positions is None:
                    pos_axes[:, t:t + n] = p
                for g in range(self.n_groups):
                    table = np.asarray(self.cm.block_table(it.req_id, g), dtype=np.int32)
                    table_views[g][s, :min(len(table), width)] = table[:width]
                    pages = table[p // ps]
                    slot_views[g][t:t + n] = np.where(pages >= 0, pages * ps + p % ps, -1)
            t += n
        for s in range(n_real, S):          # idle entries
            if keep and old_rows[s] is not None:
                for tv in table_views:
                    tv[s, :] = -1
            tok[t] = 0
            pos_axes[:, t] = 0
            cu[s + 1] = t + 1
            kvl[s], qs[s], st[s] = 1, 0, -1
            rows[r] = t
            for g in range(self.n_groups):
                slot_views[g][t] = -1
            t += 1
            r += 1
        if tok[:T].min() < 0 or tok[:T].max() >= self.vocab:
            raise ValueError(f"token ids must lie in [0, {self.vocab})")
        fs = view("feed_src")
        fs[:T] = -1
        if feed is not None:
            if len(feed) != n_real:
                raise ValueError("one source row (or -1) per item is needed")
            for s, (it, src) in enumerate(zip(items, feed)):
                if src >= 0:
                    if len(it.tokens) != 1:
                        raise ValueError("only a single token can be taken from the step before")
                    fs[cu[s]] = src
        self._dev[:total].copy_(self._host[:total], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        self.bytes_last_copy = total * 4
        o_tok, o_feed = sec["token_ids"][0], sec["feed_src"][0]
        self.last_token_ids, self.last_feed_src = self._dev[o_tok:o_tok + T], self._dev[o_feed:o_feed + T]
        self._table_rows = (layout_key, new_rows) if decode_only else None
        if not views:           # a replayed graph reads the arrays where they lie; nobody needs the views
            return None

        def dev(name):
            o, n = sec[name]
            return self._dev[o:o + n]

        groups = [GroupTables(dev(f"tables{g}").view(S, width), dev(f"slots{g}")) for g in range(self.n_groups)]
        lens = [len(it.tokens) for it in items] + [1] * pad
        ends = [it.start + len(it.tokens) for it in items] + [1] * pad
        samp = {}
        if sampling is not None:
            samp = dict(temperatures=dev("temperatures").view(torch.float32), seeds=dev("seeds").view(torch.int64),
                        sample_positions=dev("sample_positions"))
        return StepBatch(**samp,
            n_tokens=T, n_seqs=S, n_logit_rows=R, token_ids=dev("token_ids"), positions=dev("positions")[:T],
            position_axes=dev("positions").view(self.n_axes, T),
            cu_q=dev("cu_q"), kv_len=dev("kv_len"), q_start=dev("q_start"), state_slots=dev("state_slots"),
            logit_rows=dev("logit_rows"), groups=groups, host_cu_q=[int(x) for x in cu[:S + 1]],
            host_kv_len=ends, max_new_tokens=max(lens),
            max_kv_len=max(ends) if pad_to is None else width * ps, decode_only=max(lens) == 1,
            n_decode_seqs=sum(1 for n in lens if n == 1), n_prefill_seqs=sum(1 for n in lens if n > 1),
            n_prefill_tokens=sum(n for n in lens if n > 1))
