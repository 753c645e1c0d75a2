"""CUDA graphs for decode-only steps, and for short steps that bring prompt portions.

A step in which every request brings exactly one token launches a few hundred small kernels; at
small batches their launch cost exceeds their run time.  Such steps are captured once per batch
*bucket* (1, 2, 4, 8, 16, 24, 32, ... as python/tandem/executor/cuda_graph.py:34-38 of
12vivi/tandem; 12 beside them, and the most rows whose products over the model's width this
package's streaming kernel still takes, 14 for a width of 4,096: at 16 rows they are the library's) and replayed: the batch description lives in one static int32 buffer on the
device, refilled by a single copy before each replay.  Rows that pad a batch up to its bucket
carry token 0 at position 0 with a negative cache slot (the cache-write kernel skips them) and no
attention item; their outputs are never read.  Logits and sampling stay outside the graph
(cuda_graph.py:10-11 of the reference).

Only models whose mixers all declare ``capturable = True`` run under graphs: everything such a
mixer does in ``forward`` is kernel launches on the current stream, and what it knows of the batch
it reads from the device arrays of the context (``positions``, ``seq_starts``, ``state_slots``,
its own ``extras``), never from the host-side lists, which a replay does not see.  A mixer with
per-request state indexes its state tensor by ``ctx.state_slots`` on the device; padding rows
point at the state tensor's last row, which belongs to no request.  Mixers that asked for per-step
arrays (``step_arrays``) say how large they can get for a bucket through
``step_array_capacity(bucket, max_model_len, page_size, out)``.

A step that is not replayed costs the host some 15 us per kernel it launches, 4.7 ms for the 36 layers
of Qwen3-8B, while the device needs 3.3 ms for a step of up to a few hundred tokens (it streams the
weights once): the first portion of a short prompt, or a few decoded tokens beside one, would wait for
the host.  So steps of up to ``MIXED_MAX_TOKENS`` tokens are captured as well, per bucket of tokens
(8, 16, 32, 64, 128, 256) for up to as many requests as the decode graphs take: token rows beyond the
step's are padding (token 0, no cache slot, in no attention item), the attention plan keeps the layout
of its capacity (``StepContext.static_layout``), and both attention kernels run in every replay, one of
them perhaps with nothing to do.  This needs mixers that declare ``capturable_portions = True`` (what
``capturable`` says, for requests that bring several tokens too) and say how large their arrays get for
such steps (``mixed_step_array_capacity``); a step whose plan outgrows that room runs without a graph.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from tandem_b200.engine.executor import Executor, OutOfPages, StepEntry
from tandem_b200.kernels import ops
from tandem_b200.parts.base import PlanTooLarge, StepContext


def bucket_sizes(max_batch: int, also: Sequence[int] = ()) -> list:
    sizes = [b for b in (1, 2, 4, 8, 12, 16) + tuple(also) if 0 < b <= max_batch] + list(range(24, max_batch + 1, 8))
    if max_batch not in sizes:
        sizes.append(max_batch)
    return sorted(set(sizes))


class _Captured:
    """One bucket: the static batch description, its graph and its logits."""

    def __init__(self, executor: Executor, bucket: int, max_model_len: int, seqs: int = 0) -> None:
        """``bucket`` token rows; ``seqs`` = 0: as many requests, one token each; else up to ``seqs`` requests
        that share the rows among them (prompt portions beside single tokens), and one more that no request
        ever is: the rows that pad the step are its tokens, so a mixer with state sends them to the state
        tensor's spare row."""
        self.executor, self.bucket, self.seqs, self.mixed = executor, bucket, (seqs + 1) if seqs else bucket, bool(seqs)
        m = executor.manager
        self.width = -(-max_model_len // m.page_size)
        self.sizes = {"ids": bucket, "positions": bucket, "seq_of_token": bucket, "cu": self.seqs + 1, "starts": self.seqs,
                      "slots": self.seqs, "rows": self.seqs, "pending": bucket}
        for g in range(len(m.groups)):
            self.sizes[("table", g)] = self.seqs * self.width
            self.sizes[("kvslots", g)] = bucket
        capacity: dict = {}
        for mixer in executor.mixers:
            if seqs:
                mixer.mixed_step_array_capacity(bucket, self.seqs, max_model_len, m.page_size, capacity)
            elif hasattr(mixer, "step_array_capacity"):
                mixer.step_array_capacity(bucket, max_model_len, m.page_size, capacity)
        self.extra_keys = list(capacity)
        for key, n in capacity.items():
            self.sizes[("extra", key)] = n
        self.offsets, off = {}, 0
        for k, n in self.sizes.items():
            self.offsets[k] = off
            off += -(-n // 4) * 4
        # Two pinned copies of the description, used in turn: with overlap scheduling the host fills
        # step N+1 while the copy of step N may still be on its way to the device, and a buffer is
        # written again only after the copy that last read it has landed (its event).
        self.hosts = [torch.zeros(off, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.copied = [None, None]
        self.turn = 0
        self.hosts_np = [h.numpy() for h in self.hosts]
        self.host, self.host_np = self.hosts[0], self.hosts_np[0]
        self.device = torch.zeros(off, dtype=torch.int32, device=executor.device)
        self.graph = None
        self.logits = None
        self.launches = 0
        self.replays = 0

    def view(self, k):
        return self.device[self.offsets[k]: self.offsets[k] + self.sizes[k]]

    def put(self, k, values) -> None:
        o = self.offsets[k]
        self.host_np[o: o + len(values)] = values

    def fill(self, entries: Sequence[StepEntry]) -> StepContext:
        """Write this step's batch description into the pinned buffer and copy it to the device."""
        ex, m, ps, Bk, B = self.executor, self.executor.manager, self.executor.manager.page_size, self.bucket, len(entries)
        self.turn = 1 - self.turn
        self.host, self.host_np = self.hosts[self.turn], self.hosts_np[self.turn]
        if self.copied[self.turn] is not None:
            self.copied[self.turn].synchronize()  # almost always long past
        starts = [m.num_tokens(e.request_id) for e in entries]
        pad = Bk - B
        self.put("ids", [int(e.tokens[0]) if e.pending is None else 0 for e in entries] + [0] * pad)
        any_pending = any(e.pending is not None for e in entries)
        self.put("pending", [-1 if e.pending is None else e.pending for e in entries] + [-1] * pad)
        self.put("positions", starts + [0] * pad)
        self.put("seq_of_token", list(range(Bk)))
        self.put("cu", list(range(Bk + 1)))
        self.put("starts", starts + [0] * pad)
        slots = [m.slot(e.request_id) for e in entries]
        self.put("slots", slots + [ex.storage.scratch_slot] * pad)
        self.put("rows", list(range(Bk)))
        for g in range(len(m.groups)):
            o = self.offsets[("table", g)]
            block = self.host_np[o: o + Bk * self.width].reshape(Bk, self.width)
            kvslots = []
            for b, (e, s) in enumerate(zip(entries, starts)):
                t = m.table(g, e.request_id)
                block[b, : len(t)] = t
                kvslots.append(m.slot_index(g, e.request_id, s))
            self.put(("kvslots", g), kvslots + [-1] * pad)
        ctx = StepContext(
            dtype=ex.decoder.dtype, device=ex.device, num_tokens=Bk, num_seqs=Bk, token_ids=self.view("ids"),
            positions=self.view("positions"), seq_of_token=self.view("seq_of_token"), cu_seqlens=self.view("cu"),
            seq_starts=self.view("starts"), state_slots=self.view("slots"), host_starts=starts, host_lens=[1] * B,
            host_slots=slots, max_new=1, max_total=max(starts) + 1, storage=ex.storage, page_size=ps,
        )
        extras: dict = {}
        for mixer in ex.mixers:
            mixer.step_arrays(ctx, extras)
        for key in self.extra_keys:
            values = extras.get(key, [])
            if len(values) > self.sizes[("extra", key)]:
                raise RuntimeError(f"step array {key} has {len(values)} entries, the graph was captured for "
                                   f"{self.sizes[('extra', key)]}")
            self.put(("extra", key), values)
            ctx.extras[key] = self.view(("extra", key))
        for g in range(len(m.groups)):
            ctx.tables[g] = (self.view(("table", g)).view(Bk, self.width), self.view(("kvslots", g)))
        self.device.copy_(self.host, non_blocking=True)
        if self.copied[self.turn] is None:
            self.copied[self.turn] = torch.cuda.Event()
        self.copied[self.turn].record()
        ex.h2d_bytes_last = self.host.numel() * 4
        if any_pending:  # tokens of the step in flight enter the batch on the device, before the graph reads it
            ops.take_tokens(self.view("ids"), self.view("pending"), ex.pending_tokens)
        return ctx

    def fill_mixed(self, entries: Sequence[StepEntry]) -> StepContext:
        """The same for a step whose requests bring any number of tokens, ``bucket`` at most in all.  Raises
        ``PlanTooLarge`` (nothing has been copied then) if a mixer's plan does not fit its room."""
        ex, m, ps, Tb, Sb = self.executor, self.executor.manager, self.executor.manager.page_size, self.bucket, self.seqs
        starts = [m.num_tokens(e.request_id) for e in entries]
        lens = [len(e.tokens) for e in entries]
        slots = [m.slot(e.request_id) for e in entries]
        T, B = sum(lens), len(entries)
        ctx = StepContext(
            dtype=ex.decoder.dtype, device=ex.device, num_tokens=Tb, num_seqs=Sb, token_ids=self.view("ids"),
            positions=self.view("positions"), seq_of_token=self.view("seq_of_token"), cu_seqlens=self.view("cu"),
            seq_starts=self.view("starts"), state_slots=self.view("slots"), host_starts=starts, host_lens=lens,
            host_slots=slots, max_new=max(lens), max_total=max(s + n for s, n in zip(starts, lens)), storage=ex.storage,
            page_size=ps, static_layout=True,
        )
        extras: dict = {}
        for mixer in ex.mixers:  # first of all: the one thing that can fail
            mixer.step_arrays(ctx, extras)
        for key in self.extra_keys:
            if len(extras.get(key, ())) > self.sizes[("extra", key)]:
                raise PlanTooLarge(f"step array {key} has {len(extras[key])} entries, the graph has room for {self.sizes[('extra', key)]}")
        self.turn = 1 - self.turn
        self.host, self.host_np = self.hosts[self.turn], self.hosts_np[self.turn]
        if self.copied[self.turn] is not None:
            self.copied[self.turn].synchronize()  # almost always long past
        ids = np.zeros(Tb, dtype=np.int32)
        positions = np.zeros(Tb, dtype=np.int32)
        seq_of = np.full(Tb, B, dtype=np.int32)  # padding rows: the tokens of a request of their own, behind the real ones
        pending = np.full(Tb, -1, dtype=np.int32)
        cu, rows, any_pending = [0], [], False
        for b, (e, start, n) in enumerate(zip(entries, starts, lens)):
            row = cu[-1]
            ids[row: row + n] = e.tokens
            if e.pending is not None:  # only the newest token can still be on its way
                ids[row + n - 1] = 0
                pending[row + n - 1] = e.pending
                any_pending = True
            positions[row: row + n] = np.arange(start, start + n, dtype=np.int32)
            seq_of[row: row + n] = b
            rows.extend(row + w for w in e.want)
            cu.append(row + n)
        self.num_rows = len(rows)
        self.put("ids", ids)
        self.put("pending", pending)
        self.put("positions", positions)
        self.put("seq_of_token", seq_of)
        self.put("cu", cu + [Tb] * (Sb - B))
        self.put("starts", starts + [0] * (Sb - B))
        self.put("slots", slots + [ex.storage.scratch_slot] * (Sb - B))
        self.put("rows", rows + [0] * (Sb - len(rows)))
        for g in range(len(m.groups)):
            o = self.offsets[("table", g)]
            block = self.host_np[o: o + Sb * self.width].reshape(Sb, self.width)
            kvslots = np.full(Tb, -1, dtype=np.int32)
            for b, (e, start, n) in enumerate(zip(entries, starts, lens)):
                t = m.table(g, e.request_id)
                if len(t) * ps < start + n:
                    raise OutOfPages(f"request {e.request_id!r} holds {len(t)} pages, {start + n} tokens need more")
                block[b, : len(t)] = t
                pos = np.arange(start, start + n)
                pages = np.asarray(t, dtype=np.int64)[pos // ps]
                if (pages < 0).any():
                    raise RuntimeError(f"position {int(pos[pages < 0][0])} of {e.request_id!r} lies in a page that was given back")
                kvslots[cu[b]: cu[b] + n] = pages * ps + pos % ps
            self.put(("kvslots", g), kvslots)
        for key in self.extra_keys:
            self.put(("extra", key), extras.get(key, []))
            ctx.extras[key] = self.view(("extra", key))
        for g in range(len(m.groups)):
            ctx.tables[g] = (self.view(("table", g)).view(Sb, self.width), self.view(("kvslots", g)))
        self.device.copy_(self.host, non_blocking=True)
        if self.copied[self.turn] is None:
            self.copied[self.turn] = torch.cuda.Event()
        self.copied[self.turn].record()
        ex.h2d_bytes_last = self.host.numel() * 4
        if any_pending:
            ops.take_tokens(self.view("ids"), self.view("pending"), ex.pending_tokens)
        return ctx

    def capture(self, entries: Sequence[StepEntry]) -> None:
        ctx = self.fill_mixed(entries) if self.mixed else self.fill(entries)
        rows = self.view("rows")
        torch.cuda.synchronize()
        before = ops.launches
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self.executor.decoder.forward(ctx, rows)
        self.launches = ops.launches - before


MIXED_BUCKETS = (8, 16, 32, 64, 128, 256)  # token rows of the graphs for steps with prompt portions
MIXED_MAX_TOKENS = MIXED_BUCKETS[-1]  # beyond this a step keeps the device busy longer than the host needs to launch it


class DecodeGraphs:
    def __init__(self, executor: Executor, max_batch: int, max_model_len: int) -> None:
        self.executor, self.max_model_len = executor, max_model_len
        # a bucket of its own for the largest batch whose products over the model's width are still the streaming
        # kernel's (14 rows of 4,096, 11 of 5,120): one more row and all of them go to the library
        width = executor.decoder.embedding.shape[1]
        self.buckets = bucket_sizes(max_batch, (ops.streaming_row_limit(width),) if executor.decoder.dtype == torch.bfloat16 else ())
        self.captured: dict = {}
        if executor.device.type == "cuda":
            # a padded batch may be the first to reach a library product, and a library cannot be set up while a stream captures
            a = torch.zeros((16, 16), dtype=torch.bfloat16, device=executor.device)
            torch.mm(a, a)
        # steps with prompt portions: only if every mixer reads such a batch from the device arrays alone, and every
        # mixer that plans on the host can say how large such a plan gets
        self.mixed = (all(getattr(mixer, "capturable_portions", False) for mixer in executor.decoder.mixers())
                      and all(hasattr(mixer, "mixed_step_array_capacity") for mixer in executor.mixers) and self._mixed_has_room())
        self.mixed_fallbacks = 0  # steps that were meant for a graph and ran without (their plan outgrew it)

    def _mixed_has_room(self) -> bool:
        probe: dict = {}
        m = self.executor.manager
        for mixer in self.executor.mixers:
            mixer.mixed_step_array_capacity(MIXED_BUCKETS[0], min(MIXED_BUCKETS[0], self.buckets[-1]), self.max_model_len, m.page_size, probe)
        return bool(probe) or not self.executor.mixers

    @classmethod
    def maybe(cls, executor: Executor, max_batch: int, max_model_len: int):
        """Graphs need every mixer of the model to be capturable, and array capacities known for
        those that plan on the host."""
        for mixer in executor.decoder.mixers():
            if not getattr(mixer, "capturable", False):
                return None
        for mixer in executor.mixers:
            if not hasattr(mixer, "step_array_capacity"):
                return None
        return cls(executor, max_batch, max_model_len)

    def _decodes(self, entries: Sequence[StepEntry]) -> bool:
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def takes(self, entries: Sequence[StepEntry]) -> bool:
        if not (0 < len(entries) <= self.buckets[-1]
                and all(self.executor.manager.num_tokens(e.request_id) + len(e.tokens) <= self.max_model_len for e in entries)):
            return False
        if self._decodes(entries):
            return True
        tokens = sum(len(e.tokens) for e in entries)
        return (self.mixed and tokens <= MIXED_MAX_TOKENS and sum(len(e.want) for e in entries) <= self._mixed_seqs(tokens)
                and len(entries) <= self._mixed_seqs(tokens))

    def bucket_of(self, n: int) -> int:
        return next(b for b in self.buckets if b >= n)

    def _mixed_bucket(self, tokens: int) -> int:
        return next(b for b in MIXED_BUCKETS if b >= tokens)

    def _mixed_seqs(self, tokens: int) -> int:
        return min(self._mixed_bucket(tokens), self.buckets[-1])

    def launches_per_replay(self, entries: Sequence[StepEntry]) -> int:
        cap = self.captured.get(self.bucket_of(len(entries)))
        return cap.launches if cap else 0

    def capture_all(self) -> int:
        """Capture every bucket now instead of at its first step (12vivi/tandem captures its graphs when the
        engine is built: python/tandem/executor/cuda_graph.py:104-112), with requests of this method's own on
        pages that it gives back: one token each for the decode buckets, one request of as many tokens as the
        bucket has rows for those with prompt portions.  Buckets for which the pool has no room now stay for
        later.  Returns how many were captured."""
        ex, m = self.executor, self.executor.manager
        keys = list(reversed(self.buckets)) + ([("mixed", b) for b in reversed(MIXED_BUCKETS)] if self.mixed else [])
        captured = 0
        for key in keys:
            if key in self.captured:
                continue
            lens = [min(key[1], self.max_model_len)] if isinstance(key, tuple) else [1] * key
            rids = [f"__capture_{i}" for i in range(len(lens))]
            begun, room = [], len(lens) <= m.slots.num_free
            try:
                for rid, n in zip(rids, lens):
                    if not room:
                        break
                    m.begin(rid)
                    begun.append(rid)
                    room = m.grow(rid, n)  # False: no pages for so many now; the bucket is captured when a step first needs it
                entries = [StepEntry(rid, [0] * n, [n - 1]) for rid, n in zip(rids, lens)]
                if room and self.takes(entries):
                    self.run(entries)
                    captured += key in self.captured
            finally:
                for rid in begun:
                    m.end(rid)
        return captured

    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Same contract as ``Executor.run``, for the steps that ``takes`` accepts."""
        ex = self.executor
        ex.validate(entries)
        decodes = self._decodes(entries)
        tokens = sum(len(e.tokens) for e in entries)
        key = self.bucket_of(len(entries)) if decodes else ("mixed", self._mixed_bucket(tokens))
        cap = self.captured.get(key)
        if cap is None:
            logits = ex.run(entries)  # the first step of a bucket runs eagerly (this also builds what is built lazily)
            cap = _Captured(ex, key, self.max_model_len) if decodes else _Captured(ex, key[1], self.max_model_len, self._mixed_seqs(tokens))
            try:
                with torch.inference_mode():
                    cap.capture(entries)
            except PlanTooLarge:
                self.mixed_fallbacks += 1
                return logits
            self.captured[key] = cap
            return logits
        for e in entries:
            if ex.manager.num_tokens(e.request_id) == 0:
                ex.storage.reset_state(ex.manager.slot(e.request_id))
        if decodes:
            cap.fill(entries)
            wanted = len(entries)
        else:
            try:
                cap.fill_mixed(entries)
            except PlanTooLarge:
                self.mixed_fallbacks += 1
                return ex.run(entries)
            wanted = cap.num_rows
        cap.graph.replay()
        cap.replays += 1
        ops.launches += cap.launches
        ex.num_steps += 1
        return cap.logits[:wanted]
