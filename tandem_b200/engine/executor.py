"""The step function: one batch of (request, its next tokens) through the model.

``run`` takes any mix of prompt portions and single decoded tokens, cut anywhere, flattens them
into one batch, runs exactly those tokens from the cache that earlier steps left, and returns
float32 logits at the wanted places only.  It samples nothing.  12vivi/tandem's counterpart is
``ModelRunner.launch`` (python/tandem/executor/model_runner.py:83-163), which also samples;
its batch description is python/tandem/layers/flashinfer_attention.py:39-67.

``step`` is ``run`` with the cache bookkeeping around it (admit, take pages, commit, end), for
callers that drive the engine without the scheduler: trace replay and tests.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from tandem_b200.cache.manager import CacheManager, OutOfPages
from tandem_b200.cache.storage import CacheStorage
from tandem_b200.models.decoder import Decoder
from tandem_b200.parts.base import StepContext


@dataclass
class StepEntry:
    request_id: str
    tokens: Sequence[int]  # the request's next tokens
    want: Sequence[int] = field(default_factory=list)  # places among ``tokens`` whose logits are returned
    # The value of the last token is still on the device: row ``pending`` of ``Executor.pending_tokens``
    # (what the step before sampled; python/tandem/executor/model_runner.py:88-111 of 12vivi/tandem).
    pending: Optional[int] = None


class Executor:
    def __init__(self, decoder: Decoder, manager: CacheManager, storage: CacheStorage) -> None:
        self.decoder, self.manager, self.storage = decoder, manager, storage
        self.device = decoder.device
        self.vocab_size = decoder.plan.embedding.vocab_size
        self.max_position = decoder.plan.max_position
        self.mixers = [m for m in (decoder.mixers() if hasattr(decoder, "mixers") else []) if hasattr(m, "step_arrays")]
        self.num_steps = 0
        self.h2d_bytes_last = 0  # bytes of the last step's batch description copied to the device
        self.pending_tokens: Optional[torch.Tensor] = None  # int32 on the device: tokens of the step in flight

    # ------------------------------------------------------------------ batch description
    def validate(self, entries: Sequence[StepEntry]) -> None:
        """Refuse a step that cannot run, before it touches the cache: an empty portion, a token
        outside the vocabulary, a position beyond the model's table, a wanted place that is not there."""
        seen = set()
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            start = self.manager.num_tokens(e.request_id) if self.manager.has(e.request_id) else 0
            if start + n > self.max_position:
                raise ValueError(f"request {e.request_id!r} would reach position {start + n - 1}; "
                                 f"the model's position table ends at {self.max_position - 1}")
            if e.pending is not None and (self.pending_tokens is None or not 0 <= e.pending < self.pending_tokens.numel()):
                raise ValueError(f"request {e.request_id!r} takes its token from row {e.pending} of a step in flight "
                                 "that has no such row")
            toks = np.asarray(e.tokens if e.pending is None else e.tokens[:-1], dtype=np.int64)
            bad = (toks < 0) | (toks >= self.vocab_size)
            if bad.any():
                raise ValueError(f"token id {int(toks[bad][0])} of request {e.request_id!r} is outside the vocabulary "
                                 f"[0, {self.vocab_size})")
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request_id!r} wants logits at place {w} of {n} tokens")

    def build_context(self, entries: Sequence[StepEntry]) -> tuple[StepContext, list]:
        """Flatten the entries: token ids, positions, the request of each token, slots and block
        tables per cache group.  All integers travel to the device in one copy."""
        m, ps = self.manager, self.manager.page_size
        self.validate(entries)
        ids, positions, seq_of_token, cu, starts, lens, slots_host, rows = [], [], [], [0], [], [], [], []
        pending = []  # (token row, row of pending_tokens)
        for b, e in enumerate(entries):  # per-token work in numpy: a prompt portion has thousands of tokens
            n = len(e.tokens)
            start = m.num_tokens(e.request_id)
            rows.extend(cu[-1] + w for w in e.want)
            tok = np.asarray(e.tokens, dtype=np.int64).astype(np.int32)
            if e.pending is not None:
                tok[-1] = 0
                pending.append((cu[-1] + n - 1, e.pending))
            ids.append(tok)
            positions.append(np.arange(start, start + n, dtype=np.int32))
            seq_of_token.append(np.full(n, b, dtype=np.int32))
            cu.append(cu[-1] + n)
            starts.append(start)
            lens.append(n)
            slots_host.append(m.slot(e.request_id))
        ids, positions, seq_of_token = np.concatenate(ids), np.concatenate(positions), np.concatenate(seq_of_token)
        T, B = len(ids), len(entries)
        max_total = max((s + n for s, n in zip(starts, lens)), default=0)
        width = max(1, -(-max_total // ps))
        ctx = StepContext(
            dtype=self.decoder.dtype, device=self.device, num_tokens=T, num_seqs=B,
            token_ids=None, positions=None, seq_of_token=None, cu_seqlens=None, seq_starts=None, state_slots=None,
            host_starts=starts, host_lens=lens, host_slots=slots_host, max_new=max(lens, default=0),
            max_total=max_total, storage=self.storage, page_size=ps,
        )
        arrays = {"ids": ids, "positions": positions, "seq_of_token": seq_of_token, "cu": cu, "starts": starts,
                  "slots": slots_host, "rows": rows}
        if pending:
            source = [-1] * T
            for row, src in pending:
                source[row] = src
            arrays["pending"] = source
        for g in range(len(m.groups)):
            table = []
            slot_list = []
            for e, start, n in zip(entries, starts, lens):
                t = m.table(g, e.request_id)
                if len(t) * ps < start + n:
                    raise OutOfPages(f"request {e.request_id!r} holds {len(t)} pages, {start + n} tokens need more")
                table.extend(t[:width] + [-1] * (width - len(t[:width])))
                pos = np.arange(start, start + n)
                pages = np.asarray(t, dtype=np.int64)[pos // ps]
                if (pages < 0).any():  # the per-token form of CacheManager.slot_index
                    raise RuntimeError(f"position {int(pos[pages < 0][0])} of {e.request_id!r} lies in a page that was given back")
                slot_list.append((pages * ps + pos % ps).astype(np.int32))
            arrays[("table", g)] = table
            arrays[("kvslots", g)] = np.concatenate(slot_list) if slot_list else np.zeros(0, dtype=np.int32)
        extras: dict = {}
        for layer in self.mixers:  # integer arrays that mixers want on the device for this step
            layer.step_arrays(ctx, extras)
        for key, value in extras.items():
            arrays[("extra", key)] = value

        sizes = {k: len(v) for k, v in arrays.items()}
        flat = torch.empty(sum(sizes.values()) + 4 * len(sizes), dtype=torch.int32,
                           pin_memory=self.device.type == "cuda")
        offsets, off = {}, 0
        for k, v in arrays.items():  # every array starts on a 16-byte boundary
            flat[off: off + sizes[k]] = torch.from_numpy(v) if isinstance(v, np.ndarray) else torch.as_tensor(v, dtype=torch.int32).reshape(-1)
            offsets[k] = off
            off += -(-sizes[k] // 4) * 4
        dev = flat[:off].to(self.device, non_blocking=True)
        self.h2d_bytes_last = off * 4

        def view(k):
            return dev[offsets[k]: offsets[k] + sizes[k]]

        ctx.token_ids, ctx.positions, ctx.seq_of_token = view("ids"), view("positions"), view("seq_of_token")
        if pending:
            from tandem_b200.kernels import ops

            ops.take_tokens(ctx.token_ids, view("pending"), self.pending_tokens)
        ctx.cu_seqlens, ctx.seq_starts, ctx.state_slots = view("cu"), view("starts"), view("slots")
        for g in range(len(m.groups)):
            ctx.tables[g] = (view(("table", g)).view(B, width), view(("kvslots", g)))
        for key in extras:
            ctx.extras[key] = view(("extra", key))
        logit_rows = view("rows")
        return ctx, logit_rows

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Logits float32 [R, vocab] at the wanted places, in the order of the entries and of
        their ``want``.  The requests must be live and hold the pages for their new tokens."""
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        for e in entries:
            if self.manager.num_tokens(e.request_id) == 0:  # new, or recomputed from the start
                self.storage.reset_state(self.manager.slot(e.request_id))
        ctx, logit_rows = self.build_context(entries)
        logits = self.decoder.forward(ctx, logit_rows)
        self.num_steps += 1
        return logits

    def step(self, entries: Sequence[StepEntry], end: Sequence[str] = ()) -> torch.Tensor:
        """``run`` plus the bookkeeping: unknown requests are admitted, pages are taken for the new
        tokens (OutOfPages if the pool cannot give them: nothing has run then), the tokens are
        committed, and the requests in ``end`` give back what they hold afterwards."""
        m = self.manager
        self.validate(entries)
        begun = []
        try:
            for e in entries:
                if not m.has(e.request_id):
                    m.begin(e.request_id)
                    begun.append(e.request_id)
                if not m.grow(e.request_id, m.num_tokens(e.request_id) + len(e.tokens)):
                    raise OutOfPages(f"no pages left for request {e.request_id!r} "
                                     f"({m.num_tokens(e.request_id)} + {len(e.tokens)} tokens)")
        except OutOfPages:
            for rid in begun:
                m.end(rid)
            raise
        logits = self.run(entries)
        for e in entries:
            m.commit(e.request_id, len(e.tokens))
        for rid in end:
            if m.has(rid):
                m.end(rid)
        return logits
