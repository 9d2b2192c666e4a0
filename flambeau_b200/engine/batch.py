"""The descriptor of one step: which rows, at which positions, of which
sequences, against which pages, and which rows' logits are wanted.

It is packed on the host into pinned buffers with a fixed layout and sent to
the device in three copies (rows, sequences, block tables), once per step; no
kernel of the step needs the host again.  The reference uploads positions and
slot tables inside every layer and syncs the stream there
(crates/forward/src/core/composites/standard_attn.rs:315-329, 1133-1175).

A "sequence" of a step is one entry: the next tokens of one request, whether
that is a portion of its prompt or a single decoded token.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class Entry:
    request_id: object
    tokens: list
    want: list = field(default_factory=list)     # places among `tokens` whose logits are wanted


class BatchError(ValueError):
    pass


class StepBatch:
    """Device views of one step's descriptor (all int32) plus the host-side lists."""

    def __init__(self):
        self.entries: list = []
        self.n_tokens = self.n_seqs = self.n_out = 0
        self.seq_q_start: list = []
        self.seq_q_len: list = []
        self.seq_pos_start: list = []
        self.seq_slot: list = []
        self.max_q_len = 0
        self.max_kv_len = 0
        # device tensors
        self.token_ids = self.positions = self.row_seq = self.out_rows = None
        self.seq_q_start_d = self.seq_q_len_d = self.seq_pos_start_d = self.seq_slot_d = None
        self.tables: list = []
        self.h2d_bytes = 0


class BatchBuffers:
    """Pinned host staging and device storage for step descriptors, sized once."""

    ROW_FIELDS = 4      # token_ids, positions, row_seq, out_rows
    SEQ_FIELDS = 4      # q_start, q_len, pos_start, slot

    def __init__(self, device, max_tokens: int, max_seqs: int, n_groups: int, max_pages: int):
        self.device = device
        self.max_tokens, self.max_seqs, self.n_groups, self.max_pages = max_tokens, max_seqs, n_groups, max_pages
        pin = device.type == "cuda"
        self.h_rows = torch.zeros((self.ROW_FIELDS, max_tokens), dtype=torch.int32, pin_memory=pin)
        self.h_seqs = torch.zeros((self.SEQ_FIELDS, max_seqs), dtype=torch.int32, pin_memory=pin)
        self.h_tables = torch.full((max(n_groups, 1), max_seqs, max_pages), -1, dtype=torch.int32, pin_memory=pin)
        self.d_rows = torch.zeros_like(self.h_rows, device=device)
        self.d_seqs = torch.zeros_like(self.h_seqs, device=device)
        self.d_tables = torch.full_like(self.h_tables, -1, device=device)
        self.np_rows = self.h_rows.numpy()
        self.np_seqs = self.h_seqs.numpy()
        self.np_tables = self.h_tables.numpy()
        self._fill = [[0] * max_seqs for _ in range(max(n_groups, 1))]     # valid entries last written per table row

    def build(self, entries: list, cache, vocab_size: int) -> StepBatch:
        """Validate the entries against the cache manager's records and pack them.
        Pages for the new tokens must have been reserved already."""
        b = StepBatch()
        b.entries = entries
        S = len(entries)
        if not S:
            raise BatchError("a step needs at least one entry")
        if S > self.max_seqs:
            raise BatchError(f"{S} entries in one step; the engine was built for {self.max_seqs}")
        ids = [e.request_id for e in entries]
        if len(set(ids)) != S:
            raise BatchError("a request appears twice in one step")
        recs = [cache.requests[rid] for rid in ids]
        q_len = [len(e.tokens) for e in entries]
        if min(q_len) == 0:
            raise BatchError("a request brings no tokens")
        pos0 = [r.length for r in recs]
        n = sum(q_len)
        if n > self.max_tokens:
            raise BatchError(f"the step has {n} tokens; the engine was built for {self.max_tokens} a step")
        rows, seqs, tables = self.np_rows, self.np_seqs, self.np_tables
        decode_only = n == S
        if decode_only:
            starts = list(range(S))
            rows[0, :S] = [e.tokens[0] for e in entries]
            rows[1, :S] = pos0
            rows[2, :S] = starts
        else:
            starts, acc = [], 0
            for k in q_len:
                starts.append(acc)
                acc += k
            rows[0, :n] = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
            rows[1, :n] = np.concatenate([np.arange(p, p + k) for p, k in zip(pos0, q_len)])
            rows[2, :n] = np.repeat(np.arange(S), q_len)
        toks = rows[0, :n]
        if int(toks.min()) < 0 or int(toks.max()) >= vocab_size:
            raise BatchError(f"token id outside [0, {vocab_size})")
        out_rows = []
        for s, e in enumerate(entries):
            if pos0[s] + q_len[s] > recs[s].reserved_to:
                raise BatchError(f"request {e.request_id!r}: pages for positions up to {pos0[s] + q_len[s]} are not reserved")
            for w in e.want:
                if not 0 <= w < q_len[s]:
                    raise BatchError(f"request {e.request_id!r}: wanted place {w} is outside its {q_len[s]} tokens")
                out_rows.append(starts[s] + w)
        n_out = len(out_rows)
        if n_out:
            rows[3, :n_out] = out_rows
        seqs[0, :S], seqs[1, :S], seqs[2, :S] = starts, q_len, pos0
        seqs[3, :S] = [r.slot for r in recs]
        fill = self._fill
        for gi in range(cache.n_groups):
            for s, rec in enumerate(recs):
                pages = rec.pages[gi]
                k = pages.n
                if k > self.max_pages:
                    raise BatchError(f"request {ids[s]!r} holds {k} pages; tables have {self.max_pages}")
                tables[gi, s, :k] = pages.arr[:k]
                if fill[gi][s] > k:
                    tables[gi, s, k:fill[gi][s]] = -1          # what an earlier step's request left in this row
                fill[gi][s] = k
        b.seq_q_start, b.seq_q_len, b.seq_pos_start = starts, q_len, pos0
        b.seq_slot = [r.slot for r in recs]
        b.max_q_len = max(q_len)
        b.max_kv_len = max(p + k for p, k in zip(pos0, q_len))
        b.n_tokens, b.n_seqs, b.n_out = n, S, n_out
        # ---- three copies to the device ----
        width = max(n, n_out)
        self.d_rows[:, :width].copy_(self.h_rows[:, :width], non_blocking=True)
        self.d_seqs[:, :S].copy_(self.h_seqs[:, :S], non_blocking=True)
        b.h2d_bytes = 4 * (self.ROW_FIELDS * width + self.SEQ_FIELDS * S)
        if cache.n_groups:
            self.d_tables[:, :S].copy_(self.h_tables[:, :S], non_blocking=True)
            b.h2d_bytes += 4 * cache.n_groups * S * self.max_pages
        b.token_ids, b.positions, b.row_seq, b.out_rows = (self.d_rows[i] for i in range(4))
        b.seq_q_start_d, b.seq_q_len_d, b.seq_pos_start_d, b.seq_slot_d = (self.d_seqs[i] for i in range(4))
        b.tables = [self.d_tables[gi] for gi in range(cache.n_groups)]
        return b
