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

    def build(self, entries: list, cache, vocab_size: int) -> StepBatch:
        """Validate the entries against the cache manager's records and pack them.
        Pages for the new tokens must have been reserved already."""
        b = StepBatch()
        b.entries = entries
        if not entries:
            raise BatchError("a step needs at least one entry")
        if len(entries) > self.max_seqs:
            raise BatchError(f"{len(entries)} entries in one step; the engine was built for {self.max_seqs}")
        seen = set()
        row = 0
        out_rows = []
        rows, seqs, tables = self.np_rows, self.np_seqs, self.np_tables
        for s, e in enumerate(entries):
            if e.request_id in seen:
                raise BatchError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            q_len = len(e.tokens)
            if q_len == 0:
                raise BatchError(f"request {e.request_id!r} brings no tokens")
            if row + q_len > self.max_tokens:
                raise BatchError(f"the step has more than {self.max_tokens} tokens")
            rec = cache.requests[e.request_id]
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.min() < 0 or toks.max() >= vocab_size:
                raise BatchError(f"request {e.request_id!r}: token id outside [0, {vocab_size})")
            pos0 = rec.length
            if pos0 + q_len > rec.reserved_to:
                raise BatchError(f"request {e.request_id!r}: pages for positions up to {pos0 + q_len} are not reserved")
            rows[0, row:row + q_len] = toks
            rows[1, row:row + q_len] = np.arange(pos0, pos0 + q_len)
            rows[2, row:row + q_len] = s
            for w in e.want:
                if not 0 <= w < q_len:
                    raise BatchError(f"request {e.request_id!r}: wanted place {w} is outside its {q_len} tokens")
                out_rows.append(row + w)
            seqs[0, s], seqs[1, s], seqs[2, s], seqs[3, s] = row, q_len, pos0, rec.slot
            for gi in range(cache.n_groups):
                pages = rec.pages[gi]
                if len(pages) > self.max_pages:
                    raise BatchError(f"request {e.request_id!r} holds {len(pages)} pages; tables have {self.max_pages}")
                tables[gi, s, :len(pages)] = pages
                tables[gi, s, len(pages):] = -1
            b.seq_q_start.append(row)
            b.seq_q_len.append(q_len)
            b.seq_pos_start.append(pos0)
            b.seq_slot.append(rec.slot)
            b.max_q_len = max(b.max_q_len, q_len)
            b.max_kv_len = max(b.max_kv_len, pos0 + q_len)
            row += q_len
        n, S, n_out = row, len(entries), len(out_rows)
        if n_out:
            rows[3, :n_out] = out_rows
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
