"""The descriptor of one step: which rows, at which positions, of which
sequences, against which pages, and which rows' logits are wanted.

It is packed on the host (by the C++ host code of the kernel library) into
pinned buffers with a fixed layout and sent to the device in three copies
(rows, sequences, block tables), once per step; no kernel of the step needs
the host again.  The reference uploads positions and
slot tables inside every layer and syncs the stream there
(crates/forward/src/core/composites/standard_attn.rs:315-329, 1133-1175).

A "sequence" of a step is one entry: the next tokens of one request, whether
that is a portion of its prompt or a single decoded token.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import ctypes

import numpy as np
import torch


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


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
        self.tables: list = []              # per cache group: block table [sequences, table columns]
        self.table_bases: list = []         # per cache group: the logical page that column 0 of each row stands for
        self.multi_seqs_d = None            # device: the sequences that bring more than one token, in step order
        self.n_multi = 0
        self.h2d_bytes = 0


class BatchBuffers:
    """Pinned host staging and device storage for step descriptors, sized once."""

    ROW_FIELDS = 4      # token_ids, positions, row_seq, out_rows
    SEQ_FIELDS = 4      # q_start, q_len, pos_start, slot; then one row per cache group (the table rows' first
                        # page) and one with the list of the sequences that bring more than one token

    def __init__(self, device, max_tokens: int, max_seqs: int, n_groups: int, max_pages: int):
        """max_pages: columns of a block-table row = the most live pages one request holds in any group."""
        self.device = device
        self.max_tokens, self.max_seqs, self.n_groups, self.max_pages = max_tokens, max_seqs, n_groups, max_pages
        pin = device.type == "cuda"
        self.h_rows = torch.zeros((self.ROW_FIELDS, max_tokens), dtype=torch.int32, pin_memory=pin)
        self.h_seqs = torch.zeros((self.SEQ_FIELDS + n_groups + 1, max_seqs), dtype=torch.int32, pin_memory=pin)
        self.h_tables = torch.full((max(n_groups, 1), max_seqs, max_pages), -1, dtype=torch.int32, pin_memory=pin)
        self.d_rows = torch.zeros_like(self.h_rows, device=device)
        self.d_seqs = torch.zeros_like(self.h_seqs, device=device)
        self.d_tables = torch.full_like(self.h_tables, -1, device=device)
        self.np_rows = self.h_rows.numpy()
        self.np_seqs = self.h_seqs.numpy()
        self.np_tables = self.h_tables.numpy()
        self._fill = np.zeros((max(n_groups, 1), max_seqs), dtype=np.int32)   # valid entries last written per table row
        self._info = np.zeros(8, dtype=np.int32)
        from ..kernels.library import lib
        self._lib = lib()

    def _to_device(self, dst: torch.Tensor, src: torch.Tensor, rows: int, width: int, pitch: int) -> None:
        """The first `width` int32 of each of the first `rows` rows (rows `pitch` int32 apart on both sides), on
        torch's current stream.  On the GPU one asynchronous 2-d copy from the pinned buffer; torch's own copy of
        such a slice goes through a temporary and a kernel."""
        if not width or not rows:
            return
        if self.device.type != "cuda":
            dst.view(-1, pitch)[:rows, :width].copy_(src.view(-1, pitch)[:rows, :width])
            return
        from ..kernels.ops import current_stream
        if self._lib.fb_copy_rows_to_device(dst.data_ptr(), 4 * pitch, src.data_ptr(), 4 * pitch, 4 * width, rows,
                                            current_stream()) != 0:
            raise BatchError(self._lib.fb_last_error().decode(errors="replace"))

    def build(self, entries: list, cache, vocab_size: int) -> StepBatch:
        """Validate the entries against the cache manager's books and pack them (in the C++ host code,
        csrc/host_cache.cpp: fbh_build_step).  Pages for the new tokens must have been reserved already."""
        b = StepBatch()
        b.entries = entries
        S = len(entries)
        if not S:
            raise BatchError("a step needs at least one entry")
        ids = [e.request_id for e in entries]
        recs = [cache.requests[rid] for rid in ids]
        slots = np.fromiter((r.slot for r in recs), dtype=np.int32, count=S)
        q_len = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=S)
        n = int(q_len.sum())
        if n == S:
            tokens = np.fromiter((e.tokens[0] if e.tokens else 0 for e in entries), dtype=np.int64, count=S)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]) if n else np.zeros(0, np.int64)
        if tokens.size and (int(tokens.min()) < 0 or int(tokens.max()) >= vocab_size):
            raise BatchError(f"token id outside [0, {vocab_size})")
        tokens = tokens.astype(np.int32)
        n_want = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=S)
        wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=int(n_want.sum()))
        info = self._info
        code = self._lib.fbh_build_step(
            cache.books.handle, S, _p(slots), _p(q_len), _p(tokens), _p(n_want), _p(wants), int(vocab_size),
            self.max_tokens, self.max_seqs, self.max_pages, _p(self.np_rows), _p(self.np_seqs), _p(self.np_tables),
            _p(self._fill), _p(info))
        if code != 0:
            raise BatchError(self._lib.fbh_last_error().decode(errors="replace"))
        n, n_out = int(info[0]), int(info[1])
        b.seq_q_start = self.np_seqs[0, :S].tolist()
        b.seq_q_len = q_len.tolist()
        b.seq_pos_start = self.np_seqs[2, :S].tolist()
        b.seq_slot = slots.tolist()
        b.max_q_len, b.max_kv_len = int(info[2]), int(info[3])
        b.n_tokens, b.n_seqs, b.n_out = n, S, n_out
        b.n_multi = int(info[4])
        # ---- three copies to the device: the used part of each staging buffer, as one 2-d copy each ----
        width = max(n, n_out)
        self._to_device(self.d_rows, self.h_rows, self.ROW_FIELDS, width, self.max_tokens)
        self._to_device(self.d_seqs, self.h_seqs, self.SEQ_FIELDS + self.n_groups + 1, S, self.max_seqs)
        b.h2d_bytes = 4 * (self.ROW_FIELDS * width + (self.SEQ_FIELDS + self.n_groups + 1) * S)
        if cache.n_groups:
            # every group's table rows of the step's sequences: S * max_pages entries a group, contiguous
            self._to_device(self.d_tables, self.h_tables, cache.n_groups, S * self.max_pages,
                            self.max_seqs * self.max_pages)
            b.h2d_bytes += 4 * cache.n_groups * S * self.max_pages
        b.token_ids, b.positions, b.row_seq, b.out_rows = (self.d_rows[i] for i in range(4))
        b.seq_q_start_d, b.seq_q_len_d, b.seq_pos_start_d, b.seq_slot_d = (self.d_seqs[i] for i in range(4))
        b.tables = [self.d_tables[gi] for gi in range(cache.n_groups)]
        b.table_bases = [self.d_seqs[self.SEQ_FIELDS + gi] for gi in range(cache.n_groups)]
        b.multi_seqs_d = self.d_seqs[self.SEQ_FIELDS + self.n_groups]
        return b
