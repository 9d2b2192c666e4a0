"""Token choice for the wanted rows of a step, on the device.

Order, as in the reference's sampler (crates/runtime/src/sampling.rs:306-335):
penalties over the request's generated tokens, logit bias, then argmax for
greedy rows or a draw from softmax(logits / T) under top-k / top-p / min-p.
The per-row parameters travel to the device in one small copy; the logits never
leave it.
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams, uniform_for


class Sampler:
    def __init__(self, device, max_rows: int = 64):
        self.device = device
        self.max_rows = 0
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        if rows <= self.max_rows:
            return
        self.max_rows = rows
        pin = self.device.type == "cuda"
        # float fields: temperature, uniform, top_p, min_p, repetition, presence, frequency; int field: top_k
        self.h_f = torch.zeros((7, rows), dtype=torch.float32, pin_memory=pin)
        self.h_i = torch.zeros((1, rows), dtype=torch.int32, pin_memory=pin)
        self.d_f = torch.zeros_like(self.h_f, device=self.device)
        self.d_i = torch.zeros_like(self.h_i, device=self.device)
        self.out = torch.zeros(rows, dtype=torch.int32, device=self.device)
        self.h_out = torch.zeros(rows, dtype=torch.int32, pin_memory=pin)

    def sample(self, logits: torch.Tensor, rows: list) -> list:
        """`rows[i]` = (SamplingParams, generated tokens so far, draw index) for logits[i].
        Returns the chosen token ids as Python ints.  May modify `logits` (penalties, bias)."""
        n = len(rows)
        if n == 0:
            return []
        if logits.shape[0] < n:
            raise ValueError("fewer logits rows than rows to sample")
        self._grow(n)
        f, ii = self.h_f.numpy(), self.h_i.numpy()
        pen_rows, pen_tok, pen_cnt = [], [], []
        bias_rows, bias_tok, bias_val = [], [], []
        any_draw = any_filter = False
        for r, (p, history, draw) in enumerate(rows):
            f[0, r] = p.temperature
            f[1, r] = 0.0 if p.is_greedy else uniform_for(p.seed, draw)
            f[2, r] = p.top_p or 0.0
            f[3, r] = p.min_p or 0.0
            f[4, r], f[5, r], f[6, r] = p.repetition_penalty, p.presence_penalty, p.frequency_penalty
            ii[0, r] = p.top_k or 0
            any_draw |= not p.is_greedy
            any_filter |= (not p.is_greedy) and bool(p.top_k or p.top_p or p.min_p)
            if p.has_penalties and history:
                toks, cnts = np.unique(np.asarray(history, dtype=np.int64), return_counts=True)
                pen_rows += [r] * len(toks)
                pen_tok += toks.tolist()
                pen_cnt += cnts.tolist()
            if p.logit_bias:
                for tok, b in p.logit_bias.items():
                    bias_rows.append(r)
                    bias_tok.append(int(tok))
                    bias_val.append(float(b))
        if any_draw or pen_rows:
            self.d_f[:, :n].copy_(self.h_f[:, :n], non_blocking=True)
            self.d_i[:, :n].copy_(self.h_i[:, :n], non_blocking=True)
        dev = self.device
        if pen_rows:
            ops.apply_penalties(logits, torch.tensor(pen_rows, dtype=torch.int32, device=dev),
                                torch.tensor(pen_tok, dtype=torch.int32, device=dev),
                                torch.tensor(pen_cnt, dtype=torch.int32, device=dev),
                                self.d_f[4], self.d_f[5], self.d_f[6])
        if bias_rows:
            ops.apply_logit_bias(logits, torch.tensor(bias_rows, dtype=torch.int32, device=dev),
                                 torch.tensor(bias_tok, dtype=torch.int32, device=dev),
                                 torch.tensor(bias_val, dtype=torch.float32, device=dev))
        if any_draw:
            ops.sample(logits, self.out, temperature=self.d_f[0], uniform=self.d_f[1],
                       top_k=self.d_i[0] if any_filter else None, top_p=self.d_f[2] if any_filter else None,
                       min_p=self.d_f[3] if any_filter else None, n=n)
        else:
            ops.sample(logits, self.out, n=n)
        self.h_out[:n].copy_(self.out[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.h_out[:n].tolist()
