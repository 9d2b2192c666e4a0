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


class SampleHandle:
    """Tokens on their way to the host: `tokens` (device int32, one per row, valid in stream order right away)
    and a pinned copy that `Sampler.collect` reads once the event has passed."""
    __slots__ = ("n", "tokens", "host", "event")

    def __init__(self, n, tokens, host, event):
        self.n, self.tokens, self.host, self.event = n, tokens, host, event


class _Staging:
    def __init__(self, device, rows: int):
        pin = device.type == "cuda"
        # float fields: temperature, uniform, top_p, min_p, repetition, presence, frequency; int field: top_k
        self.h_f = torch.zeros((7, rows), dtype=torch.float32, pin_memory=pin)
        self.h_i = torch.zeros((1, rows), dtype=torch.int32, pin_memory=pin)
        self.d_f = torch.zeros_like(self.h_f, device=device)
        self.d_i = torch.zeros_like(self.h_i, device=device)
        self.out = torch.zeros(rows, dtype=torch.int32, device=device)
        self.h_out = torch.zeros(rows, dtype=torch.int32, pin_memory=pin)
        self.event = torch.cuda.Event() if device.type == "cuda" else None


class Sampler:
    def __init__(self, device, max_rows: int = 64):
        self.device = device
        self.max_rows = 0
        self._turn = 0
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        if rows <= self.max_rows:
            return
        self.max_rows = rows
        # two sets that take turns: a step may be launched before the tokens of the step before it are read
        self._sets = [_Staging(self.device, rows), _Staging(self.device, rows)]

    def sample(self, logits: torch.Tensor, rows: list) -> list:
        """`rows[i]` = (SamplingParams, generated tokens so far, draw index) for logits[i].
        Returns the chosen token ids as Python ints.  May modify `logits` (penalties, bias)."""
        if not rows:
            return []
        return self.collect(self.launch(logits, rows))

    def collect(self, handle: SampleHandle) -> list:
        """Wait for a launched sampling and return its token ids."""
        handle.event.synchronize()
        return handle.host[:handle.n].tolist()

    def launch(self, logits: torch.Tensor, rows: list) -> SampleHandle:
        """Launch the sampling of `rows` (as in `sample`) and the copy of the tokens to the host; nothing waits."""
        n = len(rows)
        if logits.shape[0] < n:
            raise ValueError("fewer logits rows than rows to sample")
        self._grow(n)
        st = self._sets[self._turn]
        self._turn ^= 1
        f, ii = st.h_f.numpy(), st.h_i.numpy()
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
            st.d_f[:, :n].copy_(st.h_f[:, :n], non_blocking=True)
            st.d_i[:, :n].copy_(st.h_i[:, :n], non_blocking=True)
        dev = self.device
        if pen_rows:
            ops.apply_penalties(logits, torch.tensor(pen_rows, dtype=torch.int32, device=dev),
                                torch.tensor(pen_tok, dtype=torch.int32, device=dev),
                                torch.tensor(pen_cnt, dtype=torch.int32, device=dev),
                                st.d_f[4], st.d_f[5], st.d_f[6])
        if bias_rows:
            ops.apply_logit_bias(logits, torch.tensor(bias_rows, dtype=torch.int32, device=dev),
                                 torch.tensor(bias_tok, dtype=torch.int32, device=dev),
                                 torch.tensor(bias_val, dtype=torch.float32, device=dev))
        if any_draw:
            ops.sample(logits, st.out, temperature=st.d_f[0], uniform=st.d_f[1],
                       top_k=st.d_i[0] if any_filter else None, top_p=st.d_f[2] if any_filter else None,
                       min_p=st.d_f[3] if any_filter else None, n=n)
        else:
            ops.sample(logits, st.out, n=n)
        st.h_out[:n].copy_(st.out[:n], non_blocking=True)
        st.event.record()
        return SampleHandle(n, st.out, st.h_out, st.event)
