"""Choosing next tokens for a batch of logits rows on the device.

The kernel applies, per row and in the reference's order, the repeat penalty over the
request's last generated tokens, then arg-max if the temperature is not positive,
else softmax((s - max) / T), top-k, top-p, min-p, renormalisation and an inverse-CDF
draw (crates/thuban_generate/src/sampler.rs:56-109).  The uniform number of each draw
is produced on the host by the request's own generator, so a draw can be reproduced.
"""
from __future__ import annotations

import torch

from .params import SamplingParams

MAX_CONTEXT = 64


class BatchSampler:
    def __init__(self, ops, device, max_rows: int, max_context: int = MAX_CONTEXT):
        self.ops = ops
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.max_context = max_context
        pin = self.device.type == "cuda"
        self._params_host = torch.zeros((max_rows, 8), dtype=torch.float32, pin_memory=pin)
        self._ctx_host = torch.full((max_rows, max_context), -1, dtype=torch.int32, pin_memory=pin)
        self._params = torch.zeros((max_rows, 8), dtype=torch.float32, device=self.device)
        self._ctx = torch.full((max_rows, max_context), -1, dtype=torch.int32, device=self.device)
        # the tokens land beside the kernels' error flags when the kernel set keeps such a buffer: one copy
        # to the host then brings both
        self._readback = getattr(ops, "readback", None)
        if self._readback is not None and max_rows <= ops.MAX_TOKEN_ROWS:
            self._out = ops.token_out[:max_rows]
            self._host = torch.zeros(2 + max_rows, dtype=torch.int32, pin_memory=pin)
        else:
            self._readback = None
            self._out = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
            self._host = torch.zeros(2 + max_rows, dtype=torch.int32, pin_memory=pin)
        self.last_flags = (0, 0)          # (tensor-core error, page error) as of the last read
        self._work = None

    def sample(self, logits: torch.Tensor, rows):
        """``rows``: one (SamplingParams, generator, generated_tokens) per logits row.
        Returns a list of token ids (host)."""
        R = logits.shape[0]
        if R == 0:
            return []
        assert R == len(rows) <= self.max_rows
        all_greedy = all(p.temperature <= 0 and p.repeat_penalty == 1.0 for p, _, _ in rows)
        out = self._out[:R]
        if all_greedy:
            self.ops.argmax(logits, out)
        else:
            ph, ch = self._params_host, self._ctx_host
            for i, (p, rng, generated) in enumerate(rows):
                n_ctx = 0
                if p.repeat_penalty != 1.0 and p.repeat_last_n > 0 and generated:
                    recent = generated[-min(p.repeat_last_n, self.max_context):]
                    n_ctx = len(recent)
                    ch[i, :n_ctx] = torch.tensor(recent, dtype=torch.int32)
                u = rng.next_f32() if p.temperature > 0 else 0.0
                ph[i] = torch.tensor([p.temperature, float(p.top_k), p.top_p, p.min_p, p.repeat_penalty, u,
                                      float(n_ctx), 0.0])
            self._params[:R].copy_(ph[:R], non_blocking=True)
            self._ctx[:R].copy_(ch[:R], non_blocking=True)
            if self._work is None or self._work.shape[0] < R or self._work.shape[1] != logits.shape[1]:
                self._work = torch.empty((max(R, min(self.max_rows, 64)), logits.shape[1]), dtype=torch.float32,
                                         device=self.device)
            self.ops.sample(logits, self._params[:R], self._ctx[:R], self._work[:R], out)
        # device -> host read of the step's result (synchronises)
        if self._readback is not None:
            self._host[:2 + R].copy_(self._readback[:2 + R])
            got = self._host[:2 + R].tolist()
            self.last_flags = (got[0], got[1])
            return got[2:]
        self._host[2:2 + R].copy_(out)
        return self._host[2:2 + R].tolist()
