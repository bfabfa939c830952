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

MAX_CONTEXT = 64        # width the context buffers start with; they grow to the largest repeat_last_n in use


class BatchSampler:
    """``launch`` enqueues the sampling of a step and the copy of its tokens to the host and returns a
    ticket; ``read`` waits for that copy and returns the tokens.  Two steps may be in flight (the host
    buffers alternate), so a caller can enqueue the next step before it reads this one's tokens.
    ``sample`` is the two in one."""

    def __init__(self, ops, device, max_rows: int, max_context: int = MAX_CONTEXT):
        self.ops = ops
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.max_context = max_context
        cuda = self.device.type == "cuda"
        self._params_host = [torch.zeros((max_rows, 8), dtype=torch.float32, pin_memory=cuda) for _ in range(2)]
        self._params = torch.zeros((max_rows, 8), dtype=torch.float32, device=self.device)
        self._size_context(max_context)
        # the tokens land beside the kernels' error flags when the kernel set keeps such a buffer: one copy
        # to the host then brings both, and the next step can take its tokens from there on the device
        self._readback = getattr(ops, "readback", None)
        if self._readback is not None and max_rows <= ops.MAX_TOKEN_ROWS:
            self._out = ops.token_out[:max_rows]
        else:
            self._readback = None
            self._out = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self._host = [torch.zeros(2 + max_rows, dtype=torch.int32, pin_memory=cuda) for _ in range(2)]
        self._done = [torch.cuda.Event() if cuda else None for _ in range(2)]
        self._rows = [0, 0]
        self._next = 0
        self.last_flags = (0, 0)          # (tensor-core error, page error) as of the last read
        self._work = None

    def _size_context(self, width: int):
        """Buffers for the last ``width`` generated tokens of every row (the repeat penalty's context).  The
        reference honours any ``repeat_last_n`` (crates/thuban_generate/src/sampler.rs:145-160); so the buffers
        grow when a request asks for more than they hold."""
        cuda = self.device.type == "cuda"
        self.max_context = int(width)
        self._ctx_host = [torch.full((self.max_rows, self.max_context), -1, dtype=torch.int32, pin_memory=cuda)
                          for _ in range(2)]
        self._ctx = torch.full((self.max_rows, self.max_context), -1, dtype=torch.int32, device=self.device)

    @property
    def feeds_next_step(self) -> bool:
        """The tokens stay on the device where the model's embedding can take them (StepEntry.feed)."""
        return self._readback is not None

    def launch(self, logits: torch.Tensor, rows) -> int:
        """``rows``: one (SamplingParams, generator, generated_tokens) per logits row.  Returns a ticket."""
        R = logits.shape[0]
        assert R == len(rows) <= self.max_rows
        ticket = self._next
        self._next ^= 1
        self._rows[ticket] = R
        if R == 0:
            return ticket
        all_greedy = all(p.temperature <= 0 and p.repeat_penalty == 1.0 for p, _, _ in rows)
        out = self._out[:R]
        if all_greedy:
            self.ops.argmax(logits, out)
        else:
            need = max((min(p.repeat_last_n, len(g)) for p, _, g in rows if p.repeat_penalty != 1.0 and g), default=0)
            if need > self.max_context:
                self._size_context(1 << (need - 1).bit_length())
            ph, ch = self._params_host[ticket], self._ctx_host[ticket]
            flat, any_ctx = [], False
            for i, (p, rng, generated) in enumerate(rows):
                n_ctx = 0
                if p.repeat_penalty != 1.0 and p.repeat_last_n > 0 and generated:
                    recent = generated[-min(p.repeat_last_n, self.max_context):]
                    n_ctx = len(recent)
                    ch[i, :n_ctx] = torch.tensor(recent, dtype=torch.int32)
                    any_ctx = True
                u = rng.next_f32() if p.temperature > 0 else 0.0
                flat += (p.temperature, float(p.top_k), p.top_p, p.min_p, p.repeat_penalty, u, float(n_ctx), 0.0)
            ph[:R] = torch.tensor(flat, dtype=torch.float32).view(R, 8)       # one write for all rows
            self._params[:R].copy_(ph[:R], non_blocking=True)
            if any_ctx:                     # rows without a penalty never read their context
                self._ctx[:R].copy_(ch[:R], non_blocking=True)
            if self._work is None or self._work.shape[0] < R or self._work.shape[1] != logits.shape[1]:
                self._work = torch.empty((max(R, min(self.max_rows, 64)), logits.shape[1]), dtype=torch.float32,
                                         device=self.device)
            self.ops.sample(logits, self._params[:R], self._ctx[:R], self._work[:R], out)
        # device -> host copy of the step's result, read (and waited for) by read()
        host = self._host[ticket]
        if self._readback is not None:
            host[:2 + R].copy_(self._readback[:2 + R], non_blocking=True)
        else:
            host[2:2 + R].copy_(out, non_blocking=True)
        if self._done[ticket] is not None:
            self._done[ticket].record()
        return ticket

    def read(self, ticket: int):
        """The tokens of a launched step (host list).  Blocks until they have arrived."""
        R = self._rows[ticket]
        if R == 0:
            return []
        if self._done[ticket] is not None:
            self._done[ticket].synchronize()
        got = self._host[ticket][:2 + R].tolist()
        if self._readback is not None:
            self.last_flags = (got[0], got[1])
        return got[2:]

    def sample(self, logits: torch.Tensor, rows):
        """Returns a list of token ids (host)."""
        return self.read(self.launch(logits, rows))
