"""One step's batch and the metadata the kernels read.

A batch is a list of entries, one per request: the request's slot, the position of
the first token it brings, the tokens, and the places among them whose logits are
wanted.  Entries may be portions of prompts and single decoded tokens side by side,
cut anywhere.  The reference's batch is the same thing
(``SeqChunk{tokens, seq, logit_rows}``, crates/thuban_model/src/traits.rs:12-17) with the
position kept inside the model; here the caller passes it, so that the step function
holds no per-request state and the replay tool can drive it directly.

The flattened metadata is packed into one int32 buffer and copied to the device with
a single copy: token ids, positions, slots, and the rows whose logits are wanted (the
reference uploads 8 words per row: crates/thuban_model/src/rows.rs:7-30).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..errors import ModelError


TILE_ROWS = 128        # query rows per tile of the tensor-core attention
TILE_MIN_ROWS = 16     # shorter portions go row by row


@dataclass
class StepEntry:
    slot: int              # request slot (row of the block tables, index of state slabs)
    start_pos: int         # position of tokens[0] in the request
    tokens: list           # token ids this step brings
    want: list = field(default_factory=list)   # indices into tokens whose logits are wanted


@dataclass
class StepContext:
    """Device-side view of one step, shared by every layer."""
    n_tokens: int
    ids: torch.Tensor          # [T] int32
    pos: torch.Tensor          # [T] int32
    slot: torch.Tensor         # [T] int32
    want_rows: torch.Tensor    # [R] int32 rows of the flattened batch
    n_want: int
    max_kv_len: int            # largest (position + 1) in the step, host value
    status: torch.Tensor       # [1] int32, set non-zero by a kernel that met a missing page
    entries: list              # the host-side StepEntry list
    entry_start: list          # first flattened row of each entry (host)
    # Rows of long portions, cut into tiles of up to 128 consecutive rows of one request
    # ([n, 4] int32: first row, rows, slot, position of the first row), for the tensor-core
    # attention; and the rows that are not in any tile (decoded tokens, short portions).
    tiles: torch.Tensor = None
    n_tiles: int = 0
    other_rows: torch.Tensor = None
    n_other_rows: int = 0
    attention_splits: tuple | None = None
    record: dict | None = None  # filled by parts when a test asks for internals


class StepStaging:
    """Pinned host memory and device memory for the packed metadata of a step."""

    def __init__(self, max_tokens: int, device):
        self.max_tokens = int(max_tokens)
        self.device = torch.device(device)
        self.max_tiles = self.max_tokens // 8 + 16
        n = 5 * self.max_tokens + 4 * self.max_tiles
        self.host = torch.zeros(n, dtype=torch.int32)
        if self.device.type == "cuda":
            self.host = self.host.pin_memory()
        self.dev = torch.zeros(n, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._copied = torch.cuda.Event() if self.device.type == "cuda" else None
        self._in_flight = False

    def pack(self, entries, vocab_size: int, max_positions: int, padded_tokens: int | None = None) -> StepContext:
        """Flatten, validate and upload.  ``padded_tokens`` fixes the device-side row
        count (for a captured graph of a given size)."""
        T = sum(len(e.tokens) for e in entries)
        if T == 0:
            raise ModelError("a step needs at least one token")
        if T > self.max_tokens:
            raise ModelError(f"step of {T} tokens exceeds the limit of {self.max_tokens}")
        ids, pos, slot, want, starts, tiles, others = [], [], [], [], [], [], []
        seen = set()
        max_kv = 0
        for e in entries:
            if e.slot in seen:
                raise ModelError(f"request slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise ModelError("an entry needs at least one token")
            if e.start_pos < 0 or e.start_pos + n > max_positions:
                raise ModelError(f"positions {e.start_pos}..{e.start_pos + n - 1} exceed the model's "
                                 f"{max_positions} positions")
            base = len(ids)
            starts.append(base)
            for t in e.tokens:
                if not 0 <= int(t) < vocab_size:
                    raise ModelError(f"token id {t} is outside the vocabulary of {vocab_size}")
            ids.extend(int(t) for t in e.tokens)
            pos.extend(range(e.start_pos, e.start_pos + n))
            slot.extend([e.slot] * n)
            for w in e.want:
                if not 0 <= w < n:
                    raise ModelError(f"wanted place {w} is outside the entry's {n} tokens")
                want.append(base + w)
            if n >= TILE_MIN_ROWS:
                for r in range(0, n, TILE_ROWS):
                    tiles += [base + r, min(TILE_ROWS, n - r), e.slot, e.start_pos + r]
            else:
                others.extend(range(base, base + n))
            max_kv = max(max_kv, e.start_pos + n)
        R = len(want)
        M = self.max_tokens
        h = self.host
        if self._in_flight:          # the last upload must have left the pinned buffer
            self._copied.synchronize()
        h[0:T] = torch.tensor(ids, dtype=torch.int32)
        h[M:M + T] = torch.tensor(pos, dtype=torch.int32)
        h[2 * M:2 * M + T] = torch.tensor(slot, dtype=torch.int32)
        if R:
            h[3 * M:3 * M + R] = torch.tensor(want, dtype=torch.int32)
        if others:
            h[4 * M:4 * M + len(others)] = torch.tensor(others, dtype=torch.int32)
        if tiles:
            h[5 * M:5 * M + len(tiles)] = torch.tensor(tiles, dtype=torch.int32)
        self.dev.copy_(h, non_blocking=True)
        if self._copied is not None:
            self._copied.record()
            self._in_flight = True
        d = self.dev
        return StepContext(n_tokens=T, ids=d[0:T], pos=d[M:M + T], slot=d[2 * M:2 * M + T],
                           want_rows=d[3 * M:3 * M + R], n_want=R, max_kv_len=max_kv, status=self.status,
                           entries=list(entries), entry_start=starts,
                           tiles=d[5 * M:5 * M + len(tiles)].view(-1, 4), n_tiles=len(tiles) // 4,
                           other_rows=d[4 * M:4 * M + len(others)], n_other_rows=len(others))
