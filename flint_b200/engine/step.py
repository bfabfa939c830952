"""One step's batch and the metadata the kernels read.

A batch is a list of entries, one per request: the request's slot, the position of
the first token it brings, the tokens, and the places among them whose logits are
wanted.  Entries may be portions of prompts and single decoded tokens side by side,
cut anywhere.  The reference's batch is the same thing
(``SeqChunk{tokens, seq, logit_rows}``, crates/thuban_model/src/traits.rs:12-17) with the
position kept inside the model; here the caller passes it, so that the step function
holds no per-request state and the replay tool can drive it directly.

The flattened metadata is packed (by the native runtime, ``csrc/host/runtime.cpp``) into
one pinned int32 buffer and copied to the device with a single copy: token ids, positions,
slots, and the rows whose logits are wanted (the reference uploads 8 words per row:
crates/thuban_model/src/rows.rs:7-30).
"""
from __future__ import annotations

from ctypes import c_int
from dataclasses import dataclass, field

import torch

from ..csrc import runtime as rt
from ..errors import ModelError


@dataclass(frozen=True)
class StepNeeds:
    """What a mixer asks of the step's metadata beyond ids, positions and slots: the rows of portions of at least
    ``tile_min_rows`` tokens cut into tiles of up to ``tile_rows`` consecutive rows of one request, and the list
    of the rows that are in no tile.  A mixer declares it (``Mixer.step_needs``); the step carries one tiling per
    distinct declaration (``StepContext.tiling``)."""
    tile_rows: int
    tile_min_rows: int


@dataclass
class Tiling:
    """Rows of long portions as tiles ([n, 4] int32: first row, rows, slot, position of the first row), in the
    order of their last position (a kernel whose work grows with the keys a tile sees starts from the far end),
    and the rows that are in no tile (decoded tokens, short portions)."""
    tiles: torch.Tensor
    n_tiles: int
    other_rows: torch.Tensor
    n_other_rows: int


@dataclass
class StepEntry:
    slot: int              # request slot (row of the block tables, index of state slabs)
    start_pos: int         # position of tokens[0] in the request
    tokens: list           # token ids this step brings
    want: list = field(default_factory=list)   # indices into tokens whose logits are wanted
    feed: int = -1         # >= 0: tokens[0] is not known on the host yet; it is this place of the sampler's last output


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
    longest_entry: int         # most tokens any one request brings in this step, host value
    status: torch.Tensor       # [1] int32, set non-zero by a kernel that met a missing page
    entries: list              # the host-side StepEntry list
    entry_start: list          # first flattened row of each entry (host)
    tilings: dict = field(default_factory=dict)   # StepNeeds -> Tiling, one per distinct declaration of the mixers
    attention_splits: tuple | None = None
    fed_rows: torch.Tensor = None  # [T] int32: the place in the sampler's last output that holds a row's token, or -1
    n_fed: int = 0
    even_lengths: bool = False  # a decode batch whose requests are about equally long (set by the caller)
    record: dict | None = None  # filled by parts when a test asks for internals
    plans: dict = field(default_factory=dict)     # what mixers worked out for this step (Mixer.plan_step), by kind

    def tiling(self, needs: StepNeeds) -> Tiling:
        try:
            return self.tilings[needs]
        except KeyError:
            raise ModelError(f"this step carries no tiling for {needs}: the mixer did not declare it (step_needs)") from None


class StepStaging:
    """Pinned host memory and device memory for the packed metadata of a step."""

    def __init__(self, max_tokens: int, device, status=None, needs=()):
        """``needs``: the distinct ``StepNeeds`` of the model's mixers.  The first is packed by the native runtime
        with the rest of the metadata; any further one is cut here and uploaded beside it."""
        self.max_tokens = int(max_tokens)
        self.device = torch.device(device)
        self.needs = tuple(dict.fromkeys(needs))
        smallest = min((n.tile_min_rows for n in self.needs), default=8)
        self.max_tiles = self.max_tokens // max(smallest, 1) + 16
        self._extra = None          # pinned and device buffers of the further tilings, made at first use
        n = 6 * self.max_tokens + 4 * self.max_tiles
        self.host = torch.zeros(n, dtype=torch.int32)
        if self.device.type == "cuda":
            self.host = self.host.pin_memory()
        self.dev = torch.zeros(n, dtype=torch.int32, device=self.device)
        # set non-zero by a kernel that met a position without a page (the caller may pass a flag of its own)
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=self.device)
        self._copied = torch.cuda.Event() if self.device.type == "cuda" else None
        self._in_flight = False
        self._lib = rt.lib()

    def pack(self, entries, vocab_size: int, max_positions: int) -> StepContext:
        """Flatten, validate and upload."""
        n_entries = len(entries)
        if n_entries == 0:
            raise ModelError("a step needs at least one token")
        tokens, want = [], []
        for e in entries:
            tokens.extend(e.tokens)
            want.extend(e.want)
        try:
            tok_arr, want_arr = rt.ints([int(t) for t in tokens]), rt.ints([int(w) for w in want])
        except (TypeError, ValueError, OverflowError) as err:
            raise ModelError(f"token ids and wanted places must be integers: {err}") from None
        starts = (c_int * n_entries)()
        meta = (c_int * 6)()
        M = self.max_tokens
        if self._in_flight:          # the last upload must have left the pinned buffer
            self._copied.synchronize()
        # flattening, validation and the tiles of long portions are done by the native runtime,
        # straight into the pinned buffer
        rt.checked(self._lib.flint_rt_pack_step(
            n_entries, rt.ints([e.slot for e in entries]), rt.ints([e.start_pos for e in entries]),
            rt.ints([len(e.tokens) for e in entries]), rt.ints([len(e.want) for e in entries]), tok_arr, want_arr,
            rt.ints([e.feed for e in entries]), int(vocab_size), int(max_positions), M, self.max_tiles,
            self.needs[0].tile_rows if self.needs else 1 << 30, self.needs[0].tile_min_rows if self.needs else 1 << 30,
            4096, self.host.data_ptr(), starts, meta))
        T, R, n_tiles, n_others, max_kv, n_fed = meta
        starts = list(starts)
        self.dev.copy_(self.host, non_blocking=True)
        if self._copied is not None:
            self._copied.record()
            self._in_flight = True
        d = self.dev
        tilings = {}
        if self.needs:
            tilings[self.needs[0]] = Tiling(d[5 * M:5 * M + 4 * n_tiles].view(-1, 4), n_tiles, d[4 * M:4 * M + n_others], n_others)
        for k, needs in enumerate(self.needs[1:]):
            tilings[needs] = self._cut(entries, starts, needs, k)
        return StepContext(n_tokens=T, ids=d[0:T], pos=d[M:M + T], slot=d[2 * M:2 * M + T],
                           want_rows=d[3 * M:3 * M + R], n_want=R, max_kv_len=max_kv,
                           longest_entry=max(len(e.tokens) for e in entries), status=self.status,
                           entries=list(entries), entry_start=starts, tilings=tilings,
                           fed_rows=d[5 * M + 4 * self.max_tiles:5 * M + 4 * self.max_tiles + T], n_fed=n_fed)

    def _cut(self, entries, starts, needs: StepNeeds, k: int) -> Tiling:
        """A further tiling (a model whose mixers declare different needs), cut on the host and uploaded with a
        copy of its own."""
        M, per = self.max_tokens, self.max_tokens + 4 * self.max_tiles
        if self._extra is None:
            n = per * (len(self.needs) - 1)
            host = torch.zeros(n, dtype=torch.int32)
            self._extra = (host.pin_memory() if self.device.type == "cuda" else host,
                           torch.zeros(n, dtype=torch.int32, device=self.device))
            self._extra_copied = torch.cuda.Event() if self.device.type == "cuda" else None
        host, dev = self._extra
        if k == 0 and self._extra_copied is not None and self._in_flight:
            self._extra_copied.synchronize()
        tiles, others = [], []
        for e, row0 in zip(entries, starts):
            n = len(e.tokens)
            if n < needs.tile_min_rows:
                others += range(row0, row0 + n)
                continue
            for r in range(0, n, needs.tile_rows):
                tiles += (row0 + r, min(needs.tile_rows, n - r), e.slot, e.start_pos + r)
        if len(tiles) // 4 > self.max_tiles:
            raise ModelError("a step has more tiles than its staging buffer holds")
        quads = sorted((tiles[i:i + 4] for i in range(0, len(tiles), 4)), key=lambda t: t[3] + t[1])
        tiles = [v for t in quads for v in t]
        o = per * k
        host[o:o + len(others)] = torch.tensor(others, dtype=torch.int32)
        host[o + M:o + M + len(tiles)] = torch.tensor(tiles, dtype=torch.int32)
        dev[o:o + per].copy_(host[o:o + per], non_blocking=True)
        if self._extra_copied is not None and k == len(self.needs) - 2:
            self._extra_copied.record()
        return Tiling(dev[o + M:o + M + len(tiles)].view(-1, 4), len(tiles) // 4, dev[o:o + len(others)], len(others))
