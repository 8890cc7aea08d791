"""One step's batch: what each live request contributes, flattened for the kernels.

The reference builds three differently shaped batches (single request, ``[B, 1]`` decode, B
decode tokens plus exactly one prompt chunk: ampere_kv/runner.py:219-290) and rebuilds block
tables from Python lists in every layer (ampere_kv/paged_cache.py:76, runner.py:207-213).
Here a step is any list of (request, its next tokens): prompt portions of any length beside
single decoded tokens.  All index data of the step is laid out once on the host in one int32
buffer and copied to the device in one transfer; every layer reads the same tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheManager, SequenceCache
from ..kernels import ops


@dataclass
class SeqStep:
    """A request's share of one step: its next tokens and the places among them whose logits are wanted."""

    seq: SequenceCache
    tokens: list[int]
    want: list[int] = field(default_factory=list)
    #: set when the entry's single token is the one the previous step chose in its row ``source`` and the host
    #: has not read it yet: the embedding takes it from the device (``tokens`` is then a placeholder)
    source: int | None = None


@dataclass
class GroupBatch:
    """Per cache group: where each new token's K/V goes and each sequence's page table."""

    slot_mapping: torch.Tensor      # [tokens] int32: page * page_size + offset
    block_table: torch.Tensor       # [sequences, width] int32, -1 where no page is held
    width: int


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor         # [tokens] int32
    positions: torch.Tensor         # [tokens] int32, absolute
    cu_q: torch.Tensor              # [sequences + 1] int32: first batch row of each sequence
    ctx_lens: torch.Tensor          # [sequences] int32: sequence length once this step's tokens are in
    state_slots: torch.Tensor       # [sequences] int32
    logit_rows: torch.Tensor        # [wanted] int32 batch rows
    num_logit_rows: int
    tile_seq: torch.Tensor          # attention query tiles: sequence, first batch row, rows
    tile_q0: torch.Tensor
    tile_nq: torch.Tensor
    num_tiles: int
    q_tile: int                     # most rows any tile has
    #: in a step that holds decoded tokens beside prompt portions, the tiles of the single-token sequences come
    #: first and this is their count (0 in a step of one kind): attention runs them with key splits, apart from
    #: the prompt tiles
    num_decode_tiles: int
    max_context: int                # longest ctx_lens entry (host value)
    #: (longest, mean) context of the sequences that bring one token: what the choice of key splits for their
    #: attention assumes (a captured decode step: estimates for the steps it will serve)
    decode_contexts: tuple[int, int]
    groups: list[GroupBatch]
    status: torch.Tensor | None     # int32[1] the kernels report bad indices in
    sampled: torch.Tensor | None = None   # int32 tokens the previous step chose (for entries with a ``source``)
    # host copies, for parts that loop over sequences themselves
    q_lens_host: list[int] = field(default_factory=list)
    ctx_lens_host: list[int] = field(default_factory=list)
    state_slots_host: list[int] = field(default_factory=list)
    h2d_bytes: int = 0              # size of the one host-to-device copy that carried all of the above


def _align(n: int, to: int = 4) -> int:
    return (n + to - 1) // to * to


@dataclass
class BatchLayout:
    """Sizes of one step's index buffer.  Two steps with the same layout can share device memory, which is what
    lets a decode step be replayed as a CUDA graph."""

    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    num_tiles: int
    widths: tuple[int, ...]           # block-table width per cache group
    offsets: list[int] = field(default_factory=list)

    def __post_init__(self):
        sizes = [self.num_tokens, self.num_tokens, self.num_seqs + 1, self.num_seqs, self.num_seqs,
                 max(1, self.num_logit_rows), self.num_tiles, self.num_tiles, self.num_tiles]
        for w in self.widths:
            sizes += [self.num_tokens, self.num_seqs * w]
        self.offsets = [0]
        for size in sizes:
            self.offsets.append(self.offsets[-1] + _align(size))

    @property
    def total(self) -> int:
        return self.offsets[-1]

    def key(self) -> tuple:
        return (self.num_tokens, self.num_seqs, self.num_logit_rows, self.num_tiles, self.widths)


def fill_host(manager: CacheManager, entries: list[SeqStep], layout: BatchLayout, host: np.ndarray,
              tile_rows: int) -> tuple[list[int], list[int]]:
    """Write the step's index data into ``host`` (int32, ``layout.total`` long).  Sequences, tokens and tiles
    beyond the entries (a padded layout) are filled so that they do nothing: no cache slot, no tile rows.
    Returns (q_lens, ctx_lens) of the real entries."""
    q_lens = [len(e.tokens) for e in entries]
    starts = [e.seq.length for e in entries]
    ctx_lens = [s + n for s, n in zip(starts, q_lens)]
    num_seqs, num_tokens = len(entries), sum(q_lens)
    off = layout.offsets
    host[:] = -1
    cu = np.zeros(layout.num_seqs + 1, dtype=np.int64)
    np.cumsum(q_lens, out=cu[1:num_seqs + 1])
    # padded sequences own one padded token each
    cu[num_seqs + 1:] = num_tokens + np.arange(1, layout.num_seqs - num_seqs + 1)

    def put(index: int, values) -> None:
        host[off[index]:off[index] + len(values)] = values

    host[off[0]:off[0] + layout.num_tokens] = 0
    put(0, [-(e.source + 1) if e.source is not None else t for e in entries for t in e.tokens])
    host[off[1]:off[1] + layout.num_tokens] = 0
    put(1, np.concatenate([np.arange(s, c, dtype=np.int64) for s, c in zip(starts, ctx_lens)]))
    put(2, cu)
    host[off[3]:off[3] + layout.num_seqs] = 1
    put(3, ctx_lens)
    host[off[4]:off[4] + layout.num_seqs] = 0
    put(4, [e.seq.state_slot for e in entries])
    host[off[5]:off[5] + max(1, layout.num_logit_rows)] = 0
    put(5, [int(cu[s]) + w for s, e in enumerate(entries) for w in e.want])
    tiles = [(s, int(cu[s]) + q0, min(tile_rows, n - q0)) for s, n in enumerate(q_lens) for q0 in range(0, n, tile_rows)]
    # single-token sequences first, the longest context first among them (their CTAs start in this order, and the
    # step's attention ends with the last long one); prompt tiles after them in batch order
    tiles.sort(key=lambda t: (0, -ctx_lens[t[0]]) if q_lens[t[0]] == 1 else (1, 0))
    if len(tiles) > layout.num_tiles:
        raise ValueError("the layout has too few attention tiles for this step")
    host[off[6]:off[6] + layout.num_tiles] = 0
    host[off[7]:off[7] + layout.num_tiles] = 0
    host[off[8]:off[8] + layout.num_tiles] = 0       # a tile of no rows does nothing
    put(6, [t[0] for t in tiles])
    put(7, [t[1] for t in tiles])
    put(8, [t[2] for t in tiles])
    page = manager.page_size
    for gi, (group, width) in enumerate(zip(manager.groups, layout.widths)):
        slots = np.full(layout.num_tokens, -1, dtype=np.int64)
        table = np.full((layout.num_seqs, width), -1, dtype=np.int64)
        for s, e in enumerate(entries):
            row = np.asarray(manager.table_row(e.seq, group.index), dtype=np.int64)
            if len(row) > width:
                raise ValueError("the layout's block table is too narrow for this step")
            table[s, :len(row)] = row
            pos = np.arange(starts[s], ctx_lens[s], dtype=np.int64)
            pages = row[pos // page]
            if (pages < 0).any():
                raise ValueError(f"request {e.seq.request_id!r}: a new token falls in a page that is not held")
            slots[int(cu[s]):int(cu[s + 1])] = pages * page + pos % page
        put(9 + 2 * gi, slots)
        put(10 + 2 * gi, table.reshape(-1))
    return q_lens, ctx_lens


def make_context(layout: BatchLayout, dev: torch.Tensor, *, tile_rows: int, max_context: int,
                 status: torch.Tensor | None, q_lens: list[int], ctx_lens: list[int], state_slots: list[int],
                 h2d_bytes: int, sampled: torch.Tensor | None = None,
                 decode_contexts: tuple[int, int] | None = None) -> StepContext:
    """Views into the device copy ``dev`` of a filled index buffer."""
    off = layout.offsets

    def view(index: int, size: int) -> torch.Tensor:
        return dev[off[index]:off[index] + size]

    decoding = sum(1 for n in q_lens if n == 1)
    num_decode_tiles = decoding if 0 < decoding < len(q_lens) else 0
    if decode_contexts is None:
        single = [c for n, c in zip(q_lens, ctx_lens) if n == 1] or [max_context]
        decode_contexts = (max(single), sum(single) // len(single))
    groups = []
    for gi, width in enumerate(layout.widths):
        groups.append(GroupBatch(view(9 + 2 * gi, layout.num_tokens),
                                 view(10 + 2 * gi, layout.num_seqs * width).view(layout.num_seqs, width), width))
    return StepContext(
        num_tokens=layout.num_tokens, num_seqs=layout.num_seqs, token_ids=view(0, layout.num_tokens),
        positions=view(1, layout.num_tokens), cu_q=view(2, layout.num_seqs + 1), ctx_lens=view(3, layout.num_seqs),
        state_slots=view(4, layout.num_seqs), logit_rows=view(5, layout.num_logit_rows),
        num_logit_rows=layout.num_logit_rows, tile_seq=view(6, layout.num_tiles), tile_q0=view(7, layout.num_tiles),
        tile_nq=view(8, layout.num_tiles), num_tiles=layout.num_tiles, q_tile=tile_rows,
        num_decode_tiles=num_decode_tiles, max_context=max_context, decode_contexts=decode_contexts,
        groups=groups, status=status, sampled=sampled, q_lens_host=q_lens, ctx_lens_host=ctx_lens,
        state_slots_host=state_slots, h2d_bytes=h2d_bytes)


def validate_entries(entries: list[SeqStep]) -> None:
    if not entries:
        raise ValueError("a step needs at least one entry")
    for e in entries:
        if not e.tokens:
            raise ValueError("every entry of a step needs at least one token")
        if e.source is not None and (len(e.tokens) != 1 or e.source < 0):
            raise ValueError(f"request {e.seq.request_id!r}: a token taken from the previous step's choices is "
                             f"the entry's only token")
        for w in e.want:
            if not 0 <= w < len(e.tokens):
                raise ValueError(f"request {e.seq.request_id!r}: wanted place {w} is outside its "
                                 f"{len(e.tokens)} tokens")


def exact_layout(manager: CacheManager, entries: list[SeqStep], tile_rows: int) -> BatchLayout:
    q_lens = [len(e.tokens) for e in entries]
    widths = tuple(max(1, max(len(manager.table_row(e.seq, g.index)) for e in entries)) for g in manager.groups)
    return BatchLayout(sum(q_lens), len(entries), sum(len(e.want) for e in entries),
                       sum((n + tile_rows - 1) // tile_rows for n in q_lens), widths)


def build_context(manager: CacheManager, entries: list[SeqStep], device: torch.device,
                  status: torch.Tensor | None = None, q_tile: int | None = None,
                  sampled: torch.Tensor | None = None) -> StepContext:
    """Lay out the step exactly (no padding) and copy it to the device in one transfer.  Every entry's pages
    must already be reserved for its new tokens."""
    validate_entries(entries)
    q_tile = q_tile or ops.ATTENTION_Q_TILE
    tile_rows = 1 if max(len(e.tokens) for e in entries) == 1 else q_tile
    layout = exact_layout(manager, entries, tile_rows)
    host = np.empty(layout.total, dtype=np.int32)
    q_lens, ctx_lens = fill_host(manager, entries, layout, host, tile_rows)
    staged = torch.from_numpy(host)
    if device.type == "cuda":
        staged = staged.pin_memory()
    dev = staged.to(device, non_blocking=True)
    return make_context(layout, dev, tile_rows=tile_rows, max_context=max(ctx_lens), status=status, q_lens=q_lens,
                        ctx_lens=ctx_lens, state_slots=[e.seq.state_slot for e in entries], h2d_bytes=int(host.nbytes),
                        sampled=sampled)
