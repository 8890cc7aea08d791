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
    max_context: int                # longest ctx_lens entry (host value)
    groups: list[GroupBatch]
    status: torch.Tensor | None     # int32[1] the kernels report bad indices in
    # host copies, for parts that loop over sequences themselves
    q_lens_host: list[int] = field(default_factory=list)
    ctx_lens_host: list[int] = field(default_factory=list)
    state_slots_host: list[int] = field(default_factory=list)
    h2d_bytes: int = 0              # size of the one host-to-device copy that carried all of the above


def _align(n: int, to: int = 4) -> int:
    return (n + to - 1) // to * to


def build_context(manager: CacheManager, entries: list[SeqStep], device: torch.device,
                  status: torch.Tensor | None = None, q_tile: int | None = None) -> StepContext:
    """Lay out the step.  Every entry's pages must already be reserved for its new tokens."""
    if not entries:
        raise ValueError("a step needs at least one entry")
    q_tile = q_tile or ops.ATTENTION_Q_TILE
    q_lens = [len(e.tokens) for e in entries]
    if min(q_lens) <= 0:
        raise ValueError("every entry of a step needs at least one token")
    num_seqs, num_tokens = len(entries), sum(q_lens)
    starts = [e.seq.length for e in entries]
    ctx_lens = [s + n for s, n in zip(starts, q_lens)]
    cu = np.zeros(num_seqs + 1, dtype=np.int64)
    np.cumsum(q_lens, out=cu[1:])
    tile_rows = 1 if max(q_lens) == 1 else q_tile
    tiles: list[tuple[int, int, int]] = []
    for s, n in enumerate(q_lens):
        for q0 in range(0, n, tile_rows):
            tiles.append((s, int(cu[s]) + q0, min(tile_rows, n - q0)))
    logit_rows = [int(cu[s]) + w for s, e in enumerate(entries) for w in e.want]
    for s, e in enumerate(entries):
        for w in e.want:
            if not 0 <= w < q_lens[s]:
                raise ValueError(f"request {e.seq.request_id!r}: wanted place {w} is outside its {q_lens[s]} tokens")
    widths = [max(1, max(len(manager.table_row(e.seq, g.index)) for e in entries)) for g in manager.groups]

    # one int32 buffer: [ids | positions | cu_q | ctx_lens | state_slots | logit_rows | tile_seq | tile_q0 |
    #                    tile_nq | per group: slot_mapping, block_table]
    sizes = [num_tokens, num_tokens, num_seqs + 1, num_seqs, num_seqs, max(1, len(logit_rows)),
             len(tiles), len(tiles), len(tiles)]
    for w in widths:
        sizes += [num_tokens, num_seqs * w]
    offsets = [0]
    for size in sizes:
        offsets.append(offsets[-1] + _align(size))
    host = np.full(offsets[-1], -1, dtype=np.int32)

    def put(index: int, values) -> None:
        host[offsets[index]:offsets[index] + len(values)] = values

    put(0, [t for e in entries for t in e.tokens])
    put(1, np.concatenate([np.arange(s, c, dtype=np.int64) for s, c in zip(starts, ctx_lens)]))
    put(2, cu)
    put(3, ctx_lens)
    put(4, [e.seq.state_slot for e in entries])
    put(5, logit_rows if logit_rows else [0])
    put(6, [t[0] for t in tiles])
    put(7, [t[1] for t in tiles])
    put(8, [t[2] for t in tiles])
    page = manager.page_size
    for gi, (group, width) in enumerate(zip(manager.groups, widths)):
        slots = np.empty(num_tokens, dtype=np.int64)
        table = np.full((num_seqs, width), -1, dtype=np.int64)
        for s, e in enumerate(entries):
            row = np.asarray(manager.table_row(e.seq, group.index), dtype=np.int64)
            table[s, :len(row)] = row
            pos = np.arange(starts[s], ctx_lens[s], dtype=np.int64)
            pages = row[pos // page]
            if (pages < 0).any():
                raise ValueError(f"request {e.seq.request_id!r}: a new token falls in a page that is not held")
            slots[int(cu[s]):int(cu[s + 1])] = pages * page + pos % page
        put(9 + 2 * gi, slots)
        put(10 + 2 * gi, table.reshape(-1))

    staged = torch.from_numpy(host)
    if device.type == "cuda":
        staged = staged.pin_memory()
    dev = staged.to(device, non_blocking=True)

    def view(index: int, size: int) -> torch.Tensor:
        return dev[offsets[index]:offsets[index] + size]

    groups = []
    for gi, width in enumerate(widths):
        groups.append(GroupBatch(view(9 + 2 * gi, num_tokens),
                                 view(10 + 2 * gi, num_seqs * width).view(num_seqs, width), width))
    return StepContext(
        num_tokens=num_tokens, num_seqs=num_seqs, token_ids=view(0, num_tokens), positions=view(1, num_tokens),
        cu_q=view(2, num_seqs + 1), ctx_lens=view(3, num_seqs), state_slots=view(4, num_seqs),
        logit_rows=view(5, len(logit_rows)), num_logit_rows=len(logit_rows),
        tile_seq=view(6, len(tiles)), tile_q0=view(7, len(tiles)), tile_nq=view(8, len(tiles)),
        num_tiles=len(tiles), q_tile=tile_rows, max_context=max(ctx_lens), groups=groups, status=status,
        q_lens_host=q_lens, ctx_lens_host=ctx_lens, state_slots_host=[e.seq.state_slot for e in entries],
        h2d_bytes=int(host.nbytes))
