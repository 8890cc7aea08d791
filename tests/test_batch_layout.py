"""The step's index buffer (no GPU needed): the order of the attention tiles and the context lengths that the
choice of key splits is given."""

import torch

from ampere_kv_engine_b200.cache.manager import CacheManager
from ampere_kv_engine_b200.engine.batch import SeqStep, build_context
from ampere_kv_engine_b200.parts.base import CacheSpec


def _manager():
    return CacheManager([CacheSpec("full", 2, 16)], [None], page_size=4, num_pages=200, max_seqs=8,
                        dtype=torch.float32, allocate_storage=False)


def _held(manager, name, length):
    seq = manager.open(name)
    if length:
        manager.reserve(seq, length)
        manager.commit(seq, length)
    return seq


def test_single_token_tiles_come_first_and_longest_first():
    manager = _manager()
    lengths = {"a": 30, "b": 0, "c": 90, "d": 7, "e": 55}
    seqs = {name: _held(manager, name, n) for name, n in lengths.items()}
    entries = [SeqStep(seqs["a"], [1], [0]), SeqStep(seqs["b"], list(range(21)), []), SeqStep(seqs["c"], [2], [0]),
               SeqStep(seqs["d"], [3, 4, 5], [2]), SeqStep(seqs["e"], [6], [0])]
    for e in entries:
        manager.reserve(e.seq, len(e.tokens))
    ctx = build_context(manager, entries, torch.device("cpu"), q_tile=8)
    assert ctx.num_decode_tiles == 3
    order = ctx.tile_seq.tolist()
    # the single-token sequences by falling context (91, 56, 31), then the portions' tiles in batch order
    assert order[:3] == [2, 4, 0]
    assert order[3:] == [1, 1, 1, 3]
    assert ctx.tile_nq.tolist() == [1, 1, 1, 8, 8, 5, 3]
    cu = ctx.cu_q.tolist()
    assert ctx.tile_q0.tolist() == [cu[2], cu[4], cu[0], cu[1], cu[1] + 8, cu[1] + 16, cu[3]]
    assert ctx.max_context == 91
    assert ctx.decode_contexts == (91, (91 + 56 + 31) // 3)


def test_decode_contexts_of_a_step_without_single_tokens_fall_back_to_the_longest():
    manager = _manager()
    seq = _held(manager, "p", 10)
    entries = [SeqStep(seq, [1, 2, 3, 4, 5], [4])]
    manager.reserve(seq, 5)
    ctx = build_context(manager, entries, torch.device("cpu"), q_tile=8)
    assert ctx.num_decode_tiles == 0 and ctx.decode_contexts == (15, 15)
