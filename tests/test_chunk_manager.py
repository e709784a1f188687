"""Host chunk accounting (the scheduler side of the vTensor path) and its
agreement with the allocator, on the mock driver."""
import random

import pytest

from glake_b200 import chunk_manager as cm
from glake_b200._lib import lib

MiB = 1 << 20
CH = 2 * MiB


def test_sequence_accounting_follows_the_reference_arithmetic():
    """sequence.py:342-360 by hand: 8 KiB rows (32 kv heads x 128 x bf16), 256 rows per chunk."""
    s = cm.SequenceChunks(token_size=8192)
    s.append_tokens(300)                       # prompt: (300 + 100) rows = 3.125 MiB -> 2 chunks of K, 2 of V
    assert (s.reserve_size, s.logical_block_num) == (2 * CH, 4)
    assert s.free_size == 2 * CH - 400 * 8192
    for _ in range(112):                       # 512 - 400 rows fit
        s.append_tokens(1)
    assert s.free_size == 0 and s.logical_block_num == 4
    s.append_tokens(1)                         # row 513 opens a new chunk pair
    assert (s.reserve_size, s.logical_block_num, s.free_size) == (3 * CH, 6, CH - 8192)
    t = cm.SequenceChunks(token_size=8192, headroom_tokens=0)
    t.append_tokens(256)
    assert t.logical_block_num == 2 and t.free_size == 0


def test_admission_watermark_and_cached_slots():
    m = cm.ChunkSpaceManager(max_seqs=4, num_gpu_handles=100, watermark=0.1, cache_token=2, cache_seq=2)
    assert m.free_blocks() == 100 - 2 * 2 * 2 and m.sum_all_blocks() == 100
    big = cm.SequenceChunks(8192)
    big.append_tokens(256 * 46)                # (11776 + 100) rows -> 47 chunks x 2 = 94 > 100 - 10
    assert m.can_allocate(big) == cm.AllocStatus.NEVER
    a = cm.SequenceChunks(8192)
    a.append_tokens(700)                       # 800 rows -> 4 chunks -> 8
    assert m.can_allocate(a) == cm.AllocStatus.OK
    assert m.allocate(a) and a.slot == 0       # takes a pre-cached slot, pays only the difference
    assert m.block_tables[0] == 8 and m.free_blocks() == 92 - 4
    b = cm.SequenceChunks(8192)
    b.append_tokens(10000)                     # 10100 rows -> 40 chunks -> 80
    assert m.can_allocate(b) == cm.AllocStatus.OK and m.allocate(b) and b.slot == 1
    c = cm.SequenceChunks(8192)
    c.append_tokens(2000)                      # 2100 rows -> 9 -> 18 ; free is 12
    assert m.can_allocate(c) == cm.AllocStatus.LATER
    assert m.free(a) == 0 and m.block_tables[0] == 4 and m.free_block_tables_block == 4   # keeps its cached prefix
    b.preempted = True
    assert m.free(b) == 1 and m.block_tables[1] == 0
    assert m.sum_all_blocks() == 100
    assert m.can_allocate(c) == cm.AllocStatus.OK and m.allocate(c) and c.slot == 0


@pytest.mark.parametrize("chunk_mib", [2, 8])
def test_manager_drives_the_allocator_consistently(chunk_mib):
    """A random serving trace: the manager books chunks, the allocator maps them.
    At every step the allocator holds no more than the manager booked, nothing
    the kernels need is unmapped, and budgets are conserved.  Also with 8 MiB
    chunks (vmmAllocator.set_chunk_bytes): a growth costs the driver the same per
    chunk whatever its size, so larger chunks are a tuning the accounting must follow."""
    from glake_b200 import vmmAllocator as A
    A.set_chunk_bytes(chunk_mib * MiB)
    CH = A.granularitySize
    assert cm.PHY_GRAN == CH
    layers, kvh, max_seqs = 3, 8, 6
    row = kvh * 128 * 2                         # 2 KiB -> 1024 rows per chunk
    handles = 60                                # per layer
    lib.vt_use_mock_driver(1)
    rng = random.Random(4)
    try:
        assert A.init_physical_handle(handles * layers, 0)
        segs = [A.KVcacheSegment(layers, 64 * MiB, 0, False) for _ in range(max_seqs)]
        m = cm.ChunkSpaceManager(max_seqs, handles, watermark=0.0)
        live = {}
        for step in range(400):
            # admit
            if len(live) < max_seqs and rng.random() < 0.3:
                s = cm.SequenceChunks(row)
                n = rng.randint(1, 3000)
                s.append_tokens(n)
                if m.can_allocate(s) == cm.AllocStatus.OK and m.allocate(s):
                    cm.apply_allocate(s, segs[s.slot])          # prompt + headroom mapped at admission
                    assert segs[s.slot].actual_size == s.reserve_size
                    off = A.extend_kv_cache_batch(None, None, [s.slot], [n * row], [segs[s.slot]], [0], row, False)
                    assert off == [0]
                    live[s.slot] = [s, n]
            # decode step for everybody
            extend, order = [], list(live)
            victims = []
            for slot in order:
                s, n = live[slot]
                s.append_tokens(1)
                if not m.append_slots(s, extend):
                    victims.append(slot)
            for slot in victims:                 # budget exhausted: preempt
                s, _ = live.pop(slot)
                s.preempted = True
                cm.apply_free(m.free(s), True, segs)
            cm.apply_extend([x for x in extend if x in live], segs, row)
            order = list(live)
            if order:
                offs = A.extend_kv_cache_batch(None, None, order, [row] * len(order), [segs[x] for x in order],
                                               [0] * len(order), row, True)
                for slot, o in zip(order, offs):
                    assert o == live[slot][1] * row
                    live[slot][1] += 1
            # finish
            for slot in list(live):
                if rng.random() < 0.01:
                    s, _ = live.pop(slot)
                    cm.apply_free(m.free(s), False, segs)
            # invariants
            A.wait_ready(list(range(max_seqs)))
            for slot in range(max_seqs):
                seg = segs[slot]
                seg.wait()
                held = 2 * (seg.actual_size // CH)            # K + V chunks per layer
                assert held <= m.block_tables[slot], (step, slot, held, m.block_tables[slot])
                if slot in live:
                    assert seg.actual_size >= live[slot][1] * row
            assert m.sum_all_blocks() == handles
            assert A.showFreeBlocks() == handles * layers - sum(2 * layers * (s.actual_size // CH) for s in segs)
        for s in segs:
            s.close()
    finally:
        A.shutdown()
        lib.vt_use_mock_driver(0)
        A.set_chunk_bytes(2 * MiB)
