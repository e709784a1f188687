"""Host-side chunk accounting and slot lifecycle for vTensor KV ranges.

Mirrors what the reference's scheduler side does for the vTensor path, so that
the allocator can be driven by a real scheduler instead of a synthetic loop:

* ``SequenceChunks``  — the per-sequence logical accounting of
  ``Sequence._append_tokens_to_blocks`` (GLakeServe/vllm/sequence.py:342-360):
  bytes reserved in whole 2 MiB chunks, bytes still free in the last chunk, and
  the logical chunk count (K and V counted separately, hence the factor 2).
* ``ChunkSpaceManager`` — the vTensor methods of ``BlockSpaceManagerV1``
  (GLakeServe/vllm/core/block_manager_v1.py:198-318, :436-455, :581-601): slot
  table with pre-cached slots (``--cache-seqs`` / ``--cache-tokens``), admission
  against a watermark, per-step ``append_slots`` that emits the list of slots to
  extend (the ``extend_seq_list`` handed to the model), and ``free`` with
  release-to-watermark vs. preempt semantics.

All counts are per layer, exactly as in the reference, whose worker divides the
physical budget by the layer count (GLakeServe/vllm/worker/worker.py:170-175);
the allocator multiplies by ``2 * layers`` ranges when it maps.
``apply_allocate`` / ``apply_extend`` / ``apply_free`` connect a decision to the
allocator objects of :mod:`glake_b200.vmmAllocator` (``ensure_mapped`` /
``eagerExtend`` / ``release_seq`` / ``preempt_seq``).
"""
from dataclasses import dataclass
from enum import Enum
from typing import Dict, List, Optional

PHY_GRAN = 2 * 1024 * 1024       # bytes of a physical chunk; vmmAllocator.set_chunk_bytes keeps it in step
PREFILL_HEADROOM_TOKENS = 100   # sequence.py:343: a prompt reserves room for 100 more tokens


class AllocStatus(Enum):
    OK = 0
    LATER = 1
    NEVER = 2


@dataclass
class SequenceChunks:
    """Logical chunk accounting of one sequence (sequence.py:342-360)."""
    token_size: int                 # bytes of one token row of K (or V) in one layer
    headroom_tokens: int = PREFILL_HEADROOM_TOKENS
    reserve_size: int = 0           # bytes reserved, whole chunks
    free_size: int = 0              # bytes of the reservation not yet used
    logical_block_num: int = 0      # chunks the sequence needs (K + V)
    slot: int = -1
    preempted: bool = False

    def append_tokens(self, n_tokens: int) -> None:
        plus = 0 if n_tokens == 1 else self.headroom_tokens
        need = self.token_size * (n_tokens + plus)
        if self.reserve_size == 0:
            rounded = PHY_GRAN * ((need + PHY_GRAN - 1) // PHY_GRAN)
            self.reserve_size = rounded
            self.free_size = rounded - need
            self.logical_block_num = 2 * (rounded // PHY_GRAN)
        elif self.free_size >= need:
            self.free_size -= need
        else:
            gap = need - self.free_size
            rounded = PHY_GRAN * ((gap + PHY_GRAN - 1) // PHY_GRAN)
            self.reserve_size += rounded
            self.free_size = rounded - gap
            self.logical_block_num += 2 * (rounded // PHY_GRAN)


class ChunkSpaceManager:
    """Physical chunk budget and slot table (block_manager_v1.py vTensor paths)."""

    def __init__(self, max_seqs: int, num_gpu_handles: int, watermark: float = 0.01, cache_token: int = 0,
                 cache_seq: int = 0) -> None:
        assert watermark >= 0.0
        self.max_seqs = max_seqs
        self.num_total = num_gpu_handles
        self.watermark_blocks = int(watermark * num_gpu_handles)
        self.cache_token, self.cache_seq = cache_token, cache_seq
        self.kv_cache_slot = [0] * max_seqs                       # 1 = occupied
        # physical chunks (K + V) currently held per slot
        self.block_tables: Dict[int, int] = {i: (cache_token * 2 if i < cache_seq else 0) for i in range(max_seqs)}
        self.num_free = num_gpu_handles - cache_seq * cache_token * 2
        if self.num_free < 0:
            raise ValueError("pre-cached slots exceed the chunk budget")
        self.free_block_tables_block = cache_seq * cache_token * 2  # chunks parked in idle pre-cached slots

    # -- slots ---------------------------------------------------------
    def get_free_slot(self) -> int:
        for i in range(self.max_seqs):
            if self.kv_cache_slot[i] == 0:
                self.kv_cache_slot[i] = 1
                return i
        return -1

    def get_cached_slot(self) -> int:
        for i in range(self.max_seqs):
            if self.kv_cache_slot[i] == 0 and self.cache_token and self.block_tables[i] == self.cache_token * 2:
                self.kv_cache_slot[i] = 1
                self.free_block_tables_block -= self.cache_token * 2
                return i
        return -1

    # -- admission -----------------------------------------------------
    def can_allocate(self, seq: SequenceChunks, preempted_flag: bool = False) -> AllocStatus:
        required = seq.logical_block_num + (2 if preempted_flag else 0)
        minus = self.cache_token * 2 if self.free_block_tables_block > 0 else 0
        free = self.num_free + minus
        if self.num_total - required < self.watermark_blocks:
            return AllocStatus.NEVER
        return AllocStatus.OK if free - required >= self.watermark_blocks else AllocStatus.LATER

    def allocate(self, seq: SequenceChunks) -> bool:
        slot = self.get_cached_slot()
        if slot == -1:
            slot = self.get_free_slot()
            if slot == -1:
                return False
        held = self.block_tables[slot]
        seq.slot = slot
        need = seq.logical_block_num - held
        if need > 0:
            if need > self.num_free:
                self.kv_cache_slot[slot] = 0
                if held == self.cache_token * 2 and self.cache_token:
                    self.free_block_tables_block += held
                seq.slot = -1
                return False
            self.num_free -= need
            self.block_tables[slot] += need
        return True

    # -- per decode step -----------------------------------------------
    def append_slots(self, seq: SequenceChunks, extend_seq_list: List[int]) -> bool:
        """After ``seq.append_tokens(1)``: if the sequence now needs more chunks
        than its slot holds, book one more K and one more V chunk and put the slot
        on the extend list (block_manager_v1.py:436-455).  False = budget exhausted
        (the caller preempts somebody)."""
        if self.block_tables[seq.slot] < seq.logical_block_num:
            assert seq.slot != -1
            if self.num_free < 2:
                return False
            extend_seq_list.append(seq.slot)
            self.num_free -= 2
            self.block_tables[seq.slot] += 2
        return True

    # -- end of life ---------------------------------------------------
    def free(self, seq: SequenceChunks) -> int:
        """Finished sequence: keep the pre-cached prefix of the slot if it holds at
        least that much; preempted sequence: give everything back
        (block_manager_v1.py:581-601).  Returns the slot."""
        slot = seq.slot
        if slot == -1:
            return -1
        self.kv_cache_slot[slot] = 0
        held = self.block_tables[slot]
        if not seq.preempted:
            keep = 2 * self.cache_token if held >= 2 * self.cache_token else 0
            self.num_free += held - keep
            if keep and keep == 2 * self.cache_token:
                self.free_block_tables_block += keep
            self.block_tables[slot] = keep
        else:
            self.num_free += held
            self.block_tables[slot] = 0
        seq.slot = -1
        return slot

    def sum_all_blocks(self) -> int:
        return sum(self.block_tables.values()) + self.num_free

    def free_blocks(self) -> int:
        return self.num_free


def apply_allocate(seq: SequenceChunks, segment) -> None:
    """Admission: map the sequence's whole logical reservation — the prompt plus the
    headroom of ``PREFILL_HEADROOM_TOKENS`` rows — synchronously (the reference's prefill
    growth maps ``used + tokens + 100 tokens``, vmm_allocator.cpp:322-337).  From then on
    the logical accounting runs that many rows ahead of the fill position, so
    ``append_slots`` lists a slot for background growth about 100 decode steps before
    the kernels reach the new chunk: the 2 x layers driver calls of a growth (tens of
    milliseconds for a deep model) never sit on a step's critical path."""
    segment.ensure_mapped(seq.reserve_size)


def apply_extend(extend_seq_list: List[int], segments, token_bytes: int) -> None:
    """Hand the step's extend list to the allocator: one background growth per
    listed slot (the loop of llama.py:331-337)."""
    for slot in extend_seq_list:
        if slot != -1:
            segments[slot].eagerExtend(token_bytes, slot)


def apply_free(seq_slot: int, preempted: bool, segments) -> None:
    """worker.release_seq / preempt_seq (GLakeServe/vllm/worker/worker.py:227-241)."""
    if seq_slot < 0:
        return
    if preempted:
        segments[seq_slot].preempt_seq(seq_slot)
    else:
        segments[seq_slot].release_seq(seq_slot)
