"""Prefill-first continuous batching (engine/scheduler.py:8-79, talker_llm_engine.py:11-83,
predictor_llm_engine.py:15-30 of the reference): waiting sequences are prefilled as one packed
batch, otherwise every running sequence decodes one token.  The talker variant only schedules
sequences whose next input embedding has been fed."""
from __future__ import annotations

from collections import deque

from ..config import Config
from .block_manager import BlockManager
from .sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config: Config):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.block_manager = BlockManager(config.num_kvcache_blocks, config.kvcache_block_size)
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()
        self.request_id_to_seq: dict[str, Sequence] = {}

    def is_finished(self):
        return not self.waiting and not self.running

    def add(self, seq: Sequence):
        self.waiting.append(seq)

    def _schedule_prefill(self) -> list[Sequence]:
        picked, tokens = [], 0
        while self.waiting and len(picked) < self.max_num_seqs:
            seq = self.waiting[0]
            if tokens + len(seq) > self.max_num_batched_tokens or not self.block_manager.can_allocate(seq):
                break
            self.block_manager.allocate(seq)
            tokens += len(seq) - seq.num_cached_tokens
            seq.status = SequenceStatus.RUNNING
            self.waiting.popleft()
            self.running.append(seq)
            picked.append(seq)
        return picked

    def _ready(self, seq: Sequence) -> bool:
        return True

    def _schedule_decode(self) -> list[Sequence]:
        # fast path (every steady-state decode step): all running sequences fit, all are ready and none opens a new
        # KV page this step, so the batch is the running queue in order and the queue is left as it is - exactly what
        # the general loop below produces, without its per-sequence pops and allocator calls
        n = len(self.running)
        if 0 < n <= self.max_num_seqs:
            bs, ready = self.block_manager.block_size, self._ready
            if all(s.num_tokens % bs != 1 and ready(s) for s in self.running):
                return list(self.running)
        picked = []
        for _ in range(len(self.running)):
            if not self.running or len(picked) >= self.max_num_seqs:
                break
            seq = self.running.popleft()
            if not self._ready(seq):
                self.running.append(seq)
                continue
            while not self.block_manager.can_append(seq):
                if self.running:
                    self.preempt(self.running.pop())
                else:
                    self.preempt(seq)
                    break
            else:
                self.block_manager.may_append(seq)
                picked.append(seq)
        self.running.extendleft(reversed(picked))
        return picked

    def schedule(self) -> tuple[list[Sequence], bool]:
        picked = self._schedule_prefill()
        if picked:
            return picked, True
        return self._schedule_decode(), False

    def preempt(self, seq: Sequence):
        """Drop the KV pages and queue the sequence for a full re-prefill (scheduler.py:68-71)."""
        seq.status = SequenceStatus.WAITING
        self.block_manager.deallocate(seq)
        self.waiting.appendleft(seq)

    def _finish(self, seq: Sequence):
        seq.status = SequenceStatus.FINISHED
        if seq.request_id is not None:
            self.request_id_to_seq.pop(seq.request_id, None)
        self.block_manager.deallocate(seq)
        self.running.remove(seq)

    def clear_request(self, request_id: str):
        seq = self.request_id_to_seq.pop(request_id, None)
        if seq is None:
            return
        if seq.block_table:
            self.block_manager.deallocate(seq)
        if seq in self.running:
            self.running.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)

    def postprocess(self, seqs: list[Sequence], token_ids: list[int]):
        for seq, tok in zip(seqs, token_ids):
            seq.append_token(tok, None)
            if (not seq.ignore_eos and tok == self.eos) or seq.num_completion_tokens >= seq.max_tokens:
                self._finish(seq)


class TalkerScheduler(Scheduler):
    def _ready(self, seq: Sequence) -> bool:
        return not (len(seq) > 0 and seq.decode_input_embeds is None)

    def postprocess(self, seqs, token_ids, hidden_states):
        rows = hidden_states.unbind(0)             # the row views in one call (indexing per sequence costs ~1.5 us each)
        for i, (seq, tok) in enumerate(zip(seqs, token_ids)):
            seq.append_token(tok, rows[i])
            seq.decode_input_embeds = None
            seq.batch_src = None
            hit_eos = not seq.ignore_eos and tok == self.eos
            # requests driven by the interface stop on the codec EOS there, not here
            # (talker_llm_engine.py:74-77)
            if hit_eos or (seq.request_id is None and seq.num_completion_tokens >= seq.max_tokens):
                self._finish(seq)


class PredictorScheduler(Scheduler):
    pass


class ChunkScheduler(Scheduler):
    """Continuous batching for token models whose prompts run in portions: one step carries the single pending token
    of every decoding sequence BESIDE portions of prompts, up to ``max_num_batched_tokens`` tokens.  ``schedule``
    returns ``[(sequence, tokens to run)]``; a sequence's block table grows as its portions are scheduled, and a
    sequence is admitted when a state slot and the pages of its first portion are free.  Nothing is preempted: a
    portion that does not fit is shortened, or waits for pages that finishing sequences give back."""

    def __init__(self, config: Config):
        super().__init__(config)
        from .block_manager import StateSlotPool
        self.state_slots = StateSlotPool(config.max_state_slots or config.max_num_seqs)

    def is_finished(self):
        return not self.waiting and not any(s.num_pending_tokens or not s.hold for s in self.running)

    def _fit(self, seq: Sequence, budget: int) -> int:
        n = min(seq.num_pending_tokens, budget)
        room = self.block_manager.tokens_available(seq) - seq.num_cached_tokens
        return max(0, min(n, room))

    def schedule(self) -> list[tuple[Sequence, int]]:
        picked, budget = [], self.max_num_batched_tokens
        # decoding sequences first, so that a long prompt never starves them of the token budget
        for decode_pass in (True, False):
            for seq in self.running:
                if (seq.num_pending_tokens == 1) != decode_pass or seq.num_pending_tokens == 0:
                    continue
                n = self._fit(seq, budget)
                if n > 0:
                    self.block_manager.extend(seq, seq.num_cached_tokens + n)
                    picked.append((seq, n))
                    budget -= n
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs and self.state_slots.available():
            seq = self.waiting[0]
            n = self._fit(seq, budget)
            if n <= 0 and seq.num_pending_tokens > 0:
                break
            self.waiting.popleft()
            seq.state_slot = self.state_slots.take()
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            if n > 0:
                self.block_manager.extend(seq, seq.num_cached_tokens + n)
                picked.append((seq, n))
                budget -= n
        order = {id(s): i for i, s in enumerate(self.running)}
        picked.sort(key=lambda it: order[id(it[0])])
        return picked

    def _release_state(self, seq: Sequence):
        if seq.state_slot >= 0:
            self.state_slots.give(seq.state_slot)
            seq.state_slot = -1

    def _finish(self, seq: Sequence):
        self._release_state(seq)
        super()._finish(seq)

    def clear_request(self, request_id: str):
        seq = self.request_id_to_seq.get(request_id)
        if seq is not None:
            self._release_state(seq)
            seq.status = SequenceStatus.FINISHED
        super().clear_request(request_id)

    def preempt(self, seq: Sequence):
        raise RuntimeError("ChunkScheduler never preempts")
