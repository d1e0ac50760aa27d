"""``CausalLMEngine``: the step API of token-id language models.

    add_request(token_ids, sampling_params, request_id)      a prompt to complete: sampled tokens are appended
    add_request(token_ids, request_id=..., hold=True)        a sequence whose tokens the caller feeds (replay of a
    feed(request_id, token_ids)                              recorded schedule, teacher forcing): nothing is sampled
    step(want=None) -> StepOutput                            ONE batch of everything pending: prompt portions beside
                                                             single decoded tokens, cut by the scheduler's token budget
    clear_request(request_id)                                gives pages and state slot back
    generate(prompts, sampling_params) -> completions

``want`` asks for logits: {request_id: [offsets into the tokens that request runs THIS step]}.  Sampling uses the
package's one sampler kernel; ``top_k=1`` is greedy."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ...sampling_params import SamplingParams
from ..model_runner.lm_model_runner import LMModelRunner
from ..scheduler import ChunkScheduler
from ..sequence import Sequence
from .base import LLMEngine


@dataclass
class StepOutput:
    logits: torch.Tensor | None = None                  # [wanted rows, vocab] float, in the order of ``want``
    scheduled: dict = field(default_factory=dict)       # request/sequence id -> tokens run this step
    finished: list = field(default_factory=list)        # (request_id, seq_id, completion_token_ids)
    num_tokens: int = 0


class CausalLMEngine(LLMEngine):
    runner_cls = LMModelRunner
    scheduler_cls = ChunkScheduler

    def add_request(self, token_ids: list[int], sampling_params: SamplingParams | None = None,
                    request_id: str | None = None, hold: bool = False) -> Sequence:
        if request_id is not None and request_id in self.scheduler.request_id_to_seq:
            raise ValueError(f"request {request_id!r} is live")
        seq = Sequence(list(token_ids), sampling_params or SamplingParams(), request_id=request_id)
        if not token_ids:
            seq.num_tokens = seq.num_prompt_tokens = 0
        seq.hold = hold
        if len(seq) > self.config.max_model_len:
            raise ValueError(f"prompt of {len(seq)} tokens exceeds max_model_len={self.config.max_model_len}")
        if request_id is not None:
            self.scheduler.request_id_to_seq[request_id] = seq
        self.scheduler.add(seq)
        return seq

    def feed(self, request_id: str, token_ids: list[int]):
        seq = self.scheduler.request_id_to_seq[request_id]
        if len(seq) + len(token_ids) > self.config.max_model_len:
            raise ValueError(f"request {request_id!r} would exceed max_model_len={self.config.max_model_len}")
        seq.feed(list(token_ids))

    def step(self, want: dict | None = None) -> StepOutput:
        items = self.scheduler.schedule()
        out = StepOutput()
        if not items:
            return out
        key = lambda s: s.request_id if s.request_id is not None else s.seq_id
        starts, o = {}, 0
        for seq, n in items:
            starts[key(seq)] = (o, n)
            out.scheduled[key(seq)] = n
            o += n
        out.num_tokens = o
        rows = []
        for rid, offsets in (want or {}).items():
            if rid not in starts:
                raise KeyError(f"logits wanted for {rid!r}, which runs no token this step")
            base, n = starts[rid]
            for off in offsets:
                if not 0 <= off < n:
                    raise IndexError(f"offset {off} outside the {n} tokens {rid!r} runs this step")
                rows.append(base + off)
        n_asked = len(rows)
        # sequences that complete their pending tokens and are not held get a sampled token
        sampling = [(seq, starts[key(seq)][0] + n - 1) for seq, n in items
                    if not seq.hold and seq.num_cached_tokens + n == seq.num_tokens]
        rows += [r for _, r in sampling]
        logits = self.model_runner.call("run_step", items, rows)
        for seq, n in items:
            seq.num_cached_tokens += n
        if want is not None:
            out.logits = logits[:n_asked]
        if sampling:
            groups: dict[int, list[int]] = {}
            for i, (seq, _) in enumerate(sampling):
                groups.setdefault(seq.top_k, []).append(i)
            tokens = [0] * len(sampling)
            for top_k, idx in groups.items():
                sel = logits[n_asked:] if len(idx) == len(sampling) else logits[n_asked:][torch.tensor(idx, device=logits.device)]
                ids = self.model_runner.call("sample", sel, [sampling[i][0].temperature for i in idx], top_k).tolist()
                for i, t in zip(idx, ids):
                    tokens[i] = t
            seqs = [s for s, _ in sampling]
            self.scheduler.postprocess(seqs, tokens)
            for s in seqs:
                if not s.is_finished and len(s) >= self.config.max_model_len:
                    self.scheduler._finish(s)
                if s.is_finished:
                    out.finished.append((s.request_id, s.seq_id, s.completion_token_ids))
        return out

    def generate(self, prompts: list[list[int]], sampling_params: SamplingParams | list[SamplingParams]) -> list[dict]:
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        seqs = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        done = {}
        while not self.is_finished():
            out = self.step()
            if not out.scheduled:
                raise RuntimeError("no sequence can be scheduled: the KV pool is too small for the live requests")
            for _, seq_id, toks in out.finished:
                done[seq_id] = toks
        return [{"token_ids": done[s.seq_id]} for s in seqs]
