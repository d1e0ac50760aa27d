"""Runner of token-id language models (the registry's ``LMModelRunner``): one ``run_step`` serves prompt portions and
decoded tokens together, over a paged K/V pool with per-layer shapes and a pool of per-sequence state slots.

Differences from the embedding-driven runners of this package, all behind the same ``ModelRunner`` construction:
  * the batch is a list of (sequence, tokens to run) - there is no separate prefill and decode layout; the decode
    step (every row one token) is additionally captured as CUDA graphs per batch size;
  * paged tensors and state slots are allocated per layer run from the model's ``cache_plan()`` (K and V pages of a
    layer's own head counts and sizes, or one page of latents; convolution taps, or a token-shift row), since a layer
    lists its own sizes and a layer that reuses another's weights still has a cache of its own;
  * activations and caches are bfloat16, or float32 when the engine is built with ``dtype="float32"`` (matrix
    products then run as true 32-bit library GEMMs: TF32 is switched off around this runner's calls only)."""
from __future__ import annotations

import contextlib
import os

import torch

from ...config import Config
from ...layers.sampler import Sampler
from ...models.registry import resolve_config_object
from ...utils.context import reset_context, set_context
from ..sequence import Sequence
from ..step_layout import MixedStepLayout
from .base import ModelRunner
from ...utils.graph_capture import graph_capture


class _Float32Matmul:
    """No TF32 and "highest" float32 precision inside the block."""

    def __enter__(self):
        self.saved = (torch.backends.cuda.matmul.allow_tf32, torch.get_float32_matmul_precision())
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")

    def __exit__(self, *exc):
        torch.set_float32_matmul_precision(self.saved[1])
        torch.backends.cuda.matmul.allow_tf32 = self.saved[0]
        return False


class LMModelRunner(ModelRunner):
    def pick_stack_config(self, model_config):
        return model_config

    def build_model(self):
        return resolve_config_object(self.stack_config).model_cls(self.stack_config)

    def graph_batch_sizes(self):
        if self.config.graph_batch_sizes:
            return sorted(self.config.graph_batch_sizes)
        return [b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512) if b < self.max_bs] + [self.max_bs]

    def load_model(self, state_dict):
        if isinstance(state_dict, str) and state_dict.startswith("random"):
            import importlib
            seed = int(state_dict.split(":")[1]) if ":" in state_dict else 1234
            state_dict = importlib.import_module(type(self.model).__module__).random_state_dict(self.stack_config, seed)
        if state_dict is None and self.config.model:
            path = os.path.join(self.config.model, "model.safetensors")
            if os.path.exists(path):
                from safetensors.torch import load_file
                state_dict = load_file(path)
        if state_dict is None:
            raise RuntimeError("no weights: pass state_dict= or a model directory holding model.safetensors")
        self.model.load_state_dict(state_dict)

    # ------------------------------------------------------------------ init
    def post_init(self):
        self.sampler = Sampler()
        self.top_k = 50
        self.max_step_tokens = self.config.max_num_batched_tokens
        self.layout = MixedStepLayout(self.max_step_tokens, self.max_bs, self.max_blocks, self.device)
        self.allocate_kv_cache()
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        if not self.enforce_eager:
            self.capture_cudagraph()

    def kv_block_bytes(self) -> int:
        el = 4 if self.param_dtype == torch.float32 else 2
        return sum(self.block_size * w * el for plan in self.model.cache_plan() for w in plan["paged"])

    def allocate_kv_cache(self):
        """The model says what every layer run needs (``cache_plan``): paged tensors [pages, page, width] that share one
        block table, and per-sequence state tensors [slots, ...] that share one slot id.  A layer that reuses another
        layer's weights still gets tensors of its own."""
        cfg = self.config
        if cfg.num_kvcache_blocks <= 0:
            free, _ = torch.cuda.mem_get_info(self.device)
            blocks = int(free * cfg.gpu_memory_utilization * 0.9) // max(self.kv_block_bytes(), 1)
            cfg.num_kvcache_blocks = max(1, min(blocks, self.max_bs * self.max_blocks))
        slots = cfg.max_state_slots or cfg.max_num_seqs
        self.kv_cache, self.seq_state = [], []
        for run, plan in enumerate(self.model.cache_plan()):
            paged = [torch.zeros(cfg.num_kvcache_blocks, self.block_size, w, dtype=self.param_dtype, device=self.device)
                     for w in plan["paged"]]
            state = [torch.zeros(slots, *shape, dtype=dt or self.param_dtype, device=self.device) for shape, dt in plan["state"]]
            self.model.bind_cache(run, paged, state)
            self.kv_cache.append(paged)
            self.seq_state.append(state)

    # ------------------------------------------------------------------ the step
    def true_float32(self):
        """float32 mode: library matrix products in true 32-bit while this runner's code runs (the process-wide setting
        is put back afterwards, so other models in the process keep theirs)."""
        return _Float32Matmul() if self.param_dtype == torch.float32 else contextlib.nullcontext()

    def step_body(self) -> torch.Tensor:
        lay = self.layout
        set_context(False, step_layout=lay)
        with self.true_float32():
            return self.model(lay.tokens, lay.positions)

    @torch.inference_mode()
    def capture_cudagraph(self):
        self.graph_bs = [b for b in self.graph_batch_sizes() if b <= self.max_bs]
        self.graph_pool = None
        self.graph_out: dict[int, torch.Tensor] = {}
        self.layout.fill([], self.block_size, pad_seqs=self.graph_bs[-1])       # all padding: nothing is touched
        for bs in reversed(self.graph_bs):
            self.layout.set_decode_shape(bs)
            self.step_body()                                                     # warm-up (weight packing, lazy handles)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with graph_capture(g, self.graph_pool):
                self.graph_out[bs] = self.step_body()
            if self.graph_pool is None:
                self.graph_pool = g.pool()
            self.graphs[bs] = g
        torch.cuda.synchronize()
        reset_context()

    @torch.inference_mode()
    def run_step(self, items: list[tuple[Sequence, int]], want_rows: list[int]) -> torch.Tensor:
        """Run ``items`` = [(sequence, tokens to run)] as ONE batch; K/V and state advance.  Returns float logits
        [len(want_rows), vocab] of the packed-batch rows ``want_rows`` (row = offset of the item + offset inside it)."""
        n = len(items)
        gb = self.pick_graph(n) if all(k == 1 for _, k in items) else None
        self.layout.fill(items, self.block_size, want_rows, pad_seqs=gb)
        if gb is None:
            x = self.step_body()
        else:
            self.layout.set_decode_shape(gb)
            self.graphs[gb].replay()
            x = self.graph_out[gb]
        reset_context()
        if not want_rows:
            return torch.empty(0, self.stack_config.vocab, dtype=torch.float32, device=self.device)
        rows = self.layout._view(self.layout.dev, "want_rows")[:len(want_rows)]
        with self.true_float32():
            return self.model.compute_logits(x, rows)

    @torch.inference_mode()
    def sample(self, logits: torch.Tensor, temperatures: list[float], top_k: int) -> torch.Tensor:
        t = torch.tensor(temperatures, dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        return self.sampler(logits, t, top_k=top_k)
