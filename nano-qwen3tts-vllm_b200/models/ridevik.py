"""Ridevik: a decoder-only token model whose sublayers read the 32-bit residual stream itself and are normed on the way out.

    x = embed[token] * s
    layer:  x <- x + gnorm1(mixer(shift(x)));   x <- x + gnorm2(ff(x))          (gnorm: RMS norm in groups)
    shift:  h_t + (h_(t-1) - h_t) * mu, the previous row carried in a state slot between steps
    mixer:  latent attention - one normed latent c_t and one rotated key part per token in the paged cache; head h's
            key is [W_uk,h c | kr], its value W_uv,h c; softmax with a per-head sink; causal or sliding window;
            queries direct or through a normed latent; optional sigmoid gate on the heads' outputs; W_o
    ff:     W_down xielu(W_up h + b) + b, or a softmax-over-chosen mixture of SiLU-gated experts, or absent
    logits = head gnorm(x)

Every layer carries its own sizes (``config.RidevikLayerSpec``); a layer with ``weights_of`` runs another layer's modules
over a cache and state of its own.  One forward runs a whole engine step: prompt portions and single decoded tokens side
by side, described by the step layout in the global Context.  Launches per layer: token shift, merged input GEMM,
latent preparation (norms, key rotation, cache write), [query up-projection], per-head W_uk^T (batched GEMM), attention,
per-head W_uv (batched GEMM), gate + re-layout, output GEMM, residual + group norm, the feed-forward, residual + group norm.
"""
from __future__ import annotations

import re

import torch
from torch import nn

from .. import _native as nat
from ..config import RidevikConfig, RidevikLayerSpec
from ..layers.activation import XIELU
from ..layers.attention import LatentSinkAttention
from ..layers.embed_head import ScaledTokenEmbedding
from ..layers.layernorm import GroupRMSNorm
from ..layers.linear import ColumnParallelLinear, MergedColumnParallelLinear, RowParallelLinear, linear, per_head_linear
from ..layers.moe import SoftmaxTopKGatedMoE
from ..layers.rotary_embedding import PairRotary
from ..layers.token_shift import TokenShift


class LatentAttentionMixer(nn.Module):
    """Both variants, told apart by the spec alone: ``q_rank`` (query latent or direct), ``window`` (or causal),
    ``rot.scaling`` (or plain frequencies), ``gate``."""

    def __init__(self, width: int, spec, eps: float):
        super().__init__()
        m = self.spec = spec
        self.eps = eps
        self.q_size = m.heads * (m.dim + m.rot_dim)
        self.q_in = m.q_rank if m.q_rank else self.q_size
        parts = [self.q_in, m.kv_rank + m.rot_dim] + ([m.heads * m.vdim] if m.gate else [])
        self.in_proj = MergedColumnParallelLinear(width, parts)                 # [dq | q ; dkv ; g]
        f32 = dict(dtype=torch.float32)
        if m.q_rank:
            self.q_norm = nn.Parameter(torch.ones(m.q_rank, **f32), requires_grad=False)
            self.uq = ColumnParallelLinear(m.q_rank, self.q_size)
        else:
            self.register_parameter("q_norm", None)
            self.uq = None
        self.kv_norm = nn.Parameter(torch.ones(m.kv_rank, **f32), requires_grad=False)
        self.uk = nn.Parameter(torch.empty(m.heads, m.dim, m.kv_rank), requires_grad=False)      # rows of head h: W_uk,h
        self.uv = nn.Parameter(torch.empty(m.heads, m.vdim, m.kv_rank), requires_grad=False)
        self.rotary = PairRotary(m.rot.dims, m.rot.base, m.rot.scaling)
        self.attn = LatentSinkAttention(m.heads, m.kv_rank, m.rot_dim, m.window, m.scale, self.rotary)
        self.o_proj = RowParallelLinear(m.heads * m.vdim, width)

    def forward(self, hs: torch.Tensor, cache: torch.Tensor) -> torch.Tensor:
        """hs [n, width]: the token-shifted input; cache [pages, page, kv_rank + rot_dim] of THIS layer run."""
        from ..utils.context import get_context
        m, lay = self.spec, get_context().step_layout
        n = hs.shape[0]
        u = self.in_proj(hs)
        cq = torch.empty(n, m.q_rank, dtype=hs.dtype, device=hs.device) if m.q_rank else None
        nat.latent_prep(u, 0, self.q_in, cq, self.q_norm, self.kv_norm, self.rotary.freq, self.rotary.mult, lay, cache,
                        m.q_rank, m.kv_rank, m.rot_dim, m.rot.dims, self.eps)
        q = self.uq(cq) if m.q_rank else u                                       # heads laid out [dim | rot_dim] each
        hd = m.dim + m.rot_dim
        qn = torch.as_strided(q, (m.heads, n, m.dim), (hd, q.stride(0), 1))     # un-rotated parts, head-major view
        ql = per_head_linear(qn, self.uk)                                        # [heads, n, kv_rank] = W_uk,h^T q
        o = self.attn(ql, q[:, m.dim:], (q.stride(0), hd), cache)                # [heads, n, kv_rank]
        v = per_head_linear(o, self.uv, transpose_weight=True)                   # [heads, n, vdim]
        heads_out = torch.empty(n, m.heads * m.vdim, dtype=hs.dtype, device=hs.device)
        gate = u[:, self.q_in + m.kv_rank + m.rot_dim:] if m.gate else None
        nat.gate_heads(v, (m.vdim, n * m.vdim), gate, heads_out, m.heads, m.vdim)
        return self.o_proj(heads_out)


class XieluFF(nn.Module):
    """W_down xielu(W_up h + b_up) + b_down."""

    def __init__(self, width: int, ff: int):
        super().__init__()
        self.up = ColumnParallelLinear(width, ff, bias=True)
        self.act = XIELU()
        self.down = RowParallelLinear(ff, width, bias=True)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        y = linear(h, self.up.weight)
        self.act(y, self.up.bias)                                                # bias added in float inside the activation
        return linear(y, self.down.weight, self.down.bias)


class RidevikLayer(nn.Module):
    def __init__(self, width: int, spec: RidevikLayerSpec, eps: float, groups: int):
        super().__init__()
        self.shift = TokenShift(width)
        self.mix = LatentAttentionMixer(width, spec.mixer, eps)
        self.norm1 = GroupRMSNorm(width, groups, eps)
        f = spec.mlp
        self.mlp_kind = None if f is None else f.kind
        if f is None:
            self.mlp = self.norm2 = None
        else:
            self.mlp = XieluFF(width, f.ff) if f.kind == "dense" else SoftmaxTopKGatedMoE(width, f.ff, f.experts, f.top)
            self.norm2 = GroupRMSNorm(width, groups, eps)

    def forward(self, x: torch.Tensor, cache: torch.Tensor, state: torch.Tensor, dtype: torch.dtype):
        """x [n, width] float, updated in place."""
        a = self.mix(self.shift(x, state, dtype), cache)
        h = self.norm1.add_to(x, a=a, copy_dtype=dtype if self.mlp is not None else None)
        if self.mlp_kind == "dense":
            self.norm2.add_to(x, a=self.mlp(h))
        elif self.mlp_kind == "moe":
            z, zw = self.mlp(h)
            self.norm2.add_to(x, z=z, zw=zw)


class RidevikForCausalLM(nn.Module):
    def __init__(self, config: RidevikConfig):
        super().__init__()
        self.config = c = config
        self.embed = ScaledTokenEmbedding(c.vocab, c.width, c.embedding_scale)
        # modules exist for layers with tensors of their own; `runs` maps every layer run to the module it executes
        self.layers = nn.ModuleDict({str(i): RidevikLayer(c.width, spec, c.norm_eps, c.norm_groups)
                                     for i, spec in enumerate(c.layers) if spec.weights_of is None})
        self.runs = [i if spec.weights_of is None else spec.weights_of for i, spec in enumerate(c.layers)]
        self.final_norm = GroupRMSNorm(c.width, c.norm_groups, c.norm_eps)
        self.head = nn.Parameter(torch.empty(c.vocab, c.width), requires_grad=False)
        self.caches: list = [None] * len(self.runs)          # per layer RUN: the paged latent cache
        self.states: list = [None] * len(self.runs)          # per layer RUN: the token-shift rows [slots, width] float
        self.trace_layers = None               # a list: forward() appends a copy of the residual stream after every layer run

    @property
    def dtype(self) -> torch.dtype:
        return self.head.dtype

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One engine step over the packed tokens of the batch -> the residual stream [n, width] (float)."""
        x = self.embed(tokens)
        for run, src in enumerate(self.runs):
            self.layers[str(src)](x, self.caches[run], self.states[run], self.dtype)
            if self.trace_layers is not None:
                self.trace_layers.append(x.clone())
        return x

    def compute_logits(self, x: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        return linear(self.final_norm(x, self.dtype, rows), self.head).float()

    # ------------------------------------------------------------------ cache and state
    def cache_plan(self) -> list[dict]:
        """Per layer run: widths of its paged tensors and shapes (after the slot axis) / dtypes of its state tensors."""
        return [{"paged": [spec.mixer.cache_width], "state": [((self.config.width,), torch.float32)]}
                for spec in self.config.layers]

    def bind_cache(self, run: int, paged: list, state: list):
        self.caches[run], self.states[run] = paged[0], state[0]

    # ------------------------------------------------------------------ weights
    def load_state_dict(self, state_dict, strict=True):
        """Checkpoint names: ``embed``, ``l<i>.shift``, ``l<i>.norm1|norm2``, ``l<i>.mix.{dq,dq.norm,uq | q}``,
        ``l<i>.mix.{dkv,dkv.norm,uk,uv,sink,o}``, ``l<i>.mix.g``, ``l<i>.mlp.{up,up.b,down,down.b,act}`` or
        ``l<i>.mlp.{router,router.b}`` with ``l<i>.mlp.e<j>.{gate,up,down}``, ``final.norm``, ``head``; layers that reuse
        another layer's tensors have none.  What the kernels keep in float (norm weights, shift, sinks, activation
        numbers, routers) is widened exactly."""
        seen = set()

        def put(param, value, shard=None):
            with torch.no_grad():
                if shard is not None:
                    param.weight_loader(param, value.to(param.dtype), shard)
                    return
                if param.numel() != value.numel() or (param.dim() == value.dim() and tuple(param.shape) != tuple(value.shape)):
                    raise ValueError(f"shape {tuple(value.shape)} does not fit {tuple(param.shape)}")
                param.copy_(value.to(param.dtype).reshape(param.shape))

        for name, t in state_dict.items():
            m = re.fullmatch(r"l(\d+)\.(.+)", name)
            try:
                if name == "embed":
                    put(self.embed.embed, t)
                elif name == "final.norm":
                    put(self.final_norm.weight, t)
                elif name == "head":
                    put(self.head, t)
                elif m and m.group(1) in self.layers:
                    layer, key = self.layers[m.group(1)], m.group(2)
                    mix, spec = layer.mix, layer.mix.spec
                    if key == "shift":
                        put(layer.shift.weight, t)
                    elif key == "norm1":
                        put(layer.norm1.weight, t)
                    elif key == "norm2" and layer.norm2 is not None:
                        put(layer.norm2.weight, t)
                    elif key == "mix.dq" and spec.q_rank:
                        put(mix.in_proj.weight, t, 0)
                    elif key == "mix.q" and not spec.q_rank:
                        put(mix.in_proj.weight, t, 0)
                    elif key == "mix.dq.norm" and spec.q_rank:
                        put(mix.q_norm, t)
                    elif key == "mix.uq" and spec.q_rank:
                        put(mix.uq.weight, t)
                    elif key == "mix.dkv":
                        put(mix.in_proj.weight, t, 1)
                    elif key == "mix.dkv.norm":
                        put(mix.kv_norm, t)
                    elif key == "mix.g" and spec.gate:
                        put(mix.in_proj.weight, t, 2)
                    elif key in ("mix.uk", "mix.uv"):
                        put(getattr(mix, key[4:]), t)                          # [heads * d, kv_rank] -> [heads, d, kv_rank]
                    elif key == "mix.sink":
                        put(mix.attn.sink, t)
                    elif key == "mix.o":
                        put(mix.o_proj.weight, t)
                    elif key in ("mlp.up", "mlp.down") and layer.mlp_kind == "dense":
                        put(getattr(layer.mlp, key[4:]).weight, t)
                    elif key in ("mlp.up.b", "mlp.down.b") and layer.mlp_kind == "dense":
                        put(getattr(layer.mlp, key[4:-2]).bias, t)
                    elif key == "mlp.act" and layer.mlp_kind == "dense":
                        put(layer.mlp.act.pq, t)
                    elif key == "mlp.router" and layer.mlp_kind == "moe":
                        put(layer.mlp.router, t)
                    elif key == "mlp.router.b" and layer.mlp_kind == "moe":
                        put(layer.mlp.router_bias, t)
                    elif (e := re.fullmatch(r"mlp\.e(\d+)\.(gate|up|down)", key)) and layer.mlp_kind == "moe" \
                            and int(e.group(1)) < layer.mlp.experts:
                        j, ff = int(e.group(1)), layer.mlp.ff
                        if e.group(2) == "down":
                            put(layer.mlp.down[j], t)
                        else:
                            put(layer.mlp.up[j, :ff] if e.group(2) == "gate" else layer.mlp.up[j, ff:], t)
                    else:
                        raise KeyError(name)
                else:
                    raise KeyError(name)
            except KeyError:
                if strict:
                    raise KeyError(f"unexpected tensor {name!r} in the checkpoint")
                continue
            seen.add(name)
        if strict:
            missing = sorted(set(self.checkpoint_names()) - seen)
            if missing:
                raise KeyError(f"missing tensors: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
        return seen

    def checkpoint_names(self) -> list[str]:
        return checkpoint_names(self.config)


def checkpoint_names(config: RidevikConfig) -> list[str]:
    names = ["embed", "final.norm", "head"]
    for i, spec in enumerate(config.layers):
        if spec.weights_of is not None:
            continue
        p, m = f"l{i}.", spec.mixer
        names += [p + "shift", p + "norm1", p + "mix.dkv", p + "mix.dkv.norm", p + "mix.uk", p + "mix.uv", p + "mix.sink", p + "mix.o"]
        names += [p + "mix.dq", p + "mix.dq.norm", p + "mix.uq"] if m.q_rank else [p + "mix.q"]
        if m.gate:
            names.append(p + "mix.g")
        f = spec.mlp
        if f is None:
            continue
        names.append(p + "norm2")
        if f.kind == "dense":
            names += [p + "mlp.up", p + "mlp.up.b", p + "mlp.down", p + "mlp.down.b", p + "mlp.act"]
        else:
            names += [p + "mlp.router", p + "mlp.router.b"]
            for e in range(f.experts):
                names += [f"{p}mlp.e{e}.gate", f"{p}mlp.e{e}.up", f"{p}mlp.e{e}.down"]
    return names


def random_state_dict(config: RidevikConfig, seed: int = 0) -> dict:
    """Random bfloat16 tensors under the checkpoint's names (benchmarks, tests and smoke runs; no trained weights exist)."""
    g = torch.Generator().manual_seed(seed)
    D = config.width

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16)

    sd = {"embed": rnd(config.vocab, D, std=1.0 / config.embedding_scale), "final.norm": rnd(D, mean=1.0, std=0.1),
          "head": rnd(config.vocab, D, std=D ** -0.5)}
    for i, spec in enumerate(config.layers):
        if spec.weights_of is not None:
            continue
        m, p = spec.mixer, f"l{i}."
        hd = m.dim + m.rot_dim
        sd[p + "shift"] = torch.rand(D, generator=g).to(torch.bfloat16)
        sd[p + "norm1"] = rnd(D, mean=0.5, std=0.1)
        if m.q_rank:
            sd[p + "mix.dq"] = rnd(m.q_rank, D, std=D ** -0.5)
            sd[p + "mix.dq.norm"] = rnd(m.q_rank, mean=1.0, std=0.1)
            sd[p + "mix.uq"] = rnd(m.heads * hd, m.q_rank, std=m.q_rank ** -0.5)
        else:
            sd[p + "mix.q"] = rnd(m.heads * hd, D, std=D ** -0.5)
        sd[p + "mix.dkv"] = rnd(m.kv_rank + m.rot_dim, D, std=D ** -0.5)
        sd[p + "mix.dkv.norm"] = rnd(m.kv_rank, mean=1.0, std=0.1)
        sd[p + "mix.uk"] = rnd(m.heads * m.dim, m.kv_rank, std=m.kv_rank ** -0.5)
        sd[p + "mix.uv"] = rnd(m.heads * m.vdim, m.kv_rank, std=m.kv_rank ** -0.5)
        sd[p + "mix.sink"] = rnd(m.heads, std=1.0)
        if m.gate:
            sd[p + "mix.g"] = rnd(m.heads * m.vdim, D, std=D ** -0.5)
        sd[p + "mix.o"] = rnd(D, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
        f = spec.mlp
        if f is None:
            continue
        sd[p + "norm2"] = rnd(D, mean=0.5, std=0.1)
        if f.kind == "dense":
            sd[p + "mlp.up"] = rnd(f.ff, D, std=D ** -0.5)
            sd[p + "mlp.up.b"] = rnd(f.ff, std=0.1)
            sd[p + "mlp.down"] = rnd(D, f.ff, std=f.ff ** -0.5)
            sd[p + "mlp.down.b"] = rnd(D, std=0.1)
            sd[p + "mlp.act"] = rnd(2, std=0.5)
        else:
            sd[p + "mlp.router"] = rnd(f.experts, D, std=D ** -0.5)
            sd[p + "mlp.router.b"] = rnd(f.experts, std=0.2)
            for e in range(f.experts):
                sd[f"{p}mlp.e{e}.gate"] = rnd(f.ff, D, std=D ** -0.5)
                sd[f"{p}mlp.e{e}.up"] = rnd(f.ff, D, std=D ** -0.5)
                sd[f"{p}mlp.e{e}.down"] = rnd(D, f.ff, std=f.ff ** -0.5)
    return sd
