"""Bokenex: a decoder-only token model of parallel layers over a 32-bit residual stream.

    x = embed[token] + pos[position]
    layer:  h = gain_norm(x);  x <- x + m * (mixer(h) + ff(h))            (one norm, both sublayers read it)
    mixer:  q|k|v = W_qkv h -> short causal convolution per channel -> RMS norm per head on q and k
            -> sliding-window sigmoid attention with a logarithmic distance bias -> W_o
    ff:     W_down relu(W_up h)^2, dense or as a sigmoid top-k mixture of experts, or absent
    logits = head gain_norm(x)

Every layer carries its own sizes (``config.LayerSpec``).  One forward runs a whole engine step: prompt portions and
single decoded tokens side by side, described by the step layout in the global Context.  Launches per layer: merged
q|k|v GEMM, convolution + head norm + K/V write, attention, output GEMM, the feed-forward (two GEMMs and an
activation, or router + two grouped GEMMs), and one residual kernel that also applies the NEXT layer's norm.
"""
from __future__ import annotations

import re

import torch
from torch import nn

from .. import _native as nat
from ..config import BokenexConfig, LayerSpec
from ..layers.attention import WindowSigmoidAttention
from ..layers.embed_head import TokenPositionEmbedding
from ..layers.layernorm import GainRMSNorm
from ..layers.linear import MergedColumnParallelLinear, RowParallelLinear, ColumnParallelLinear, linear, linear_relu_sq
from ..layers.moe import SigmoidTopKMoE
from ..layers.short_conv import ShortConvQKV


class BokenexAttentionMixer(nn.Module):
    def __init__(self, width: int, spec, eps: float):
        super().__init__()
        m = spec
        self.qkv_proj = MergedColumnParallelLinear(width, [m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim])
        self.conv = ShortConvQKV(m.heads, m.kv_heads, m.dim, m.vdim, m.conv, eps)
        self.attn = WindowSigmoidAttention(m.heads, m.kv_heads, m.dim, m.vdim, m.window, m.scale)
        self.o_proj = RowParallelLinear(m.heads * m.vdim, width)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        u = self.qkv_proj(h)
        q = self.conv(u, self.attn.k_cache, self.attn.v_cache)
        return self.o_proj(self.attn(q))


class BokenexDenseFF(nn.Module):
    def __init__(self, width: int, ff: int):
        super().__init__()
        self.up = ColumnParallelLinear(width, ff)
        self.down = RowParallelLinear(ff, width)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.down(linear_relu_sq(h, self.up.weight))


class BokenexLayer(nn.Module):
    def __init__(self, width: int, spec: LayerSpec, eps: float):
        super().__init__()
        self.norm1 = GainRMSNorm(eps)
        self.mix = BokenexAttentionMixer(width, spec.mixer, eps)
        f = spec.mlp
        self.mlp_kind = None if f is None else f.kind
        if f is None:
            self.mlp = None
        elif f.kind == "dense":
            self.mlp = BokenexDenseFF(width, f.ff)
        else:
            self.mlp = SigmoidTopKMoE(width, f.ff, f.experts, f.top, f.router_scale)

    def forward(self, x: torch.Tensor, h: torch.Tensor, mult: float, next_norm: GainRMSNorm | None):
        """x [n, width] float (updated in place), h = norm1(x) -> the next layer's normed input (or None)."""
        a = self.mix(h)
        b = z = zw = None
        if self.mlp_kind == "dense":
            b = self.mlp(h)
        elif self.mlp_kind == "moe":
            z, zw = self.mlp(h)
        h_next = torch.empty_like(h) if next_norm is not None else None
        nat.residual_norm(x, a, b, z, zw, mult, h_next, next_norm.gain() if next_norm is not None else None,
                          self.norm1.eps, h.dtype)
        return h_next


class BokenexForCausalLM(nn.Module):
    def __init__(self, config: BokenexConfig):
        super().__init__()
        self.config = config
        c = config
        self.embed = TokenPositionEmbedding(c.vocab, c.max_positions, c.width)
        self.layers = nn.ModuleList([BokenexLayer(c.width, spec, c.norm_eps) for spec in c.layers])
        self.final_norm = GainRMSNorm(c.norm_eps)
        self.head = nn.Parameter(torch.empty(c.vocab, c.width), requires_grad=False)
        self.trace_layers = None               # a list: forward() appends a copy of the residual stream after every layer

    @property
    def dtype(self) -> torch.dtype:
        return self.head.dtype

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One engine step over the packed tokens of the batch -> the residual stream [n, width] (float)."""
        n_layers = len(self.layers)
        first = self.layers[0].norm1 if n_layers else None
        x, h = self.embed(tokens, positions, first)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].norm1 if i + 1 < n_layers else None
            h = layer(x, h, self.config.residual_mult, nxt)
            if self.trace_layers is not None:
                self.trace_layers.append(x.clone())
        return x

    def compute_logits(self, x: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        """Logits (float) of the residual rows ``rows`` (all rows if None): final norm on the gathered rows, then the head."""
        hw = self.final_norm(x, self.dtype, rows)
        return linear(hw, self.head).float()

    # ------------------------------------------------------------------ weights
    def cache_modules(self):
        """(attention, convolution) module pairs in layer order: what cache and state are bound to."""
        return [(l.mix.attn, l.mix.conv) for l in self.layers]

    def cache_plan(self) -> list[dict]:
        """Per layer: widths of its paged tensors (K, V) and the shape (after the slot axis) of its convolution state."""
        return [{"paged": [l.mixer.kv_heads * l.mixer.dim, l.mixer.kv_heads * l.mixer.vdim],
                 "state": [((max(l.mixer.conv - 1, 1), l.mixer.channels), None)]} for l in self.config.layers]

    def bind_cache(self, run: int, paged: list, state: list):
        attn, conv = self.cache_modules()[run]
        attn.k_cache, attn.v_cache = paged
        conv.state = state[0]

    def load_state_dict(self, state_dict, strict=True):
        """Checkpoint names: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.mix.{q,k,v,o}``, ``l<i>.mix.{q,k,v}.conv``,
        ``l<i>.mix.{q,k}.norm``, ``l<i>.mix.{r1,r2,pb}``, ``l<i>.mlp.{up,down}`` or ``l<i>.mlp.router`` with
        ``l<i>.mlp.e<j>.{up,down}``, ``final.norm``, ``head``.  Tensors are bfloat16 in the file; what the kernels
        keep in float (gains, head norms, per-head constants, convolution taps, routers) is widened exactly."""
        seen = set()
        c = self.config

        def put(param, value, shard=None):
            with torch.no_grad():
                if shard is not None:
                    param.weight_loader(param, value.to(param.dtype), shard)
                else:
                    if tuple(param.shape) != tuple(value.shape):
                        raise ValueError(f"shape {tuple(value.shape)} does not fit {tuple(param.shape)}")
                    param.copy_(value.to(param.dtype))

        for name, t in state_dict.items():
            m = re.fullmatch(r"l(\d+)\.(.+)", name)
            try:
                if name == "embed":
                    put(self.embed.embed, t)
                elif name == "pos":
                    put(self.embed.pos, t)
                elif name == "final.norm":
                    put(self.final_norm.weight, t.reshape(()))
                elif name == "head":
                    put(self.head, t)
                elif m and int(m.group(1)) < len(self.layers):
                    layer, key = self.layers[int(m.group(1))], m.group(2)
                    mix, spec = layer.mix, c.layers[int(m.group(1))].mixer
                    offs = {"q": 0, "k": spec.heads * spec.dim, "v": spec.heads * spec.dim + spec.kv_heads * spec.dim}
                    rows = {"q": spec.heads * spec.dim, "k": spec.kv_heads * spec.dim, "v": spec.kv_heads * spec.vdim}
                    if key == "norm1":
                        put(layer.norm1.weight, t.reshape(()))
                    elif key in ("mix.q", "mix.k", "mix.v"):
                        put(mix.qkv_proj.weight, t, "qkv".index(key[-1]))
                    elif key in ("mix.q.conv", "mix.k.conv", "mix.v.conv"):
                        ch = key[4]
                        put(mix.conv.weight[offs[ch]:offs[ch] + rows[ch]], t)
                    elif key == "mix.q.norm":
                        put(mix.conv.q_norm, t)
                    elif key == "mix.k.norm":
                        put(mix.conv.k_norm, t)
                    elif key in ("mix.r1", "mix.r2", "mix.pb"):
                        put(getattr(mix.attn, key[4:]), t)
                    elif key == "mix.o":
                        put(mix.o_proj.weight, t)
                    elif key in ("mlp.up", "mlp.down") and layer.mlp_kind == "dense":
                        put(getattr(layer.mlp, key[4:]).weight, t)
                    elif key == "mlp.router" and layer.mlp_kind == "moe":
                        put(layer.mlp.router, t)
                    elif (e := re.fullmatch(r"mlp\.e(\d+)\.(up|down)", key)) and layer.mlp_kind == "moe":
                        put(getattr(layer.mlp, e.group(2))[int(e.group(1))], t)
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
        names = ["embed", "pos", "final.norm", "head"]
        for i, spec in enumerate(self.config.layers):
            p = f"l{i}."
            names += [p + "norm1", p + "mix.o", p + "mix.q.norm", p + "mix.k.norm", p + "mix.r1", p + "mix.r2", p + "mix.pb"]
            for ch in "qkv":
                names += [f"{p}mix.{ch}", f"{p}mix.{ch}.conv"]
            if spec.mlp is None:
                continue
            if spec.mlp.kind == "dense":
                names += [p + "mlp.up", p + "mlp.down"]
            else:
                names.append(p + "mlp.router")
                for e in range(spec.mlp.experts):
                    names += [f"{p}mlp.e{e}.up", f"{p}mlp.e{e}.down"]
        return names


def random_state_dict(config: BokenexConfig, seed: int = 0) -> dict:
    """Random bfloat16 tensors under the checkpoint's names (benchmarks and smoke runs; no trained weights exist)."""
    g = torch.Generator().manual_seed(seed)
    D = config.width

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16)

    sd = {"embed": rnd(config.vocab, D), "pos": rnd(config.max_positions, D, std=0.5), "final.norm": rnd(mean=1.0, std=0.05),
          "head": rnd(config.vocab, D, std=D ** -0.5)}
    for i, spec in enumerate(config.layers):
        m, p = spec.mixer, f"l{i}."
        sd[p + "norm1"] = rnd(mean=1.0, std=0.05)
        for ch, rows in (("q", m.heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)):
            sd[f"{p}mix.{ch}"] = rnd(rows, D, std=D ** -0.5)
            sd[f"{p}mix.{ch}.conv"] = rnd(rows, m.conv, std=0.5)
        sd[p + "mix.q.norm"] = rnd(m.dim, mean=1.0, std=0.1)
        sd[p + "mix.k.norm"] = rnd(m.dim, mean=1.0, std=0.1)
        sd[p + "mix.r1"] = rnd(m.heads, mean=0.5, std=0.2)
        sd[p + "mix.r2"] = rnd(m.heads, mean=0.5, std=0.1).abs()
        sd[p + "mix.pb"] = rnd(m.heads, mean=-2.0, std=0.5)
        sd[p + "mix.o"] = rnd(D, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
        f = spec.mlp
        if f is None:
            continue
        if f.kind == "dense":
            sd[p + "mlp.up"] = rnd(f.ff, D, std=D ** -0.5)
            sd[p + "mlp.down"] = rnd(D, f.ff, std=f.ff ** -0.5)
        else:
            sd[p + "mlp.router"] = rnd(f.experts, D, std=D ** -0.5)
            for e in range(f.experts):
                sd[f"{p}mlp.e{e}.up"] = rnd(f.ff, D, std=D ** -0.5)
                sd[f"{p}mlp.e{e}.down"] = rnd(D, f.ff, std=f.ff ** -0.5)
    return sd
