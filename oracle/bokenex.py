"""Plain, slow restatement of the Bokenex decoder (test infrastructure only: nothing in the package imports it).

One function per mechanism, whole sequences at a time, no cache and no batching: every position is
recomputed from the full prefix, so the engine's paged cache, short-convolution state, portions and
mixed batches have something independent to be compared with.  Arithmetic is done in the dtype of the
weights handed in (float64 in the tests).

Notation: x [T, D] residual stream, h = norm(x), H query heads over G key/value heads, d the query/key
size per head, dv the value size, W the number of keys a position sees (itself included).
"""
from __future__ import annotations

import math

import torch


def gain_rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * g with ONE gain g for all coordinates."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain.reshape(())


def vector_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm over the last axis with a plain (not one-plus) weight vector."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def causal_short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([u.new_zeros(taps - 1, C), u], 0)
    y = u.new_zeros(T, C)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    r = torch.relu(z)
    return r * r


def windowed_sigmoid_attention(q, k, v, scale, window, r1, r2, pb):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].

    weight(i, j) = sigmoid(q_i . k_j * scale - r1_h * ln(1 + r2_h * (i - j)) + pb_h) for 0 <= i - j < window,
    else 0; the weights are NOT normalised over j."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = q.new_zeros(T, H, v.shape[-1])
    idx = torch.arange(T)
    dist = (idx[:, None] - idx[None, :])
    visible = (dist >= 0) & (dist < window)
    distf = dist.clamp(min=0).to(q.dtype)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        s = s - r1[h] * torch.log1p(r2[h] * distf) + pb[h]
        w = torch.sigmoid(s) * visible
        out[:, h] = w @ v[:, g]
    return out


def attention_mixer(h, p, m, eps):
    """p: the mixer's tensors by short name (q, k, v, q.conv, k.conv, v.conv, q.norm, k.norm, r1, r2, pb, o);
    m: its sizes (heads, kv_heads, dim, vdim, scale, mask.size)."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = causal_short_conv(h @ p["q"].T, p["q.conv"]).view(T, H, d)
    k = causal_short_conv(h @ p["k"].T, p["k.conv"]).view(T, G, d)
    v = causal_short_conv(h @ p["v"].T, p["v.conv"]).view(T, G, dv)
    q = vector_rms_norm(q, p["q.norm"], eps)
    k = vector_rms_norm(k, p["k.norm"], eps)
    o = windowed_sigmoid_attention(q, k, v, m["scale"], m["mask"]["size"], p["r1"], p["r2"], p["pb"])
    return o.reshape(T, H * dv) @ p["o"].T


def dense_ff(h, up, down):
    return relu_squared(h @ up.T) @ down.T


def moe_route(h, router, top, scale):
    """-> (chosen expert ids [T, top], their weights [T, top]): sigmoid scores, the `top` largest, divided by
    their sum (+ 1e-20), times `scale`."""
    s = torch.sigmoid(h @ router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20) * scale


def moe_ff(h, router, ups, downs, top, scale):
    idx, w = moe_route(h, router, top, scale)
    out = h.new_zeros(h.shape[0], downs[0].shape[0])
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] = out[t] + w[t, j] * dense_ff(h[t:t + 1], ups[e], downs[e])[0]
    return out


def forward(cfg: dict, sd: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (positions 0..T-1).  ``sd``: tensors by checkpoint name."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    T = tok.numel()
    x = sd["embed"][tok] + sd["pos"][:T]
    trail = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = gain_rms_norm(x, sd[pre + "norm1"], eps)
        assert layer["type"] == "attention"
        p = {k[len(pre) + 4:]: v for k, v in sd.items() if k.startswith(pre + "mix.")}
        y = attention_mixer(h, p, layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = y + dense_ff(h, sd[pre + "mlp.up"], sd[pre + "mlp.down"])
            else:
                r = mlp["router"]
                ups = [sd[f"{pre}mlp.e{e}.up"] for e in range(r["experts"])]
                downs = [sd[f"{pre}mlp.e{e}.down"] for e in range(r["experts"])]
                y = y + moe_ff(h, sd[pre + "mlp.router"], ups, downs, r["top"], r["scale"])
        x = x + mult * y
        trail.append(x)
    logits = gain_rms_norm(x, sd["final.norm"], eps) @ sd["head"].T
    return (logits, torch.stack(trail)) if return_layers else logits


def random_config(seed: int, width=48, vocab=40, n_layers=3, max_positions=96, heads=4, kv_heads=2, dim=8, vdim=12,
                  window=9, taps=3, ff=40, experts=5, top=2, expert_ff=24, residual_mult=0.7, scale=0.3,
                  router_scale=1.5, eps=1e-5, kinds=("dense", "moe", None)) -> dict:
    """A small configuration in the checkpoint's config.json layout; layer i's feed-forward kind cycles over ``kinds``."""
    layers = []
    for i in range(n_layers):
        kind = kinds[i % len(kinds)]
        mlp = None
        if kind == "dense":
            mlp = {"kind": "dense", "ff": ff + 8 * i}
        elif kind == "moe":
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "scale": router_scale}}
        layers.append({"type": "attention", "mlp": mlp,
                       "mixer": {"conv": taps, "dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv_heads,
                                 "mask": {"size": window + i}, "scale": scale}})
    return {"architecture": "Bokenex", "layers": layers, "max_positions": max_positions, "norm": {"eps": eps},
            "residual_mult": residual_mult, "vocab": vocab, "width": width, "seed": seed}


def random_weights(cfg: dict, seed: int = 0, dtype=torch.float64) -> dict:
    """Random tensors under the checkpoint's names, rounded to bfloat16 values (what a checkpoint can hold)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16).to(dtype)

    sd = {"embed": rnd(cfg["vocab"], D), "pos": rnd(cfg["max_positions"], D, std=0.5),
          "final.norm": rnd(std=0.1, mean=1.0), "head": rnd(cfg["vocab"], D, std=D ** -0.5)}
    for i, layer in enumerate(cfg["layers"]):
        m, pre = layer["mixer"], f"l{i}."
        H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        sd[pre + "norm1"] = rnd(std=0.1, mean=1.0)
        for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            sd[f"{pre}mix.{name}"] = rnd(rows, D, std=D ** -0.5)
            sd[f"{pre}mix.{name}.conv"] = rnd(rows, taps, std=0.6)
        sd[pre + "mix.q.norm"] = rnd(d, std=0.2, mean=1.0)
        sd[pre + "mix.k.norm"] = rnd(d, std=0.2, mean=1.0)
        sd[pre + "mix.r1"] = rnd(H, std=0.3, mean=0.5)
        sd[pre + "mix.r2"] = rnd(H, std=0.2, mean=0.6).abs()
        sd[pre + "mix.pb"] = rnd(H, std=0.5, mean=-1.0)
        sd[pre + "mix.o"] = rnd(D, H * dv, std=(H * dv) ** -0.5)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            sd[pre + "mlp.up"] = rnd(mlp["ff"], D, std=D ** -0.5)
            sd[pre + "mlp.down"] = rnd(D, mlp["ff"], std=mlp["ff"] ** -0.5)
        else:
            f, r = mlp["expert"]["ff"], mlp["router"]
            sd[pre + "mlp.router"] = rnd(r["experts"], D, std=2.0 * D ** -0.5)
            for e in range(r["experts"]):
                sd[f"{pre}mlp.e{e}.up"] = rnd(f, D, std=D ** -0.5)
                sd[f"{pre}mlp.e{e}.down"] = rnd(D, f, std=f ** -0.5)
    return sd
