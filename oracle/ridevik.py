"""Plain, slow restatement of the Ridevik decoder (test infrastructure only: nothing in the package imports it).

One function per mechanism, whole sequences at a time, no cache, no state and no batching: every position is
recomputed from the full prefix (keys and values are expanded per head from the latent, nothing is absorbed into the
queries), so the engine's paged latent cache, token-shift state, portions and mixed batches have something independent
to be compared with.  Arithmetic is done in the dtype of the tensors handed in (float64 in the tests).

Notation: x [T, D] residual stream, H heads, dn / dr the un-rotated / rotated query-key sizes per head, dv the value
size, r the latent size, W the number of keys a position sees (itself included; None = all earlier ones).
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def grouped_rms_norm(x, weight, eps, groups):
    """The last axis is cut into ``groups`` equal consecutive parts; each is divided by its own root mean square."""
    T, D = x.shape
    g = x.reshape(T, groups, D // groups)
    g = g / torch.sqrt((g * g).mean(-1, keepdim=True) + eps)
    return g.reshape(T, D) * weight


def token_shift(h, mu):
    """h_t <- h_t + (h_(t-1) - h_t) * mu with h_(-1) = 0 (the un-shifted predecessor is used)."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


def rotary_frequencies(dims, base, scaling=None, dtype=torch.float64):
    """f_i = base^(-2i/dims), i < dims/2, optionally blended with f_i / factor by a linear ramp over i (YaRN);
    returns (frequencies, multiplier of cos and sin)."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def corr(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(corr(float(scaling["fast"]))), 0)
    hi = min(math.ceil(corr(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v, positions, freqs, mult, dims):
    """v [..., T, n]: the first ``dims`` coordinates are rotated pairwise (2i with 2i+1) by the angle p * f_i."""
    a = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    c, s = torch.cos(a) * mult, torch.sin(a) * mult
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def sink_softmax_attention(q, k, v, scale, window, sink):
    """q, k [T, H, d], v [T, H, dv] -> [T, H, dv].  Softmax over the visible keys j (0 <= i - j < window, or all
    j <= i) whose denominator also holds exp(sink_h): a slot without key or value."""
    T, H, _ = q.shape
    idx = torch.arange(T)
    dist = idx[:, None] - idx[None, :]
    visible = dist >= 0
    if window is not None:
        visible &= dist < window
    out = q.new_zeros(T, H, v.shape[-1])
    for h in range(H):
        s = (q[:, h] @ k[:, h].T) * scale
        s = s.masked_fill(~visible, -math.inf)
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[h])
        e = torch.exp(s - m)
        out[:, h] = (e @ v[:, h]) / (e.sum(-1, keepdim=True) + torch.exp(sink[h] - m))
    return out


def latent_attention(h, p, spec, eps):
    """The mixer.  ``p``: tensors by their short names (dq, dq.norm, uq | q; dkv, dkv.norm, uk, uv, sink, g?, o).
    ``spec``: heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims, scaling?}, mask {size}? (no mask = causal)."""
    T = h.shape[0]
    H, dn, dr, dv, r = spec["heads"], spec["dim"], spec["rot_dim"], spec["vdim"], spec["kv_rank"]
    if "dq" in p:
        q = rms_norm(h @ p["dq"].T, p["dq.norm"], eps) @ p["uq"].T
    else:
        q = h @ p["q"].T
    q = q.reshape(T, H, dn + dr)
    ckr = h @ p["dkv"].T
    c = rms_norm(ckr[:, :r], p["dkv.norm"], eps)
    rot = spec["rot"]
    f, mult = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"), dtype=h.dtype)
    pos = torch.arange(T)
    kr = rotate_pairs(ckr[:, r:], pos, f, mult, rot["dims"])                       # [T, dr], one for all heads
    qr = rotate_pairs(q[:, :, dn:].transpose(0, 1), pos, f, mult, rot["dims"]).transpose(0, 1)
    kn = (c @ p["uk"].T).reshape(T, H, dn)
    v = (c @ p["uv"].T).reshape(T, H, dv)
    qq = torch.cat([q[:, :, :dn], qr], -1)
    kk = torch.cat([kn, kr[:, None, :].expand(T, H, dr)], -1)
    window = spec["mask"]["size"] if spec.get("mask") else None
    o = sink_softmax_attention(qq, kk, v, spec["scale"], window, p["sink"]).reshape(T, H * dv)
    if "g" in p:
        o = o * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    sp = torch.nn.functional.softplus
    pos = sp(p) * z * z + 0.5 * z
    neg = (0.5 + sp(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1 - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(h, p):
    return xielu(h @ p["up"].T + p["up.b"], p["act"][0], p["act"][1]) @ p["down"].T + p["down.b"]


def softmax_topk_moe(h, p, experts, top):
    """Router logits W_r h + b; the ``top`` largest are chosen; weights = softmax over the chosen logits; experts are
    gated feed-forwards W_down (silu(W_gate h) * (W_up h))."""
    z = h @ p["router"].T + p["router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(val, -1)
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            g = h[t] @ p[f"e{e}.gate"].T
            u = h[t] @ p[f"e{e}.up"].T
            out[t] += w[t, k] * ((torch.nn.functional.silu(g) * u) @ p[f"e{e}.down"].T)
    return out


def _sub(sd, prefix):
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def forward(sd: dict, config: dict, tokens, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one whole sequence.  ``sd``: checkpoint tensors by name; ``config``: the config.json dict."""
    sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x = sd["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."
        h = token_shift(x, sd[p + "shift"])
        a = latent_attention(h, _sub(sd, p + "mix."), layer["mixer"], eps)
        x = x + grouped_rms_norm(a, sd[p + "norm1"], eps, groups)
        f = layer.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                b = dense_ff(x, _sub(sd, p + "mlp."))
            else:
                b = softmax_topk_moe(x, _sub(sd, p + "mlp."), f["router"]["experts"], f["router"]["top"])
            x = x + grouped_rms_norm(b, sd[p + "norm2"], eps, groups)
        if layers_out is not None:
            layers_out.append(x.clone())
    return grouped_rms_norm(x, sd["final.norm"], eps, groups) @ sd["head"].T


# ------------------------------------------------------------------------------------------------ test material
def random_config(seed: int = 0, *, width=48, vocab=61, n_layers=4, heads=(3, 2), dim=(8, 16), rot_dim=(8, 4), rot_dims=None,
                  vdim=(16, 8), kv_rank=(24, 16), q_rank=12, window=9, groups=2, ff=40, expert_ff=24, experts=5, top=2,
                  kinds=("dense", "moe", None, "moe"), types=("latent_attention_2", "latent_attention"), share=None,
                  scaling=True, embedding_scale=3.0, eps=1e-5) -> dict:
    """A small config.json dict.  ``types`` / ``kinds`` cycle over the layers; index 0 of the size pairs belongs to
    "latent_attention_2", index 1 to "latent_attention".  ``share`` = {layer: earlier layer whose tensors it reuses}."""
    layers = []
    for i in range(n_layers):
        t = types[i % len(types)]
        k = 1 if t == "latent_attention" else 0
        rd = rot_dim[k]
        mixer = {"heads": heads[k], "dim": dim[k], "rot_dim": rd, "vdim": vdim[k], "kv_rank": kv_rank[k],
                 "scale": (dim[k] + rd) ** -0.5 * (1.0 + 0.25 * k),
                 "rot": {"base": 10000.0 if k == 0 else 500.0, "dims": rd if rot_dims is None else rot_dims[k]}}
        if k == 1:
            mixer["q_rank"] = q_rank
            mixer["mask"] = {"size": window}
            if scaling:
                mixer["rot"]["scaling"] = {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 0.5}
        kind = kinds[i % len(kinds)]
        mlp = None
        if kind == "dense":
            mlp = {"kind": "dense", "ff": ff}
        elif kind == "moe":
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
        layers.append({"type": t, "mixer": mixer, "mlp": mlp})
    for i, j in (share or {}).items():
        layers[i] = dict(layers[j], weights_of=j)
    return {"architecture": "Ridevik", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale},
            "norm": {"eps": eps, "groups": groups}, "layers": layers}


def random_weights(config: dict, seed: int = 0) -> dict:
    """Random tensors under the checkpoint's names, rounded to bfloat16 values (held as float64)."""
    g = torch.Generator().manual_seed(seed)
    D = config["width"]

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16).double()

    sd = {"embed": rnd(config["vocab"], D, std=0.5), "final.norm": rnd(D, mean=1.0, std=0.2), "head": rnd(config["vocab"], D, std=D ** -0.5)}
    for i, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        m, p = layer["mixer"], f"l{i}."
        H, hd, r = m["heads"], m["dim"] + m["rot_dim"], m["kv_rank"]
        sd[p + "shift"] = torch.rand(D, generator=g).to(torch.bfloat16).double()
        sd[p + "norm1"] = rnd(D, mean=0.6, std=0.2)
        if "q_rank" in m:
            sd[p + "mix.dq"] = rnd(m["q_rank"], D, std=D ** -0.5)
            sd[p + "mix.dq.norm"] = rnd(m["q_rank"], mean=1.0, std=0.2)
            sd[p + "mix.uq"] = rnd(H * hd, m["q_rank"], std=2 * m["q_rank"] ** -0.5)
        else:
            sd[p + "mix.q"] = rnd(H * hd, D, std=2 * D ** -0.5)
        sd[p + "mix.dkv"] = rnd(r + m["rot_dim"], D, std=D ** -0.5)
        sd[p + "mix.dkv.norm"] = rnd(r, mean=1.0, std=0.2)
        sd[p + "mix.uk"] = rnd(H * m["dim"], r, std=2 * r ** -0.5)
        sd[p + "mix.uv"] = rnd(H * m["vdim"], r, std=r ** -0.5)
        sd[p + "mix.sink"] = rnd(H, std=1.5)
        if layer["type"] == "latent_attention":
            sd[p + "mix.g"] = rnd(H * m["vdim"], D, std=D ** -0.5)
        sd[p + "mix.o"] = rnd(D, H * m["vdim"], std=(H * m["vdim"]) ** -0.5)
        f = layer["mlp"]
        if f is None:
            continue
        sd[p + "norm2"] = rnd(D, mean=0.6, std=0.2)
        if f["kind"] == "dense":
            sd[p + "mlp.up"] = rnd(f["ff"], D, std=D ** -0.5)
            sd[p + "mlp.up.b"] = rnd(f["ff"], std=0.3)
            sd[p + "mlp.down"] = rnd(D, f["ff"], std=f["ff"] ** -0.5)
            sd[p + "mlp.down.b"] = rnd(D, std=0.3)
            sd[p + "mlp.act"] = rnd(2, std=0.7)
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            sd[p + "mlp.router"] = rnd(E, D, std=D ** -0.5)
            sd[p + "mlp.router.b"] = rnd(E, std=0.3)
            for e in range(E):
                sd[f"{p}mlp.e{e}.gate"] = rnd(ff, D, std=D ** -0.5)
                sd[f"{p}mlp.e{e}.up"] = rnd(ff, D, std=D ** -0.5)
                sd[f"{p}mlp.e{e}.down"] = rnd(D, ff, std=ff ** -0.5)
    return sd
