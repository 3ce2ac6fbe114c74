"""The Pipesun decoder stated plainly: whole sequences, no cache, no batching, one function per mechanism.

Written from the design's equations in this file's own notation; it shares no code with the product.
``forward(config, weights, tokens)`` returns the logits at every position (in the dtype of the weights:
tests use float64).  Notation: T tokens, E stream width, H heads, G key/value heads, D query/key size,
V value size, C latent size, R size of the turned part.
"""
from __future__ import annotations

import math

import torch


# ---- configurations and weights of the tests --------------------------------------------------------
def differential_layer(*, heads, kv_heads, dim, vdim, diff=0.4, scale=None, kv_from=None, ff=48):
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, diff=diff,
                 scale=scale if scale is not None else dim ** -0.5)
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return dict(type="attention", mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def latent_layer(*, heads, dim, rot_dim, vdim, kv_rank, rot_dims=None, base=10000.0, scale=None, ff=48):
    mixer = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
                 rot=dict(base=base, dims=rot_dim if rot_dims is None else rot_dims),
                 scale=scale if scale is not None else (dim + rot_dim) ** -0.5)
    return dict(type="latent_attention", mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def model_config(layers, *, vocab, width, eps=1e-5):
    return dict(architecture="Pipesun", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)


def tensor_shapes(cfg):
    E = cfg["width"]
    shapes = {"embed": (cfg["vocab"], E), "final.norm": (E,), "head": (cfg["vocab"], E)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes.update({p + "norm1": (E,), p + "norm1b": (E,), p + "shift": (E,), p + "dwa": (i + 2,)})
        if layer["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (2 * H * D, E), p + "mix.q.b": (2 * H * D,), p + "mix.q.norm": (D,),
                           p + "mix.o": (E, H * V)})
            shapes.update({p + f"mix.{n}": (D,) for n in ("lq1", "lk1", "lq2", "lk2")})
            if "kv_from" not in m:
                shapes.update({p + "mix.k": (2 * G * D, E), p + "mix.k.b": (2 * G * D,), p + "mix.k.norm": (D,),
                               p + "mix.v": (G * V, E), p + "mix.v.b": (G * V,)})
        else:
            H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * (D + R), E), p + "mix.dkv": (C + R, E), p + "mix.dkv.norm": (C,),
                           p + "mix.uk": (H * D, C), p + "mix.uv": (H * V, C), p + "mix.sink": (H,),
                           p + "mix.g": (H * V, E), p + "mix.o": (E, H * V)})
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            shapes.update({p + "norm2": (E,), p + "norm2b": (E,), p + "mlp.gate": (F, E), p + "mlp.up": (F, E),
                           p + "mlp.down": (E, F)})
    return shapes


def random_weights(cfg, seed, dtype=torch.float32):
    """Random tensors that bfloat16 holds exactly; scales chosen so that every mechanism moves the logits."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1", "norm2", "norm1b", "norm2b"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif leaf == "shift":
            t = torch.rand(shape, generator=gen)
        elif leaf == "dwa":
            t = torch.randn(shape, generator=gen) * 0.3
            t[-1] += 1.0
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = torch.randn(shape, generator=gen) * 0.3
        elif leaf in ("sink", "b"):
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) * (2.0 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16).to(dtype)
    return out


# ---- mechanisms ------------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / torch.sqrt(torch.mean(x * x, dim=-1, keepdim=True) + eps)


def shift_towards_previous(y, mix):
    """y_t + (y_{t-1} - y_t) * mix, with zeros in front of the first token."""
    previous = torch.zeros_like(y)
    previous[1:] = y[:-1]
    return y + (previous - y) * mix


def causal_weights(scores, sink=None):
    """Softmax over the keys j <= i of scores [heads, T, T]; ``sink`` [heads] joins every denominator once."""
    T = scores.shape[-1]
    hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    scores = scores.masked_fill(hidden, -math.inf)
    top = scores.amax(-1, keepdim=True)
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(scores - top)
    total = e.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink[:, None, None] - top)
    return e / total


def turn_pairs(x, positions, base, dims):
    """Entries (2i, 2i+1), i < dims/2, of the last axis turned by positions * base^(-2i/dims); x [T, ..., n]."""
    out = x.clone()
    if dims == 0:
        return out
    i = torch.arange(dims // 2, dtype=torch.float64)
    angle = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (dims // 2,)
    c, s = torch.cos(angle).reshape(shape).to(x.dtype), torch.sin(angle).reshape(shape).to(x.dtype)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def differential_keys_values(y, w, p, m, eps):
    T, G, D, V = y.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = (y @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, 2, D)
    v = (y @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, V)
    return unit_rms(k, eps) * w[p + "k.norm"], v


def differential_attention(y, w, p, m, eps, keys_values):
    T, H, G, D, V = y.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((y @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, 2, D), eps) * w[p + "q.norm"]
    k, v = keys_values
    per = H // G
    lam = (torch.exp(torch.dot(w[p + "lq1"], w[p + "lk1"])) - torch.exp(torch.dot(w[p + "lq2"], w[p + "lk2"]))
           + m["diff"])
    heads = []
    for h in range(H):
        g = h // per
        a = [causal_weights((q[:, h, n] @ k[:, g, n].T)[None] * m["scale"])[0] @ v[:, g] for n in range(2)]
        heads.append(unit_rms(a[0] - lam * a[1], eps) * (1.0 - m["diff"]))
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def latent_attention(y, w, p, m, eps):
    T, H, D, R, V, C = y.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    q = (y @ w[p + "q"].T).reshape(T, H, D + R)
    down = y @ w[p + "dkv"].T
    latent = unit_rms(down[:, :C], eps) * w[p + "dkv.norm"]
    shared = turn_pairs(down[:, C:], positions, m["rot"]["base"], m["rot"]["dims"])            # [T, R]
    q_turned = turn_pairs(q[:, :, D:], positions, m["rot"]["base"], m["rot"]["dims"])          # [T, H, R]
    keys = (latent @ w[p + "uk"].T).reshape(T, H, D)
    values = (latent @ w[p + "uv"].T).reshape(T, H, V)
    scores = torch.stack([q[:, h, :D] @ keys[:, h].T + q_turned[:, h] @ shared.T for h in range(H)]) * m["scale"]
    weights = causal_weights(scores, w[p + "sink"])
    mixed = torch.cat([weights[h] @ values[:, h] for h in range(H)], dim=-1)
    return (mixed * torch.sigmoid(y @ w[p + "g"].T)) @ w[p + "o"].T


def gated_feed_forward(y, w, p):
    gate = y @ w[p + "gate"].T
    return (gate * torch.sigmoid(gate) * (y @ w[p + "up"].T)) @ w[p + "down"].T


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab].  ``streams``: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    results = [x]
    keys_values = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        y = shift_towards_previous(unit_rms(x, eps) * w[p + "norm1"], w[p + "shift"])
        if layer["type"] == "attention":
            source = m.get("kv_from")
            keys_values[i] = (keys_values[source] if source is not None
                              else differential_keys_values(y, w, p + "mix.", m, eps))
            mixed = differential_attention(y, w, p + "mix.", m, eps, keys_values[i])
        else:
            mixed = latent_attention(y, w, p + "mix.", m, eps)
        x = x + unit_rms(mixed, eps) * w[p + "norm1b"]
        if layer["mlp"] is not None:
            x = x + unit_rms(gated_feed_forward(unit_rms(x, eps) * w[p + "norm2"], w, p + "mlp."), eps) * w[p + "norm2b"]
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    return (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
