"""A plain, slow, cache-less statement of the Toposun decoder, one function per mechanism.

Everything works on whole sequences ``[T, ...]`` with torch's elementary operations in the
dtype of the tensors it is given (the tests use float64 or float32); nothing here is shared
with the product path.  ``cfg`` is the dict a model folder's config.json holds, ``w`` a dict
from tensor name to tensor.
"""
from __future__ import annotations

import math

import torch


def layer_norm_scale_only(x, weight, eps):
    """Centre, divide by the root of the biased variance plus eps, multiply by a weight; no shift."""
    mean = x.mean(-1, keepdim=True)
    centred = x - mean
    var = (centred * centred).mean(-1, keepdim=True)
    return centred / torch.sqrt(var + eps) * weight


def rms_over_projection(x, weight, eps):
    """``x / sqrt(mean(x^2) + eps) * weight`` with the mean over the whole last axis (all heads at once)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def rotate_leading_dims(x, positions, base, dims):
    """Half-layout rotation of the first ``dims`` entries of each head of ``x [T, heads, D]``:
    entry i pairs with entry i + dims/2 and turns by ``position * base^(-2i/dims)``."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)).to(torch.float32)          # 32-bit table, as served
    angle = positions.to(torch.float32)[:, None] * freq[None, :]          # 32-bit angles
    cos, sin = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def visible(num_tokens, window, keep_first):
    """``[T, T]`` mask: query i sees key j when j <= i and (i - j < window or j < keep_first)."""
    i = torch.arange(num_tokens)[:, None]
    j = torch.arange(num_tokens)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def attention_mixer(h, w, prefix, m, eps, positions=None):
    """Grouped-query attention whose values are the raw key projection."""
    tokens = h.shape[0]
    heads, kv_heads, dim = m["heads"], m["kv_heads"], m["dim"]
    positions = torch.arange(tokens) if positions is None else positions
    q = h @ w[f"{prefix}.q"].T + w[f"{prefix}.q.b"]
    k = h @ w[f"{prefix}.k"].T + w[f"{prefix}.k.b"]
    v = k.view(tokens, kv_heads, dim)
    q = rms_over_projection(q, w[f"{prefix}.q.norm"], eps).view(tokens, heads, dim)
    k = rms_over_projection(k, w[f"{prefix}.k.norm"], eps).view(tokens, kv_heads, dim)
    q = rotate_leading_dims(q, positions, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_leading_dims(k, positions, m["rot"]["base"], m["rot"]["dims"])
    mask = visible(tokens, m["mask"]["size"], m["mask"]["keep_first"])
    group = heads // kv_heads
    out = torch.empty(tokens, heads, dim, dtype=h.dtype)
    for head in range(heads):
        g = head // group
        scores = (q[:, head] @ k[:, g].T) * m["scale"]
        scores = scores.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, g]
    return out.reshape(tokens, heads * dim) @ w[f"{prefix}.o"].T + w[f"{prefix}.o.b"]


def clamped_gated_ff(h, w, prefix, limit):
    """``down(g * sigmoid(1.702 g) * (u + 1))`` with g capped above and u clamped on both sides."""
    g = torch.clamp(h @ w[f"{prefix}.gate"].T, max=limit)
    u = torch.clamp(h @ w[f"{prefix}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{prefix}.down"].T


def silu_gated_ff(h, w, prefix):
    g = h @ w[f"{prefix}.gate"].T
    return (g * torch.sigmoid(g) * (h @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def route(h, router_weight, top):
    """Sigmoid scores, the ``top`` largest per token: (expert ids [T, top], their scores)."""
    scores = torch.sigmoid(h @ router_weight.T)
    values, ids = torch.topk(scores, top, dim=-1)
    return ids, values


def mixture_ff(h, w, prefix, mlp, margins=None):
    """Routed experts fed with ``score * h`` (scores not renormalised) plus a gated shared expert.
    ``margins`` (a list) receives, per token, the gap between the last chosen and the first unchosen score."""
    ids, scores = route(h, w[f"{prefix}.router"], mlp["router"]["top"])
    if margins is not None and mlp["router"]["top"] < mlp["router"]["experts"]:
        ordered = torch.sigmoid(h @ w[f"{prefix}.router"].T).sort(dim=-1, descending=True).values
        margins.append(ordered[:, mlp["router"]["top"] - 1] - ordered[:, mlp["router"]["top"]])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), scores[t]):
            out[t] += silu_gated_ff((s * h[t])[None], w, f"{prefix}.e{e}")[0]
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(h @ w[f"{prefix}.shared.sg"].T)            # [T, 1]
        out = out + gate * silu_gated_ff(h, w, f"{prefix}.shared")
    return out


def feed_forward(h, w, prefix, mlp, margins=None):
    if mlp["kind"] == "dense":
        return clamped_gated_ff(h, w, prefix, mlp["limit"])
    if mlp["kind"] == "moe":
        return mixture_ff(h, w, prefix, mlp, margins)
    raise ValueError(mlp["kind"])


def layer(x, w, index, spec, eps, positions=None, margins=None):
    """Both sub-layers read the same stream: ``x + (mixer(norm1 x) + ff(norm2 x))``."""
    prefix = f"l{index}"
    if spec["type"] != "attention":
        raise ValueError(spec["type"])
    a = attention_mixer(layer_norm_scale_only(x, w[f"{prefix}.norm1"], eps), w, f"{prefix}.mix",
                        spec["mixer"], eps, positions)
    if spec.get("mlp") is None:
        return x + a
    f = feed_forward(layer_norm_scale_only(x, w[f"{prefix}.norm2"], eps), w, f"{prefix}.mlp", spec["mlp"], margins)
    return x + (a + f)


def forward(cfg, w, tokens, collect=None, margins=None):
    """Logits ``[T, vocab]`` of one sequence; ``collect`` (a list) receives the stream after each layer,
    ``margins`` (a list) every mixture layer's per-token gap between chosen and unchosen scores."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for index, spec in enumerate(cfg["layers"]):
        x = layer(x, w, index, spec, eps, margins=margins)
        if collect is not None:
            collect.append(x)
    return layer_norm_scale_only(x, w["final.norm"], eps) @ w["embed"].T


def random_weights(cfg, seed, dtype=torch.float32, std=0.08):
    """Random tensors under the design's names (bf16-representable values, so that a bfloat16 model
    folder and this oracle hold the same numbers)."""
    gen = torch.Generator().manual_seed(seed)
    width = cfg["width"]

    def mat(*shape, scale=std):
        return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16).to(dtype)

    def around_one(n):
        return (1.0 + 0.1 * torch.randn(n, generator=gen)).to(torch.bfloat16).to(dtype)

    w = {"embed": mat(cfg["vocab"], width, scale=0.5), "final.norm": around_one(width)}
    for index, spec in enumerate(cfg["layers"]):
        p, m = f"l{index}", spec["mixer"]
        q_rows, k_rows = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
        w[f"{p}.norm1"] = around_one(width)
        w[f"{p}.mix.q"], w[f"{p}.mix.q.b"] = mat(q_rows, width), mat(q_rows)
        w[f"{p}.mix.k"], w[f"{p}.mix.k.b"] = mat(k_rows, width), mat(k_rows)
        w[f"{p}.mix.q.norm"], w[f"{p}.mix.k.norm"] = around_one(q_rows), around_one(k_rows)
        w[f"{p}.mix.o"], w[f"{p}.mix.o.b"] = mat(width, m["heads"] * m["vdim"]), mat(width)
        mlp = spec.get("mlp")
        if mlp is None:
            continue
        w[f"{p}.norm2"] = around_one(width)

        def gated(prefix, ff):
            w[f"{prefix}.gate"], w[f"{prefix}.up"], w[f"{prefix}.down"] = mat(ff, width), mat(ff, width), mat(width, ff)

        if mlp["kind"] == "dense":
            gated(f"{p}.mlp", mlp["ff"])
        else:
            for e in range(mlp["router"]["experts"]):
                gated(f"{p}.mlp.e{e}", mlp["expert"]["ff"])
            w[f"{p}.mlp.router"] = mat(mlp["router"]["experts"], width, scale=0.3)
            if mlp.get("shared") is not None:
                gated(f"{p}.mlp.shared", mlp["shared"]["ff"])
                w[f"{p}.mlp.shared.sg"] = mat(1, width)
    return w


def attention_layer_config(heads=4, kv_heads=2, dim=16, window=8, keep_first=2, rot_dims=8, base=10000.0,
                           scale=None, mlp=None):
    return {"type": "attention",
            "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": dim,
                      "mask": {"keep_first": keep_first, "size": window},
                      "rot": {"base": base, "dims": rot_dims},
                      "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))},
            "mlp": mlp}


def dense_mlp(ff, limit=7.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe_mlp(experts, top, ff, shared_ff=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff is not None:
        out["shared"] = {"ff": shared_ff}
    return out


def model_config(layers, vocab=96, width=32, eps=1e-5):
    return {"architecture": "Toposun", "layers": list(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width}
