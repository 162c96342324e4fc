"""A plain, slow implementation of the Fasolorn decoder in float64: one function per mechanism,
whole sequences at once, no code shared with the package.

``weights`` maps the names of the design's own weight file (``embed``, ``l0.mix.q``,
``l1.mlp.e3.up``, ...) to tensors; ``config`` is the design's config.json as a dict.

Notation.  The stream starts as ``x = E[token] * embedding.scale``; a layer is

    x += mixer(N1(x));   x += ff(N2(x))      (the second line only where the layer has a feed-forward)

with N an RMS norm with a weight; the logits are ``E N(x)``.  Two mixers.  ``attention``: grouped
queries, interleaved rotary pairs over the first values of a head, a window, a softmax whose
denominator also holds ``exp(sink_h)``, values blended with the values the first blending layer made
for the same token, heads multiplied by ``sigmoid(W_g h)``.  ``latent_attention``: keys and values are
products of a cached normed latent, with one rotated key part (pairs ``(i, i + r/2)``) shared by the
heads, a window and a plain softmax.  Feed-forwards: a gated unit with silu, or a mixture of
``relu(.)^2`` units chosen by softmax scores plus a correction, some of whose experts return their
input, beside a shared unit.
"""
import math

import torch

F = torch.float64


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def frequencies(dims, base):
    """f_i = base^(-2i/dims), i < dims/2."""
    return float(base) ** (-2.0 * torch.arange(dims // 2, dtype=F) / dims)


def _angles(x, positions, dims, base):
    angle = positions.to(F)[:, None] * frequencies(dims, base)[None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return cos, sin


def rotate_interleaved(x, positions, rot):
    """x [T, ..., d]: values (2i, 2i + 1) of the first rot.dims turn by position * f_i; the rest stay."""
    dims = int(rot["dims"])
    cos, sin = _angles(x, positions, dims, rot["base"])
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def rotate_halves(x, positions, rot):
    """x [T, ..., d]: values (i, i + dims/2) of the first rot.dims turn by position * f_i; the rest stay."""
    dims = int(rot["dims"])
    half = dims // 2
    cos, sin = _angles(x, positions, dims, rot["base"])
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def visible(count, mask):
    """visible[i, j]: 0 <= i - j < mask.size (every j <= i without a mask)."""
    i = torch.arange(count)[:, None]
    j = torch.arange(count)[None, :]
    seen = j <= i
    if mask is not None:
        seen = seen & (i - j < int(mask["size"]))
    return seen


def softmax_with_sink(scores, seen, sink):
    """scores [H, T, T]; the denominator also holds exp(sink_h), a term that stands for no token.  Without a sink
    (None) an ordinary softmax."""
    scores = scores.masked_fill(~seen, float("-inf"))
    top = scores.max(dim=-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.to(F)[:, None, None])
    weights = torch.exp(scores - top)
    total = weights.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink.to(F)[:, None, None] - top)
    return weights / total


def attention_values(h, w, prefix):
    """The values a layer projects, before any blending: [T, kv_heads * vdim]."""
    return h @ w[f"{prefix}.v"].to(F).T


def attention(h, w, prefix, mixer, value):
    """h [T, width]; `value` [T, kv_heads * vdim] are the (blended) values of this layer."""
    heads, groups, d, dv = (int(mixer[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
    count = h.shape[0]
    positions = torch.arange(count)
    q = (h @ w[f"{prefix}.q"].to(F).T).reshape(count, heads, d)
    k = (h @ w[f"{prefix}.k"].to(F).T).reshape(count, groups, d)
    if mixer.get("rot") is not None:
        q = rotate_interleaved(q, positions, mixer["rot"])
        k = rotate_interleaved(k, positions, mixer["rot"])
    v = value.reshape(count, groups, dv)
    per = heads // groups
    k = k.repeat_interleave(per, dim=1)
    v = v.repeat_interleave(per, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(mixer["scale"])
    weights = softmax_with_sink(scores, visible(count, mixer.get("mask")), w[f"{prefix}.sink"])
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(count, heads * dv)
    out = out * torch.sigmoid(h @ w[f"{prefix}.g"].to(F).T)
    return out @ w[f"{prefix}.o"].to(F).T


def latent_attention(h, w, prefix, mixer, eps):
    heads, d, dr, dv, rank = (int(mixer[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    count = h.shape[0]
    positions = torch.arange(count)
    q = (h @ w[f"{prefix}.q"].to(F).T).reshape(count, heads, d + dr)
    down = h @ w[f"{prefix}.dkv"].to(F).T
    latent = rms_norm(down[:, :rank], w[f"{prefix}.dkv.norm"].to(F), eps)
    key_rot = rotate_halves(down[:, rank:], positions, mixer["rot"])
    q_rot = rotate_halves(q[..., d:], positions, mixer["rot"])
    key = (latent @ w[f"{prefix}.uk"].to(F).T).reshape(count, heads, d)
    value = (latent @ w[f"{prefix}.uv"].to(F).T).reshape(count, heads, dv)
    scores = torch.einsum("ihd,jhd->hij", q[..., :d], key) + torch.einsum("ihd,jd->hij", q_rot, key_rot)
    weights = softmax_with_sink(scores * float(mixer["scale"]), visible(count, mixer.get("mask")), None)
    out = torch.einsum("hij,jhd->ihd", weights, value).reshape(count, heads * dv)
    return out @ w[f"{prefix}.o"].to(F).T


def dense_ff(h, w, prefix):
    gate = h @ w[f"{prefix}.gate"].to(F).T
    return (gate * torch.sigmoid(gate) * (h @ w[f"{prefix}.up"].to(F).T)) @ w[f"{prefix}.down"].to(F).T


def squared_relu_unit(h, w, prefix):
    return torch.relu(h @ w[f"{prefix}.up"].to(F).T) ** 2 @ w[f"{prefix}.down"].to(F).T


def route(h, w, prefix, router):
    """(chosen [T, top], weights [T, top], margin [T]): the experts with the largest score + correction,
    weighted by their scores over the scores' sum, times router.scale.  The margin is the gap between
    the last chosen and the best expert left out."""
    top = int(router["top"])
    scores = torch.softmax(h @ w[f"{prefix}.router"].to(F).T, dim=-1)
    choice = scores + w[f"{prefix}.correction"].to(F)
    ranked = choice.sort(dim=-1, descending=True)
    chosen = ranked.indices[:, :top]
    margin = ranked.values[:, top - 1] - ranked.values[:, top] if top < scores.shape[1] else \
        torch.full((h.shape[0],), float("inf"), dtype=F)
    picked = torch.gather(scores, 1, chosen)
    weights = picked / (picked.sum(-1, keepdim=True) + 1e-20) * float(router.get("scale", 1.0))
    return chosen, weights, margin


def mixture(h, w, prefix, mlp, margins=None):
    router = mlp["router"]
    real = int(router["experts"])   # the router's outputs beyond these return their input
    chosen, weights, margin = route(h, w, prefix, router)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weights[t]):
            out[t] += s * (h[t] if e >= real else squared_relu_unit(h[t], w, f"{prefix}.e{e}"))
    if mlp.get("shared") is not None:
        out = out + squared_relu_unit(h, w, f"{prefix}.shared")
    return out


def forward(config, weights, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one sequence; with `return_layers` also the stream after every layer.  A list
    given as `margins` receives every router's margin [T]."""
    w = weights
    eps = float(config["norm"]["eps"])
    x = w["embed"].to(F)[torch.tensor(tokens)] * float(config.get("embedding", {}).get("scale", 1.0))
    first_values, streams = None, []
    for index, layer in enumerate(config["layers"]):
        p, mixer = f"l{index}", layer["mixer"]
        h = rms_norm(x, w[f"{p}.norm1"].to(F), eps)
        if layer["type"] == "attention":
            value = attention_values(h, w, f"{p}.mix")
            if mixer.get("v_mix"):
                if first_values is None:
                    first_values = value
                else:
                    blend = w[f"{p}.mix.vmix"].to(F)
                    value = (1.0 - blend) * value + blend * first_values
            x = x + attention(h, w, f"{p}.mix", mixer, value)
        elif layer["type"] == "latent_attention":
            x = x + latent_attention(h, w, f"{p}.mix", mixer, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[f"{p}.norm2"].to(F), eps)
            x = x + (dense_ff(h, w, f"{p}.mlp") if mlp["kind"] == "dense" else mixture(h, w, f"{p}.mlp", mlp, margins))
        streams.append(x.clone())
    logits = rms_norm(x, w["final.norm"].to(F), eps) @ w["embed"].to(F).T
    return (logits, torch.stack(streams)) if return_layers else logits
