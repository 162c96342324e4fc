"""A plain, slow implementation of the Pugovik decoder in float64: one function per mechanism,
whole sequences at once (the recurrence token by token), no code shared with the package.

``weights`` maps the names of the design's own weight file (``embed``, ``l0.mix.q``,
``l0.rg1.b``, ...) to tensors; ``config`` is the design's config.json as a dict.

Notation.  With m the residual multiplier, a layer is

    h = N1(x);  y = mixer(h) * sigmoid(R1 h + r1);  x += m * (N1b(y) * s1)
    h = N2(x);  y = ff(h)    * sigmoid(R2 h + r2);  x += m * (N2b(y) * s2)

where every N is an RMS norm over equal consecutive groups of the row.  Mixers: attention over a
cached latent (each head's unrotated keys and its values are products of the latent, one rotated
key part is shared by the heads; interleaved rotary pairs with YaRN frequencies; an output
gate), and linear attention with one constant decay per head.  The feed-forward is a mixture of
gated units chosen by sigmoid scores within the best groups of experts.
"""
import math

import torch

F = torch.float64


def silu(x):
    return x * torch.sigmoid(x)


def grouped_rms_norm(x, weight, eps, groups):
    """Each of `groups` equal consecutive parts of a row is divided by its own root mean square."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(x.shape) * weight


def rotary_frequencies(dims, base, scaling):
    """Frequencies of the dims/2 pairs; YaRN blends each with its slowed form by a ramp over the
    pair index.  Returns (frequencies, stretch of cos and sin)."""
    index = torch.arange(dims // 2, dtype=F)
    freq = base ** (-2.0 * index / dims)
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    high = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((index - low) / max(high - low, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, rot):
    """x [T, ..., d]: values (2i, 2i + 1) of the first rot.dims turn by position * f_i."""
    dims = int(rot["dims"])
    freq, stretch = rotary_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle) * stretch, torch.sin(angle) * stretch
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_and_key(h, w, prefix, mixer, eps):
    """What a latent-attention layer caches: the normed latent [T, rank] and the rotated shared key
    part [T, rot_dim]."""
    rank = int(mixer["kv_rank"])
    positions = torch.arange(h.shape[0])
    down = h @ w[f"{prefix}.dkv"].to(F).T
    latent = down[:, :rank]
    latent = latent / torch.sqrt((latent * latent).mean(-1, keepdim=True) + eps) * w[f"{prefix}.dkv.norm"].to(F)
    return latent, rotate_pairs(down[:, rank:], positions, mixer["rot"])


def latent_attention(h, w, prefix, mixer, eps, kept):
    """h [T, width]; `kept` = (latent, rotated key) of the layer whose cache this layer reads."""
    heads, d, dr, dv = (int(mixer[k]) for k in ("heads", "dim", "rot_dim", "vdim"))
    count = h.shape[0]
    latent, key_rot = kept
    q = (h @ w[f"{prefix}.q"].to(F).T).reshape(count, heads, d + dr)
    q_plain = q[..., :d]
    q_rot = rotate_pairs(q[..., d:], torch.arange(count), mixer["rot"])
    k_plain = (latent @ w[f"{prefix}.uk"].to(F).T).reshape(count, heads, d)
    value = (latent @ w[f"{prefix}.uv"].to(F).T).reshape(count, heads, dv)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, key_rot)
    scores = scores * float(mixer["scale"])
    visible = torch.tril(torch.ones(count, count, dtype=torch.bool))
    scores = scores.masked_fill(~visible, float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", weights, value).reshape(count, heads * dv)
    out = out * torch.sigmoid(h @ w[f"{prefix}.g"].to(F).T)
    return out @ w[f"{prefix}.o"].to(F).T


def lightning(h, w, prefix, mixer, eps):
    """Linear attention token by token: S = decay_h S + k v^T, o = S^T q, S zero at the start."""
    heads, d, dv = (int(mixer[k]) for k in ("heads", "dim", "vdim"))
    count = h.shape[0]
    q = silu(h @ w[f"{prefix}.q"].to(F).T).reshape(count, heads, d)
    k = silu(h @ w[f"{prefix}.k"].to(F).T).reshape(count, heads, d)
    v = silu(h @ w[f"{prefix}.v"].to(F).T).reshape(count, heads, dv)
    decay = torch.tensor([float(x) for x in mixer["decay"]], dtype=F)
    state = torch.zeros(heads, d, dv, dtype=F)
    out = torch.zeros(count, heads, dv, dtype=F)
    for t in range(count):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    out = out.reshape(count, heads * dv)
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w[f"{prefix}.norm"].to(F)
    out = out * torch.sigmoid(h @ w[f"{prefix}.g"].to(F).T)
    return out @ w[f"{prefix}.o"].to(F).T


def route(scores, top, group_count, keep):
    """scores [T, experts] -> (chosen expert indices [T, top], their weights).  A group's score is the
    sum of its two largest scores (its only one where groups hold one expert); experts outside the
    `keep` best groups cannot be chosen."""
    count, experts = scores.shape
    per_group = experts // group_count
    grouped = scores.reshape(count, group_count, per_group)
    group_score = grouped.topk(min(2, per_group), dim=-1).values.sum(-1)
    best = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(count, group_count, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = grouped.masked_fill(~allowed[:, :, None], float("-inf")).reshape(count, experts)
    chosen = masked.topk(top, dim=-1).indices
    return chosen, torch.gather(scores, 1, chosen)


def route_margin(scores, top, group_count, keep):
    """Per token, how far the choice is from another one: the smaller of the gap between the last
    kept group's score and the best dropped one's, and the gap between the last chosen expert's
    score and the best allowed one left out (infinite where there is no such rival)."""
    count, experts = scores.shape
    per_group = experts // group_count
    grouped = scores.reshape(count, group_count, per_group)
    group_score = grouped.topk(min(2, per_group), dim=-1).values.sum(-1)
    margin = torch.full((count,), float("inf"), dtype=scores.dtype)
    order = group_score.sort(dim=-1, descending=True)
    if keep < group_count:
        margin = torch.minimum(margin, order.values[:, keep - 1] - order.values[:, keep])
    allowed = torch.zeros(count, group_count, dtype=torch.bool)
    allowed.scatter_(1, order.indices[:, :keep], True)
    masked = grouped.masked_fill(~allowed[:, :, None], float("-inf")).reshape(count, experts)
    if top < keep * per_group:
        ranked = masked.sort(dim=-1, descending=True).values
        margin = torch.minimum(margin, ranked[:, top - 1] - ranked[:, top])
    return margin


def mixture(h, w, prefix, mlp, margins=None):
    router = mlp["router"]
    scores = torch.sigmoid(h @ w[f"{prefix}.router"].to(F).T)
    chosen, weight = route(scores, int(router["top"]), int(router["groups"]["count"]), int(router["groups"]["keep"]))
    if margins is not None:
        margins.append(route_margin(scores, int(router["top"]), int(router["groups"]["count"]), int(router["groups"]["keep"])))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weight[t]):
            gate, up, down = (w[f"{prefix}.e{e}.{n}"].to(F) for n in ("gate", "up", "down"))
            out[t] += s * (down @ (silu(gate @ h[t]) * (up @ h[t])))
    return out


def forward(config, weights, tokens, return_layers=False, margins=None):
    """Logits [T, vocab] of one sequence; with `return_layers` also the stream after every layer.  A list
    given as `margins` receives every mixture's route_margin [T]."""
    w = weights
    eps, groups = float(config["norm"]["eps"]), int(config["norm"]["groups"])
    mult = float(config["residual_mult"])

    def norm(x, name):
        return grouped_rms_norm(x, w[name].to(F), eps, groups)

    x = norm(w["embed"].to(F)[torch.tensor(tokens)], "embed.norm")
    kept, streams = {}, []
    for index, layer in enumerate(config["layers"]):
        p, mixer = f"l{index}", layer["mixer"]
        h = norm(x, f"{p}.norm1")
        if layer["type"] == "latent_attention":
            source = mixer.get("kv_from")
            if source is None:
                kept[index] = latent_and_key(h, w, f"{p}.mix", mixer, eps)
                source = index
            y = latent_attention(h, w, f"{p}.mix", mixer, eps, kept[source])
        elif layer["type"] == "lightning":
            y = lightning(h, w, f"{p}.mix", mixer, eps)
        else:
            raise ValueError(layer["type"])
        y = y * torch.sigmoid(h @ w[f"{p}.rg1"].to(F).T + w[f"{p}.rg1.b"].to(F))
        x = x + mult * (norm(y, f"{p}.norm1b") * w[f"{p}.ls1"].to(F))
        if layer.get("mlp") is not None:
            h = norm(x, f"{p}.norm2")
            y = mixture(h, w, f"{p}.mlp", layer["mlp"], margins)
            y = y * torch.sigmoid(h @ w[f"{p}.rg2"].to(F).T + w[f"{p}.rg2.b"].to(F))
            x = x + mult * (norm(y, f"{p}.norm2b") * w[f"{p}.ls2"].to(F))
        streams.append(x.clone())
    logits = norm(x, "final.norm") @ w["head"].to(F).T
    return (logits, torch.stack(streams)) if return_layers else logits
