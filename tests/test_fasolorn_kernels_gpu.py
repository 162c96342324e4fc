"""The kernels' options that Fasolorn brought, each alone against a plain 64-bit restatement of the same
operation: attention with a learned sink and an output gate (the general kernel, the tcgen05 flash
kernel's ending, the split-key kernel's combine), rotation with published and blended values, and the
mixture with units without a gate, a correction, identity outputs and always-used units in its three
forms."""
import math
import os

import numpy as np
import pytest
import torch

from test_kernels_gpu import _give_back_passed_pages, _ops, _paged_case, _rel

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sunk_gated_reference(q, keys, values, lengths, counts, heads, kv_heads, scale, window, sink, gate):
    """out[t, h] = sigmoid(gate[t, h]) * sum_j p_j v_j with p_j = e^{s_j} / (e^{sink_h} + sum e^{s_j})."""
    out = torch.zeros_like(q, dtype=torch.float64)
    group = heads // kv_heads
    t = 0
    for e, (n, c) in enumerate(zip(lengths, counts)):
        for i in range(c):
            position = n - c + i
            first = max(0, position - window + 1) if window else 0
            for h in range(heads):
                k = keys[e][first:position + 1, h // group].double()
                v = values[e][first:position + 1, h // group].double()
                s = torch.cat([(k @ q[t, h].double()) * scale, sink[h:h + 1].double()])
                w = torch.softmax(s, dim=0)[:-1]
                out[t, h] = (w @ v) * torch.sigmoid(gate[t, h].double())
            t += 1
    return out


@pytest.mark.parametrize("heads,kv_heads,d,page", [(4, 2, 64, 16), (3, 1, 128, 64), (5, 5, 48, 8), (6, 2, 128, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 50])
def test_attention_with_a_learned_sink_and_an_output_gate(heads, kv_heads, d, page, dtype, window):
    """Portions beside single tokens; sinks from far below to far above the scores; the gate's
    pre-activations sit behind other columns of a wider 32-bit tensor, as behind q, k and v."""
    ops = _ops()
    lengths = [70, 200, 131, 64, 5, 300]
    counts = [70, 67, 1, 2, 5, 1]
    entries = len(lengths)
    lengths, counts, table, k_pool, v_pool, keys, values, q = _paged_case(
        entries, heads, kv_heads, d, page, dtype, seed=heads * 10 + d, lengths=lengths, counts=counts)
    scale = 1.0 / math.sqrt(d)
    total = sum(counts)
    g = torch.Generator().manual_seed(5)
    sink = torch.linspace(-6.0, 6.0, heads)
    offset = 24
    wide = torch.randn(total, offset + heads * d + 8, generator=g) * 2.0
    gate = wide[:, offset:offset + heads * d].reshape(total, heads, d)
    want = _sunk_gated_reference(q, keys, values, lengths, counts, heads, kv_heads, scale, window, sink, gate)
    plain = _sunk_gated_reference(q, keys, values, lengths, counts, heads, kv_heads, scale, window,
                                  torch.full((heads,), -80.0), torch.full_like(gate, 80.0))
    assert _rel(plain, want) > 0.1      # sink and gate matter
    _give_back_passed_pages(table, k_pool, v_pool, lengths, counts, page, window)
    qd = q.to(dtype).reshape(total, heads * d).to(DEV)
    kp, vp, tb = k_pool.to(DEV), v_pool.to(DEV), table.to(DEV)
    sink_d, wide_d = sink.to(DEV), wide.to(DEV)
    positions, token_seq = [], []
    for e, (n, c) in enumerate(zip(lengths, counts)):
        positions += list(range(n - c, n))
        token_seq += [e] * c
    positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    token_seq = torch.tensor(token_seq, dtype=torch.int32, device=DEV)
    out = torch.full_like(qd, float("nan"))
    ops.attention(qd, out, kp, vp, token_seq=token_seq, positions=positions, block_table=tb, num_heads=heads,
                  num_kv_heads=kv_heads, head_dim=d, scale=scale, window=window, sink=True, sink_values=sink_d,
                  gate=wide_d, gate_offset=offset)
    limit = 3e-6 if dtype == torch.float32 else 1e-2
    assert _rel(out.float().cpu().view(total, heads, d), want) < limit
    if dtype != torch.bfloat16 or d not in ops.TC_ATTENTION_HEAD_DIMS:
        return
    starts = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    pos0 = torch.tensor([n - c for n, c in zip(lengths, counts)], dtype=torch.int32, device=DEV)
    # the flash kernel alone, then the two kernels of a mixed step together
    out2 = torch.full_like(qd, float("nan"))
    ops.attention_prefill(qd, out2, kp, vp, entry_starts=starts, entry_pos0=pos0, block_table=tb, num_entries=entries,
                          num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=scale, window=window, sink=True,
                          sink_values=sink_d, gate=wide_d, gate_offset=offset)
    assert _rel(out2.float().cpu().view(total, heads, d), want) < limit
    out3 = torch.full_like(qd, float("nan"))
    ops.attention_prefill(qd, out3, kp, vp, entry_starts=starts, entry_pos0=pos0, block_table=tb, num_entries=entries,
                          num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=scale, window=window, sink=True,
                          sink_values=sink_d, gate=wide_d, gate_offset=offset, skip_single=True)
    for chunk, splits in (ops.decode_splits(entries, kv_heads, 300, ops.sm_count(DEV)), (32, 10)):
        scratch = torch.full((ops.attention_decode_scratch_floats(entries, heads, d, splits),), float("nan"), device=DEV)
        out4 = out3.clone()
        ops.attention_decode(qd, out4, kp, vp, positions=pos0, block_table=tb, num_heads=heads, num_kv_heads=kv_heads,
                             head_dim=d, scale=scale, window=window, chunk=chunk, num_splits=splits, scratch=scratch,
                             entry_starts=starts, sink=True, sink_values=sink_d, gate=wide_d, gate_offset=offset)
        assert _rel(out4.float().cpu().view(total, heads, d), want) < limit, (chunk, splits)
    # a step of single tokens: the last token of every entry
    last = [int(starts[e + 1]) - 1 for e in range(entries)]
    q1 = qd[last].contiguous()
    wide1 = wide_d[last].contiguous()
    position1 = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    chunk, splits = ops.decode_splits(entries, kv_heads, 300, ops.sm_count(DEV))
    # the one-kernel forms (a cluster of 8 or 16 blocks per entry and KV head, with and without the next
    # keys on their way) and the two-kernel form
    for cluster in ("8", "8p", "16", "16p", "0"):
        os.environ["VIPERA_ATTENTION_CLUSTER"] = cluster
        try:
            scratch = torch.full((ops.attention_decode_scratch_floats(entries, heads, d, splits),), float("nan"), device=DEV)
            out5 = torch.full_like(q1, float("nan"))
            ops.attention_decode(q1, out5, kp, vp, positions=position1, block_table=tb, num_heads=heads,
                                 num_kv_heads=kv_heads, head_dim=d, scale=scale, window=window, chunk=chunk,
                                 num_splits=splits, scratch=scratch, sink=True, sink_values=sink_d, gate=wide1,
                                 gate_offset=offset)
        finally:
            os.environ.pop("VIPERA_ATTENTION_CLUSTER", None)
        assert _rel(out5.float().cpu().view(entries, heads, d), want[last]) < limit, cluster


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style_name,rot_dims", [("interleaved", 6), ("interleaved", 10), ("neox", 4), ("none", 0)])
def test_rotation_with_published_and_blended_values(style_name, rot_dims, dtype):
    ops = _ops()
    heads, kv_heads, d, dv, page, tokens = 3, 2, 10, 7, 4, 9
    style = {"interleaved": ops.ROPE_INTERLEAVED, "neox": ops.ROPE_NEOX, "none": ops.ROPE_NONE}[style_name]
    g = torch.Generator().manual_seed(11)
    extra = 5      # columns behind q, k and v that the kernel must leave alone
    width = (heads + kv_heads) * d + kv_heads * dv
    qkv = torch.randn(tokens, width + extra, generator=g)
    other = torch.randn(tokens, kv_heads * dv, generator=g)
    blend = torch.tensor([0.3])
    positions = torch.tensor([5, 6, 7, 0, 1, 2, 3, 40, 41], dtype=torch.int32)
    token_seq = torch.tensor([0, 0, 0, 1, 1, 1, 1, 2, 2], dtype=torch.int32)
    table = torch.tensor([[3, 7, -1, -1, -1, -1, -1, -1, -1, -1, -1], [1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1],
                          [-1, -1, -1, -1, -1, -1, -1, -1, -1, -1, 5]], dtype=torch.int32)
    half = max(rot_dims // 2, 1)
    # the tables hold a row per position
    angle = torch.arange(64, dtype=torch.float64)[:, None] * (100.0 ** (-2.0 * torch.arange(half, dtype=torch.float64) / max(rot_dims, 2)))[None, :]
    cos_table, sin_table = torch.cos(angle).float(), torch.sin(angle).float()
    cos, sin = cos_table[positions.long()], sin_table[positions.long()]

    def turned(x):   # [tokens, n, d] in 64-bit
        out = x.clone()
        for i in range(rot_dims // 2):
            a, b = (2 * i, 2 * i + 1) if style_name == "interleaved" else (i, i + rot_dims // 2)
            c, s = cos[:, i].double()[:, None], sin[:, i].double()[:, None]
            out[..., a] = x[..., a] * c - x[..., b] * s
            out[..., b] = x[..., b] * c + x[..., a] * s
        return out

    q_want = turned(qkv[:, :heads * d].double().reshape(tokens, heads, d)) if style_name != "none" else qkv[:, :heads * d].double().reshape(tokens, heads, d)
    k_want = qkv[:, heads * d:(heads + kv_heads) * d].double().reshape(tokens, kv_heads, d)
    k_want = turned(k_want) if style_name != "none" else k_want
    v_raw = qkv[:, (heads + kv_heads) * d:width].double()
    for mode in ("publish", "blend"):
        k_pool = torch.full((9, page, kv_heads, d), float("nan"), dtype=dtype, device=DEV)
        v_pool = torch.full((9, page, kv_heads, dv), float("nan"), dtype=dtype, device=DEV)
        q_out = torch.full((tokens, heads * d), float("nan"), dtype=dtype, device=DEV)
        publish = torch.full((tokens, kv_heads * dv), float("nan"), device=DEV) if mode == "publish" else None
        ops.rope_cache_blend(qkv.to(DEV), q_out, num_heads=heads, num_kv_heads=kv_heads, head_dim=d, value_dim=dv,
                             rot_dims=rot_dims, positions=positions.to(DEV), cos=cos_table.to(DEV) if rot_dims else None,
                             sin=sin_table.to(DEV) if rot_dims else None, style=style, k_pool=k_pool, v_pool=v_pool,
                             token_seq=token_seq.to(DEV), block_table=table.to(DEV), page_size=page, write_cache=True,
                             publish=publish, blend_with=other.to(DEV) if mode == "blend" else None,
                             blend=blend.to(DEV) if mode == "blend" else None)
        limit = 1e-6 if dtype == torch.float32 else 6e-3
        assert _rel(q_out.float().cpu().view(tokens, heads, d), q_want) < limit
        v_want = v_raw if mode == "publish" else 0.7 * v_raw + 0.3 * other.double()
        if mode == "publish":
            assert torch.equal(publish.cpu(), v_raw.float())
        for t in range(tokens):
            p, e = int(positions[t]), int(token_seq[t])
            physical = int(table[e, p // page])
            assert _rel(k_pool[physical, p % page].float().cpu(), k_want[t]) < limit
            assert _rel(v_pool[physical, p % page].float().cpu().reshape(-1), v_want[t]) < limit
        written = sorted({int(table[int(token_seq[t]), int(positions[t]) // page]) for t in range(tokens)})
        untouched = [p for p in range(9) if p not in written]
        assert torch.isnan(k_pool[untouched].float()).all() and torch.isnan(v_pool[untouched].float()).all()


def _mixture_reference(h, router, correction, up, down, top, identity, always, route_scale, eps):
    """64-bit: softmax scores, the choice by score + correction, weights score / (sum + eps) * scale;
    outputs beyond the units with matrices return the row; the last `always` units count for all."""
    tokens, hidden = h.shape
    outputs = router.shape[0]
    real = outputs - identity
    scores = torch.softmax(h.double() @ router.double().T, dim=-1)
    choice = scores + correction.double()
    chosen = choice.topk(top, dim=-1).indices
    picked = torch.gather(scores, 1, chosen)
    weights = picked / (picked.sum(-1, keepdim=True) + eps) * route_scale
    margin = choice.sort(dim=-1, descending=True).values
    margin = margin[:, top - 1] - margin[:, top] if top < outputs else torch.full((tokens,), 1.0)

    def unit(x, e):
        return (torch.relu(up[e].double() @ x) ** 2) @ down[e].double().T

    out = torch.zeros(tokens, hidden, dtype=torch.float64)
    for t in range(tokens):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            out[t] += w * (h[t].double() if e >= real else unit(h[t].double(), e))
        for extra in range(always):
            out[t] += unit(h[t].double(), real + extra)
    return out, margin


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,hidden,ff,experts,identity,always,top", [
    (5, 64, 32, 6, 2, 2, 3),        # few assignments: tiles of 8 rows
    (300, 128, 64, 12, 3, 1, 4),    # bfloat16: grouped tensor-core products; 32-bit: tiles of 32 rows
    (70, 72, 24, 5, 0, 0, 2),       # an inner size the tensor-core form refuses; no identity outputs, no extra units
    (200, 256, 48, 3, 1, 3, 4),     # every router output chosen
])
def test_mixture_of_units_without_a_gate(tokens, hidden, ff, experts, identity, always, top, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(tokens + hidden)
    outputs = experts + identity
    matrices = experts + always
    h = torch.randn(tokens, hidden, generator=g).to(dtype)
    router = torch.randn(outputs, hidden, generator=g) * 0.3
    correction = torch.randn(outputs, generator=g) * 0.2
    up = (torch.randn(matrices, ff, hidden, generator=g) * 0.2).to(dtype)
    down = (torch.randn(matrices, hidden, ff, generator=g) * 0.2).to(dtype)
    want, margin = _mixture_reference(h.float(), router, correction, up.float(), down.float(), top, identity, always, 2.5, 1e-20)
    slots = top + always
    chosen = torch.full((tokens, slots), -7, dtype=torch.int32, device=DEV)
    weight = torch.full((tokens, slots), float("nan"), device=DEV)
    scratch = torch.zeros(ops.moe_scratch_words(tokens, slots, matrices), dtype=torch.int32, device=DEV)
    capacity = ops.moe_capacity(tokens, slots, matrices)
    act = torch.full((capacity, ff), float("nan"), dtype=dtype, device=DEV)
    rows = torch.full((tokens, slots * hidden), float("nan"), device=DEV)
    xs = torch.full((capacity, hidden), float("nan"), dtype=dtype, device=DEV)
    ys = torch.full((capacity, hidden), float("nan"), device=DEV)
    ops.moe(h.to(DEV), router=router.to(DEV), gate_up=up.to(DEV), down=down.to(DEV), gate_group=ops.MOE_GATE_GROUP, top=top,
            groups=1, keep=1, group_top=1, softmax_scores=True, renormalize=True, activation=ops.ACT_RELU2, chosen=chosen,
            weight=weight, scratch=scratch, act=act, rows=rows, xs=xs, ys=ys, gated=False, correction=correction.to(DEV),
            identity=identity, always=always, route_scale=2.5, renorm_eps=1e-20)
    got = rows.view(tokens, slots, hidden).double().sum(1).cpu()
    assert torch.isfinite(got).all()
    clear = margin > 1e-4      # (a choice that hangs on the last bits may come out either way)
    assert clear.float().mean() > 0.95
    limit = 2e-5 if dtype == torch.float32 else 2e-2
    assert _rel(got[clear], want[clear]) < limit
    # the always-used units sit in the last places with weight one; identity outputs are marked below zero
    assert (weight[:, top:] == 1.0).all() and (chosen[:, top:].cpu() == torch.arange(experts, experts + always, dtype=torch.int32)).all()
    assert ((chosen[:, :top] < 0).any().item()) == (identity > 0 and bool((_chosen_identity(h, router, correction, top, experts)).any()))
    assert torch.allclose(weight[:, :top].sum(-1).cpu(), torch.full((tokens,), 2.5), atol=1e-4)


def _chosen_identity(h, router, correction, top, experts):
    scores = torch.softmax(h.double() @ router.double().T, dim=-1) + correction.double()
    return scores.topk(top, dim=-1).indices >= experts
