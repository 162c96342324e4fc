"""Pugovik without a GPU: configuration, tensor names, what the layers keep between steps, the
frequency tables, and the plain implementation against other ways of writing its mechanisms."""
import json
import math

import numpy as np
import pytest
import torch

import pugovik_cases as cases
import plain_pugovik as plain
import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors
from vipera_rs_b200.cache.pools import plan_groups
from vipera_rs_b200.config import architecture_of
from vipera_rs_b200.engine.planner import plan_memory, spec_cache_requests
from vipera_rs_b200.parts.base import FixedState, PagedKV
from vipera_rs_b200.parts.rotary import rotary_tables


def spec_of(name):
    arch = architecture_of(cases.CONFIGS[name])
    return arch, arch.model_spec(arch.config_from_dict(cases.CONFIGS[name]))


def copy_of(config):
    return json.loads(json.dumps(config))


def test_configuration_reads_back_and_refuses_what_it_does_not_know():
    arch, spec = spec_of("mixed")
    config = arch.config_from_dict(cases.MIXED)
    assert arch.config_from_dict(config.to_dict()) == config
    assert config.norm_groups == 3 and config.residual_mult == 0.8
    assert [layer.kind for layer in config.layers] == ["lightning", "latent_attention", "lightning", "latent_attention"]
    assert config.layers[3].mixer["kv_from"] == 1 and config.layers[2].mlp is None
    # the layer that reads another's latents is scheduled on that layer's cache slot, without writing it
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False)]
    bad = copy_of(cases.MIXED)
    bad["layers"][0]["type"] = "lstm"
    with pytest.raises(errors.UnsupportedError):
        arch.config_from_dict(bad)
    bad = copy_of(cases.MIXED)
    bad["layers"][3]["mixer"]["kv_from"] = 0          # not a latent layer
    with pytest.raises(errors.InvalidArgumentError):
        arch.config_from_dict(bad)
    bad = copy_of(cases.MIXED)
    bad["layers"][3]["mixer"]["kv_rank"] = 48         # the shared cache has another geometry
    with pytest.raises(errors.InvalidArgumentError):
        arch.config_from_dict(bad)
    bad = copy_of(cases.MIXED)
    bad["layers"][0]["mixer"]["decay"] = [0.5]        # one decay per head
    with pytest.raises(errors.InvalidArgumentError):
        arch.config_from_dict(bad)
    bad = copy_of(cases.MIXED)
    bad["layers"][1]["mlp"]["router"]["top"] = 7      # more than the kept groups hold
    with pytest.raises(errors.InvalidArgumentError):
        arch.config_from_dict(bad)
    bad = copy_of(cases.MIXED)
    bad["layers"][1]["mlp"]["kind"] = "dense"
    with pytest.raises(errors.UnsupportedError):
        arch.config_from_dict(bad)
    bad = copy_of(cases.MIXED)
    bad["norm"]["groups"] = 5                          # does not divide the width
    with pytest.raises(errors.InvalidArgumentError):
        arch.config_from_dict(bad)


def test_tensor_names_of_a_written_folder():
    path = cases.folder("mixed", "bfloat16", scaling="none")
    _, weights = cases.read(path)
    names = set(weights)
    assert {"embed", "embed.norm", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.ls1",
            "l0.ls2", "l0.rg1", "l0.rg1.b", "l0.rg2", "l0.rg2.b", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g",
            "l0.mix.o", "l0.mix.norm", "l0.mlp.router", "l0.mlp.e0.gate", "l0.mlp.e5.down", "l1.mix.dkv",
            "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l1.mix.g", "l3.mix.uk", "l3.mlp.e3.up"} <= names
    assert "l3.mix.dkv" not in names and "l3.mix.dkv.norm" not in names      # it reads layer 1's latents
    assert "l2.norm2" not in names and "l2.rg2" not in names and "l2.mlp.router" not in names   # no feed-forward
    assert tuple(weights["l1.mix.q"].shape) == (3 * (16 + 8), 72) and tuple(weights["l1.mix.dkv"].shape) == (40 + 8, 72)
    assert tuple(weights["l3.mix.uk"].shape) == (5 * 8, 40) and tuple(weights["l3.mix.uv"].shape) == (5 * 12, 40)
    assert tuple(weights["l0.mix.norm"].shape) == (3 * 20,) and tuple(weights["l1.mlp.router"].shape) == (9, 72)


def test_what_layers_keep_between_steps():
    _, spec = spec_of("mixed")
    requests = spec_cache_requests(spec)
    assert requests == {0: FixedState((3 * 12 * 20,), torch.float32), 1: PagedKV(1, 40, None, value_dim=8),
                        2: FixedState((2 * 20 * 8,), torch.float32)}
    groups, states = plan_groups(requests)
    assert len(groups) == 1 and len(states) == 2
    assert groups[0].bytes_per_token(2) == (40 + 8) * 2          # one latent and one rotated key part, once for both layers
    plan = plan_memory(spec, 256, 4, "bfloat16", device_bytes=10**9)
    assert plan["feasible"] and plan["kv_bytes_per_token"] == 96


def test_frequency_tables_follow_the_ramp():
    scaling = cases.ONLY_LATENT["layers"][0]["mixer"]["rot"]["scaling"]
    cos, sin = rotary_tables(8, 5000.0, 60, "cpu", scaling).pair
    want, stretch = plain.rotary_frequencies(8, 5000.0, scaling)
    unscaled, _ = plain.rotary_frequencies(8, 5000.0, None)
    kinds = {"kept": 0, "slowed": 0, "blended": 0}
    for f, g in zip(unscaled.tolist(), want.tolist()):
        kinds["kept" if g == f else "slowed" if abs(g - f / 4.0) < 1e-15 else "blended"] += 1
    assert min(kinds.values()) >= 1, kinds          # the constants reach all three branches
    assert stretch == pytest.approx(0.1 * math.log(4.0) + 1.0)
    angle = torch.arange(60, dtype=torch.float64)[:, None] * want[None, :]
    assert torch.allclose(cos.double(), torch.cos(angle) * stretch, atol=3e-5)
    assert torch.allclose(sin.double(), torch.sin(angle) * stretch, atol=3e-5)


def test_rotation_turns_neighbouring_values_and_leaves_the_rest():
    x = torch.arange(2 * 3 * 10, dtype=torch.float64).reshape(2, 3, 10) / 7.0
    rot = {"dims": 6, "base": 100.0, "scaling": None}
    out = plain.rotate_pairs(x, torch.tensor([0, 5]), rot)
    assert torch.equal(out[0], x[0]) and torch.equal(out[1, :, 6:], x[1, :, 6:])
    freq = 100.0 ** (-2.0 * 1 / 6)
    u, v = x[1, 2, 2], x[1, 2, 3]
    assert out[1, 2, 2] == pytest.approx(float(u * math.cos(5 * freq) - v * math.sin(5 * freq)))
    assert out[1, 2, 3] == pytest.approx(float(v * math.cos(5 * freq) + u * math.sin(5 * freq)))


def test_plain_mechanisms_against_other_ways_of_writing_them():
    torch.manual_seed(3)
    # linear attention: the recurrence unrolled as a sum over earlier tokens
    config, weights = cases.read(cases.folder("lightning", "float32", scaling="sharp"))
    w = {k: v.double() for k, v in weights.items()}
    m = config["layers"][0]["mixer"]
    h = torch.randn(9, config["width"], dtype=torch.float64)
    heads, d, dv = m["heads"], m["dim"], m["vdim"]
    q = plain.silu(h @ w["l0.mix.q"].T).reshape(9, heads, d)
    k = plain.silu(h @ w["l0.mix.k"].T).reshape(9, heads, d)
    v = plain.silu(h @ w["l0.mix.v"].T).reshape(9, heads, dv)
    out = torch.zeros(9, heads, dv, dtype=torch.float64)
    for t in range(9):
        for s in range(t + 1):
            for head in range(heads):
                out[t, head] += m["decay"][head] ** (t - s) * (q[t, head] @ k[s, head]) * v[s, head]
    out = out.reshape(9, heads * dv)
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + config["norm"]["eps"]) * w["l0.mix.norm"]
    out = (out * torch.sigmoid(h @ w["l0.mix.g"].T)) @ w["l0.mix.o"].T
    assert torch.allclose(out, plain.lightning(h, w, "l0.mix", m, config["norm"]["eps"]), rtol=1e-9, atol=1e-9)

    # latent attention: keys and values expanded against the heads attending to the latents themselves
    config, weights = cases.read(cases.folder("latent", "float32", scaling="sharp"))
    w = {k: v.double() for k, v in weights.items()}
    m = config["layers"][0]["mixer"]
    eps = config["norm"]["eps"]
    h = torch.randn(11, config["width"], dtype=torch.float64)
    latent, key_rot = plain.latent_and_key(h, w, "l0.mix", m, eps)
    heads, d, r, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ w["l0.mix.q"].T).reshape(11, heads, d + r)
    q_rot = plain.rotate_pairs(q[..., d:], torch.arange(11), m["rot"])
    up_k = w["l0.mix.uk"].reshape(heads, d, -1)
    up_v = w["l0.mix.uv"].reshape(heads, dv, -1)
    absorbed = torch.einsum("thd,hdr->thr", q[..., :d], up_k)
    out = torch.zeros(11, heads, dv, dtype=torch.float64)
    for t in range(11):
        for head in range(heads):
            scores = (latent[:t + 1] @ absorbed[t, head] + key_rot[:t + 1] @ q_rot[t, head]) * m["scale"]
            out[t, head] = up_v[head] @ (torch.softmax(scores, 0) @ latent[:t + 1])
    out = (out.reshape(11, -1) * torch.sigmoid(h @ w["l0.mix.g"].T)) @ w["l0.mix.o"].T
    assert torch.allclose(out, plain.latent_attention(h, w, "l0.mix", m, eps, (latent, key_rot)), rtol=1e-9, atol=1e-9)


def test_the_router_keeps_to_the_best_groups():
    scores = torch.tensor([[0.9, 0.1, 0.5, 0.55, 0.6, 0.2, 0.05, 0.8],      # groups of two: sums 1.0, 1.05, 0.8, 0.85
                           [0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8]], dtype=torch.float64)
    chosen, weight = plain.route(scores, top=3, group_count=4, keep=2)
    assert chosen[0].tolist() == [0, 3, 2] and weight[0].tolist() == [0.9, 0.55, 0.5]    # 0.8 and 0.6 lie in lost groups
    assert chosen[1].tolist() == [7, 6, 5]
    chosen, _ = plain.route(scores, top=3, group_count=4, keep=4)
    assert chosen[0].tolist() == [0, 7, 4]
    # groups of one expert: the group's score is the expert's own
    chosen, _ = plain.route(scores, top=2, group_count=8, keep=3)
    assert chosen[0].tolist() == [0, 7]
    # groups of four: the two largest of each count (1.45 against 1.4)
    chosen, _ = plain.route(scores, top=2, group_count=2, keep=1)
    assert chosen[0].tolist() == [0, 3]


def test_the_plain_model_shows_what_the_tests_rely_on():
    """Sharp weights: a far token, one more visible key and a lost state each move the logits."""
    path = cases.folder("mixed", "float32", scaling="sharp")
    vocab = cases.MIXED["vocab"]
    tokens = torch.randint(0, vocab, (200,), generator=torch.Generator().manual_seed(5)).tolist()
    want = cases.plain_logits(path, tokens)
    changed = list(tokens)
    changed[3] = (changed[3] + 1) % vocab
    moved = cases.plain_logits(path, changed)
    assert np.abs(want[-10:] - moved[-10:]).max() / np.abs(want).max() > 1e-3
    # the latents alone carry token 3 that far in the latent-only model (the states are out of it)
    path = cases.folder("shared", "float32", scaling="sharp")
    want = cases.plain_logits(path, tokens)
    moved = cases.plain_logits(path, changed)
    assert np.abs(want[-10:] - moved[-10:]).max() / np.abs(want).max() > 1e-3
    # a request that starts later is another request: the first tokens matter
    assert np.abs(want[-1] - cases.plain_logits(path, tokens[1:])[-1]).max() / np.abs(want).max() > 1e-3
