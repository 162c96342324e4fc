"""Fasolorn without a GPU: configuration, tensor names, what the layers keep between steps, and the
plain implementation against other ways of writing its mechanisms; what the tests' sharpened weights
make visible (a window's edge, the sink, the blend of the values, a far key)."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import fasolorn_cases as cases
import helpers
import plain_fasolorn as plain
import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors
from vipera_rs_b200.cache.pools import plan_groups
from vipera_rs_b200.config import architecture_of
from vipera_rs_b200.engine.planner import plan_memory, spec_cache_requests
from vipera_rs_b200.parts.base import PagedKV

F = torch.float64


def spec_of(name):
    arch = architecture_of(cases.CONFIGS[name])
    return arch, arch.model_spec(arch.config_from_dict(cases.CONFIGS[name]))


def test_configuration_reads_back_and_refuses_what_it_does_not_know():
    arch, spec = spec_of("mixed")
    config = arch.config_from_dict(cases.MIXED)
    assert arch.config_from_dict(config.to_dict()) == config
    assert config.embedding_scale == 1.7 and spec.embedding_scale == 1.7 and spec.head_name is None
    assert [layer.kind for layer in config.layers] == ["attention", "attention", "latent_attention", "attention", "attention"]
    assert [layer.block for layer in spec.layers] == ["prenorm", "prenorm", "prenorm_mixer", "prenorm", "prenorm"]
    # the first layer that blends publishes its values, the later ones blend with them
    assert [layer.parts["mixer"].params.get("value_mix") for layer in spec.layers] == [None, "source", None, "blend", "blend"]
    assert spec.layers[4].parts["mixer"].params["window"] is None and spec.layers[4].parts["mixer"].params["position"].kind == "none"
    ffn = spec.layers[1].parts["ffn"].params
    assert (ffn["experts"], ffn["identity"], ffn["top"], ffn["shared_size"], ffn["route_scale"]) == (7, 2, 3, 40, 1.5)
    assert arch.config_from_dict(cases.ODD).embedding_scale == 1.0
    for path, value, error in ((("layers", 0, "type"), "lstm", errors.UnsupportedError),
                               (("layers", 0, "mixer", "kv_heads"), 4, errors.InvalidArgumentError),   # 6 heads
                               (("layers", 0, "mixer", "rot", "dims"), 18, errors.InvalidArgumentError),  # beyond the head
                               (("layers", 2, "mixer", "rot", "dims"), 6, errors.InvalidArgumentError),   # not the rotated part
                               (("layers", 3, "mixer", "vdim"), 16, errors.InvalidArgumentError),   # blended rows of another size
                               (("layers", 1, "mlp", "router", "top"), 8, errors.InvalidArgumentError),
                               (("layers", 1, "mlp", "kind"), "sparse", errors.UnsupportedError)):
        bad = copy.deepcopy(cases.MIXED)
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            arch.config_from_dict(bad)


def test_tensor_names_of_a_written_folder():
    path = cases.folder("mixed", "bfloat16", scaling="none")
    _, weights = cases.read(path)
    names = set(weights)
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g", "l0.mix.o",
            "l0.mix.sink", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.vmix", "l1.mlp.router", "l1.mlp.correction",
            "l1.mlp.e0.up", "l1.mlp.e4.down", "l1.mlp.shared.up", "l1.mlp.shared.down", "l2.mix.dkv", "l2.mix.dkv.norm",
            "l2.mix.uk", "l2.mix.uv", "l2.mix.q", "l2.mix.o", "l3.mix.vmix", "l4.mix.vmix"} <= names
    assert "head" not in names and "l0.mix.vmix" not in names and "l2.norm2" not in names and "l2.mix.g" not in names
    assert "l1.mlp.e5.up" not in names and "l1.mlp.e0.gate" not in names     # identity outputs and units without a gate
    assert "l3.mlp.shared.up" not in names
    assert tuple(weights["l1.mix.vmix"].shape) == () and tuple(weights["l0.mix.sink"].shape) == (6,)
    assert tuple(weights["l1.mlp.router"].shape) == (7, 72) and tuple(weights["l1.mlp.correction"].shape) == (7,)
    assert tuple(weights["l1.mlp.shared.up"].shape) == (40, 72) and tuple(weights["l2.mix.dkv"].shape) == (40 + 8, 72)
    assert tuple(weights["l0.mix.g"].shape) == (6 * 12, 72) and tuple(weights["l0.mix.v"].shape) == (2 * 12, 72)


def test_what_layers_keep_between_steps():
    _, spec = spec_of("mixed")
    requests = spec_cache_requests(spec)
    assert requests == {0: PagedKV(2, 16, 24, value_dim=12), 1: PagedKV(3, 12, 17, value_dim=8),
                        2: PagedKV(1, 40, 21, value_dim=8), 3: PagedKV(3, 8, 30), 4: PagedKV(1, 20, None, value_dim=24)}
    groups, states = plan_groups(requests)
    assert len(groups) == 5 and not states        # every window and geometry has pages of its own
    plan = plan_memory(spec, 256, 4, "bfloat16", device_bytes=10**9)
    assert plan["feasible"]


def test_the_sink_is_one_more_score_without_a_value():
    torch.manual_seed(3)
    scores = torch.randn(3, 5, 5, dtype=F) * 4
    sink = torch.tensor([-2.0, 0.5, 7.0], dtype=F)
    seen = plain.visible(5, {"size": 3})
    got = plain.softmax_with_sink(scores, seen, sink)
    padded = torch.cat([scores.masked_fill(~seen, float("-inf")), sink[:, None, None].expand(3, 5, 1)], dim=-1)
    assert torch.allclose(got, torch.softmax(padded, dim=-1)[..., :5], atol=1e-14)
    assert (got.sum(-1) < 1).all() and got[2].sum(-1).max() < 0.9     # a large sink takes most of the weight
    assert torch.allclose(plain.softmax_with_sink(scores, seen, None).sum(-1), torch.ones(3, 5, dtype=F))
    assert seen.sum(-1).tolist() == [1, 2, 3, 3, 3] and bool(seen[4, 2]) and not bool(seen[4, 1])


def test_the_two_pairings_of_the_rotation():
    x = torch.arange(2 * 3 * 10, dtype=F).reshape(2, 3, 10) / 7.0
    rot = {"dims": 6, "base": 100.0}
    position = torch.tensor([0, 5])
    freq = 100.0 ** (-2.0 * 1 / 6)
    for rotate, (a, b) in ((plain.rotate_interleaved, (2, 3)), (plain.rotate_halves, (1, 4))):
        out = rotate(x, position, rot)
        assert torch.equal(out[0], x[0]) and torch.equal(out[1, :, 6:], x[1, :, 6:])
        u, v = x[1, 2, a], x[1, 2, b]
        assert out[1, 2, a] == pytest.approx(float(u * math.cos(5 * freq) - v * math.sin(5 * freq)))
        assert out[1, 2, b] == pytest.approx(float(v * math.cos(5 * freq) + u * math.sin(5 * freq)))
    # a dot product of two rotated vectors depends on the distance of their positions only
    q, k = torch.randn(1, 6, dtype=F), torch.randn(1, 6, dtype=F)
    for rotate in (plain.rotate_interleaved, plain.rotate_halves):
        near = (rotate(q, torch.tensor([9]), rot) * rotate(k, torch.tensor([4]), rot)).sum()
        far = (rotate(q, torch.tensor([109]), rot) * rotate(k, torch.tensor([104]), rot)).sum()
        assert near == pytest.approx(float(far))


def test_latent_attention_with_absorbed_matrices():
    """q . (U c) = (U^T q) . c and sum_j p_j V c_j = V sum_j p_j c_j: the form the kernels use."""
    path = cases.folder("latent", "float32", scaling="mild")
    config, w = cases.read(path)
    mixer = config["layers"][0]["mixer"]
    heads, d, dr, dv, rank = (mixer[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    torch.manual_seed(1)
    h = torch.randn(50, config["width"], dtype=F)
    want = plain.latent_attention(h, w, "l0.mix", mixer, config["norm"]["eps"])
    positions = torch.arange(50)
    q = (h @ w["l0.mix.q"].to(F).T).reshape(50, heads, d + dr)
    down = h @ w["l0.mix.dkv"].to(F).T
    c = plain.rms_norm(down[:, :rank], w["l0.mix.dkv.norm"].to(F), config["norm"]["eps"])
    kr = plain.rotate_halves(down[:, rank:], positions, mixer["rot"])
    up_k = w["l0.mix.uk"].to(F).reshape(heads, d, rank)
    up_v = w["l0.mix.uv"].to(F).reshape(heads, dv, rank)
    qa = torch.einsum("thd,hdr->thr", q[..., :d], up_k)
    scores = torch.einsum("ihr,jr->hij", qa, c) + torch.einsum("ihd,jd->hij", plain.rotate_halves(q[..., d:], positions, mixer["rot"]), kr)
    p = plain.softmax_with_sink(scores * mixer["scale"], plain.visible(50, mixer["mask"]), None)
    out = torch.einsum("hvr,ihr->ihv", up_v, torch.einsum("hij,jr->ihr", p, c)).reshape(50, heads * dv)
    assert torch.allclose(out @ w["l0.mix.o"].to(F).T, want, atol=1e-9)


def test_a_shared_unit_is_the_sum_of_its_pieces():
    """D relu(U h)^2 is a sum over the inner features: cut into pieces of another size, the last one
    filled up with zero features, the pieces add up to the whole."""
    torch.manual_seed(2)
    h = torch.randn(9, 24, dtype=F)
    w = {"s.up": torch.randn(40, 24, dtype=F), "s.down": torch.randn(24, 40, dtype=F)}
    whole = plain.squared_relu_unit(h, w, "s")
    up = torch.cat([w["s.up"], torch.zeros(8, 24, dtype=F)])
    down = torch.cat([w["s.down"], torch.zeros(24, 8, dtype=F)], dim=1)
    pieces = sum(plain.squared_relu_unit(h, {"p.up": up[i:i + 16], "p.down": down[:, i:i + 16]}, "p") for i in range(0, 48, 16))
    assert torch.allclose(pieces, whole, atol=1e-10)


def test_the_router_chooses_with_the_correction_and_weighs_without_it():
    torch.manual_seed(5)
    h = torch.randn(200, 16, dtype=F)
    w = {"m.router": torch.randn(6, 16, dtype=F), "m.correction": torch.tensor([0.0, 0.3, -0.3, 0.0, 0.2, -0.1], dtype=F)}
    router = {"experts": 4, "identity": 2, "top": 2, "scale": 2.5}
    chosen, weights, margin = plain.route(h, w, "m", router)
    scores = torch.softmax(h @ w["m.router"].T, dim=-1)
    plainly = scores.topk(2, dim=-1).indices
    assert (chosen.sort(-1).values != plainly.sort(-1).values).any()         # the correction changes choices
    assert torch.allclose(weights.sum(-1), torch.full((200,), 2.5, dtype=F))   # scores over their sum, times the scale
    assert torch.allclose(weights[:, 0] / weights[:, 1], torch.gather(scores, 1, chosen)[:, 0] / torch.gather(scores, 1, chosen)[:, 1])
    assert (chosen >= 4).any() and (margin > 0).all()
    # an identity output returns the row itself
    w.update({f"m.e{k}.up": torch.randn(8, 16, dtype=F) for k in range(4)})
    w.update({f"m.e{k}.down": torch.randn(16, 8, dtype=F) for k in range(4)})
    out = plain.mixture(h, w, "m", {"router": router})
    t = int(torch.where((chosen >= 4).all(-1))[0][0]) if (chosen >= 4).all(-1).any() else None
    if t is not None:
        assert torch.allclose(out[t], 2.5 * h[t])


def _logits(name, tokens, change=None, scaling="sharp"):
    config, weights = cases.read(cases.folder(name, "float32", scaling=scaling))
    config = copy.deepcopy(config)
    weights = dict(weights)
    if change is not None:
        change(config, weights)
    return plain.forward(config, weights, tokens).numpy()


def test_what_the_sharpened_weights_make_visible():
    """The GPU tests rest on this: with the tests' weights a window that is one key off, a sink that
    is left out, values that are not blended and a far key all move the logits by far more than the
    tolerances."""
    tokens = helpers.random_tokens(cases.MIXED["vocab"], 80, 5)
    want = _logits("mixed", tokens)
    scale = np.abs(want).max()

    def moved(change, rows=slice(40, None)):
        return float(np.abs(_logits("mixed", tokens, change)[rows] - want[rows]).max() / scale)

    for layer in (0, 1, 2, 3):
        for step in (-1, 1):
            def window(config, weights, layer=layer, step=step):
                config["layers"][layer]["mixer"]["mask"]["size"] += step
            assert moved(window) > 0.02, (layer, step)

    def no_sink(config, weights):
        weights["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], -50.0)
    assert moved(no_sink) > 0.02

    def no_blend(config, weights):
        weights["l3.mix.vmix"] = torch.zeros_like(weights["l3.mix.vmix"])
    assert moved(no_blend) > 0.02

    def no_gate(config, weights):
        weights["l1.mix.g"] = torch.zeros_like(weights["l1.mix.g"])
    assert moved(no_gate) > 0.02

    def no_correction(config, weights):
        weights["l1.mlp.correction"] = torch.zeros_like(weights["l1.mlp.correction"])
    assert moved(no_correction, slice(0, None)) > 0.02

    # without masks a token counts however far back it lies
    tokens = helpers.random_tokens(cases.FAR["vocab"], 260, 6)
    changed = list(tokens)
    changed[3] = (changed[3] + 1) % cases.FAR["vocab"]
    a, b = _logits("far", tokens), _logits("far", changed)
    assert np.abs(a[-20:] - b[-20:]).max() / np.abs(a).max() > 1e-3


def test_exact_angle_tables_stay_good_far_out():
    """The design's tables are formed in 64-bit and rounded once: at position 100,000 an entry is as good
    as at position 1, where a 32-bit angle is off by thousands of times more."""
    from vipera_rs_b200.parts.rotary import rotary_tables

    dims, base, reach = 16, 10000.0, 100001
    exact = rotary_tables(dims, base, reach, "cpu", None, exact=True).pair
    plain32 = rotary_tables(dims, base, reach, "cpu", None).pair
    angle = torch.arange(reach, dtype=F)[:, None] * plain.frequencies(dims, base)[None, :]
    want_cos, want_sin = torch.cos(angle), torch.sin(angle)
    assert (exact[0].double() - want_cos).abs().max() < 1e-7 and (exact[1].double() - want_sin).abs().max() < 1e-7
    assert (plain32[0].double() - want_cos)[-1000:].abs().max() > 1e-4
    arch, spec = spec_of("mixed")
    assert spec.layers[0].parts["mixer"].params["position"].params["exact_angles"] is True
    assert spec.layers[2].parts["mixer"].params["position"].params["exact_angles"] is True
