"""Small Fasolorn configurations and model folders for the tests, with weights scaled so that the
mechanisms show: sharp attention (a window that is one key off, a lost sink or a missing blend of
the values moves the logits), routers whose choices are clear, corrections that change choices."""
from __future__ import annotations

import functools
import json
import os
import tempfile
from typing import Dict, Sequence

import numpy as np
import torch

import plain_fasolorn as plain


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=5, identity=2, top=3, scale=1.5, shared=40):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def attention(heads=6, kv_heads=2, dim=16, vdim=12, window=24, rot_dims=8, base=5000.0, scale=0.3, v_mix=False, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        mixer["mask"] = {"size": window}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent(heads=3, dim=16, rot_dim=8, vdim=24, rank=40, window=21, base=3000.0, scale=0.3, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
             "rot": {"dims": rot_dim, "base": base}}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def config(layers, width=72, vocab=211, eps=3e-6, scale=1.7):
    out = {"architecture": "Fasolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if scale is not None:
        out["embedding"] = {"scale": scale}
    return out


# Sizes that share nothing: grouped queries, a head turned in part, a layer without a feed-forward, values
# blended from the second layer on (not the first), a layer without mask and rotation, a shared unit whose
# inner size is no multiple of the experts', a mixture without identity outputs and without a shared unit.
MIXED = config([attention(mlp=dense()),
                attention(heads=3, kv_heads=3, dim=12, vdim=8, window=17, rot_dims=12, v_mix=True, mlp=moe()),
                latent(),
                attention(heads=6, kv_heads=3, dim=8, vdim=8, window=30, rot_dims=4, scale=0.5, v_mix=True,
                          mlp=moe(ff=16, experts=4, identity=0, top=1, scale=1.0, shared=0)),
                attention(heads=2, kv_heads=1, dim=20, vdim=24, window=0, rot_dims=0, scale=0.25, v_mix=True, mlp=dense(56))])
# Sizes the tensor-core products take, head sizes of 64 and 128 with values as long as keys.
WIDE = config([attention(heads=4, kv_heads=2, dim=64, vdim=64, window=70, rot_dims=32, base=10000.0, scale=0.12, v_mix=True,
                         mlp=moe(ff=64, experts=8, identity=2, top=2, scale=2.0, shared=128)),
               latent(heads=4, dim=64, rot_dim=32, vdim=64, rank=128, window=50, base=10000.0, scale=0.1, mlp=dense(512)),
               attention(heads=2, kv_heads=1, dim=128, vdim=128, window=100, rot_dims=128, base=10000.0, scale=0.09, v_mix=True,
                         mlp=moe(ff=128, experts=16, identity=0, top=4, scale=1.0, shared=64)),
               latent(heads=2, dim=32, rot_dim=32, vdim=128, rank=128, window=33, base=10000.0, scale=0.15)],
              width=256, vocab=640, eps=2e-5, scale=0.8)
# Values the others make equal, even or absent: a width that is no multiple of 8, no embedding scale, one
# head, a window of one key (a token sees itself only), a window longer than any request, a rotation of two
# values, every router output chosen, one expert beside one identity output, a rank that is no multiple
# of 8, an unrotated part shorter than the rotated one, a single blending layer (nothing to blend with).
ODD = config([attention(heads=1, kv_heads=1, dim=6, vdim=7, window=1, rot_dims=2, scale=0.7, v_mix=True,
                        mlp=moe(ff=9, experts=1, identity=1, top=2, scale=0.5, shared=5)),
              latent(heads=1, dim=6, rot_dim=10, vdim=7, rank=19, window=1000, scale=0.7, mlp=moe(ff=12, experts=3, identity=0, top=3, shared=12)),
              attention(heads=5, kv_heads=5, dim=10, vdim=3, window=9, rot_dims=10, scale=1.0, mlp=dense(17)),
              latent(heads=6, dim=4, rot_dim=2, vdim=3, rank=33, window=2, scale=1.0, mlp=moe(ff=8, experts=2, identity=3, top=1, shared=0))],
             width=100, vocab=97, eps=1e-4, scale=None)
# A larger one for long steps: many experts, more heads, a latent that is no multiple of 16.
LARGE = config([attention(heads=8, kv_heads=4, dim=32, vdim=48, window=150, rot_dims=16, base=20000.0, scale=0.15, v_mix=True,
                          mlp=moe(ff=112, experts=30, identity=2, top=6, scale=2.5, shared=160)),
                latent(heads=8, dim=32, rot_dim=16, vdim=48, rank=136, window=90, base=20000.0, scale=0.11, mlp=dense(640)),
                attention(heads=4, kv_heads=2, dim=64, vdim=96, window=64, rot_dims=64, base=20000.0, scale=0.12, v_mix=True,
                          mlp=moe(ff=48, experts=6, identity=1, top=2, scale=1.0, shared=48)),
                latent(heads=4, dim=16, rot_dim=16, vdim=32, rank=72, window=200, base=20000.0, scale=0.2)],
               width=384, vocab=1000, eps=1e-5, scale=0.6)
ONLY_ATTENTION = config([attention()])
ONLY_BLEND = config([attention(v_mix=True), attention(heads=4, kv_heads=1, dim=12, vdim=24, window=11, rot_dims=6, v_mix=True)])
ONLY_LATENT = config([latent()])
ONLY_MOE = config([attention(heads=1, kv_heads=1, dim=4, vdim=4, window=3, rot_dims=0, mlp=moe(ff=32, experts=9, identity=3, top=3))])
# No mask anywhere: a key counts however far back it lies.
FAR = config([attention(window=0, mlp=dense()), latent(window=0), attention(heads=3, kv_heads=3, dim=12, vdim=8, window=0, rot_dims=12)])

CONFIGS = {"mixed": MIXED, "wide": WIDE, "odd": ODD, "large": LARGE, "attention": ONLY_ATTENTION, "blend": ONLY_BLEND,
           "latent": ONLY_LATENT, "moe": ONLY_MOE, "far": FAR}

# How stored tensors are changed (by the end of their names): ("mul", x) or ("add", x).
SHARP = {".mix.q": ("mul", 25.0), ".mix.k": ("mul", 12.0), ".mix.v": ("mul", 10.0), ".mix.dkv": ("mul", 4.0),
         ".mix.uk": ("mul", 4.0), ".mix.uv": ("mul", 10.0), ".mix.g": ("mul", 20.0), ".mlp.router": ("mul", 8.0),
         ".mlp.correction": ("mul", 3.0), ".up": ("mul", 20.0), ".gate": ("mul", 20.0)}
MILD = {".mix.q": ("mul", 10.0), ".mix.k": ("mul", 6.0), ".mix.v": ("mul", 10.0), ".mix.uv": ("mul", 10.0),
        ".mix.g": ("mul", 20.0), ".mlp.router": ("mul", 8.0), ".mlp.correction": ("mul", 3.0), ".up": ("mul", 20.0),
        ".gate": ("mul", 20.0)}
RULES = {"sharp": SHARP, "mild": MILD, "none": {}}


@functools.lru_cache(maxsize=None)
def folder(name: str, store_dtype: str = "float32", seed: int = 7, scaling: str = "sharp") -> str:
    """A model folder of configuration `name` with seeded random weights, scaled."""
    import vipera_rs_b200  # noqa: F401
    from safetensors.torch import load_file, save_file
    from vipera_rs_b200.engine import write_random_model

    path = tempfile.mkdtemp(prefix=f"vipera_fasolorn_{name}_{store_dtype}_{scaling}_")
    write_random_model(path, CONFIGS[name], seed, store_dtype)
    file = os.path.join(path, "model.safetensors")
    tensors = load_file(file)
    for tensor_name in list(tensors):
        for ending, (how, amount) in RULES[scaling].items():
            if tensor_name.endswith(ending):
                value = tensors[tensor_name].to(torch.float32)
                value = value + amount if how == "add" else value * amount
                tensors[tensor_name] = value.to(tensors[tensor_name].dtype)
    save_file(tensors, file)
    return path


def read(path: str):
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as handle:
        return json.load(handle), load_file(os.path.join(path, "model.safetensors"))


_PLAIN: Dict[tuple, tuple] = {}


def _plain(path: str, tokens: Sequence[int]) -> tuple:
    key = (path, tuple(tokens))
    if key not in _PLAIN:
        config, weights = read(path)
        margins = []
        logits = plain.forward(config, weights, list(tokens), margins=margins).numpy()
        least = torch.stack(margins).min(dim=0).values.numpy() if margins else np.full(len(tokens), np.inf)
        _PLAIN[key] = (logits, least)
    return _PLAIN[key]


def plain_logits(path: str, tokens: Sequence[int]) -> np.ndarray:
    return _plain(path, tokens)[0]


def plain_margins(path: str, tokens: Sequence[int]) -> np.ndarray:
    """Per position, the least margin of any router's choice (plain.route)."""
    return _plain(path, tokens)[1]


def drawn(seed: int) -> dict:
    """A configuration whose sizes, order of layers and constants are drawn from `seed`: head sizes with and
    without tensor-core forms, grouped and single heads, windows shorter than a page and longer than a
    request, layers without masks, rotations of part of a head, ranks that are no multiples of 8, mixtures
    with and without identity outputs and shared units."""
    import random

    rng = random.Random(seed)
    width = rng.choice([64, 96, 128, 200, 256])
    value_row = rng.choice([32, 64, 128])        # kv_heads * vdim of every blending layer
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            mlp = dense(rng.choice([24, 40, 64, 136]))
        elif kind == "moe":
            experts, identity = rng.choice([1, 2, 5, 8, 19]), rng.choice([0, 0, 1, 3])
            ff = rng.choice([8, 16, 24, 64])
            mlp = moe(ff=ff, experts=experts, identity=identity, top=rng.randint(1, min(experts + identity, 4)),
                      scale=rng.choice([1.0, 0.5, 2.5]), shared=rng.choice([0, ff // 2, ff, 2 * ff + 8]))
        else:
            mlp = None
        window = rng.choice([0, 1, 5, 33, 64, 65, 100, 500])
        if rng.random() < 0.6:
            blends = rng.random() < 0.6
            if blends:
                kv_heads = rng.choice([1, 2, 4])
                vdim = value_row // kv_heads
                dim = rng.choice([vdim, vdim, 16, 24])
            else:
                kv_heads = rng.choice([1, 2, 3])
                dim = rng.choice([8, 16, 48, 64, 128])
                vdim = rng.choice([dim, dim, 8, 40])
            heads = kv_heads * rng.choice([1, 1, 2, 3])
            rot_dims = rng.choice([0, 2, dim // 2 // 2 * 2, dim])
            layers.append(attention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=window, rot_dims=rot_dims,
                                    base=rng.choice([100.0, 10000.0, 500000.0]), scale=dim ** -0.5, v_mix=blends, mlp=mlp))
        else:
            dim, rot_dim = rng.choice([8, 16, 32, 64]), rng.choice([2, 8, 16, 32, 64])
            layers.append(latent(heads=rng.choice([1, 2, 3, 8]), dim=dim, rot_dim=rot_dim, vdim=rng.choice([8, 24, 64, 80]),
                                 rank=rng.choice([16, 19, 64, 96, 136, 200]), window=window,
                                 base=rng.choice([100.0, 10000.0]), scale=(dim + rot_dim) ** -0.5, mlp=mlp))
    return config(layers, width=width, vocab=rng.randint(50, 600), eps=rng.choice([1e-5, 1e-6, 3e-4]),
                  scale=rng.choice([None, 0.5, 1.0, 3.0]))


for _seed in range(16):
    CONFIGS[f"drawn{_seed}"] = drawn(_seed)
