"""Small Pugovik configurations and model folders for the tests, with weights scaled so that the
mechanisms show: sharp attention (one wrong key moves the logits), decays near one (a token
counts hundreds of tokens later), routers whose choices are clear."""
from __future__ import annotations

import functools
import json
import os
import tempfile
from typing import Dict, Sequence

import numpy as np
import torch

import plain_pugovik as plain


def moe(ff=24, experts=6, top=2, groups=3, keep=2):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def latent_layer(heads=3, dim=16, rot_dim=8, vdim=24, rank=40, scale=0.3, base=5000.0, scaling=True, kv_from=None, mlp=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 512, "fast": 4.0, "slow": 0.5}
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def lightning_layer(heads=3, dim=12, vdim=20, decay=(0.5, 0.93, 0.998), mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def config(layers, width=72, vocab=211, eps=3e-6, groups=3, mult=0.8):
    return {"architecture": "Pugovik", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "residual_mult": mult, "layers": layers}


# Sizes that share nothing with each other; a layer that reads an earlier layer's latents with other heads.
MIXED = config([lightning_layer(mlp=moe()),
                latent_layer(mlp=moe(ff=40, experts=9, top=4, groups=3, keep=2)),
                lightning_layer(heads=2, dim=20, vdim=8, decay=(0.8, 0.99)),
                latent_layer(heads=5, dim=8, vdim=12, scale=0.5, kv_from=1, mlp=moe(ff=16, experts=4, top=1, groups=2, keep=1))])
# Sizes the tensor-core products take; a shared cache two layers back.
WIDE = config([latent_layer(heads=4, dim=64, rot_dim=32, vdim=64, rank=128, scale=0.1, base=10000.0,
                            mlp=moe(ff=128, experts=8, top=2, groups=2, keep=1)),
               lightning_layer(heads=4, dim=64, vdim=64, decay=(0.7, 0.9, 0.97, 0.999),
                               mlp=moe(ff=64, experts=16, top=4, groups=4, keep=2)),
               latent_layer(heads=2, dim=32, rot_dim=32, vdim=128, rank=128, scale=0.15, base=10000.0, kv_from=0),
               lightning_layer(heads=2, dim=128, vdim=32, decay=(0.95, 0.9999), mlp=moe(ff=256, experts=4, top=2, groups=1, keep=1))],
              width=256, vocab=640, eps=2e-5, groups=4, mult=0.6)
# Values the others make equal, even or absent: a width that is no multiple of 8, one norm group, a
# multiplier of one, one head, groups of one expert, every expert used, one expert in all, a rotated
# part of two values, no frequency scaling, unrotated size below the rotated one, a decay of one
# (nothing forgotten) and of zero (nothing kept), a rank that is no multiple of 8.
ODD = config([latent_layer(heads=1, dim=6, rot_dim=10, vdim=7, rank=19, scale=0.7, scaling=False,
                           mlp=moe(ff=9, experts=5, top=2, groups=5, keep=3)),
              lightning_layer(heads=1, dim=7, vdim=40, decay=(1.0,), mlp=moe(ff=12, experts=3, top=3, groups=1, keep=1)),
              latent_layer(heads=6, dim=4, rot_dim=2, vdim=3, rank=33, scale=1.0, scaling=False, mlp=moe(ff=8, experts=1, top=1, groups=1, keep=1)),
              lightning_layer(heads=2, dim=37, vdim=5, decay=(0.0, 0.5)),
              latent_layer(heads=2, dim=5, rot_dim=10, vdim=9, rank=19, scale=0.4, scaling=False, kv_from=0)],
             width=100, vocab=97, eps=1e-4, groups=1, mult=1.0)
# A larger one for long steps: a latent that is no multiple of 16, more heads, many experts in groups, a
# layer that reads the first layer's pages with other heads, a last layer without a feed-forward.
LARGE = config([latent_layer(heads=8, dim=32, rot_dim=16, vdim=48, rank=136, scale=0.11, base=20000.0,
                             mlp=moe(ff=112, experts=32, top=6, groups=8, keep=3)),
                lightning_layer(heads=4, dim=48, vdim=96, decay=(0.6, 0.9, 0.99, 0.9995), mlp=moe(ff=64, experts=4, top=2, groups=2, keep=2)),
                latent_layer(heads=4, dim=16, rot_dim=16, vdim=32, rank=136, scale=0.2, base=20000.0, kv_from=0,
                             mlp=moe(ff=48, experts=6, top=1, groups=3, keep=2)),
                lightning_layer(heads=2, dim=64, vdim=64, decay=(0.97, 0.5))],
               width=384, vocab=1000, eps=1e-5, groups=2, mult=0.9)
ONLY_LATENT = config([latent_layer()])
ONLY_SHARED = config([latent_layer(), latent_layer(heads=2, dim=12, vdim=10, scale=0.4, kv_from=0)])
ONLY_LIGHTNING = config([lightning_layer()])
ONLY_MOE = config([lightning_layer(heads=1, dim=4, vdim=4, decay=(0.5,), mlp=moe(ff=32, experts=12, top=3, groups=4, keep=2))])

CONFIGS = {"mixed": MIXED, "wide": WIDE, "odd": ODD, "large": LARGE, "latent": ONLY_LATENT, "shared": ONLY_SHARED,
           "lightning": ONLY_LIGHTNING, "moe": ONLY_MOE}

# How stored tensors are changed (by the end of their names): ("mul", x) or ("add", x).
SHARP = {".mix.q": ("mul", 25.0), ".mix.dkv": ("mul", 4.0), ".mix.uk": ("mul", 4.0), ".mix.uv": ("mul", 10.0),
         ".mix.k": ("mul", 20.0), ".mix.v": ("mul", 20.0), ".mlp.router": ("mul", 8.0), ".gate": ("mul", 20.0),
         ".up": ("mul", 20.0), ".rg1": ("mul", 10.0), ".rg2": ("mul", 10.0)}
MILD = {".mix.q": ("mul", 10.0), ".mix.uv": ("mul", 10.0), ".mix.k": ("mul", 20.0), ".mix.v": ("mul", 20.0),
        ".mlp.router": ("mul", 8.0), ".gate": ("mul", 20.0), ".up": ("mul", 20.0), ".rg1": ("mul", 10.0),
        ".rg2": ("mul", 10.0)}
RULES = {"sharp": SHARP, "mild": MILD, "none": {}}


@functools.lru_cache(maxsize=None)
def folder(name: str, store_dtype: str = "float32", seed: int = 7, scaling: str = "sharp") -> str:
    """A model folder of configuration `name` with seeded random weights, scaled."""
    import vipera_rs_b200  # noqa: F401
    from safetensors.torch import load_file, save_file
    from vipera_rs_b200.engine import write_random_model

    path = tempfile.mkdtemp(prefix=f"vipera_pugovik_{name}_{store_dtype}_{scaling}_")
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
    """Per position, the least margin of any mixture's choice of experts (plain.route_margin)."""
    return _plain(path, tokens)[1]
