"""Typed configuration of the Pugovik decoder, read from the keys of its own config.json, and
its description in terms of parts.

The design: the embedding rows pass a norm; every sublayer sits between two norms, its output
is gated by the sublayer's own input and scaled per channel before it joins the stream with a
constant multiplier m:

    h = N1(x);  y = mixer(h) * sigmoid(R1 h + r1);  x += m * s1 * N1b(y)
    h = N2(x);  y = ff(h)    * sigmoid(R2 h + r2);  x += m * s2 * N2b(y)

Every N is an RMS norm over ``norm.groups`` equal consecutive parts of the row.  Two mixers:
``latent_attention`` (causal softmax attention whose keys and values are products of a cached
low-rank latent, with one rotated key part shared by all heads, interleaved rotary pairs with
YaRN frequencies and an output gate; a layer may read another layer's cache, ``kv_from``) and
``lightning`` (linear attention with one constant decay per head, a norm over the concatenated
heads and an output gate).  The feed-forward is a mixture of gated units: sigmoid scores, experts
in groups of neighbours of which the best ``groups.keep`` (by the sum of their two best scores)
may be chosen from, the ``top`` best experts weighted by their scores as they are.

config.json keys: ``architecture`` ("Pugovik"), ``vocab``, ``width``, ``residual_mult``,
``norm.eps``, ``norm.groups`` and ``layers`` (a list of ``{type, mixer, mlp}``).  Tensor names in
the weight file: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.ls1``,
``l<i>.rg1`` (bias ``l<i>.rg1.b``), the same with 2 for the feed-forward, ``l<i>.mix.<name>``,
``l<i>.mlp.router``, ``l<i>.mlp.e<k>.gate|up|down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import InvalidArgumentError, UnsupportedError
from .nobupel import DEFAULT_MAX_POSITIONS, _integer, _need, _number, nobupel_stored_name, nobupel_tensor_alias
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class PugovikLayer:
    kind: str                       # "latent_attention" or "lightning"
    mixer: Dict[str, Any]           # the mixer's sizes and constants, checked
    mlp: Optional[Dict[str, Any]]   # the mixture's sizes, None for a layer without a feed-forward


@dataclass(frozen=True)
class PugovikConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    residual_mult: float
    layers: Tuple[PugovikLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Pugovik"
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "PugovikConfig":
        _need("the configuration", data, ("vocab", "width", "layers", "norm", "residual_mult"))
        _need("norm", data["norm"], ("eps",))
        width = _integer("width", data["width"])
        groups = _integer("norm.groups", data["norm"].get("groups", 1))
        if width % groups:
            raise InvalidArgumentError(f"norm.groups {groups} does not divide the width {width}")
        if not isinstance(data["layers"], list) or not data["layers"]:
            raise InvalidArgumentError("layers must be a list with at least one layer")
        layers: List[PugovikLayer] = []
        for index, entry in enumerate(data["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, ("type", "mixer"))
            kind, mixer = entry["type"], entry["mixer"]
            if kind == "latent_attention":
                checked = cls._latent(f"{where}.mixer", mixer, index, layers)
            elif kind == "lightning":
                checked = cls._lightning(f"{where}.mixer", mixer)
            else:
                raise UnsupportedError(f"{where}: unknown mixer type {kind!r}; known: latent_attention, lightning")
            mlp = entry.get("mlp")
            layers.append(PugovikLayer(kind, checked, None if mlp is None else cls._mixture(f"{where}.mlp", mlp)))
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
        return cls(vocab=_integer("vocab", data["vocab"]), width=width, eps=_number("norm.eps", data["norm"]["eps"]),
                   norm_groups=groups, residual_mult=_number("residual_mult", data["residual_mult"], positive=False),
                   layers=tuple(layers),
                   max_positions=_integer("max_positions", data.get("max_positions", DEFAULT_MAX_POSITIONS)),
                   eos_token_ids=eos_ids, raw=dict(data))

    @staticmethod
    def _latent(where: str, mixer: Dict[str, Any], index: int, earlier: List[PugovikLayer]) -> Dict[str, Any]:
        _need(where, mixer, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"))
        out = {key: _integer(f"{where}.{key}", mixer[key]) for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        out["scale"] = _number(f"{where}.scale", mixer["scale"])
        rot = mixer["rot"]
        _need(f"{where}.rot", rot, ("dims", "base"))
        dims = _integer(f"{where}.rot.dims", rot["dims"])
        if dims != out["rot_dim"] or dims % 2:
            raise InvalidArgumentError(f"{where}: rot.dims {dims} must be even and equal rot_dim {out['rot_dim']}")
        scaling = rot.get("scaling")
        if scaling is not None:
            _need(f"{where}.rot.scaling", scaling, ("factor", "original", "fast", "slow"))
            scaling = {key: _number(f"{where}.rot.scaling.{key}", scaling[key])
                       for key in ("factor", "original", "fast", "slow")}
        out["rot"] = {"dims": dims, "base": _number(f"{where}.rot.base", rot["base"]), "scaling": scaling}
        out["kv_from"] = None
        if mixer.get("kv_from") is not None:
            source = _integer(f"{where}.kv_from", mixer["kv_from"], 0)
            if source >= index or earlier[source].kind != "latent_attention" or earlier[source].mixer["kv_from"] is not None:
                raise InvalidArgumentError(f"{where}.kv_from {source} must name an earlier latent_attention layer "
                                           "that has a cache of its own")
            theirs = earlier[source].mixer
            if any(theirs[key] != out[key] for key in ("kv_rank", "rot_dim", "rot")):
                raise InvalidArgumentError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {source}")
            out["kv_from"] = source
        return out

    @staticmethod
    def _lightning(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        _need(where, mixer, ("heads", "dim", "vdim", "decay"))
        out = {key: _integer(f"{where}.{key}", mixer[key]) for key in ("heads", "dim", "vdim")}
        decay = mixer["decay"]
        if not isinstance(decay, list) or len(decay) != out["heads"]:
            raise InvalidArgumentError(f"{where}.decay must list one decay per head")
        out["decay"] = tuple(_number(f"{where}.decay[{i}]", value, positive=False) for i, value in enumerate(decay))
        return out

    @staticmethod
    def _mixture(where: str, mlp: Dict[str, Any]) -> Dict[str, Any]:
        _need(where, mlp, ("kind", "expert", "router"))
        if mlp["kind"] != "moe":
            raise UnsupportedError(f"{where}: unknown kind {mlp['kind']!r}; known: moe")
        _need(f"{where}.expert", mlp["expert"], ("ff",))
        router = mlp["router"]
        _need(f"{where}.router", router, ("experts", "top"))
        experts = _integer(f"{where}.router.experts", router["experts"])
        top = _integer(f"{where}.router.top", router["top"])
        groups = router.get("groups") or {"count": 1, "keep": 1}
        _need(f"{where}.router.groups", groups, ("count", "keep"))
        count = _integer(f"{where}.router.groups.count", groups["count"])
        keep = _integer(f"{where}.router.groups.keep", groups["keep"])
        if experts % count or keep > count or top > keep * (experts // count):
            raise InvalidArgumentError(f"{where}.router: {experts} experts in {count} groups of which {keep} are kept "
                                       f"cannot give {top} experts a token")
        return {"ff": _integer(f"{where}.expert.ff", mlp["expert"]["ff"]), "experts": experts, "top": top,
                "groups": count, "keep": keep}

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        layers = []
        for layer in self.layers:
            mixer = {k: (list(v) if isinstance(v, tuple) else v) for k, v in layer.mixer.items() if v is not None}
            if "rot" in mixer:
                mixer["rot"] = {k: v for k, v in mixer["rot"].items() if v is not None}
            mlp = None
            if layer.mlp is not None:
                m = layer.mlp
                mlp = {"kind": "moe", "expert": {"ff": m["ff"]},
                       "router": {"experts": m["experts"], "top": m["top"],
                                  "groups": {"count": m["groups"], "keep": m["keep"]}}}
            layers.append({"type": layer.kind, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps, "groups": self.norm_groups},
                               "residual_mult": self.residual_mult, "layers": layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def pugovik_model_spec(config: PugovikConfig) -> ModelSpec:
    """Pugovik in parts.  A layer that reads another layer's latent cache is a schedule entry that
    names that layer's cache slot and does not write it."""
    norm = PartSpec("rmsnorm", {"size": config.width, "eps": config.eps, "groups": config.norm_groups})
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for index, layer in enumerate(config.layers):
        m = layer.mixer
        if layer.kind == "latent_attention":
            rot = m["rot"]
            position = PartSpec("rope_interleaved", {"head_dim": m["rot_dim"], "rotary_dims": rot["dims"],
                                                     "theta": rot["base"], "scaling": rot["scaling"],
                                                     "max_positions": config.max_positions})
            mixer = PartSpec("latent_attention", {
                "hidden_size": config.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "softmax_scale": m["scale"], "norm_eps": config.eps,
                "own_cache": m["kv_from"] is None, "output_gate": True, "position": position})
            source = index if m["kv_from"] is None else m["kv_from"]
            schedule.append(ScheduleEntry(layer=index, cache=source, writes_cache=m["kv_from"] is None))
        else:
            mixer = PartSpec("lightning", {
                "hidden_size": config.width, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "decay": tuple(m["decay"]), "norm_eps": config.eps})
            schedule.append(ScheduleEntry(layer=index, cache=index))
        parts = {"mixer_norm": norm, "mixer": mixer, "mixer_out_norm": norm}
        names = {"mixer_norm": "norm1", "mixer": "mix", "mixer_out_norm": "norm1b", "mixer_scale": "ls1",
                 "mixer_gate": "rg1", "ffn_norm": "norm2", "ffn": "mlp", "ffn_out_norm": "norm2b", "ffn_scale": "ls2",
                 "ffn_gate": "rg2"}
        if layer.mlp is not None:
            f = layer.mlp
            parts.update(ffn_norm=norm, ffn_out_norm=norm, ffn=PartSpec("moe_mlp", {
                "hidden_size": config.width, "intermediate_size": f["ff"], "experts": f["experts"], "top": f["top"],
                "groups": f["groups"], "keep_groups": f["keep"], "score": "sigmoid", "group_score_top": 2,
                "renormalize": False, "activation": "silu", "projection_names": ("gate", "up", "down")}))
        layers.append(LayerSpec(block="sandwich", prefix=f"l{index}", parts=parts, names=names,
                                params={"hidden_size": config.width, "residual_mult": config.residual_mult,
                                        "layer_scale": True, "gated": True}))
    spec = ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        max_position_embeddings=config.max_positions,
        embedding_name="embed.weight",
        layers=layers,
        schedule=schedule,
        final_norm=norm,
        final_norm_name="final.norm",
        head_name="head.weight",
        embedding_norm=norm,
        embedding_norm_name="embed.norm",
    )
    spec.validate()
    return spec


_SECOND_SUBLAYER = re.compile(r"^l(\d+)\.(norm2|norm2b|ls2|rg2)\.(weight|bias)$")


def pugovik_ignorable(config: PugovikConfig, name: str) -> bool:
    """A file may hold the second sublayer's norms, scale and gate for a layer without a
    feed-forward; nothing reads them."""
    match = _SECOND_SUBLAYER.match(name)
    return bool(match) and int(match.group(1)) < len(config.layers) and config.layers[int(match.group(1))].mlp is None


register_architecture("Pugovik", PugovikConfig.from_dict, pugovik_model_spec,
                      tensor_alias=nobupel_tensor_alias, stored_name=nobupel_stored_name, ignorable=pugovik_ignorable)
