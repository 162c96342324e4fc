"""Typed configuration of the Fasolorn decoder, read from the keys of its own config.json, and
its description in terms of parts.

The design: embedding rows times a constant; pre-norm layers ``x += mixer(N1(x))`` and, where the
layer has a feed-forward, ``x += ff(N2(x))``; a final norm; the embedding matrix again as the output
matrix.  Two mixers.  ``attention``: grouped-query attention with interleaved rotary pairs over the
first ``rot.dims`` values of a head, a sliding window, a softmax whose denominator also holds
``exp(sink_h)`` (a learned number per head), values that, in every layer marked ``v_mix`` but the first
such, are blended with the first such layer's values of the same token (``(1 - b) v + b v_first``), and
heads multiplied by ``sigmoid(W_g h)`` before the output matrix.  ``latent_attention``: attention over
a cached normed low-rank latent with one rotated key part (pairs ``(i, i + r/2)``) shared by the heads,
a sliding window and a plain softmax.  Two feed-forwards.  ``dense``: a gated unit with silu.
``moe``: units ``D relu(U h)^2`` chosen by softmax scores plus a correction (the weights are the scores
themselves over their sum, times a constant); the last ``router.identity`` router outputs return their
input; a shared unit of the same form is added for every token.

config.json keys: ``architecture`` ("Fasolorn"), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps`` and ``layers`` (a list of ``{type, mixer, mlp}``).  Tensor names in the weight file:
``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.<name>``, ``l<i>.mlp.<name>``,
``l<i>.mlp.e<k>.up|down``, ``l<i>.mlp.shared.up|down``, ``final.norm``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import InvalidArgumentError, UnsupportedError
from .nobupel import DEFAULT_MAX_POSITIONS, _integer, _need, _number, nobupel_stored_name, nobupel_tensor_alias
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class FasolornLayer:
    kind: str                       # "attention" or "latent_attention"
    mixer: Dict[str, Any]           # the mixer's sizes and constants, checked
    mlp: Optional[Dict[str, Any]]   # the feed-forward's, None for a layer without one


def _mask(where: str, mixer: Dict[str, Any]) -> Optional[int]:
    mask = mixer.get("mask")
    if mask is None:
        return None
    _need(f"{where}.mask", mask, ("size",))
    return _integer(f"{where}.mask.size", mask["size"])


def _rot(where: str, mixer: Dict[str, Any], most: int) -> Optional[Dict[str, Any]]:
    rot = mixer.get("rot")
    if rot is None:
        return None
    _need(f"{where}.rot", rot, ("dims", "base"))
    dims = _integer(f"{where}.rot.dims", rot["dims"], 0)
    if dims % 2 or dims > most:
        raise InvalidArgumentError(f"{where}: rot.dims {dims} must be even and at most {most}")
    return {"dims": dims, "base": _number(f"{where}.rot.base", rot["base"])} if dims else None


@dataclass(frozen=True)
class FasolornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[FasolornLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Fasolorn"
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "FasolornConfig":
        _need("the configuration", data, ("vocab", "width", "layers", "norm"))
        _need("norm", data["norm"], ("eps",))
        width = _integer("width", data["width"])
        if not isinstance(data["layers"], list) or not data["layers"]:
            raise InvalidArgumentError("layers must be a list with at least one layer")
        layers: List[FasolornLayer] = []
        for index, entry in enumerate(data["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, ("type", "mixer"))
            kind, mixer = entry["type"], entry["mixer"]
            if kind == "attention":
                checked = cls._attention(f"{where}.mixer", mixer)
            elif kind == "latent_attention":
                checked = cls._latent(f"{where}.mixer", mixer)
            else:
                raise UnsupportedError(f"{where}: unknown mixer type {kind!r}; known: attention, latent_attention")
            mlp = entry.get("mlp")
            layers.append(FasolornLayer(kind, checked, None if mlp is None else cls._mlp(f"{where}.mlp", mlp)))
        blended = [layer.mixer for layer in layers if layer.kind == "attention" and layer.mixer["v_mix"]]
        if any(m["kv_heads"] * m["vdim"] != blended[0]["kv_heads"] * blended[0]["vdim"] for m in blended):
            raise InvalidArgumentError("layers with v_mix must have value rows of one size (kv_heads * vdim)")
        embedding = data.get("embedding") or {}
        eos = data.get("eos_token_id")
        eos_ids = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(x) for x in eos))
        return cls(vocab=_integer("vocab", data["vocab"]), width=width, eps=_number("norm.eps", data["norm"]["eps"]),
                   embedding_scale=_number("embedding.scale", embedding.get("scale", 1.0), positive=False),
                   layers=tuple(layers),
                   max_positions=_integer("max_positions", data.get("max_positions", DEFAULT_MAX_POSITIONS)),
                   eos_token_ids=eos_ids, raw=dict(data))

    @staticmethod
    def _attention(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        _need(where, mixer, ("heads", "dim", "vdim", "scale"))
        mixer = {"kv_heads": mixer["heads"], **mixer}      # without kv_heads every query head has keys of its own
        out = {key: _integer(f"{where}.{key}", mixer[key]) for key in ("heads", "kv_heads", "dim", "vdim")}
        if out["heads"] % out["kv_heads"]:
            raise InvalidArgumentError(f"{where}: heads {out['heads']} is not a multiple of kv_heads {out['kv_heads']}")
        out["scale"] = _number(f"{where}.scale", mixer["scale"])
        out["mask"] = _mask(where, mixer)
        out["rot"] = _rot(where, mixer, out["dim"])
        out["v_mix"] = bool(mixer.get("v_mix", False))
        return out

    @staticmethod
    def _latent(where: str, mixer: Dict[str, Any]) -> Dict[str, Any]:
        _need(where, mixer, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"))
        out = {key: _integer(f"{where}.{key}", mixer[key]) for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        out["scale"] = _number(f"{where}.scale", mixer["scale"])
        out["mask"] = _mask(where, mixer)
        out["rot"] = _rot(where, mixer, out["rot_dim"])
        if out["rot"] is None or out["rot"]["dims"] != out["rot_dim"]:
            raise InvalidArgumentError(f"{where}: rot.dims must equal rot_dim {out['rot_dim']}")
        return out

    @staticmethod
    def _mlp(where: str, mlp: Dict[str, Any]) -> Dict[str, Any]:
        _need(where, mlp, ("kind",))
        if mlp["kind"] == "dense":
            _need(where, mlp, ("ff",))
            return {"kind": "dense", "ff": _integer(f"{where}.ff", mlp["ff"])}
        if mlp["kind"] != "moe":
            raise UnsupportedError(f"{where}: unknown kind {mlp['kind']!r}; known: dense, moe")
        _need(where, mlp, ("expert", "router"))
        _need(f"{where}.expert", mlp["expert"], ("ff",))
        router = mlp["router"]
        _need(f"{where}.router", router, ("experts", "top"))
        experts = _integer(f"{where}.router.experts", router["experts"])
        identity = _integer(f"{where}.router.identity", router.get("identity", 0), 0)
        top = _integer(f"{where}.router.top", router["top"])
        if top > experts + identity:
            raise InvalidArgumentError(f"{where}.router: {top} of {experts + identity} experts cannot be chosen")
        shared = mlp.get("shared")
        if shared is not None:
            _need(f"{where}.shared", shared, ("ff",))
            shared = _integer(f"{where}.shared.ff", shared["ff"])
        return {"kind": "moe", "ff": _integer(f"{where}.expert.ff", mlp["expert"]["ff"]), "experts": experts,
                "identity": identity, "top": top, "scale": _number(f"{where}.router.scale", router.get("scale", 1.0)),
                "shared": shared}

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer = {k: v for k, v in m.items() if k not in ("mask", "rot", "v_mix")}
            if m["mask"] is not None:
                mixer["mask"] = {"size": m["mask"]}
            if m["rot"] is not None:
                mixer["rot"] = dict(m["rot"])
            if m.get("v_mix"):
                mixer["v_mix"] = True
            mlp = None
            if layer.mlp is not None and layer.mlp["kind"] == "dense":
                mlp = {"kind": "dense", "ff": layer.mlp["ff"]}
            elif layer.mlp is not None:
                f = layer.mlp
                mlp = {"kind": "moe", "expert": {"ff": f["ff"]},
                       "router": {"experts": f["experts"], "identity": f["identity"], "top": f["top"], "scale": f["scale"]}}
                if f["shared"] is not None:
                    mlp["shared"] = {"ff": f["shared"]}
            layers.append({"type": layer.kind, "mixer": mixer, "mlp": mlp})
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


# What the design fixes: the sum the router's weights are divided by holds this beside the scores.
ROUTER_SUM_EPS = 1e-20


def fasolorn_model_spec(config: FasolornConfig) -> ModelSpec:
    """Fasolorn in parts.  The first layer marked ``v_mix`` publishes its values to the later ones of
    the same step; every layer has a cache slot of its own."""
    norm = PartSpec("rmsnorm", {"size": config.width, "eps": config.eps})
    layers: List[LayerSpec] = []
    source_seen = False
    for index, layer in enumerate(config.layers):
        m = layer.mixer
        if layer.kind == "attention":
            rot = m["rot"]
            position = PartSpec("none", {}) if rot is None else PartSpec("rope_interleaved", {
                "head_dim": m["dim"], "rotary_dims": rot["dims"], "theta": rot["base"], "scaling": None,
                "exact_angles": True, "max_positions": config.max_positions})
            value_mix = None
            if m["v_mix"]:
                value_mix = "blend" if source_seen else "source"
                source_seen = True
            mixer = PartSpec("gqa_attention", {
                "hidden_size": config.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                "head_dim": m["dim"], "value_dim": m["vdim"], "qkv_bias": False, "window": m["mask"],
                "sink": "learned", "output_gate": True, "gate_name": "g", "value_mix": value_mix,
                "softmax_scale": m["scale"], "position": position, "projection_names": ("q", "k", "v", "o")})
        else:
            rot = m["rot"]
            position = PartSpec("rope_neox", {"head_dim": m["rot_dim"], "rotary_dims": rot["dims"], "theta": rot["base"],
                                              "scaling": None, "exact_angles": True,
                                              "max_positions": config.max_positions})
            mixer = PartSpec("latent_attention", {
                "hidden_size": config.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "softmax_scale": m["scale"], "norm_eps": config.eps,
                "own_cache": True, "output_gate": False, "window": m["mask"], "position": position})
        parts = {"mixer_norm": norm, "mixer": mixer}
        names = {"mixer_norm": "norm1", "mixer": "mix"}
        block = "prenorm_mixer"
        if layer.mlp is not None:
            f = layer.mlp
            block = "prenorm"
            if f["kind"] == "dense":
                ffn = PartSpec("gated_mlp", {"hidden_size": config.width, "intermediate_size": f["ff"],
                                             "activation": "silu", "bias": False,
                                             "projection_names": ("gate", "up", "down")})
            else:
                ffn = PartSpec("moe_mlp", {
                    "hidden_size": config.width, "intermediate_size": f["ff"], "experts": f["experts"] + f["identity"],
                    "identity": f["identity"], "top": f["top"], "groups": 1, "keep_groups": 1, "score": "softmax",
                    "correction": True, "renormalize": True, "renorm_eps": ROUTER_SUM_EPS, "route_scale": f["scale"],
                    "gated": False, "activation": "relu2", "shared_size": f["shared"],
                    "projection_names": ("gate", "up", "down")})
            parts.update(ffn_norm=norm, ffn=ffn)
            names.update(ffn_norm="norm2", ffn="mlp")
        layers.append(LayerSpec(block=block, prefix=f"l{index}", parts=parts, names=names))
    spec = ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=config.width,
        max_position_embeddings=config.max_positions,
        embedding_name="embed.weight",
        layers=layers,
        schedule=[ScheduleEntry(layer=index, cache=index) for index in range(len(layers))],
        final_norm=norm,
        final_norm_name="final.norm",
        head_name=None,
        embedding_scale=config.embedding_scale,
    )
    spec.validate()
    return spec


register_architecture("Fasolorn", FasolornConfig.from_dict, fasolorn_model_spec,
                      tensor_alias=nobupel_tensor_alias, stored_name=nobupel_stored_name)
