"""Parts a decoder is put together from.  Importing this package registers the built-in
kinds: ``rmsnorm`` and ``layernorm``; ``rope_neox``, ``rope_interleaved`` and ``none``; ``gqa_attention``, ``latent_attention``, ``mlstm``, ``mamba1``, ``gla``, ``lightning`` and ``parallel``; ``swiglu`` (also ``gated_mlp``) and ``moe_mlp``; ``prenorm``, ``prenorm_mixer``, ``outnorm_conv`` and ``sandwich``."""
from . import attention, block, gla, latent, lightning, mamba, mlp, mlstm, moe, norm, parallel, rotary  # noqa: F401  (registration)
from .base import (
    CacheBundle,
    FeedForward,
    FixedState,
    Mixer,
    Norm,
    PagedKV,
    PagedKVView,
    Part,
    PositionEncoding,
    StateView,
    StepContext,
    Workspace,
)
from .block import Block
from .linear import Linear, NormedInput, interleave_gate_up
from .model import DecoderModel, model_schema

__all__ = [
    "CacheBundle", "FeedForward", "FixedState", "Mixer", "Norm", "PagedKV", "PagedKVView", "Part", "PositionEncoding",
    "StateView", "StepContext", "Workspace", "Block", "Linear", "NormedInput", "interleave_gate_up", "DecoderModel", "model_schema",
]
