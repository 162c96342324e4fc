"""Rotary position encoding, NeoX pairing ``(i, i + d/2)``.

Angles as the reference computes them, in 32-bit: ``inv_i = 1 / base^(2i/d)``,
``angle = position * inv_i`` (crates/vipera-backend-cpu/src/model.rs:4204-4206).  The
reference builds the table once per position and step and shares it between layers
(model.rs:970-973); here one table is built on the host for the positions the engine can
reach (``prepare``; the model's own limit where nobody says) and shared by every layer with
the same head size and base.  Tables live as long as a part holds them.
"""
from __future__ import annotations

import math
import weakref

import torch

from ..errors import InvalidArgumentError

from ..config.registry import POSITION_ENCODINGS
from ..kernels import ops
from .base import PositionEncoding

class _Tables:
    """(cos, sin) held by the parts that use them; the shared table forgets them with the last part."""

    def __init__(self, cos, sin):
        self.pair = (cos, sin)


_TABLES = weakref.WeakValueDictionary()


def yarn_blend(inverse: torch.Tensor, dims: int, theta: float, scaling: dict):
    """YaRN scaling of the frequencies ``inverse`` [dims/2] of a rotation over ``dims`` values:
    (blended frequencies, stretch of cos and sin).  ``scaling`` holds ``factor``, ``original``
    (the length the model first saw), and ``fast`` and ``slow``, the numbers of full turns within
    that length above which a pair keeps its frequency and below which it is slowed by the
    factor; pairs in between are blended by a linear ramp over the pair index.  The pair that
    makes t turns within the original length has index dims ln(original / (2 pi t)) / (2 ln theta).
    Both tables are stretched by 0.1 ln(factor) + 1."""
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if not (factor > 0 and original > 0 and float(scaling["fast"]) > 0 and float(scaling["slow"]) > 0):
        raise InvalidArgumentError("YaRN scaling needs positive factor, original, fast and slow")

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    low = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    high = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    index = torch.arange(dims // 2, dtype=torch.float64)
    ramp = torch.clamp((index - low) / max(high - low, 0.001), 0.0, 1.0).to(torch.float32)
    blended = inverse / torch.tensor(factor, dtype=torch.float32) * ramp + inverse * (1.0 - ramp)
    return blended, 0.1 * math.log(factor) + 1.0


def wavelength_blend(inverse: torch.Tensor, scaling: dict) -> torch.Tensor:
    """Frequency scaling by wavelength, as Llama 3.1 does it.  With l = 2 pi / f a pair's wavelength:
    f stays where l < original / high, becomes f / factor where l > original / low, and in between
    is (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  ``scaling`` holds
    ``factor``, ``low``, ``high`` and ``original`` (the length the model first saw)."""
    factor, original = float(scaling["factor"]), float(scaling["original"])
    low, high = float(scaling["low"]), float(scaling["high"])
    if not (factor > 0 and original > 0 and high > low):
        raise InvalidArgumentError("wavelength scaling needs a positive factor and original, and high above low")
    f = inverse.to(torch.float64)
    wavelength = 2.0 * math.pi / f
    s = (original / wavelength - low) / (high - low)
    blended = (1.0 - s) * f / factor + s * f
    out = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blended))
    return out.to(torch.float32)


def rotary_tables(head_dim: int, theta: float, max_positions: int, device, scaling=None, exact: bool = False) -> _Tables:
    """cos and sin, each float32 [max_positions, head_dim / 2], on ``device``; ``head_dim`` is the
    count of values that turn.  ``scaling``: None, the YaRN constants (see ``yarn_blend``), or with
    ``kind = "llama3"`` the constants of ``wavelength_blend``.  ``exact`` (without scaling): frequencies,
    angles, cosines and sines are formed in 64-bit and rounded once, so that a table entry is as good
    at position 100,000 as at position 1 (a 32-bit angle p f_i carries p f_i 2^-24 of error)."""
    frozen = None if not scaling else tuple(sorted((str(k), str(v)) for k, v in scaling.items()))
    key = (head_dim, float(theta), max_positions, str(device), frozen, bool(exact))
    cached = _TABLES.get(key)
    if cached is not None:
        return cached
    half = head_dim // 2
    if exact and not scaling:
        frequency = torch.pow(torch.tensor(float(theta), dtype=torch.float64),
                              -2.0 * torch.arange(half, dtype=torch.float64) / float(head_dim))
        angle = torch.arange(max_positions, dtype=torch.float64)[:, None] * frequency[None, :]
        tables = _Tables(torch.cos(angle).to(torch.float32).contiguous().to(device),
                         torch.sin(angle).to(torch.float32).contiguous().to(device))
        _TABLES[key] = tables
        return tables
    index = torch.arange(half, dtype=torch.float32)
    exponent = 2.0 * index / torch.tensor(float(head_dim), dtype=torch.float32)
    inverse = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), exponent)
    stretch = 1.0
    if scaling and scaling.get("kind") == "llama3":
        # this family's frequencies are formed in 64-bit and rounded once
        exact = torch.pow(torch.tensor(float(theta), dtype=torch.float64),
                          -2.0 * torch.arange(half, dtype=torch.float64) / float(head_dim))
        inverse = wavelength_blend(exact, scaling)
    elif scaling:
        inverse, stretch = yarn_blend(inverse, head_dim, float(theta), scaling)
    position = torch.arange(max_positions, dtype=torch.float32)
    angle = position[:, None] * inverse[None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    if stretch != 1.0:
        cos, sin = cos * stretch, sin * stretch
    tables = _Tables(cos.contiguous().to(device), sin.contiguous().to(device))
    _TABLES[key] = tables
    return tables


class RopeNeox(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``max_positions`` and, optionally, ``rotary_dims`` (only
    the first that many values of a head turn, value i with value i + rotary_dims/2; default: the
    whole head), ``scaling`` (the YaRN constants, see ``yarn_blend``) and ``exact_angles`` (true, without
    scaling: the tables are formed in 64-bit and rounded once).  No tensors."""

    style = ops.ROPE_NEOX
    kernels = ("rope_cache",)

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        self.rot_dims = int(params.get("rotary_dims") or self.head_dim)
        if self.rot_dims % 2 or not 0 < self.rot_dims <= self.head_dim:
            raise InvalidArgumentError(f"rotary_dims {self.rot_dims} must be even and within the head size {self.head_dim}")
        self.scaling = dict(params["scaling"]) if params.get("scaling") else None
        self.exact = bool(params.get("exact_angles", False))
        self.reach = None   # positions the tables cover; the model's own limit where nobody says
        self._tables = None

    def prepare(self, max_positions: int) -> None:
        """An engine reaches positions below `max_positions` only: the tables are sized for the
        furthest any engine on this model has asked for, and never shrink."""
        reach = min(self.max_positions, int(max_positions))
        if self.reach is not None and reach <= self.reach:
            return
        self.reach = reach
        if self._tables is not None:
            # Tables in use move: graphs that captured their addresses are stale.
            self._tables = None
            ops.buffer_generation += 1

    def tables(self):
        if self._tables is None:
            if self.reach is None:
                self.reach = self.max_positions
            self._tables = rotary_tables(self.rot_dims, self.theta, self.reach, self.device, self.scaling, self.exact)
        return self._tables.pair


class RopeInterleaved(RopeNeox):
    """The same angles with the other pairing: values ``(2i, 2i + 1)`` turn together.  No fused
    ending knows it; the rotation kernel behind the q/k/v product does (so it runs unfused)."""

    style = ops.ROPE_INTERLEAVED


class NoPositions(PositionEncoding):
    """Leaves q and k as they are."""

    style = ops.ROPE_NONE

    def tables(self):
        return (None, None)


POSITION_ENCODINGS.register("rope_neox", RopeNeox)
POSITION_ENCODINGS.register("rope_interleaved", RopeInterleaved)
POSITION_ENCODINGS.register("none", NoPositions)
