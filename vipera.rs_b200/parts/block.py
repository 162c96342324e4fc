"""Arrangements of a layer's parts.

An arrangement declares its roles: which named parts it reads from the layer's description
and which registry each comes from.  ``Block`` builds them, so a new arrangement (four norms
around the two sub-layers, a mixer beside the feed-forward, one norm only) is a subclass
that names its roles and writes ``forward``; nothing else changes.

``prenorm``: ``x += mixer(norm(x))``, then ``x += ffn(norm(x))`` — the order of
crates/vipera-backend-cpu/src/model.rs:977-1198.  The residual stream is 32-bit; mixers
and feed-forwards add into it themselves, so that the addition can be the ending of their
last product.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Registry
from ..errors import UnsupportedError
from ..kernels import ops
from ..weights import TensorSpec
from .base import CacheBundle, FixedState, StateView
from .conv import CausalConv
from .linear import Linear, NormedInput
from .norm import LayerNorm


class Block:
    """Base of all arrangements.  ``roles`` maps a role's name to the registry its part is
    looked up in; the built parts are attributes of the same names.  ``cache_role`` names the
    role whose part says what the layer keeps between steps (``cache_request()``); the layer's
    cache slot is handed to ``forward`` and the arrangement passes it on to that part."""

    roles: Dict[str, Registry] = {}
    cache_role = "mixer"

    def __init__(self, layer_spec, tensors, dtype, device):
        self.spec = layer_spec
        self.params = layer_spec.params
        self._parts = {}
        for role, registry in self.roles.items():
            part_spec = self._role_spec(layer_spec, role)
            part = registry.find(part_spec.kind)(part_spec.params, layer_spec.part_prefix(role), tensors, dtype, device)
            setattr(self, role, part)
            self._parts[role] = part

    @classmethod
    def _role_spec(cls, layer_spec, role):
        from ..errors import InvalidArgumentError

        try:
            return layer_spec.parts[role]
        except KeyError:
            raise InvalidArgumentError(
                f"the {layer_spec.block!r} arrangement needs a part for the role {role!r}; "
                f"layer {layer_spec.prefix} gives {sorted(layer_spec.parts)}") from None

    @classmethod
    def schema(cls, layer_spec):
        schema = {}
        for role, registry in cls.roles.items():
            part_spec = cls._role_spec(layer_spec, role)
            schema.update(registry.find(part_spec.kind).schema(part_spec.params, layer_spec.part_prefix(role)))
        return schema

    def parts(self):
        return tuple(self._parts.values())

    def cache_request(self):
        """What this layer keeps between steps: PagedKV, FixedState or None."""
        part = self._parts.get(self.cache_role)
        return None if part is None else part.cache_request()

    @classmethod
    def cache_request_for(cls, layer_spec):
        """The same from the description alone (no weights): for memory plans."""
        if cls.cache_role not in cls.roles:
            return None
        part_spec = cls._role_spec(layer_spec, cls.cache_role)
        return cls.roles[cls.cache_role].find(part_spec.kind).cache_request_for(part_spec.params)

    @classmethod
    def workspace_bytes(cls, layer_spec, tokens, element_bytes):
        """Workspace of one execution of the layer in a step of `tokens` tokens: what its parts
        ask for, together (their buffers have names of their own and live side by side)."""
        total = 0
        for role, registry in cls.roles.items():
            part_spec = cls._role_spec(layer_spec, role)
            total += registry.find(part_spec.kind).workspace_bytes(part_spec.params, tokens, element_bytes)
        return total

    def forward(self, ctx, residual, cache, writes_cache):
        raise NotImplementedError

    @staticmethod
    def _input(part, normed: NormedInput):
        """A part that sets ``takes_lazy_input`` receives the normalised input as a NormedInput
        and may fuse the norm into its first product; any other part receives a tensor."""
        return normed if getattr(part, "takes_lazy_input", False) else normed.tensor()


class PreNormBlock(Block):
    roles = {"mixer_norm": NORMS, "mixer": MIXERS, "ffn_norm": NORMS, "ffn": FEED_FORWARDS}

    def forward(self, ctx, residual, cache, writes_cache):
        h = NormedInput(ctx, self.mixer_norm, residual)
        self.mixer.forward(ctx, self._input(self.mixer, h), residual, cache, writes_cache)
        h = NormedInput(ctx, self.ffn_norm, residual)
        self.ffn.forward(ctx, self._input(self.ffn, h), residual)


class PreNormMixerBlock(Block):
    """A layer without a feed-forward: ``x += mixer(norm(x))`` and nothing more."""

    roles = {"mixer_norm": NORMS, "mixer": MIXERS}

    def forward(self, ctx, residual, cache, writes_cache):
        h = NormedInput(ctx, self.mixer_norm, residual)
        self.mixer.forward(ctx, self._input(self.mixer, h), residual, cache, writes_cache)


class OutNormConvBlock(Block):
    """``x += norm(mixer(c(x)))`` and, where the layer has a feed-forward, ``x += norm(ffn(c(x)))``:
    the norms act on the sublayers' outputs, and what a sublayer reads is the residual stream
    itself with a short causal convolution over time added to it, ``c(h) = h + conv(h)``
    (``params``: ``taps``, ``hidden_size``; tensors ``<layer>.<mixer_conv>.weight`` and
    ``<layer>.<ffn_conv>.weight``, [hidden, taps]).  The last ``taps - 1`` rows of the stream in
    front of each sublayer are kept per request beside what the mixer keeps.

    A sublayer adds its output into the 32-bit stream it is handed; here that is a cleared
    buffer of the stream's shape, which the norm then adds into the stream."""

    roles = {"mixer": MIXERS, "mixer_norm": NORMS}
    optional_roles = {"ffn": FEED_FORWARDS, "ffn_norm": NORMS}
    conv_roles = ("mixer_conv", "ffn_conv")

    def __init__(self, layer_spec, tensors, dtype, device):
        self.roles = self._roles_of(layer_spec)
        super().__init__(layer_spec, tensors, dtype, device)
        self.hidden = int(layer_spec.params["hidden_size"])
        self.has_ffn = "ffn" in layer_spec.parts
        self.mixer_conv = CausalConv(layer_spec.part_prefix("mixer_conv"), tensors, device, add_input=True)
        self.ffn_conv = (CausalConv(layer_spec.part_prefix("ffn_conv"), tensors, device, add_input=True)
                         if self.has_ffn else None)

    @classmethod
    def _roles_of(cls, layer_spec):
        roles = dict(cls.roles)
        if "ffn" in layer_spec.parts:
            roles.update(cls.optional_roles)
        return roles

    @classmethod
    def _conv_state(cls, layer_spec):
        convs = 2 if "ffn" in layer_spec.parts else 1
        taps, hidden = int(layer_spec.params["taps"]), int(layer_spec.params["hidden_size"])
        return FixedState((convs, taps - 1, hidden), torch.float32) if taps > 1 else None

    @classmethod
    def schema(cls, layer_spec):
        schema = {}
        for role, registry in cls._roles_of(layer_spec).items():
            part_spec = cls._role_spec(layer_spec, role)
            schema.update(registry.find(part_spec.kind).schema(part_spec.params, layer_spec.part_prefix(role)))
        taps, hidden = int(layer_spec.params["taps"]), int(layer_spec.params["hidden_size"])
        for role in cls.conv_roles[:2 if "ffn" in layer_spec.parts else 1]:
            schema.update(CausalConv.schema(layer_spec.part_prefix(role), hidden, taps))
        return schema

    def parts(self):
        return tuple(self._parts.values()) + (self.mixer_conv,)

    def cache_request(self):
        return CacheBundle.of(conv=self._conv_state(self.spec), mixer=self.mixer.cache_request())

    @classmethod
    def cache_request_for(cls, layer_spec):
        part_spec = cls._role_spec(layer_spec, "mixer")
        return CacheBundle.of(conv=cls._conv_state(layer_spec),
                              mixer=MIXERS.find(part_spec.kind).cache_request_for(part_spec.params))

    @classmethod
    def workspace_bytes(cls, layer_spec, tokens, element_bytes):
        total = tokens * int(layer_spec.params["hidden_size"]) * (4 + element_bytes)   # the cleared stream and c(x)
        for role, registry in cls._roles_of(layer_spec).items():
            part_spec = cls._role_spec(layer_spec, role)
            total += registry.find(part_spec.kind).workspace_bytes(part_spec.params, tokens, element_bytes)
        return total

    def forward(self, ctx, residual, cache, writes_cache):
        ws = ctx.workspace
        cache = cache or {}
        conv_state = cache.get("conv")
        branch = ws.get("block.branch", (ctx.num_tokens, self.hidden), torch.float32)
        h = ws.get("block.h", (ctx.num_tokens, self.hidden), ctx.dtype)
        self.mixer_conv(ctx, residual, None if conv_state is None else StateView(conv_state.data[:, 0]),
                        out=h, clear=branch)
        self.mixer.forward(ctx, h, branch, cache.get("mixer"), writes_cache)
        self.mixer_norm.add_into(ctx, branch, residual)
        if self.has_ffn:
            self.ffn_conv(ctx, residual, None if conv_state is None else StateView(conv_state.data[:, 1]),
                          out=h, clear=branch)
            self.ffn.forward(ctx, h, branch)
            self.ffn_norm.add_into(ctx, branch, residual)


class SandwichBlock(Block):
    """Norms before and after each sublayer, the sublayer's output gated by its own input and
    scaled per channel, a constant multiplier on what joins the stream:

        h = N(x);  y = sublayer(h) * sigmoid(R h + r);  x += m * s * Nb(y)

    first for the mixer, then (where the layer has one) for the feed-forward.  ``params``:
    ``hidden_size``, ``residual_mult`` (m), ``layer_scale`` (true: tensors ``<layer>.<mixer_scale>.weight``
    and ``<layer>.<ffn_scale>.weight`` [hidden], the s above) and ``gated`` (true: matrices
    ``<layer>.<mixer_gate>.weight`` [hidden, hidden] with ``.bias``, and the same for ``ffn_gate``).
    The norms after the sublayers are of the RMS kind (a weight, an eps and a count of groups):
    one kernel gates the sublayer's output, norms it, scales it and adds it into the stream.

    A sublayer adds its output into the 32-bit stream it is handed; here that is a cleared buffer.
    A feed-forward may instead leave several rows per token to be added (``forward`` returning
    ``(rows, count)``), which the same kernel sums in a fixed order."""

    roles = {"mixer_norm": NORMS, "mixer": MIXERS, "mixer_out_norm": NORMS}
    optional_roles = {"ffn_norm": NORMS, "ffn": FEED_FORWARDS, "ffn_out_norm": NORMS}
    kernels = ("groupnorm",)

    def __init__(self, layer_spec, tensors, dtype, device):
        self.roles = self._roles_of(layer_spec)
        super().__init__(layer_spec, tensors, dtype, device)
        self.hidden = int(layer_spec.params["hidden_size"])
        self.mult = float(layer_spec.params.get("residual_mult", 1.0))
        self.has_ffn = "ffn" in layer_spec.parts
        self.sides = ("mixer", "ffn") if self.has_ffn else ("mixer",)
        self.gates, self.coefficients = {}, {}
        for side in self.sides:
            out_norm = self._parts[f"{side}_out_norm"]
            if getattr(out_norm, "weight", None) is None or not hasattr(out_norm, "eps") or isinstance(out_norm, LayerNorm):
                raise UnsupportedError(f"{layer_spec.prefix}: the norm after a sublayer must be an RMS norm")
            # everything that multiplies the normed output per channel, as one 32-bit vector
            coefficient = out_norm.weight * self.mult
            if layer_spec.params.get("layer_scale", False):
                scale = tensors[f"{layer_spec.part_prefix(side + '_scale')}.weight"]
                coefficient = coefficient * scale.to(device=device, dtype=torch.float32)
            self.coefficients[side] = coefficient.contiguous()
            self.gates[side] = None
            if layer_spec.params.get("gated", False):
                prefix = layer_spec.part_prefix(side + "_gate")
                self.gates[side] = Linear(tensors[f"{prefix}.weight"], dtype, device, bias=tensors[f"{prefix}.bias"])
                setattr(self, f"{side}_gate", self.gates[side])

    @classmethod
    def _roles_of(cls, layer_spec):
        roles = dict(cls.roles)
        if "ffn" in layer_spec.parts:
            roles.update(cls.optional_roles)
        return roles

    @classmethod
    def schema(cls, layer_spec):
        schema = {}
        for role, registry in cls._roles_of(layer_spec).items():
            part_spec = cls._role_spec(layer_spec, role)
            schema.update(registry.find(part_spec.kind).schema(part_spec.params, layer_spec.part_prefix(role)))
        hidden = int(layer_spec.params["hidden_size"])
        for side in ("mixer", "ffn") if "ffn" in layer_spec.parts else ("mixer",):
            if layer_spec.params.get("layer_scale", False):
                schema[f"{layer_spec.part_prefix(side + '_scale')}.weight"] = TensorSpec((hidden,), init="norm", store="float32")
            if layer_spec.params.get("gated", False):
                prefix = layer_spec.part_prefix(side + "_gate")
                schema[f"{prefix}.weight"] = TensorSpec((hidden, hidden))
                schema[f"{prefix}.bias"] = TensorSpec((hidden,), init="bias")
        return schema

    @classmethod
    def cache_request_for(cls, layer_spec):
        part_spec = cls._role_spec(layer_spec, "mixer")
        return MIXERS.find(part_spec.kind).cache_request_for(part_spec.params)

    @classmethod
    def workspace_bytes(cls, layer_spec, tokens, element_bytes):
        total = tokens * int(layer_spec.params["hidden_size"]) * (8 + element_bytes)   # cleared stream, gate, h
        for role, registry in cls._roles_of(layer_spec).items():
            part_spec = cls._role_spec(layer_spec, role)
            total += registry.find(part_spec.kind).workspace_bytes(part_spec.params, tokens, element_bytes)
        return total

    def parts(self):
        # the arrangement itself launches kernels and owns matrices, so it counts among its parts
        return tuple(self._parts.values()) + (self,)

    def kernel_families(self):
        names = self.kernels
        for gate in self.gates.values():
            if gate is not None:
                names += gate.kernel_families()
        return tuple(dict.fromkeys(names))

    def _join(self, ctx, side, h, branch, parts, residual):
        gate = None
        if self.gates[side] is not None:
            gate = ctx.workspace.get("block.gate", (ctx.num_tokens, self.hidden), torch.float32)
            self.gates[side](ctx, h, epilogue=ops.EPI_STORE, out=gate)
        out_norm = self._parts[f"{side}_out_norm"]
        ops.gated_norm_add(branch, parts, gate, self.coefficients[side], residual, out_norm.eps,
                           int(getattr(out_norm, "groups", 1)))

    def forward(self, ctx, residual, cache, writes_cache):
        ws = ctx.workspace
        branch = ws.get("block.branch", (ctx.num_tokens, self.hidden), torch.float32)
        h = NormedInput(ctx, self.mixer_norm, residual).tensor()
        branch.zero_()
        self.mixer.forward(ctx, h, branch, cache, writes_cache)
        self._join(ctx, "mixer", h, branch, 1, residual)
        if self.has_ffn:
            h = NormedInput(ctx, self.ffn_norm, residual).tensor()
            rows = self.ffn.forward(ctx, h, None) if getattr(self.ffn, "leaves_rows", False) else None
            if rows is None:
                branch.zero_()
                self.ffn.forward(ctx, h, branch)
                rows = (branch, 1)
            self._join(ctx, "ffn", h, rows[0], rows[1], residual)


BLOCKS.register("prenorm", PreNormBlock)
BLOCKS.register("sandwich", SandwichBlock)
BLOCKS.register("outnorm_conv", OutNormConvBlock)
BLOCKS.register("prenorm_mixer", PreNormMixerBlock)
