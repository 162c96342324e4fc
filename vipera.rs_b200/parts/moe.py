"""A mixture of gated feed-forward units.

``z = R h`` in 32-bit gives a score per expert, ``s = sigmoid(z)`` (or ``softmax(z)``).  The experts
form ``groups`` equal groups of neighbours; a group's score is the sum of its ``group_score_top``
largest scores, and only experts of the ``keep_groups`` best groups may be chosen.  A token uses the
``top`` experts with the largest scores among those, weighted by their scores (divided by their
sum with ``renormalize``): ``y = sum_e w_e D_e (act(G_e h) * (U_e h))``.

The step's (token, expert) assignments are sorted by expert on the device and each expert's run is
cut into tiles of rows, so that a tile's products read one expert's matrices; the grid depends on
the step's size only, and the step can be captured in a CUDA graph (``csrc/kernels/moe.cu``).  Each
chosen expert's weighted output stays a 32-bit row of its own: an arrangement that takes rows
(``leaves_rows``) sums a token's rows in the order of its places; handed a stream, the part sums
them into it itself.
"""
from __future__ import annotations

import torch

from ..config.registry import FEED_FORWARDS
from ..errors import UnsupportedError
from ..kernels import ops
from ..weights import TensorSpec
from .base import FeedForward


class MixtureOfExperts(FeedForward):
    """params: hidden_size, intermediate_size (of one expert), experts, top and, optionally,
    ``groups`` (default 1), ``keep_groups`` (default: all), ``group_score_top`` (1 or 2, default 2),
    ``score`` (``sigmoid``, the default, or ``softmax``), ``renormalize`` (default false),
    ``activation`` (``silu`` or ``gelu_tanh``), ``projection_names`` (default gate, up, down).
    Tensors: ``<prefix>.router.weight`` [experts, hidden] and, per expert k, ``<prefix>.e<k>.<gate|up>.weight``
    [intermediate, hidden] and ``<prefix>.e<k>.<down>.weight`` [hidden, intermediate]."""

    kernels = ("moe",)
    leaves_rows = True   # forward(ctx, h, None) returns (rows [tokens, top * hidden] float32, top)

    @staticmethod
    def _names(params):
        return params.get("projection_names", ("gate", "up", "down"))

    @classmethod
    def schema(cls, params, prefix):
        hidden, inter, experts = params["hidden_size"], params["intermediate_size"], int(params["experts"])
        gate, up, down = cls._names(params)
        schema = {f"{prefix}.router.weight": TensorSpec((experts, hidden), store="float32")}
        for k in range(experts):
            schema[f"{prefix}.e{k}.{gate}.weight"] = TensorSpec((inter, hidden))
            schema[f"{prefix}.e{k}.{up}.weight"] = TensorSpec((inter, hidden))
            schema[f"{prefix}.e{k}.{down}.weight"] = TensorSpec((hidden, inter))
        return schema

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        top, experts = int(params["top"]), int(params["experts"])
        assignments = tokens * top
        return (assignments * (params["intermediate_size"] * element_bytes + params["hidden_size"] * 4 + 16)
                + 12 * ops.moe_max_tiles(tokens, top, experts) + 4)

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.experts, self.top = int(params["experts"]), int(params["top"])
        self.groups = int(params.get("groups") or 1)
        self.keep = int(params.get("keep_groups") or self.groups)
        self.group_top = int(params.get("group_score_top", 2))
        score = str(params.get("score", "sigmoid"))
        if score not in ("sigmoid", "softmax"):
            raise UnsupportedError(f"{prefix}: router scores are sigmoid or softmax, not {score!r}")
        self.softmax_scores = score == "softmax"
        self.renormalize = bool(params.get("renormalize", False))
        name = str(params.get("activation", "silu"))
        if name not in ops.ACTIVATIONS:
            raise UnsupportedError(f"activation {name!r}; the gated unit knows: " + ", ".join(sorted(ops.ACTIVATIONS)))
        self.activation = ops.ACTIVATIONS[name]
        if (self.experts % self.groups or not 0 < self.keep <= self.groups or self.group_top not in (1, 2)
                or not 0 < self.top <= self.keep * (self.experts // self.groups) or self.experts > ops.MOE_MAX_EXPERTS):
            raise UnsupportedError(f"{prefix}: {self.experts} experts in {self.groups} groups of which {self.keep} are kept "
                                   f"cannot give a token {self.top} experts")
        gate, up, down = self._names(params)
        self.router = tensors[f"{prefix}.router.weight"].to(device=device, dtype=torch.float32).contiguous()

        def stacked(which):
            return torch.stack([tensors[f"{prefix}.e{k}.{which}.weight"] for k in range(self.experts)]).to(
                device=device, dtype=dtype).contiguous()

        self.gate, self.up, self.down = stacked(gate), stacked(up), stacked(down)

    def forward(self, ctx, h, residual):
        count, ws = ctx.num_tokens, ctx.workspace
        assignments = count * self.top
        tiles = ops.moe_max_tiles(count, self.top, self.experts)
        chosen = ws.get("moe.chosen", (count, self.top), torch.int32)
        weight = ws.get("moe.weight", (count, self.top), torch.float32)
        scratch = ws.get("moe.scratch", (2 * assignments + 1 + 3 * tiles,), torch.int32)
        act = ws.get("moe.act", (assignments, self.inter), ctx.dtype)
        rows = ws.get("moe.rows", (count, self.top * self.hidden), torch.float32)
        ops.moe(h, router=self.router, gate=self.gate, up=self.up, down=self.down, top=self.top, groups=self.groups,
                keep=self.keep, group_top=self.group_top, softmax_scores=self.softmax_scores,
                renormalize=self.renormalize, activation=self.activation, chosen=chosen, weight=weight, scratch=scratch,
                act=act, rows=rows)
        if residual is None:
            return rows, self.top
        ops.add_rows(rows, self.top, residual)
        return None


FEED_FORWARDS.register("moe_mlp", MixtureOfExperts)
