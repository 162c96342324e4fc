"""A mixture of gated feed-forward units.

``z = R h`` in 32-bit gives a score per expert, ``s = sigmoid(z)`` (or ``softmax(z)``).  The experts
form ``groups`` equal groups of neighbours; a group's score is the sum of its ``group_score_top``
largest scores, and only experts of the ``keep_groups`` best groups may be chosen.  A token uses the
``top`` experts with the largest scores among those, weighted by their scores (divided by their
sum with ``renormalize``): ``y = sum_e w_e D_e (act(G_e h) * (U_e h))``.

The step's (token, expert) assignments are sorted by expert on the device and each expert's run is
cut into tiles of rows, so that a tile's products read one expert's matrices; the grid depends on
the step's size only, and the step can be captured in a CUDA graph (``csrc/kernels/moe.cu``).  A
step of few assignments streams each used expert's matrices once through tiles of 8 rows; a long
step in bfloat16 pads every expert's run to whole tiles of 128 rows and runs the two products as
grouped products on the tensor cores, the gated unit as the first one's ending.  Each
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

    kernels = ("moe", "gemm_tc")
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
        hidden, inter = params["hidden_size"], params["intermediate_size"]
        capacity = ops.moe_capacity(tokens, top, experts)
        return (capacity * (inter * element_bytes + hidden * (element_bytes + 4)) + tokens * top * (hidden * 4 + 8)
                + 4 * ops.moe_scratch_words(tokens, top, experts) + 1024)

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

        # gate and up rows in one tensor: interleaved in sixteens where the tensor-core ending can
        # read them (bfloat16, an inner size of whole sixteens), else all gate rows, then all up rows
        self.gate_group = ops.MOE_GATE_GROUP if dtype == torch.bfloat16 and self.inter % ops.MOE_GATE_GROUP == 0 else self.inter
        pieces = self.inter // self.gate_group
        self.gate_up = torch.stack([stacked(gate).view(self.experts, pieces, self.gate_group, self.hidden),
                                    stacked(up).view(self.experts, pieces, self.gate_group, self.hidden)],
                                   dim=2).reshape(self.experts, 2 * self.inter, self.hidden).contiguous()
        self.down = stacked(down)

    def forward(self, ctx, h, residual):
        count, ws = ctx.num_tokens, ctx.workspace
        capacity = ops.moe_capacity(count, self.top, self.experts)
        chosen = ws.get("moe.chosen", (count, self.top), torch.int32)
        weight = ws.get("moe.weight", (count, self.top), torch.float32)
        scratch = ws.get("moe.scratch", (ops.moe_scratch_words(count, self.top, self.experts),), torch.int32)
        act = ws.get("moe.act", (capacity, self.inter), ctx.dtype)
        rows = ws.get("moe.rows", (count, self.top * self.hidden), torch.float32)
        xs = ys = None
        if ops.moe_form(count, self.top, self.hidden, self.inter, self.gate_group, ctx.dtype)[1]:
            xs = ws.get("moe.xs", (capacity, self.hidden), ctx.dtype)
            ys = ws.get("moe.ys", (capacity, self.hidden), torch.float32)
        ops.moe(h, router=self.router, gate_up=self.gate_up, down=self.down, gate_group=self.gate_group, top=self.top,
                groups=self.groups, keep=self.keep, group_top=self.group_top, softmax_scores=self.softmax_scores,
                renormalize=self.renormalize, activation=self.activation, chosen=chosen, weight=weight, scratch=scratch,
                act=act, rows=rows, xs=xs, ys=ys)
        if residual is None:
            return rows, self.top
        ops.add_rows(rows, self.top, residual)
        return None


FEED_FORWARDS.register("moe_mlp", MixtureOfExperts)
