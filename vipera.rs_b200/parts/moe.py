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

Further options.  Units without a gate, ``y_e = D_e act(U_e h)`` (``gated`` false; ``act`` may then be
``relu2``, the square of relu).  A correction per router output that is added to the scores for the
choice only (``correction``).  Router outputs without matrices (``identity``: the last that many),
which return the token's own row times their weight.  ``renorm_eps`` joins the sum the weights are
divided by, ``route_scale`` multiplies them.  A shared unit of the same form (``shared_size``, its
inner size) that every token uses: since ``D act(U h)`` is a sum over the inner features, it is cut
into pieces of the experts' inner size (the last filled up with zero features) that ride along as
further units with weight 1, through the same tiles and products.
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
    ``activation`` (``silu`` or ``gelu_tanh``; without a gate also ``relu2``), ``projection_names``
    (default gate, up, down), ``gated`` (default true; false: no gate matrices), ``identity`` (default 0:
    the last that many of the ``experts`` router outputs have no matrices), ``correction`` (true: tensor
    ``<prefix>.correction.weight`` [experts]), ``route_scale`` (default 1), ``renorm_eps`` (default 0),
    ``shared_size`` (default none: the inner size of a shared unit, tensors ``<prefix>.shared.<name>.weight``).
    Tensors: ``<prefix>.router.weight`` [experts, hidden] and, per expert k that has matrices,
    ``<prefix>.e<k>.<gate|up>.weight`` [intermediate, hidden] and ``<prefix>.e<k>.<down>.weight``
    [hidden, intermediate]."""

    kernels = ("moe", "gemm_tc")
    leaves_rows = True   # forward(ctx, h, None) returns (rows [tokens, top * hidden] float32, top)

    @staticmethod
    def _names(params):
        return params.get("projection_names", ("gate", "up", "down"))

    @classmethod
    def schema(cls, params, prefix):
        hidden, inter, experts = params["hidden_size"], params["intermediate_size"], int(params["experts"])
        gate, up, down = cls._names(params)
        gated = bool(params.get("gated", True))
        schema = {f"{prefix}.router.weight": TensorSpec((experts, hidden), store="float32")}
        if params.get("correction", False):
            schema[f"{prefix}.correction.weight"] = TensorSpec((experts,), init="correction", store="float32")
        units = [(f"e{k}", inter) for k in range(experts - int(params.get("identity") or 0))]
        if params.get("shared_size"):
            units.append(("shared", int(params["shared_size"])))
        for unit, size in units:
            if gated:
                schema[f"{prefix}.{unit}.{gate}.weight"] = TensorSpec((size, hidden))
            schema[f"{prefix}.{unit}.{up}.weight"] = TensorSpec((size, hidden))
            schema[f"{prefix}.{unit}.{down}.weight"] = TensorSpec((hidden, size))
        return schema

    @staticmethod
    def _counts(params):
        """(matrices, a token's places): the units with matrices and the assignments a token has."""
        inter = int(params["intermediate_size"])
        pieces = -(-int(params["shared_size"]) // inter) if params.get("shared_size") else 0
        return int(params["experts"]) - int(params.get("identity") or 0) + pieces, int(params["top"]) + pieces

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        experts, top = cls._counts(params)
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
        self.gated = bool(params.get("gated", True))
        name = str(params.get("activation", "silu"))
        known = ops.ACTIVATIONS if self.gated else ops.UNIT_ACTIVATIONS
        if name not in known:
            raise UnsupportedError(f"activation {name!r}; the unit knows: " + ", ".join(sorted(known)))
        self.activation = known[name]
        self.identity = int(params.get("identity") or 0)
        self.route_scale = float(params.get("route_scale", 1.0))
        self.renorm_eps = float(params.get("renorm_eps", 0.0))
        self.shared_size = int(params.get("shared_size") or 0)
        self.always = -(-self.shared_size // self.inter) if self.shared_size else 0
        self.matrices, self.slots = self._counts(params)
        if not 0 <= self.identity < self.experts or self.matrices > ops.MOE_MAX_EXPERTS:
            raise UnsupportedError(f"{prefix}: {self.identity} of {self.experts} router outputs without matrices")
        self.correction = None
        if params.get("correction", False):
            self.correction = tensors[f"{prefix}.correction.weight"].to(device=device, dtype=torch.float32).contiguous()
        if (self.experts % self.groups or not 0 < self.keep <= self.groups or self.group_top not in (1, 2)
                or not 0 < self.top <= self.keep * (self.experts // self.groups) or self.experts > ops.MOE_MAX_EXPERTS):
            raise UnsupportedError(f"{prefix}: {self.experts} experts in {self.groups} groups of which {self.keep} are kept "
                                   f"cannot give a token {self.top} experts")
        gate, up, down = self._names(params)
        self.router = tensors[f"{prefix}.router.weight"].to(device=device, dtype=torch.float32).contiguous()

        def stacked(which, features_last=False):
            """The units' matrices [matrices, ...]: the experts', then the shared unit's cut into pieces of
            the experts' inner size along its features (the last piece filled up with zeros)."""
            units = [tensors[f"{prefix}.e{k}.{which}.weight"] for k in range(self.experts - self.identity)]
            if self.always:
                whole = tensors[f"{prefix}.shared.{which}.weight"]
                spare = self.always * self.inter - self.shared_size
                if features_last:
                    whole = torch.cat([whole, whole.new_zeros(self.hidden, spare)], dim=1)
                    units.extend(whole[:, i * self.inter:(i + 1) * self.inter] for i in range(self.always))
                else:
                    whole = torch.cat([whole, whole.new_zeros(spare, self.hidden)], dim=0)
                    units.extend(whole[i * self.inter:(i + 1) * self.inter] for i in range(self.always))
            return torch.stack(units).to(device=device, dtype=dtype).contiguous()

        # gate and up rows in one tensor: interleaved in sixteens where the tensor-core ending can
        # read them (bfloat16, an inner size of whole sixteens), else all gate rows, then all up rows
        self.gate_group = ops.MOE_GATE_GROUP if dtype == torch.bfloat16 and self.inter % ops.MOE_GATE_GROUP == 0 else self.inter
        if self.gated:
            pieces = self.inter // self.gate_group
            self.gate_up = torch.stack([stacked(gate).view(self.matrices, pieces, self.gate_group, self.hidden),
                                        stacked(up).view(self.matrices, pieces, self.gate_group, self.hidden)],
                                       dim=2).reshape(self.matrices, 2 * self.inter, self.hidden).contiguous()
        else:
            self.gate_up = stacked(up)
        self.down = stacked(down, features_last=True)

    def forward(self, ctx, h, residual):
        count, ws = ctx.num_tokens, ctx.workspace
        capacity = ops.moe_capacity(count, self.slots, self.matrices)
        chosen = ws.get("moe.chosen", (count, self.slots), torch.int32)
        weight = ws.get("moe.weight", (count, self.slots), torch.float32)
        scratch = ws.get("moe.scratch", (ops.moe_scratch_words(count, self.slots, self.matrices),), torch.int32)
        act = ws.get("moe.act", (capacity, self.inter), ctx.dtype)
        rows = ws.get("moe.rows", (count, self.slots * self.hidden), torch.float32)
        xs = ys = None
        # (units without a gate take the tensor-core form with the activation its store ending knows)
        grouped_ok = self.gated or self.activation == ops.ACT_RELU2
        if grouped_ok and ops.moe_form(count, self.slots, self.hidden, self.inter,
                                       self.gate_group if self.gated else ops.MOE_GATE_GROUP, ctx.dtype)[1]:
            xs = ws.get("moe.xs", (capacity, self.hidden), ctx.dtype)
            ys = ws.get("moe.ys", (capacity, self.hidden), torch.float32)
        ops.moe(h, router=self.router, gate_up=self.gate_up, down=self.down, gate_group=self.gate_group, top=self.top,
                groups=self.groups, keep=self.keep, group_top=self.group_top, softmax_scores=self.softmax_scores,
                renormalize=self.renormalize, activation=self.activation, chosen=chosen, weight=weight, scratch=scratch,
                act=act, rows=rows, xs=xs, ys=ys, gated=self.gated, correction=self.correction, identity=self.identity,
                always=self.always, route_scale=self.route_scale, renorm_eps=self.renorm_eps)
        if residual is None:
            return rows, self.slots
        ops.add_rows(rows, self.slots, residual)
        return None


FEED_FORWARDS.register("moe_mlp", MixtureOfExperts)
