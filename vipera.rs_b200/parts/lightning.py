"""Linear attention with one constant decay per head, as a mixer with a state of fixed size.

Per head a matrix S [d, dv] in 32-bit floats, zero at a request's start.  From the mixer's input
h: ``q = silu(W_q h)``, ``k = silu(W_k h)``, ``v = silu(W_v h)``; for each token

    S = lambda_h S + k v^T        o = S^T q

with a decay ``lambda_h`` per head that the configuration gives.  The concatenated heads' o is
divided by its root mean square over the whole row and multiplied by a weight per value, then by
``sigmoid(W_g h)``, and sent through the output matrix, which adds into the stream the mixer is
handed.  q, k, v and the gate come from one product with the concatenated matrix; its result stays
32-bit, as do the activations, the state, the products with it and the norm
(``csrc/kernels/lightning.cu``).
"""
from __future__ import annotations

import os

import torch

from ..config.registry import MIXERS
from ..errors import InvalidArgumentError
from ..kernels import ops
from ..weights import TensorSpec
from .base import FixedState, Mixer
from .linear import Linear


class LightningAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (size of q and k per head), value_dim, decay (one
    number per head), norm_eps.  Tensors under ``<prefix>``: q, k [heads * head_dim, hidden], v, g
    [heads * value_dim, hidden], o [hidden, heads * value_dim], norm [heads * value_dim]."""

    kernels = ("lightning",)
    # Steps of this many tokens and more run their chunks side by side (the recurrence computed
    # twice); shorter ones walk each entry's tokens in one launch.
    CHUNKED_FROM = int(os.environ.get("VIPERA_SCAN_CHUNKED_FROM", 256))

    @classmethod
    def schema(cls, params, prefix):
        hidden, heads = params["hidden_size"], params["num_heads"]
        d, dv = params["head_dim"], params["value_dim"]
        return {
            f"{prefix}.q.weight": TensorSpec((heads * d, hidden)),
            f"{prefix}.k.weight": TensorSpec((heads * d, hidden)),
            f"{prefix}.v.weight": TensorSpec((heads * dv, hidden)),
            f"{prefix}.g.weight": TensorSpec((heads * dv, hidden)),
            f"{prefix}.o.weight": TensorSpec((hidden, heads * dv)),
            f"{prefix}.norm.weight": TensorSpec((heads * dv,), init="norm"),
        }

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden, self.heads = int(params["hidden_size"]), int(params["num_heads"])
        self.dim, self.vdim = int(params["head_dim"]), int(params["value_dim"])
        self.norm_eps = float(params["norm_eps"])
        decay = [float(x) for x in params["decay"]]
        if len(decay) != self.heads:
            raise InvalidArgumentError(f"{prefix}: one decay per head is needed")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(device=device, dtype=torch.float32).contiguous()
        rows = [tensors[f"{prefix}.{n}.weight"] for n in ("q", "k", "v", "g")]
        widths = [r.shape[0] for r in rows]
        self.offsets = tuple(sum(widths[:i]) for i in range(4))
        self.proj = Linear(torch.cat(rows, dim=0), dtype, device)
        self.out = Linear(tensors[f"{prefix}.o.weight"], dtype, device)
        self.norm_weight = tensors[f"{prefix}.norm.weight"].to(device=device, dtype=torch.float32).contiguous()

    def kernel_families(self):
        return tuple(dict.fromkeys(("lightning",) + self.proj.kernel_families() + self.out.kernel_families()))

    @classmethod
    def cache_request_for(cls, params):
        return FixedState((int(params["num_heads"]) * int(params["head_dim"]) * int(params["value_dim"]),), torch.float32)

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        heads, d, dv = params["num_heads"], params["head_dim"], params["value_dim"]
        return tokens * (heads * (2 * d + 2 * dv) * 4 + heads * dv * (4 + element_bytes))

    def forward(self, ctx, h, residual, cache, writes_cache):
        count, ws = ctx.num_tokens, ctx.workspace
        proj = ws.get("lightning.proj", (count, self.proj.out_features), torch.float32)
        self.proj(ctx, h, epilogue=ops.EPI_STORE, out=proj)
        raw = ws.get("lightning.raw", (count, self.heads * self.vdim), torch.float32)
        mixed = ws.get("lightning.out", (count, self.heads * self.vdim), ctx.dtype)
        chunk_state = None
        if not ctx.all_single and count >= self.CHUNKED_FROM:
            chunk_state = ws.get("lightning.chunk_states",
                                 (ops.scan_jobs(count, ctx.num_entries), self.heads * self.dim * self.vdim), torch.float32)
        ops.lightning(proj, offsets=self.offsets, heads=self.heads, dim=self.dim, vdim=self.vdim, decay=self.decay,
                      norm_weight=self.norm_weight, norm_eps=self.norm_eps, state=cache.data,
                      entry_starts=ctx.entry_starts, state_slots=ctx.state_slots, fresh=ctx.fresh,
                      num_entries=ctx.num_entries, raw=raw, out=mixed, chunk_state=chunk_state)
        self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)


MIXERS.register("lightning", LightningAttention)
