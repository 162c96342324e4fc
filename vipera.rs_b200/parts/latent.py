"""Attention over a cached low-rank latent.

From the mixer's input h: ``q = W_q h`` (head by head ``[d unrotated | r rotated]``) and
``W_dkv h = [c' | k_r']``; the latent ``c = rmsnorm(c') * w`` [rank] and the rotated key part
``k_r = rot(k_r')`` [r], shared by all heads, are all a token leaves in the cache.  Head h's key
is ``[U_h c | k_r]`` and its value ``V_h c``; the score is ``scale * (q_d . U_h c + rot(q_r) . k_r)``,
the mask causal, the softmax plain.  The concatenated heads are multiplied by ``sigmoid(W_g h)``
(where the mixer has an output gate) and sent through the output matrix, which adds into the stream
the mixer is handed.

Since ``q . (U_h c) = (U_h^T q) . c`` and ``sum_j p_j V_h c_j = V_h sum_j p_j c_j``, the heads attend
to the latents themselves (``csrc/kernels/latent.cu``): no earlier token's keys or values are ever
expanded.  The pages hold the latents where other attention keeps keys (one "KV head" of ``rank``
values) and the rotated key part where it keeps values (``rot_dim`` values).  A layer built with
``own_cache = False`` has no down projection: it reads the pages another layer of the same latent
geometry wrote in this step (the schedule hands it that layer's cache slot without write access).
Scores, softmax, the sums over keys, the latent's norm and the rotation are 32-bit.  In bfloat16
the fold over the keys runs on the tensor cores, sixteen (token, head) rows of one request to a
block, and a step of few tokens cuts its keys between blocks.
"""
from __future__ import annotations

import torch

from ..config.registry import MIXERS, POSITION_ENCODINGS
from ..errors import UnsupportedError
from ..kernels import ops
from ..weights import TensorSpec
from .base import Mixer, PagedKV
from .linear import Linear


HEAD_MAJOR_FROM = 64   # tokens of a step from which the up products run head by head on the tensor cores


class LatentAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (unrotated q/k values per head), rot_dim (rotated
    values per head; the key's are shared), value_dim, kv_rank, softmax_scale, norm_eps, position (a
    PartSpec of a rotary encoding over rot_dim values: interleaved pairs or halves) and, optionally,
    ``own_cache`` (default true), ``output_gate`` (default false), ``window`` (a query at position p
    sees keys p - window + 1 .. p; pages the window has left are given back).  Tensors under ``<prefix>``: q [heads * (head_dim +
    rot_dim), hidden], dkv [kv_rank + rot_dim, hidden] and dkv.norm [kv_rank] (with a cache of its
    own), uk [heads * head_dim, kv_rank], uv [heads * value_dim, kv_rank], g [heads * value_dim,
    hidden] (with a gate), o [hidden, heads * value_dim]."""

    kernels = ("latent",)

    @classmethod
    def schema(cls, params, prefix):
        hidden, heads = params["hidden_size"], params["num_heads"]
        d, r, dv, rank = params["head_dim"], params["rot_dim"], params["value_dim"], params["kv_rank"]
        schema = {
            f"{prefix}.q.weight": TensorSpec((heads * (d + r), hidden)),
            f"{prefix}.uk.weight": TensorSpec((heads * d, rank)),
            f"{prefix}.uv.weight": TensorSpec((heads * dv, rank)),
            f"{prefix}.o.weight": TensorSpec((hidden, heads * dv)),
        }
        if params.get("own_cache", True):
            schema[f"{prefix}.dkv.weight"] = TensorSpec((rank + r, hidden))
            schema[f"{prefix}.dkv.norm.weight"] = TensorSpec((rank,), init="norm")
        if params.get("output_gate", False):
            schema[f"{prefix}.g.weight"] = TensorSpec((heads * dv, hidden))
        return schema

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden, self.heads = int(params["hidden_size"]), int(params["num_heads"])
        self.dim, self.rot, self.vdim = int(params["head_dim"]), int(params["rot_dim"]), int(params["value_dim"])
        self.rank = int(params["kv_rank"])
        self.scale, self.norm_eps = float(params["softmax_scale"]), float(params["norm_eps"])
        self.own_cache = bool(params.get("own_cache", True))
        self.gated = bool(params.get("output_gate", False))
        self.window = int(params.get("window") or 0)
        if self.rank > ops.LATENT_MAX_RANK or self.rot > ops.LATENT_MAX_ROT or self.rot % 2:
            raise UnsupportedError(f"{prefix}: latent attention takes a rank up to {ops.LATENT_MAX_RANK} and an even "
                                   f"rotated part up to {ops.LATENT_MAX_ROT}")
        # one product for everything that reads h: q, the gate's pre-activation, the down projection
        names = ["q"] + (["g"] if self.gated else []) + (["dkv"] if self.own_cache else [])
        rows = [tensors[f"{prefix}.{name}.weight"] for name in names]
        starts = {name: sum(r.shape[0] for r in rows[:i]) for i, name in enumerate(names)}
        self.q_off, self.g_off, self.kv_off = starts["q"], starts.get("g", -1), starts.get("dkv", -1)
        self.proj = Linear(torch.cat(rows, dim=0), dtype, device)
        self.up_k = tensors[f"{prefix}.uk.weight"].to(device=device, dtype=dtype).contiguous()
        # each head's value matrix transposed, [heads, rank, value_dim]: neighbouring threads read neighbouring values
        self.up_v = tensors[f"{prefix}.uv.weight"].to(device=device, dtype=dtype).view(
            self.heads, self.vdim, self.rank).transpose(1, 2).contiguous()
        # for long steps in bfloat16 both products run as grouped tensor-core products, a head a group:
        # U_h transposed [heads, rank, d] and V_h as stored [heads, value_dim, rank]
        self.head_major = (dtype == torch.bfloat16 and self.rank % 8 == 0 and self.rot % 8 == 0 and self.dim % 8 == 0)
        self.up_k_t = self.up_v_rows = None
        if self.head_major:
            self.up_k_t = self.up_k.view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
            self.up_v_rows = tensors[f"{prefix}.uv.weight"].to(device=device, dtype=dtype).view(
                self.heads, self.vdim, self.rank).contiguous()
        self.latent_norm = None
        if self.own_cache:
            self.latent_norm = tensors[f"{prefix}.dkv.norm.weight"].to(device=device, dtype=torch.float32).contiguous()
        self.out = Linear(tensors[f"{prefix}.o.weight"], dtype, device)
        position = params["position"]
        self.position = POSITION_ENCODINGS.find(position.kind)(position.params, prefix, tensors, dtype, device)
        if self.position.style not in (ops.ROPE_INTERLEAVED, ops.ROPE_NEOX) or \
                int(getattr(self.position, "rot_dims", 0)) != self.rot:
            raise UnsupportedError(f"{prefix}: the rotated part turns as pairs over all its {self.rot} values")

    def kernel_families(self):
        grouped = ("gemm_tc",) if self.head_major else ()
        return tuple(dict.fromkeys(("latent",) + grouped + self.proj.kernel_families() + self.out.kernel_families()))

    def prepare(self, max_positions: int) -> None:
        self.position.prepare(max_positions)

    @classmethod
    def cache_request_for(cls, params):
        return PagedKV(1, int(params["kv_rank"]), params.get("window") or None, value_dim=int(params["rot_dim"]))

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        heads, rank, r = params["num_heads"], params["kv_rank"], params["rot_dim"]
        width = heads * (params["head_dim"] + r + params["value_dim"]) + rank + r
        # (the splits of a step of few tokens: at most some 600 blocks of 16 rows more than the step's own)
        padded = tokens + 127
        head_major = heads * padded * (params["head_dim"] * 2 + rank * 6 + params["value_dim"] * 4) + tokens * heads * r * 4 + 4096
        return (tokens * (width * 4 + heads * (2 * rank + r) * 4 + heads * params["value_dim"] * element_bytes)
                + 16 * (rank + 2) * 4 * 1300 + head_major)

    def forward(self, ctx, h, residual, cache, writes_cache):
        if writes_cache != self.own_cache:
            raise UnsupportedError(f"{self.prefix}: a layer with a down projection writes its cache, one without reads another's")
        count, ws = ctx.num_tokens, ctx.workspace
        proj = ws.get("latent.proj", (count, self.proj.out_features), torch.float32)
        self.proj(ctx, h, epilogue=ops.EPI_STORE, out=proj)
        qa = ws.get("latent.qa", (count, self.heads, self.rank + self.rot), torch.float32)
        mixed_latent = ws.get("latent.mixed", (count, self.heads, self.rank), torch.float32)
        mixed = ws.get("latent.out", (count, self.heads * self.vdim), ctx.dtype)
        cos, sin = self.position.tables()
        max_keys = max(int(ctx.max_kv_len), 1)
        # (with a window the splits past it see no key and leave at once; the combine skips them)
        floats = ops.latent_part_floats(count, self.heads, self.rank, max_keys, ops.sm_count(h.device)) if ctx.dtype == torch.bfloat16 else 0
        part = ws.get("latent.part", (floats,), torch.float32) if floats else None
        head_major = None
        if self.head_major and count >= HEAD_MAJOR_FROM:
            padded = -(-count // 128) * 128
            head_major = {
                "padded": padded, "up_k_t": self.up_k_t, "up_v_rows": self.up_v_rows,
                "a_heads": ws.get("latent.a_heads", (self.heads * padded, self.dim), torch.bfloat16),
                "qa_heads": ws.get("latent.qa_heads", (self.heads * padded, self.rank), torch.float32),
                "q_rot": ws.get("latent.q_rot", (count, self.heads * self.rot), torch.float32),
                "l_heads": ws.get("latent.l_heads", (self.heads * padded, self.rank), torch.bfloat16),
                "o_heads": ws.get("latent.o_heads", (self.heads * padded, self.vdim), torch.float32),
                "tile_group": ws.get("latent.tile_group", (self.heads * padded // 128,), torch.int32),
            }
        ops.latent_attention(proj, q_off=self.q_off, g_off=self.g_off, kv_off=self.kv_off, up_k=self.up_k, up_v=self.up_v,
                             norm_weight=self.latent_norm, eps=self.norm_eps, positions=ctx.positions,
                             token_entry=ctx.token_entry, block_table=ctx.block_tables[cache.group], cos=cos, sin=sin,
                             k_pool=cache.k, v_pool=cache.v, qa=qa, latent_out=mixed_latent, out=mixed, heads=self.heads,
                             head_dim=self.dim, rot_dim=self.rot, value_dim=self.vdim, scale=self.scale, max_keys=max_keys,
                             part=part, head_major=head_major, window=self.window, pairing=self.position.style)
        self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)


MIXERS.register("latent_attention", LatentAttention)
