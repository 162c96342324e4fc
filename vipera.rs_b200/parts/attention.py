"""Grouped-query attention over the paged cache.

In the reference's order (crates/vipera-backend-cpu/src/model.rs:1005-1126): q, k, v products
from the normalised input, bias added after the product and before the rotation, rotation
of q and k, keys and values written to their pages, attention of every new token over its
request's keys, output product added to the residual stream.  Query head h reads KV head
h // group (model.rs:1813-1826).

Here q, k and v come from one product with the concatenated matrix (the reference keeps
three products, model.rs:1005-1025); the rotation and the cache write are one kernel; the
output product adds into the 32-bit residual stream in its own ending.
"""
from __future__ import annotations

import os

import torch

from ..config.registry import MIXERS, POSITION_ENCODINGS
from ..errors import UnsupportedError
from ..kernels import ops
from ..weights import TensorSpec
from .base import Mixer, PagedKV
from .linear import Linear, NormedInput


class GQAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, window (None or a
    count of keys), softmax_scale, position (a PartSpec of a position encoding) and,
    optionally, ``projection_names`` (defaults q_proj, k_proj, v_proj, o_proj), ``value_dim`` (the
    size of a value row and of a head's output, default head_dim), ``keep_first`` (with a window:
    the first that many keys of a request stay visible to every later query, at their true
    positions) and ``sink`` (true: a key of score 0 without a value joins every softmax, which
    adds one to its denominator).  A position encoding may turn only the first values of a head
    (its ``rot_dims``).  Further options: ``chunk`` (instead of a window, a mask of chunks: position
    i sees j <= i with floor(i / chunk) = floor(j / chunk), chunks counted from a request's
    position 0); ``values_from_keys`` (no value projection: the values are the keys as projected,
    before norm and rotation); ``row_norm`` with ``norm_eps`` (the whole q row and the whole k row
    are each divided by their root mean square and multiplied by a weight per value,
    ``<q>.norm.weight`` and ``<k>.norm.weight``, before the rotation); ``talking_heads`` (the
    softmax weights of the heads are mixed by ``<prefix>.talk.weight`` [heads, heads] before they
    meet the values, ``w_h = sum_g M[h, g] p_g``); ``out_scale`` (multiplies the mixer's output);
    ``sink = "learned"`` (the sink's score is a number per query head, ``<prefix>.sink.weight`` [heads]:
    ``exp(sink_h)`` joins the denominator, unscaled); ``output_gate`` (the concatenated heads are
    multiplied by ``sigmoid(W_g h)``, ``<prefix>.<gate_name>.weight`` [heads * value_dim, hidden],
    ``gate_name`` ``g`` by default; the gate's rows join the q/k/v product); ``value_mix``:
    ``"source"`` publishes the values of the step's tokens as projected, ``"blend"`` caches
    ``(1 - b) v + b v_source`` with ``b = <prefix>.vmix.weight`` (a single number) and ``v_source`` what
    the source layer published for the same token earlier in the step (both kinds hold the tensor;
    the source does not read it)."""

    kernels = ("rope_cache", "attention", "attention_mma", "attention_tc")
    takes_lazy_input = True
    # With mixed head weights: steps of this many tokens and more that bring portions run every
    # (query head, KV head) pair through the tensor-core flash kernel; shorter ones and steps of
    # single tokens run the split-key kernels.
    TALK_PAIRS_FROM = int(os.environ.get("VIPERA_TALK_PAIRS_FROM", 64))

    @staticmethod
    def _names(params):
        return params.get("projection_names", ("q_proj", "k_proj", "v_proj", "o_proj"))

    @classmethod
    def schema(cls, params, prefix):
        hidden, d = params["hidden_size"], params["head_dim"]
        dv = params.get("value_dim") or d
        q_width, kv_width = params["num_heads"] * d, params["num_kv_heads"] * d
        v_width = params["num_kv_heads"] * dv
        qn, kn, vn, on = cls._names(params)
        schema = {
            f"{prefix}.{qn}.weight": TensorSpec((q_width, hidden)),
            f"{prefix}.{kn}.weight": TensorSpec((kv_width, hidden)),
            f"{prefix}.{vn}.weight": TensorSpec((v_width, hidden)),
            f"{prefix}.{on}.weight": TensorSpec((hidden, params["num_heads"] * dv)),
        }
        if params.get("values_from_keys", False):
            del schema[f"{prefix}.{vn}.weight"]
        if params.get("row_norm", False):
            schema[f"{prefix}.{qn}.norm.weight"] = TensorSpec((q_width,), init="norm")
            schema[f"{prefix}.{kn}.norm.weight"] = TensorSpec((kv_width,), init="norm")
        if params.get("talking_heads", False):
            schema[f"{prefix}.talk.weight"] = TensorSpec((params["num_heads"], params["num_heads"]), init="mix")
        if params.get("sink") == "learned":
            schema[f"{prefix}.sink.weight"] = TensorSpec((params["num_heads"],), init="sink", store="float32")
        if params.get("output_gate", False):
            schema[f"{prefix}.{params.get('gate_name', 'g')}.weight"] = TensorSpec((params["num_heads"] * dv, hidden))
        if params.get("value_mix"):
            schema[f"{prefix}.vmix.weight"] = TensorSpec((), init="blend", store="float32")
        if params.get("qkv_bias", False):
            schema[f"{prefix}.{qn}.bias"] = TensorSpec((q_width,), init="bias")
            schema[f"{prefix}.{kn}.bias"] = TensorSpec((kv_width,), init="bias")
            schema[f"{prefix}.{vn}.bias"] = TensorSpec((v_width,), init="bias")
        return schema

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.window = params.get("window")
        self.keep_first = int(params.get("keep_first") or 0) if self.window else 0
        self.sink = bool(params.get("sink", False))
        self.sink_values = None
        if params.get("sink") == "learned":
            self.sink_values = tensors[f"{prefix}.sink.weight"].to(device=device, dtype=torch.float32).contiguous()
        elif params.get("sink") not in (None, False, True):
            raise UnsupportedError(f"{prefix}: sink is true or \"learned\", not {params.get('sink')!r}")
        self.gated = bool(params.get("output_gate", False))
        self.value_mix = params.get("value_mix") or None
        if self.value_mix not in (None, "source", "blend"):
            raise UnsupportedError(f"{prefix}: value_mix is \"source\" or \"blend\", not {self.value_mix!r}")
        self.blend = None
        if self.value_mix == "blend":
            self.blend = tensors[f"{prefix}.vmix.weight"].to(device=device, dtype=torch.float32).reshape(1).contiguous()
        self.scale = float(params["softmax_scale"])
        for size in (self.head_dim, self.value_dim):
            if not 0 < size <= 256:
                raise UnsupportedError(f"head size {size}: the attention kernels take sizes up to 256")
        if self.num_heads % self.num_kv_heads:
            raise UnsupportedError("the number of heads must be a multiple of the number of KV heads")
        qn, kn, vn, on = self._names(params)
        self.chunk = int(params.get("chunk") or 0)
        self.values_from_keys = bool(params.get("values_from_keys", False))
        self.row_norm = bool(params.get("row_norm", False))
        self.norm_eps = float(params.get("norm_eps", 0.0))
        self.out_scale = float(params.get("out_scale", 1.0))
        self.talk = None
        if self.chunk and self.window:
            raise UnsupportedError("attention: a mask is a window or chunks, not both")
        if self.values_from_keys and self.value_dim != self.head_dim:
            raise UnsupportedError("attention: values that are the keys have the keys' size")
        if params.get("talking_heads", False):
            if self.window or self.chunk or self.sink or self.gated or self.value_mix:
                raise UnsupportedError("attention: mixed head weights come with a plain causal mask only")
            self.talk = tensors[f"{prefix}.talk.weight"].to(device=device, dtype=torch.float32).contiguous()
        self.q_norm = self.k_norm = None
        if self.row_norm:
            self.q_norm = tensors[f"{prefix}.{qn}.norm.weight"].to(device=device, dtype=torch.float32).contiguous()
            self.k_norm = tensors[f"{prefix}.{kn}.norm.weight"].to(device=device, dtype=torch.float32).contiguous()
        if (self.gated or self.value_mix) and (self.values_from_keys or self.row_norm):
            raise UnsupportedError("attention: an output gate or blended values do not come with a norm over whole "
                                   "rows or values that are the keys")
        names = (qn, kn) if self.values_from_keys else (qn, kn, vn)
        # the gate reads the mixer's input like q, k and v: its rows are the last of the one product
        self.gate_offset = sum(tensors[f"{prefix}.{n}.weight"].shape[0] for n in names)
        if self.gated:
            names = names + (params.get("gate_name", "g"),)
        fused = torch.cat([tensors[f"{prefix}.{n}.weight"] for n in names], dim=0)
        bias = None
        if params.get("qkv_bias", False):
            bias = torch.cat([tensors[f"{prefix}.{n}.bias"].to(torch.float32) for n in (qn, kn, vn)], dim=0)
            if self.gated:
                bias = torch.cat([bias, torch.zeros(fused.shape[0] - bias.shape[0])])
        self.qkv = Linear(fused, dtype, device, bias=bias)
        self.out = Linear(tensors[f"{prefix}.{on}.weight"], dtype, device)
        position = params["position"]
        self.position = POSITION_ENCODINGS.find(position.kind)(position.params, prefix, tensors, dtype, device)
        self.rot_dims = int(getattr(self.position, "rot_dims", self.head_dim))
        # The fused endings and the tensor-core attention kernels know the common form only: values as
        # long as keys, whole heads that turn, a plain window, a plain softmax.
        self.common_form = (self.value_dim == self.head_dim and self.rot_dims == self.head_dim
                            and not self.keep_first and not self.sink and self.head_dim % 16 == 0
                            and not self.chunk and not self.values_from_keys and not self.row_norm
                            and self.talk is None and self.out_scale == 1.0 and not self.gated
                            and self.value_mix is None)

    def kernel_families(self):
        # the tensor-core attention kernels serve bfloat16 with head sizes 64 and 128; everything
        # else runs through the general kernel
        own = ["rope_cache", "attention"]
        if self.talk is not None:
            own.append("attention_talk")
            if self.dtype == torch.bfloat16 and self.head_dim in ops.MMA_HEAD_DIMS and self.value_dim == self.head_dim:
                own.append("attention_mma")
        plain_mask = self.talk is None and self.out_scale == 1.0
        if plain_mask and self.dtype == torch.bfloat16 and self.head_dim in (64, 128) and self.value_dim == self.head_dim:
            own.append("attention_mma")
            if (self.head_dim in ops.TC_ATTENTION_HEAD_DIMS and not self.keep_first and not self.chunk
                    and (not self.sink or self.sink_values is not None)):
                own.append("attention_tc")
        return tuple(dict.fromkeys(tuple(own) + self.qkv.kernel_families() + self.out.kernel_families()
                                   + self.position.kernel_families()))

    def prepare(self, max_positions: int) -> None:
        prepare = getattr(self.position, "prepare", None)
        if prepare is not None:
            prepare(max_positions)

    @classmethod
    def cache_request_for(cls, params):
        value_dim = int(params.get("value_dim") or params["head_dim"])
        window = params.get("window")
        return PagedKV(int(params["num_kv_heads"]), int(params["head_dim"]), window,
                       value_dim=value_dim if value_dim != int(params["head_dim"]) else None,
                       keep_first=int(params.get("keep_first") or 0) if window else 0)

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        dv = params.get("value_dim") or params["head_dim"]
        q_width = params["num_heads"] * params["head_dim"]
        qkv_width = q_width + params["num_kv_heads"] * (params["head_dim"] + dv)
        if params.get("output_gate", False):
            qkv_width += params["num_heads"] * dv
        if params.get("value_mix"):
            qkv_width += params["num_kv_heads"] * dv   # the published values, 32-bit
        # q and the attention's output in the run's type, and the 32-bit q/k/v product of the unfused route
        return tokens * ((q_width + params["num_heads"] * dv) * element_bytes + qkv_width * 4)

    def forward(self, ctx, h, residual, cache, writes_cache):
        count = ctx.num_tokens
        heads, kv_heads, d, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        ws = ctx.workspace
        q = ws.get("attention.q", (count, heads * d), ctx.dtype)
        table = ctx.block_tables[cache.group]
        style = self.position.style
        if self.common_form and self.qkv.takes_small(count) and style in (ops.ROPE_NONE, ops.ROPE_NEOX):
            # few tokens: one kernel for norm, q/k/v product, bias, rotation and cache write
            cos, sin = self.position.tables()
            rope = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, style=style, positions=ctx.positions,
                        cos=cos, sin=sin, q_out=q, write_cache=writes_cache, k_pool=cache.k, v_pool=cache.v,
                        token_entry=ctx.token_entry, block_table=table, page_size=cache.page_size)
            if isinstance(h, NormedInput) and h.fusable:
                ops.gemv_small(self.qkv.weight, x=h.residual, norm_weight=h.norm.weight, eps=h.norm.eps,
                               tokens=count, epilogue=ops.GEMV_ROPE_CACHE, bias=self.qkv.bias, rope=rope)
            else:
                ops.gemv_small(self.qkv.weight, a=h.tensor() if isinstance(h, NormedInput) else h,
                               epilogue=ops.GEMV_ROPE_CACHE, bias=self.qkv.bias, rope=rope)
            mixed = ws.get("attention.out", (count, heads * d), ctx.dtype)
            self._attend(ctx, q, mixed, cache, table)
            self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)
            return
        if (self.common_form and ctx.dtype == torch.bfloat16 and style in (ops.ROPE_NONE, ops.ROPE_NEOX)
                and self.qkv.tensor_core
                and ops.gemm_tc_rope_takes(count, self.qkv.out_features, self.qkv.in_features, d)):
            # many tokens: the tensor-core product ends with bias, rotation and cache write
            cos, sin = self.position.tables()
            a = h.tensor() if isinstance(h, NormedInput) else h
            ops.gemm_tc_rope(a, self.qkv.weight, bias=self.qkv.bias, q_out=q, num_heads=heads, num_kv_heads=kv_heads,
                             head_dim=d, positions=ctx.positions, cos=cos, sin=sin, style=style, k_pool=cache.k,
                             v_pool=cache.v, token_entry=ctx.token_entry, block_table=table,
                             page_size=cache.page_size, write_cache=writes_cache)
            mixed = ws.get("attention.out", (count, heads * d), ctx.dtype)
            self._attend(ctx, q, mixed, cache, table)
            self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)
            return
        qkv = ws.get("attention.qkv", (count, self.qkv.out_features), torch.float32)
        self.qkv(ctx, h, epilogue=ops.EPI_STORE, out=qkv)
        if self.row_norm or self.values_from_keys:
            if style is None:
                raise UnsupportedError("attention: a norm over whole rows needs a position encoding of the rotary kind")
            cos, sin = self.position.tables()
            ops.qk_prepare(qkv, q, num_heads=heads, num_kv_heads=kv_heads, head_dim=d, value_dim=dv,
                           rot_dims=self.rot_dims, q_norm=self.q_norm, k_norm=self.k_norm, eps=self.norm_eps,
                           values_from_keys=self.values_from_keys, positions=ctx.positions, cos=cos, sin=sin,
                           style=style, k_pool=cache.k, v_pool=cache.v, token_seq=ctx.token_entry,
                           block_table=table, page_size=cache.page_size, write_cache=writes_cache)
            mixed = ws.get("attention.out", (count, heads * dv), ctx.dtype)
            self._attend(ctx, q, mixed, cache, table)
            self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)
            return
        if style is None:
            # An encoding the fused kernel does not know: the part applies it to the 32-bit
            # product itself, then the kernel only converts and stores.
            q_view = qkv[:, : heads * d].unflatten(1, (heads, d))
            k_view = qkv[:, heads * d : (heads + kv_heads) * d].unflatten(1, (kv_heads, d))
            self.position.apply(ctx, q_view, k_view)
            style, cos, sin = ops.ROPE_NONE, None, None
        else:
            cos, sin = self.position.tables()
        if self.gated or self.value_mix:
            publish = blend_with = None
            if self.value_mix == "source":
                publish = ws.get("attention.value_mix", (count, kv_heads * dv), torch.float32)
                ctx.extras["attention.value_mix"] = publish
            elif self.value_mix == "blend":
                blend_with = ctx.extras.get("attention.value_mix")
                if blend_with is None or tuple(blend_with.shape) != (count, kv_heads * dv):
                    raise UnsupportedError(f"{self.prefix}: no earlier layer of this step published values of this "
                                           "layer's size to blend with")
            ops.rope_cache_blend(qkv, q, num_heads=heads, num_kv_heads=kv_heads, head_dim=d, value_dim=dv,
                                 rot_dims=self.rot_dims if style != ops.ROPE_NONE else 0, positions=ctx.positions,
                                 cos=cos, sin=sin, style=style, k_pool=cache.k, v_pool=cache.v,
                                 token_seq=ctx.token_entry, block_table=table, page_size=cache.page_size,
                                 write_cache=writes_cache, publish=publish, blend_with=blend_with, blend=self.blend)
        else:
            ops.rope_cache(qkv, q, num_heads=heads, num_kv_heads=kv_heads, head_dim=d,
                           positions=ctx.positions, cos=cos, sin=sin, style=style,
                           k_pool=cache.k, v_pool=cache.v, token_seq=ctx.token_entry, block_table=table,
                           page_size=cache.page_size, write_cache=writes_cache, value_dim=dv, rot_dims=self.rot_dims)
        mixed = ws.get("attention.out", (count, heads * dv), ctx.dtype)
        self._attend(ctx, q, mixed, cache, table, gate=qkv if self.gated else None)
        self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)

    def _attend(self, ctx, q, mixed, cache, table, gate=None):
        """Choose the attention kernel: on the bfloat16 path with a head size the tensor-core
        kernels are built for, the split-key kernel for steps of single tokens and the flash
        kernel otherwise; in every other case the general kernel."""
        heads, kv_heads, d = self.num_heads, self.num_kv_heads, self.head_dim
        window = self.window or 0
        if self.talk is not None:
            count = ctx.num_tokens
            tensor_cores = (ctx.dtype == torch.bfloat16 and d in ops.MMA_HEAD_DIMS and self.value_dim == d
                            and heads * kv_heads <= 4096 and os.environ.get("VIPERA_TALK_PAIRS", "1") != "0")
            if ctx.all_single and tensor_cores:
                # single tokens: the same pairs through the split-key kernel, which streams the history
                # through shared memory once per pair of KV heads
                chunk, splits = ops.decode_splits(ctx.num_entries, kv_heads * kv_heads, max(ctx.max_kv_len, 1),
                                                  ops.sm_count(q.device))
                scratch = ctx.workspace.get(
                    "attention.partials",
                    (ops.attention_decode_scratch_floats(ctx.num_entries, heads * kv_heads, d, splits),), torch.float32)
                pairs = ctx.workspace.get("attention.talk_pairs", (count, heads * kv_heads * d), torch.float32)
                ops.attention_talk_decode(q, mixed, pairs, cache.k, cache.v, self.talk, positions=ctx.positions,
                                          block_table=table, num_heads=heads, num_kv_heads=kv_heads, head_dim=d,
                                          scale=self.scale, chunk=chunk, num_splits=splits, scratch=scratch,
                                          out_scale=self.out_scale)
                return
            if not ctx.all_single and tensor_cores and count >= self.TALK_PAIRS_FROM:
                # steps with portions on the tensor cores: every (query head, KV head) pair through the
                # flash kernel, then the mix of the pairs' outputs
                pairs = ctx.workspace.get("attention.talk_pairs", (count, heads * kv_heads * d), torch.float32)
                ops.attention_talk_prefill(q, mixed, pairs, cache.k, cache.v, self.talk, entry_starts=ctx.entry_starts,
                                           entry_pos0=ctx.entry_pos0, block_table=table, num_entries=ctx.num_entries,
                                           num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=self.scale,
                                           out_scale=self.out_scale)
                return
            keys, splits = ops.talk_splits(count, max(ctx.max_kv_len, 1), ops.sm_count(q.device))
            stats = ctx.workspace.get("attention.talk_stats", (count, splits, heads, 2), torch.float32)
            partial = None if splits == 1 else ctx.workspace.get(
                "attention.talk_partial", (splits, count, heads * self.value_dim), torch.float32)
            ops.attention_talk(q, mixed, cache.k, cache.v, self.talk, token_seq=ctx.token_entry,
                               positions=ctx.positions, block_table=table, num_heads=heads, num_kv_heads=kv_heads,
                               head_dim=d, value_dim=self.value_dim, scale=self.scale, out_scale=self.out_scale,
                               split_keys=keys, num_splits=splits, stats=stats, partial=partial)
            return
        # a learned sink and an output gate are endings of the tcgen05 flash kernel and of the split-key
        # kernel's combine (plain windows only); elsewhere they run through the general kernel
        extended = self.sink_values is not None or gate is not None
        extended_ok = (not self.keep_first and not self.chunk and ops.attention_tc_takes_gate(gate, self.gate_offset)
                       and d in ops.TC_ATTENTION_HEAD_DIMS and os.environ.get("VIPERA_ATTENTION_TC", "1") != "0")
        if (self.out_scale == 1.0 and ctx.dtype == torch.bfloat16 and d in ops.MMA_HEAD_DIMS and self.value_dim == d
                and (not extended or extended_ok)):
            # Kept first keys and the sink are options of the mma.sync kernels (the flash kernel folds
            # the kept keys as tiles of their own, the split-key kernel as a split of its own); the
            # tcgen05 flash kernel serves attention without them.
            kept = dict(keep_first=self.keep_first, sink=self.sink, mask_chunk=self.chunk, sink_values=self.sink_values,
                        gate=gate, gate_offset=self.gate_offset)
            places = 1 if self.keep_first else 0
            if ctx.all_single:
                chunk, splits = ops.decode_splits(ctx.num_entries, kv_heads, max(ctx.max_kv_len, 1),
                                                  ops.sm_count(q.device))
                scratch = ctx.workspace.get(
                    "attention.partials",
                    (ops.attention_decode_scratch_floats(ctx.num_entries, heads, d, splits + places),), torch.float32)
                ops.attention_decode(q, mixed, cache.k, cache.v, positions=ctx.positions, block_table=table,
                                     num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=self.scale,
                                     window=window, chunk=chunk, num_splits=splits, scratch=scratch, **kept)
            else:
                # portions through the flash kernel; the single tokens beside them (the running
                # decodes of a mixed step) through the split-key kernel, which streams their
                # history once per KV head instead of once per head and tile of 128 queries
                ops.attention_prefill(q, mixed, cache.k, cache.v, entry_starts=ctx.entry_starts,
                                      entry_pos0=ctx.entry_pos0, block_table=table, num_entries=ctx.num_entries,
                                      num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=self.scale,
                                      window=window, skip_single=ctx.any_single, **kept)
                if ctx.any_single:
                    chunk, splits = ops.decode_splits(ctx.num_entries, kv_heads, max(ctx.max_kv_len, 1),
                                                      ops.sm_count(q.device))
                    scratch = ctx.workspace.get(
                        "attention.partials",
                        (ops.attention_decode_scratch_floats(ctx.num_entries, heads, d, splits + places),), torch.float32)
                    ops.attention_decode(q, mixed, cache.k, cache.v, positions=ctx.entry_pos0, block_table=table,
                                         num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=self.scale,
                                         window=window, chunk=chunk, num_splits=splits, scratch=scratch,
                                         entry_starts=ctx.entry_starts, **kept)
            return
        ops.attention(q, mixed, cache.k, cache.v, token_seq=ctx.token_entry, positions=ctx.positions,
                      block_table=table, num_heads=heads, num_kv_heads=kv_heads, head_dim=d,
                      scale=self.scale, window=window, value_dim=self.value_dim, keep_first=self.keep_first,
                      sink=self.sink, chunk=self.chunk, out_scale=self.out_scale, sink_values=self.sink_values,
                      gate=gate, gate_offset=self.gate_offset)


MIXERS.register("gqa_attention", GQAttention)
