"""Causal grouped-query attention over the paged cache: the "attention" mixer.

Order of work as the reference's layer body (dynalm/src/model/transformer.cpp:607-654): q, k, v
projections (here one product against the row-wise concatenation [Wq; Wk; Wv], which changes no
result), position encoding of q and k, write of k and v into the cache, attention of every row over
its request's keys, output projection. The mixer keeps sizes and constants from its spec only.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import POSITIONS, CacheSpec, TensorDecl, register_mixer


@register_mixer("attention")
class PagedAttention:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts (and graph_key) only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        qw, kw = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return {
            "q": TensorDecl((qw, spec.width)),
            "k": TensorDecl((kw, spec.width)),
            "v": TensorDecl((kw, spec.width)),
            "o": TensorDecl((spec.width, qw)),
            "q_bias": TensorDecl((qw,), role="vector", required=False, init="bias"),
            "k_bias": TensorDecl((kw,), role="vector", required=False, init="bias"),
            "v_bias": TensorDecl((kw,), role="vector", required=False, init="bias"),
            "o_bias": TensorDecl((spec.width,), role="vector", required=False, init="bias"),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        if spec.head_dim % 16 or not 0 < spec.head_dim <= 256:
            raise Unsupported(f"attention: head_dim {spec.head_dim} must be a multiple of 16, at most 256")
        if spec.num_heads % spec.num_kv_heads:
            raise Unsupported(f"attention: {spec.num_heads} heads do not divide into {spec.num_kv_heads} KV heads")
        self.spec = spec
        self.rt = runtime
        self.q_width = spec.num_heads * spec.head_dim
        self.kv_width = spec.num_kv_heads * spec.head_dim
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        biases = [tensors.get("q_bias"), tensors.get("k_bias"), tensors.get("v_bias")]
        if any(b is not None for b in biases):
            widths = (self.q_width, self.kv_width, self.kv_width)
            self.b_qkv = torch.cat([b if b is not None else torch.zeros(w, dtype=torch.float32, device=runtime.device)
                                    for b, w in zip(biases, widths)]).contiguous()
        else:
            self.b_qkv = None
        self.w_o = tensors["o"]
        self.b_o = tensors.get("o_bias")
        pos = spec.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if pos is not None else None

    def step_plans(self) -> list:
        """What this mixer wants worked out once per step on the host and sent with the step's integers: the query
        tiles of its prompt kernels (kernels/attention.py)."""
        from ..kernels import attention as fast
        plans = [fast.QUERY_TILES]
        if fast.DECODE_PLANNED and fast.decode_uses_tensor_cores(self.spec):
            plans.append(fast.decode_units_plan(self.spec))
        if fast.TILE_PARTS and self.spec.head_dim in ops.PREFILL_TCGEN05_HEAD_DIMS:
            plans.append(fast.tile_parts_plan(self.spec))
        return plans

    def first_weights(self) -> torch.Tensor:
        """The weights this part streams first (a block may say so to the kernel in front, kernels/ops.stream_ahead)."""
        return self.w_qkv

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(kind="pages", entry_shape=(self.spec.num_kv_heads, self.spec.head_dim), tensors=2,
                         window=self.spec.get("window", 0))

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] normed input in the compute dtype -> [rows, width]."""
        s, rt = self.spec, self.rt
        rows = x.shape[0]
        k_cache, v_cache = cache.arrays
        table = self.position.table() if self.position is not None else None
        if owns_cache and self._fused_projection_applies(x, table):
            # one kernel projects, rotates and writes the cache
            qkv = rt.buffer("attn_qkv", (rows, self.q_width + 2 * self.kv_width))
            step_angles = getattr(self.position, "step_angles", None)
            angles = step_angles(ctx, rt) if rows > ops.SKINNY_FAST_ROWS and step_angles is not None else None
            ops.gemm_qkv_rope(x, self.w_qkv, qkv, ctx.positions, ctx.row_slot, cache.block_table, k_cache, v_cache,
                              table[0], table[2], s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size, angles)
            return self._attend_and_project(qkv, cache, ctx, rows)
        if owns_cache:
            qkv = rt.buffer("attn_qkv", (rows, self.q_width + 2 * self.kv_width))
            linear(x, self.w_qkv, qkv, self.b_qkv)
        else:
            # a layer that reads another entry's cache makes queries only
            qkv = rt.buffer("attn_qkv", (rows, self.q_width + 2 * self.kv_width))[:, :self.q_width]
            linear(x, self.w_qkv[:self.q_width], qkv, self.b_qkv[:self.q_width] if self.b_qkv is not None else None)
        if self.position is not None and table is None:
            q = qkv[:, :self.q_width].unflatten(1, (s.num_heads, s.head_dim))
            k = qkv[:, self.q_width:self.q_width + self.kv_width].unflatten(1, (s.num_kv_heads, s.head_dim)) \
                if owns_cache else None
            self.position.apply(q, k, ctx.positions[:rows])
        inv_freq, rot, pos_scale = table if table is not None else (None, 0, 1.0)
        ops.rope_cache_write(qkv, ctx.positions, ctx.row_slot, cache.block_table, k_cache, v_cache, inv_freq, rot,
                             pos_scale, s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size, write_cache=owns_cache)
        return self._attend_and_project(qkv, cache, ctx, rows)

    def _fused_projection_applies(self, x: torch.Tensor, table) -> bool:
        """bfloat16, no bias, the rotation covers the whole head, and either few rows (the weight-streaming
        kernel) or enough tiles for the tcgen05 kernel with a head size it takes (ops.QKV_ROPE_TCGEN05_MIN_ROUNDS)."""
        if not (table is not None and table[0] is not None and table[1] == self.spec.head_dim and self.b_qkv is None
                and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0):
            return False
        if x.shape[0] <= ops.SKINNY_FAST_ROWS:
            return True
        from ..kernels.gemm import rotating_epilogue_pays, tcgen05_ok
        if not rotating_epilogue_pays(x.shape[0], self.w_qkv.shape[0], self.spec.head_dim):
            return False
        qkv = self.rt.buffer("attn_qkv", (x.shape[0], self.q_width + 2 * self.kv_width))
        return tcgen05_ok(x, self.w_qkv, qkv, self.w_qkv.shape[0])

    def _attend_and_project(self, qkv: torch.Tensor, cache, ctx, rows: int) -> torch.Tensor:
        s, rt = self.spec, self.rt
        attn = rt.buffer("attn_out", (rows, self.q_width))
        if rows <= ops.SKINNY_FAST_ROWS:
            ops.stream_ahead(self.w_o)                 # taken by the decode attention, read by the product after it
        self.attend(qkv, cache, ctx, attn)
        ops.stream_ahead(None)
        if self.b_o is None:
            return linear_partial(attn, self.w_o, rt, "mixer_out")
        out = rt.buffer("mixer_out", (rows, s.width))
        linear(attn, self.w_o, out, self.b_o)
        return out

    def graph_key(self, ctx) -> tuple:
        from ..kernels import attention as fast
        if fast.DECODE_PLANNED and fast.decode_uses_tensor_cores(self.spec):
            planned = ctx.extras.get(fast.decode_units_plan(self.spec).name)
            if planned is not None and planned[1][0] > 0:
                return ()         # the grid of the planned decode kernel depends on the number of rows alone
        return (("attn_splits", fast.decode_plan(ctx, self.spec)),)

    def attend(self, qkv: torch.Tensor, cache, ctx, out: torch.Tensor) -> None:
        s = self.spec
        k_cache, v_cache = cache.arrays
        from ..kernels import attention as fast
        if fast.paged_attention(qkv, cache, ctx, out, s, self.rt):
            return
        ops.paged_attention_generic(qkv, k_cache, v_cache, cache.block_table, ctx.positions, ctx.row_slot, out,
                                    s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size, float(s.scale), s.get("window", 0))


@register_mixer("gated_attention")
class GatedNormedAttention(PagedAttention):
    """Grouped-query attention with keys of head_dim and values of value_dim numbers, a rotation of the first
    `rotary_dim` numbers of every head, a window, and what its parameters switch on:

    qk_norm     "projection": queries and keys normed over their WHOLE projection before the heads are cut and before
                the rotation (one statistic for all H * d numbers of q, one for the G * d of k; weights q_norm, k_norm);
                "head": after the rotation every head of q and k is divided by its own root mean square (no weight);
                "none".
    gated       the concatenated heads times sigmoid(W_g h) before the output projection (one product gives
                [q | k | v | gate]).
    sink        "zero": the softmax's denominator holds one more term of score 0, which carries no value; "none".
    keep_first  with a window: keys at positions below it stay visible behind the window, at their true positions.
    position    "rotary" (pairs i, i + rotary_dim / 2) or, with qk_norm "head" or "none", "rotary_interleaved" (pairs 2i,
                2i + 1).
    Biases of the four projections are taken when the model has them (q_bias, k_bias, v_bias, o_bias).

    Parameters: num_heads, num_kv_heads, head_dim, value_dim, scale, window, keep_first, eps, qk_norm, gated, sink,
    position. Tensors: q, k, v, o, and by the parameters q_norm, k_norm, gate.

    Where keys and values have one size the cache is the plain attention's (two arrays) and so are the kernels that
    read it, as far as they know the mask and the softmax asked for; otherwise a token's keys and values form one record
    [k | v] in one array, read by the plain kernel. With `keep_first` the pages behind the window are kept (the first
    of them are still read)."""

    out_name = "mixer_out"     # the workspace buffer of the result; a mixer that holds this one may name another

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        qw, kw, vw = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.num_kv_heads * spec.value_dim
        ow = spec.num_heads * spec.value_dim
        normed, gated = spec.get("qk_norm", "none") == "projection", bool(spec.get("gated", False))
        return {
            "q": TensorDecl((qw, spec.width)), "k": TensorDecl((kw, spec.width)), "v": TensorDecl((vw, spec.width)),
            "o": TensorDecl((spec.width, ow)),
            "q_norm": TensorDecl((qw,), role="vector", required=normed, init="around_one"),
            "k_norm": TensorDecl((kw,), role="vector", required=normed, init="around_one"),
            "gate": TensorDecl((ow, spec.width), required=gated),
            "q_bias": TensorDecl((qw,), role="vector", required=False, init="bias"),
            "k_bias": TensorDecl((kw,), role="vector", required=False, init="bias"),
            "v_bias": TensorDecl((vw,), role="vector", required=False, init="bias"),
            "o_bias": TensorDecl((spec.width,), role="vector", required=False, init="bias"),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        if not 0 < spec.head_dim <= 256 or not 0 < spec.value_dim <= 256:
            raise Unsupported(f"gated_attention: head_dim {spec.head_dim} and value_dim {spec.value_dim} must be at most 256")
        if spec.num_heads % spec.num_kv_heads:
            raise Unsupported(f"gated_attention: {spec.num_heads} heads do not divide into {spec.num_kv_heads} KV heads")
        if spec.get("qk_norm", "none") not in ("projection", "head", "none"):
            raise Unsupported(f"gated_attention: no query/key norm '{spec.qk_norm}' (projection, head, none)")
        if spec.get("sink", "none") not in ("zero", "none"):
            raise Unsupported(f"gated_attention: no sink '{spec.sink}' (zero, none)")
        self.spec = spec
        self.rt = runtime
        self.q_width = spec.num_heads * spec.head_dim
        self.kv_width = spec.num_kv_heads * spec.head_dim
        self.v_width = spec.num_kv_heads * spec.value_dim
        self.o_width = spec.num_heads * spec.value_dim
        self.normed = spec.get("qk_norm", "none") == "projection"
        self.head_normed = spec.get("qk_norm", "none") == "head"
        self.sink = spec.get("sink", "none") == "zero"
        self.window = int(spec.get("window", 0))
        self.keep_first = int(spec.get("keep_first", 0)) if self.window > 0 else 0
        self.gated = bool(spec.get("gated", False))
        self.same = spec.head_dim == spec.value_dim          # keys and values of one size: the plain attention's cache
        mats = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["gate"]] if self.gated else [])
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        biases = [tensors.get("q_bias"), tensors.get("k_bias"), tensors.get("v_bias")]
        self.b_qkv = None
        if any(b is not None for b in biases):
            widths = [self.q_width, self.kv_width, self.v_width] + ([self.o_width] if self.gated else [])
            self.b_qkv = torch.cat([b if b is not None else torch.zeros(w, dtype=torch.float32, device=runtime.device)
                                    for b, w in zip(biases + [None], widths)]).contiguous()
        self.q_norm, self.k_norm = (tensors["q_norm"], tensors["k_norm"]) if self.normed else (None, None)
        self.w_o = tensors["o"]
        self.b_o = tensors.get("o_bias")
        self.eps = float(spec.get("eps", 1e-6))
        pos = spec.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if pos is not None else None
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        if self.position is not None and self.position.table() is None and not self.interleaved:
            raise Unsupported("gated_attention: the rotation runs inside its kernel and takes a position encoding with a table")
        if self.interleaved and self.normed:
            raise Unsupported("gated_attention: the interleaved rotation goes with the norm per head or with none")
        # the kernels of the plain attention's cache know a window and an ordinary softmax
        self.plain_mask = not self.sink and self.keep_first == 0

    def step_plans(self) -> list:
        if self.same and self.plain_mask:
            return super().step_plans()
        from ..kernels import attention as fast
        return [fast.QUERY_TILES]                  # the masked flash kernel walks the step's query tiles

    def graph_key(self, ctx) -> tuple:
        if self.same and self.plain_mask:
            return super().graph_key(ctx) if self.rt.dtype == torch.bfloat16 else ()
        return (("masked_flash_parts", self._decode_parts(ctx)),) if self.rt.dtype == torch.bfloat16 else ()

    def _decode_parts(self, ctx) -> int:
        """Into how many parts a step of single tokens deals a row's keys (part of the launch shape, so of the graph key)."""
        if not ctx.decode_only:
            return 1
        s = self.spec
        span = ctx.max_kv_len if self.window <= 0 else min(ctx.max_kv_len, self.window + self.keep_first)
        bucket = 256
        while bucket < span:
            bucket *= 2
        group = s.num_heads // s.num_kv_heads
        return ops.masked_flash_parts(ctx.num_tokens, s.num_kv_heads if 1 < group <= 64 else s.num_heads, bucket)

    def cache_spec(self) -> Optional[CacheSpec]:
        s = self.spec
        window = self.window if self.keep_first == 0 else 0      # kept first tokens: no page is given back
        if self.same:
            return CacheSpec(kind="pages", entry_shape=(s.num_kv_heads, s.head_dim), tensors=2, window=window)
        return CacheSpec(kind="pages", entry_shape=(self.kv_width + self.v_width,), tensors=1, window=window)

    def _kv(self, cache):
        """(keys of the first token, elements between tokens, values of the first token, elements between tokens)."""
        if self.same:
            k_cache, v_cache = cache.arrays
            return k_cache, self.kv_width, v_cache, self.v_width
        (records,) = cache.arrays
        row = self.kv_width + self.v_width
        return records, row, records.view(-1)[self.kv_width:], row

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if not owns_cache:
            raise Unsupported("gated_attention: every run of the layer keeps a cache of its own")
        rows = x.shape[0]
        proj = rt.buffer("gattn_proj", (rows, self.w_qkv.shape[0]))
        by_projection = self.normed or (not self.head_normed and not self.interleaved)
        # a bias joins in the kernel that turns and norms, where that kernel takes one; else in the product (the plain one)
        linear(x, self.w_qkv, proj, self.b_qkv if (by_projection or self.gated) else None)
        k_cache, k_row, v_cache, v_row = self._kv(cache)
        if by_projection:
            inv_freq, rot, pos_scale = self.position.table() if self.position is not None else (None, 0, 1.0)
            ops.qk_proj_norm_cache(proj, self.q_norm, self.k_norm, self.eps, self.normed, inv_freq, rot, pos_scale,
                                   ctx.positions, ctx.row_slot, cache.block_table, k_cache, k_row, v_cache, v_row,
                                   s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, cache.page_size)
        else:
            # the rotation first (either layout), then every head by itself
            if self.position is None:
                inv_freq, rot = None, 0
            elif self.interleaved:
                inv_freq, rot = self.position.inv_freq, self.position.rotary_dim
            else:
                inv_freq, rot, pos_scale = self.position.table()
                if pos_scale != 1.0:
                    raise Unsupported("gated_attention: stretched positions go with the norm over the projection")
            ops.qk_rot_head_norm_cache(proj, inv_freq, rot, self.interleaved, self.head_normed, self.eps, ctx.positions,
                                       ctx.row_slot, cache.block_table, k_cache, k_row, v_cache, v_row, s.num_heads,
                                       s.num_kv_heads, s.head_dim, s.value_dim, cache.page_size,
                                       bias=None if self.gated else self.b_qkv)
        attn = rt.buffer("gattn_out", (rows, self.o_width))
        self.attend(proj, cache, ctx, attn)
        if self.gated:
            ops.sigmoid_gate(attn, proj[:, self.q_width + self.kv_width + self.v_width:])
        if self.b_o is None:
            return linear_partial(attn, self.w_o, rt, self.out_name)
        if attn.dtype == torch.float32:
            out = rt.buffer(self.out_name, (rows, s.width))
            linear(attn, self.w_o, out, self.b_o)
            return out
        # 16-bit operands: the product leaves float32 sums (whole, or split-K partial sums) and the bias joins those
        from ..kernels.gemm import skinny_ok, use_stream
        if use_stream(attn, self.w_o) or skinny_ok(attn, self.w_o):
            out = linear_partial(attn, self.w_o, rt, self.out_name)
            ops.add_bias(out[0] if out.dim() == 3 else out, self.b_o)
            return out
        out = rt.buffer(self.out_name + "_wide", (rows, s.width), torch.float32)
        linear(attn, self.w_o, out)
        ops.add_bias(out, self.b_o)
        return out

    def _flash_applies(self, qkv: torch.Tensor, cache, ctx) -> bool:
        """bfloat16, sizes the masked flash kernel has, a step built with the query tiles, aligned rows."""
        from ..kernels import attention as fast
        s = self.spec
        return (qkv.dtype == torch.bfloat16 and (s.head_dim, s.value_dim) in ops.MASKED_FLASH_SIZES
                and fast.query_tiles(ctx) is not None and cache.page_size & (cache.page_size - 1) == 0
                and qkv.stride(0) % 8 == 0 and self.kv_width % 8 == 0 and self.v_width % 8 == 0)

    def attend(self, qkv: torch.Tensor, cache, ctx, out: torch.Tensor) -> None:
        s = self.spec
        if not (self.same and self.plain_mask) and self._flash_applies(qkv, cache, ctx):
            from ..kernels import attention as fast
            q_tiles, n_tiles, _, _ = fast.query_tiles(ctx)
            k_cache, k_row, v_cache, v_row = self._kv(cache)
            parts = self._decode_parts(ctx)
            partial = None
            if parts > 1:
                most = max(self.rt.max_requests, qkv.shape[0])
                partial = self.rt.flat(f"masked_flash_parts_{s.num_heads}x{s.value_dim}",
                                       ops.masked_flash_partial_floats(most, s.num_heads, s.value_dim, ops.MASKED_FLASH_MAX_PARTS))
            ops.masked_flash_attention(qkv, k_cache, k_row, v_cache, v_row, cache.block_table, q_tiles, n_tiles, out,
                                       s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, cache.page_size,
                                       float(s.scale), self.window, self.keep_first, self.sink,
                                       one_token_tiles=ctx.decode_only, parts=parts, partial=partial)
            return
        if self.same and self.plain_mask:
            from ..kernels import attention as fast
            if fast.paged_attention(qkv, cache, ctx, out, s, self.rt):
                return
        k_cache, k_row, v_cache, v_row = self._kv(cache)
        ops.paged_attention_generic_kv(qkv, k_cache, k_row, v_cache, v_row, cache.block_table, ctx.positions, ctx.row_slot,
                                       out, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, cache.page_size,
                                       float(s.scale), self.window, self.keep_first, self.sink)
