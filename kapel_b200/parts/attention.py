"""Grouped-query attention over the paged cache.

q, k, v come from one stacked product (Kapel stacks them at load: crates/kapel-models/src/model.rs:415-480,
1506-1517); one kernel rotates q and k and appends k and v to the cache at the rows' lines
(Kapel: rope_any twice and write_rows_any twice, model.rs:1561-1579); attention reads the pages
through the block table with scale, soft cap and window as arguments (model.rs:1580-1590);
then the output product (model.rs:1633-1637).

A spec may ask for more than that: a norm over the whole query and key projections, values of
another size than keys, first keys that stay visible below the window, a sigmoid gate on the
heads' outputs. Such a layer runs the general path: one stacked product q|k|v|g in 32-bit, one
kernel that norms q and k and appends k and v to the cache, the row-wise attention kernel (which
knows the kept first keys and the values' size), the gate, the output product.

A spec with an RMS norm over every head's query and key (`q_head_norm`, `k_head_norm`: one weight
of the head's size for all heads) runs the third path: the stacked product in 32-bit, one kernel
that norms each head, rotates it and appends keys and values (of their own size) to the cache,
then the tensor-core kernels where keys and values have one size and the row-wise kernel elsewhere.

A spec with biases, pooled blocks below the window, a number a head on the scores, mixed heads'
weights or values mixed with another layer's runs the fourth path (`forward_pooled`): the stacked
product in 32-bit; one kernel for biases, the norms over the whole projections, the rotation (either
pairing), the value mix and the append; one that leaves the means of every block the step completes
in the request's slot of the layer's state table; then the attention kernel over window and blocks.

A spec with short convolutions on queries and keys whose values are its keys runs the fifth path
(`forward_convolved`): the stacked product q|k in 32-bit; one kernel that adds the biases, convolves every
channel over the last rows (the rows before the step from the request's state) and appends the keys, which
are also the values (one table); the row-wise attention kernel with the block mask and 1 in the
denominator; the output product, whose bias the caller may add (`forward_unbiased`, `out_bias`).
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache import CacheNeeds, PagedKV, StateSpec
from .base import Part, linear, matrix_named, pad_columns, product_width, require_product_widths, stack_rows
from .registry import build_part


class Attention(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        dv = spec.v_head_dim or spec.head_dim
        qd, kvd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        w = spec.weights
        if spec.values_are_keys:
            out = {w["q"]: (qd, spec.hidden), w["k"]: (kvd, spec.hidden), w["o"]: (spec.hidden, qd)}
            if spec.conv:
                out[w["q_conv"]], out[w["k_conv"]] = (qd, spec.conv), (kvd, spec.conv)
            if spec.qk_bias:
                out[w["q_bias"]], out[w["k_bias"]] = (qd,), (kvd,)
            if spec.out_bias:
                out[w["o_bias"]] = (spec.hidden,)
            return out
        out = {w["q"]: (qd, spec.hidden), w["k"]: (kvd, spec.hidden), w["v"]: (spec.num_kv_heads * dv, spec.hidden),
               w["o"]: (spec.hidden, spec.num_heads * dv)}
        if spec.gated:
            out[w["g"]] = (spec.num_heads * dv, spec.hidden)
        for n in (spec.q_norm, spec.k_norm, spec.q_head_norm, spec.k_head_norm):
            if n is not None:
                out[n.weight] = (n.width,)
        if spec.bias:
            out[w["q_bias"]], out[w["k_bias"]], out[w["v_bias"]] = (qd,), (kvd,), (spec.num_kv_heads * dv,)
        if spec.head_temp:
            out[w["temp"]] = (spec.num_heads,)
        if spec.talk:
            out[w["talk"]] = (spec.num_heads, spec.num_heads)
        if spec.value_mix == "mix":
            out[w["vmix"]] = ()
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"attention: {spec.num_heads} heads over {spec.num_kv_heads} kv heads")
        self.v_dim = spec.v_head_dim or spec.head_dim
        self.by_head = bool(spec.q_head_norm or spec.k_head_norm)
        self.convolved = bool(spec.conv or spec.values_are_keys or spec.block_mask or spec.unit_sink or spec.qk_bias or spec.out_bias)
        self.out_bias = None
        if self.convolved:
            if not (spec.values_are_keys and 1 <= spec.conv <= 16):
                raise ValueError("attention: a block mask, 1 in the denominator or biases on q, k and o are built for the path with "
                                 f"convolutions (1 to 16 rows, got {spec.conv}) whose values are its keys")
            if (self.by_head or spec.gated or spec.q_norm or spec.k_norm or spec.keep_first or spec.softcap or spec.window or spec.bias
                    or spec.pool or spec.head_temp or spec.talk or spec.value_mix or spec.v_head_dim not in (None, spec.head_dim)):
                raise ValueError("attention: convolutions together with norms, a gate, a window, a soft cap, pooled blocks, mixed heads or "
                                 "values of their own are not built")
            if spec.block_mask < 0:
                raise ValueError(f"attention: blocks of {spec.block_mask} positions")
        self.pooled = bool(spec.bias or spec.pool or spec.head_temp or spec.talk or spec.value_mix)
        if self.pooled:
            if self.by_head or spec.gated or spec.keep_first or spec.softcap:
                raise ValueError("attention: biases, pooled blocks, head temperatures, mixed heads or mixed values together with norms "
                                 "over each head, a gate, kept first keys or a soft cap are not built")
            if spec.pool and (not spec.window or spec.pool_blocks <= 0):
                raise ValueError(f"attention: blocks of {spec.pool} need a window (got {spec.window}) and a count of blocks (got {spec.pool_blocks})")
            if spec.value_mix not in (None, "source", "mix"):
                raise ValueError(f"attention: value_mix {spec.value_mix!r} is not known (\"source\", \"mix\")")
        self.general = bool(spec.gated or spec.q_norm or spec.k_norm or spec.keep_first or self.v_dim != spec.head_dim) and not self.by_head \
            and not self.pooled
        if self.by_head and (spec.q_norm or spec.k_norm or spec.keep_first or spec.window):
            raise ValueError("attention: norms over each head together with norms over the whole projection, a window or kept first keys are not built")
        for n in (spec.q_head_norm, spec.k_head_norm):
            if n is not None and (n.kind != "rms" or n.width != spec.head_dim):
                raise ValueError(f"attention: a norm over each head must be an RMS norm of width {spec.head_dim}")
        if not self.general and not self.by_head and not self.pooled and not self.convolved and spec.head_dim % 16:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be a multiple of 16 for the kernels")
        if spec.keep_first < 0 or (spec.keep_first and not spec.window):
            raise ValueError(f"attention: {spec.keep_first} first keys kept with window {spec.window}")
        for n, width in ((spec.q_norm, spec.num_heads * spec.head_dim), (spec.k_norm, spec.num_kv_heads * spec.head_dim)):
            if n is not None and (n.kind != "rms" or n.width != width):
                raise ValueError(f"attention: a norm over the whole projection must be an RMS norm of width {width}")
        if not self.general and not self.by_head and not self.pooled and not self.convolved:
            require_product_widths(ctx, "attention", hidden_size=spec.hidden,
                                   **{"num_attention_heads x value size": spec.num_heads * self.v_dim})
        self.position = build_part("position", spec.position, ctx)
        if self.general and self.position.rotary_dim:
            raise ValueError("attention: a rotation together with projection norms, a gate, kept first keys or another value size is not built")
        if self.convolved and self.position.rotary_dim:
            raise ValueError("attention: a rotation together with convolutions is not built")
        if not self.pooled and getattr(self.position, "neighbours", False):
            raise ValueError("attention: the rotation of neighbouring components is built for the path with biases, pooled blocks or mixed heads only")

    def load_convolved(self, tensors):
        s, w, dev = self.spec, self.spec.weights, self.ctx.device
        self.w_qkv = stack_rows(self.ctx, tensors, [w["q"], w["k"]], "attention")
        self.w_o = pad_columns(self.ctx, matrix_named(self.ctx, tensors, w["o"]))
        f32 = lambda n: tensors[n].to(dev).float().contiguous()
        self.conv = torch.cat([f32(w["q_conv"]), f32(w["k_conv"])], dim=0).contiguous()
        self.qk_bias = torch.cat([f32(w["q_bias"]), f32(w["k_bias"])]).contiguous() if s.qk_bias else None
        self.out_bias = f32(w["o_bias"]) if s.out_bias else None
        self.ones = torch.ones((s.hidden,), dtype=torch.float32, device=dev) if s.out_bias else None
        self.sinks = torch.zeros((s.num_heads,), dtype=torch.float32, device=dev) if s.unit_sink else None      # e^0 = 1 in the denominator

    def load(self, tensors):
        if self.convolved:
            return self.load_convolved(tensors)
        w = self.spec.weights
        names = [w["q"], w["k"], w["v"]] + ([w["g"]] if self.spec.gated else [])
        self.w_qkv = stack_rows(self.ctx, tensors, names, "attention")
        self.w_o = matrix_named(self.ctx, tensors, w["o"])
        if (self.general and self.spec.gated) or self.by_head or self.pooled:
            self.w_o = pad_columns(self.ctx, self.w_o)
        if self.pooled:
            dev = self.ctx.device
            small = lambda name: (tensors[name].to(dev).float() if self.ctx.is_f32 else tensors[name].to(dev)).contiguous()
            self.biases = tuple(small(w[r]) for r in ("q_bias", "k_bias", "v_bias")) if self.spec.bias else None
            self.temp = tensors[w["temp"]].to(dev).float().contiguous() if self.spec.head_temp else None
            self.talk = tensors[w["talk"]].to(dev).float().contiguous() if self.spec.talk else None
            self.v_weight = small(w["vmix"]).reshape(1) if self.spec.value_mix == "mix" else None
        self.proj_norms = []
        for n in (self.spec.q_head_norm, self.spec.k_head_norm) if self.by_head else (self.spec.q_norm, self.spec.k_norm):
            if n is None:
                self.proj_norms.append(None)
                continue
            t = tensors[n.weight]
            t = t.to(self.ctx.device) if t.device != self.ctx.device else t
            self.proj_norms.append((t.float() if self.ctx.is_f32 else t.contiguous(), n.eps, n.offset))

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        if self.convolved:
            # one table: a key is also the value. A block mask gives no pages back (a block's pages stay until the request ends).
            states = (("conv", StateSpec((K.conv_state_floats(s.num_heads, s.num_kv_heads, s.head_dim, s.conv),))),)
            return CacheNeeds(paged=PagedKV(s.num_kv_heads, s.head_dim, None, 0, None, shared_values=True), states=states)
        if self.pooled and s.pool:
            # The pages keep the window's tokens, and a block's tokens until its last one has come (the
            # means are taken from the pages then); the means of a request's blocks are its state.
            kept = max(s.window, s.pool)
            return CacheNeeds(paged=PagedKV(s.num_kv_heads, s.head_dim, kept, 0, self.v_dim if self.v_dim != s.head_dim else None),
                              state=StateSpec((s.pool_blocks, s.num_kv_heads, s.head_dim + self.v_dim)))
        return CacheNeeds(paged=PagedKV(s.num_kv_heads, s.head_dim, s.window, s.keep_first if s.window else 0,
                                        self.v_dim if self.v_dim != s.head_dim else None))

    def forward_pooled(self, h, batch, cache):
        s, dv = self.spec, self.v_dim
        nq, nk = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        stacked = linear(self.ctx, h, self.w_qkv, out_dtype=torch.float32, keep_split=True)
        k_table, v_table = cache.tables()
        group = batch.groups[cache.group]
        rotary = self.position.rotary_dim
        v_other = None
        if s.value_mix == "mix":
            v_other = batch.memo.get(("value_mix", s.value_mix_key))
            if v_other is None:
                raise ValueError(f"attention: values are mixed with those of {s.value_mix_key!r}, which no earlier layer of the step has kept")
        q, kept = K.proj_rope_append(
            stacked, 0, nq, nq + nk, self.biases, self.proj_norms[0], self.proj_norms[1],
            self.position.tables(batch) if rotary else None, rotary, getattr(self.position, "neighbours", False),
            v_other, self.v_weight if v_other is not None else None, s.value_mix == "source", group.lines, k_table, v_table,
            s.num_heads, s.num_kv_heads, s.head_dim, dv, cache.owns, self.ctx.dtype)
        if kept is not None:
            batch.memo[("value_mix", s.value_mix_key)] = kept
        pooled = None
        if s.pool:
            pooled = cache.state()
            if cache.owns:
                K.pool_blocks(k_table, v_table, group.block_table, batch.row_entry, batch.positions, group.lines, batch.slots, pooled, s.pool)
        splits, split_keys = batch.pooled_slices(s.window, s.pool) if hasattr(batch, "pooled_slices") else (1, 0)
        tiles = batch.pooled_tiles() if hasattr(batch, "pooled_tiles") else None
        y = K.pooled_attention(q, k_table, v_table, pooled, group.block_table, batch.row_entry, batch.row_count, batch.slots,
                               self.talk, self.temp, self.ctx.page_size, s.window, s.pool, s.scale, splits, split_keys, tiles,
                               batch.longest_count() if tiles is not None else None)
        width = product_width(self.ctx, s.num_heads * dv)
        y = y.view(y.shape[0], s.num_heads * dv)
        if width != y.shape[1]:
            y = K.pad_cols(y, width)
        return linear(self.ctx, y, self.w_o, keep_split=True)

    def forward_unbiased(self, h, batch, cache):
        """`forward` without the output product's bias (`out_bias`), for a caller that adds it in a kernel of its own."""
        if not self.convolved:
            return self.forward(h, batch, cache)
        s = self.spec
        nq = s.num_heads * s.head_dim
        stacked = linear(self.ctx, h, self.w_qkv, out_dtype=torch.float32, keep_split=True)
        k_table, _ = cache.tables()
        group = batch.groups[cache.group]
        q = K.conv_append(stacked, 0, nq, self.qk_bias, self.conv, cache.state_of("conv"), batch.row_entry, batch.entry_ranges(),
                          batch.slots, batch.entries, group.lines, k_table, s.num_heads, s.num_kv_heads, s.head_dim, s.conv, cache.owns,
                          self.ctx.dtype)
        q = q.view(-1, s.num_heads, s.head_dim)
        heads_per_kv = s.num_heads // s.num_kv_heads
        y = None
        if s.head_dim % 16 == 0 and K.attention_mma_takes(q.dtype, s.head_dim, heads_per_kv):
            # prompt portions go to the tensor-core kernel, which knows the block mask and the sink (in one slot: a row
            # reads at most a block of keys); a pass of single tokens stays with the row-wise kernel below
            decode, tiles, _, _, _ = batch.attention_tiles(heads_per_kv, s.num_kv_heads, None, s.head_dim, "mma", keep_first=0)
            if not decode:
                y = K.paged_attention_mma(q, k_table, k_table, group.block_table, batch.row_count, tiles, self.ctx.page_size, None,
                                          s.scale, None, 0, 0, 1, False, block=s.block_mask, sinks=self.sinks)
        if y is None:
            y = K.paged_attention_rows(q, k_table, k_table, group.block_table, batch.row_entry, batch.row_count, self.ctx.page_size,
                                       None, s.scale, None, batch.attention_slots(s.block_mask or None), sinks=self.sinks,
                                       block=s.block_mask)
        y = y.view(y.shape[0], nq)
        width = product_width(self.ctx, nq)
        if width != nq:
            y = K.pad_cols(y, width)
        return linear(self.ctx, y, self.w_o, keep_split=True)

    def forward_general(self, h, batch, cache):
        s, dv = self.spec, self.v_dim
        nq, nk = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        stacked = linear(self.ctx, h, self.w_qkv, out_dtype=torch.float32, keep_split=True)
        k_table, v_table = cache.tables()
        group = batch.groups[cache.group]
        q = K.proj_norm_append(stacked, 0, nq, nq + nk, self.proj_norms[0], self.proj_norms[1], group.lines, k_table, v_table,
                               s.num_heads, s.num_kv_heads, s.head_dim, dv, cache.owns, self.ctx.dtype)
        heads_per_kv = s.num_heads // s.num_kv_heads
        y = None
        if dv == s.head_dim and K.attention_mma_takes(q.dtype, s.head_dim, heads_per_kv):
            # prompt portions go to the tensor-core kernel, which knows the kept first keys; a pass of
            # single tokens stays with the row-wise kernel below
            decode, tiles, split, slots, _ = batch.attention_tiles(heads_per_kv, s.num_kv_heads, s.window, s.head_dim, "mma",
                                                                   keep_first=s.keep_first if s.window else 0)
            if not decode:
                y = K.paged_attention_mma(q, k_table, v_table, group.block_table, batch.row_count, tiles, self.ctx.page_size,
                                          s.window, s.scale, s.softcap, 0, split, slots, False,
                                          keep_first=s.keep_first if s.window else 0)
        if y is None:
            y = K.paged_attention_rows(
                q, k_table, v_table, group.block_table, batch.row_entry, batch.row_count, self.ctx.page_size, s.window, s.scale,
                s.softcap, batch.attention_slots(s.window, s.keep_first), s.keep_first)
        if s.gated:
            y = K.head_gate(y, stacked, nq + nk + s.num_kv_heads * dv, None, False, 0.0, self.ctx.dtype,
                            pad_to=product_width(self.ctx, s.num_heads * dv))
            return linear(self.ctx, y, self.w_o, keep_split=True)
        return linear(self.ctx, y.view(y.shape[0], s.num_heads * dv), self.w_o, keep_split=True)

    def forward_by_head(self, h, batch, cache):
        s, dv = self.spec, self.v_dim
        nq, nk = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        stacked = linear(self.ctx, h, self.w_qkv, out_dtype=torch.float32, keep_split=True)
        k_table, v_table = cache.tables()
        group = batch.groups[cache.group]
        rotary = self.position.rotary_dim
        q = K.head_norm_rope_append(stacked, 0, nq, nq + nk, self.proj_norms[0], self.proj_norms[1],
                                    self.position.tables(batch) if rotary else None, rotary, group.lines, k_table, v_table,
                                    s.num_heads, s.num_kv_heads, s.head_dim, dv, cache.owns, self.ctx.dtype)
        heads_per_kv = s.num_heads // s.num_kv_heads
        if dv == s.head_dim and s.head_dim % 16 == 0 and K.attention_mma_takes(q.dtype, s.head_dim, heads_per_kv):
            decode, tiles, split, slots, relative = batch.attention_tiles(
                heads_per_kv, s.num_kv_heads, None, s.head_dim,
                K.attention_prompt_kernel(s.num_heads, s.num_kv_heads, s.head_dim, self.ctx.page_size, s.softcap))
            y = K.paged_attention_mma(q, k_table, v_table, group.block_table, batch.row_count, tiles, self.ctx.page_size, None,
                                      s.scale, s.softcap, decode, split, slots, relative, pairs=getattr(batch, "pairs", None))
        else:
            y = K.paged_attention_rows(q, k_table, v_table, group.block_table, batch.row_entry, batch.row_count, self.ctx.page_size,
                                       None, s.scale, s.softcap, batch.attention_slots(None))
        width = product_width(self.ctx, s.num_heads * dv)
        if s.gated:
            y = K.head_gate(y, stacked, nq + nk + s.num_kv_heads * dv, None, False, 0.0, self.ctx.dtype, pad_to=width)
        else:
            y = y.view(y.shape[0], s.num_heads * dv)
            if width != y.shape[1]:
                y = K.pad_cols(y, width)
        return linear(self.ctx, y, self.w_o, keep_split=True)

    def forward(self, h, batch, cache):
        s = self.spec
        if self.convolved:
            y = self.forward_unbiased(h, batch, cache)
            return K.weighted_sum2(y, self.ones, None, None, self.out_bias) if self.out_bias is not None else y
        if self.pooled:
            return self.forward_pooled(h, batch, cache)
        if self.by_head:
            return self.forward_by_head(h, batch, cache)
        if self.general:
            return self.forward_general(h, batch, cache)
        qkv = linear(self.ctx, h, self.w_qkv, keep_split=True)
        k_table, v_table = cache.tables()
        group = batch.groups[cache.group]
        heads_per_kv = s.num_heads // s.num_kv_heads
        if K.attention_decode_fused_takes(qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.position.rotary_dim,
                                          self.ctx.page_size, self.ctx.dtype):
            decode, tiles, split, slots, relative = batch.attention_tiles(
                heads_per_kv, s.num_kv_heads, s.window, s.head_dim,
                K.attention_prompt_kernel(s.num_heads, s.num_kv_heads, s.head_dim, self.ctx.page_size, s.softcap))
            if decode and relative:         # every request brings one token: rotation, the cache's new line and attention in one kernel
                y = K.paged_attention_decode_fused(
                    qkv, self.position.tables(batch), group.lines, k_table, v_table, group.block_table, batch.row_count,
                    s.num_heads, s.num_kv_heads, s.head_dim, cache.owns, self.ctx.page_size, s.window, s.scale, s.softcap,
                    split, slots)
                return linear(self.ctx, y.view(y.shape[0], s.num_heads * s.head_dim), self.w_o, keep_split=True)
        q = K.rope_append(
            qkv, self.position.tables(batch), group.lines, k_table, v_table,
            s.num_heads, s.num_kv_heads, s.head_dim, self.position.rotary_dim, write_kv=cache.owns,
            out_dtype=self.ctx.dtype,
        )
        if K.attention_mma_takes(q.dtype, s.head_dim, heads_per_kv):
            decode, tiles, split, slots, relative = batch.attention_tiles(
                heads_per_kv, s.num_kv_heads, s.window, s.head_dim,
                K.attention_prompt_kernel(s.num_heads, s.num_kv_heads, s.head_dim, self.ctx.page_size, s.softcap))
            y = K.paged_attention_mma(
                q, k_table, v_table, group.block_table, batch.row_count, tiles,
                self.ctx.page_size, s.window, s.scale, s.softcap, decode, split, slots, relative,
                pairs=getattr(batch, "pairs", None),
            )
        else:                   # the 32-bit path, and sizes the tensor-core kernel does not take
            y = K.paged_attention_rows(
                q, k_table, v_table, group.block_table, batch.row_entry, batch.row_count,
                self.ctx.page_size, s.window, s.scale, s.softcap, batch.attention_slots(s.window),
            )
        return linear(self.ctx, y.view(y.shape[0], s.num_heads * s.head_dim), self.w_o, keep_split=True)
