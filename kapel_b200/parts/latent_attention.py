"""Attention whose queries and whose keys and values come through low-rank latents.

Only the normed key/value latent c [kv_rank] and the one rotated key part [rot_dim] of a row are
kept: they are one line of a paged cache with a single kv head, whose value table is the key
table itself (a line's first kv_rank components are its value). The heads' own key and value
matrices never meet the cache: a head's plain score q_plain . (uk_h c) is (uk_h^T q_plain) . c, so each
query is carried into the latent's space once a row (`head_linear` with uk), attention runs with
all heads on the one cached line (keys of kv_rank + rot_dim, values of kv_rank), and the head's
output uv_h (sum_j p_j c_j) is one more small product a head, which also applies the output gate.

    stacked = [dq; dkv; g] h            one product, 32-bit sums
    c_q, cache line                     `latent_append`: both RMS norms, the key part's rotation, the append
    q = uq c_q                          [rows, heads, head_dim + rot_dim]
    q' = [uk_h^T q_plain | rot(q_rot)]  `head_linear` with the rotation of the tail
    y = attention(q', lines, sink)      the tensor-core kernel for such lines (bfloat16) or the row-wise kernel; the sink in the denominator
    o = (uv_h y) * sigmoid(g)           `head_linear` with the gate, then the output product

A rotation of neighbouring components (2i, 2i+1) runs through the same kernels, which pair component i
with i + rot/2: the rotated parts only ever meet in the dot product q_rot . k_rot, which does not change
when both are reordered alike, so the rows of uq and dkv that make them are reordered once at load (the
even components first, then the odd ones).
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache import CacheNeeds, PagedKV
from .base import Part, linear, matrix_named, pad_columns, product_width, stack_rows
from .registry import build_part


class LatentAttention(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w, H = spec.weights, spec.num_heads
        out = {
            w["dq"]: (spec.q_rank, spec.hidden), w["dq_norm"]: (spec.q_rank,),
            w["uq"]: (H * (spec.head_dim + spec.rot_dim), spec.q_rank),
            w["dkv"]: (spec.kv_rank + spec.rot_dim, spec.hidden), w["dkv_norm"]: (spec.kv_rank,),
            w["uk"]: (H * spec.head_dim, spec.kv_rank), w["uv"]: (H * spec.v_head_dim, spec.kv_rank),
            w["o"]: (spec.hidden, H * spec.v_head_dim),
        }
        if spec.sink:
            out[w["sink"]] = (H,)
        if spec.gated:
            out[w["g"]] = (H * spec.v_head_dim, spec.hidden)
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.rot_dim % 2:
            raise ValueError(f"latent_attention: a rotated part of {spec.rot_dim} components must be even")
        self.position = build_part("position", spec.position, ctx)
        if self.position.rotary_dim != spec.rot_dim:
            raise ValueError(f"latent_attention: the rotation covers {self.position.rotary_dim} of the {spec.rot_dim} rotated components")

    def load(self, tensors):
        s, w, ctx = self.spec, self.spec.weights, self.ctx
        H = s.num_heads
        names = [w["dq"], w["dkv"]] + ([w["g"]] if s.gated else [])
        self.w_down = stack_rows(ctx, tensors, names, "latent_attention")
        w_uq = matrix_named(ctx, tensors, w["uq"])
        if getattr(self.position, "neighbours", False):
            r, d = s.rot_dim, s.head_dim
            order = torch.cat([torch.arange(0, r, 2), torch.arange(1, r, 2)]).to(ctx.device)
            at = s.q_rank + s.kv_rank
            self.w_down[at : at + r] = self.w_down[at : at + r].index_select(0, order)
            w_uq = w_uq.clone().view(H, d + r, -1)
            w_uq[:, d:] = w_uq[:, d:].index_select(1, order)
            w_uq = w_uq.view(H * (d + r), -1)
        self.w_uq = pad_columns(ctx, w_uq)           # the append kernel writes the latent this wide
        self.w_o = pad_columns(ctx, matrix_named(ctx, tensors, w["o"]))
        dev = ctx.device
        # a matrix a head. In 32-bit [heads, in, out] for the FMA kernel: uk as it is stored (rows are a head's plain
        # components), uv turned. In bfloat16 [heads, out, in] for the tensor-core kernel: uk turned, uv as it is stored.
        uk = tensors[w["uk"]].to(dev).to(ctx.dtype).view(H, s.head_dim, s.kv_rank)
        uv = tensors[w["uv"]].to(dev).to(ctx.dtype).view(H, s.v_head_dim, s.kv_rank)
        self.turned = not ctx.is_f32
        self.m_uk = (uk.transpose(1, 2) if self.turned else uk).contiguous()
        self.m_uv = (uv if self.turned else uv.transpose(1, 2)).contiguous()
        norm = lambda n: (tensors[n].to(dev).float() if ctx.is_f32 else tensors[n].to(dev).contiguous())
        self.norm_q, self.norm_kv = norm(w["dq_norm"]), norm(w["dkv_norm"])
        if self.norm_q.dtype != self.norm_kv.dtype:
            self.norm_q, self.norm_kv = self.norm_q.float(), self.norm_kv.float()
        self.sinks = tensors[w["sink"]].to(dev).float().contiguous() if s.sink else None

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(paged=PagedKV(1, s.kv_rank + s.rot_dim, None, 0, None, shared_values=True))

    def forward(self, h, batch, cache):
        s, ctx = self.spec, self.ctx
        H, d, r = s.num_heads, s.head_dim, s.rot_dim
        stacked = linear(ctx, h, self.w_down, out_dtype=torch.float32, keep_split=True)
        k_table, _ = cache.tables()
        group = batch.groups[cache.group]
        cos_sin = self.position.tables(batch)
        c_q = K.latent_append(stacked, 0, s.q_rank, s.q_rank, s.kv_rank, r, self.norm_q, self.norm_kv, s.eps,
                              cos_sin, group.lines, k_table, cache.owns, ctx.dtype, pad_to=self.w_uq.shape[1])
        q = linear(ctx, c_q, self.w_uq, out_dtype=torch.float32, keep_split=True)
        q_lat = K.head_linear(q, H, d + r, 0, self.m_uk, y_head=s.kv_rank + r, tail_off=d, tail=r, cos_sin=cos_sin, transposed=self.turned)
        if K.latent_attention_mma_takes(q_lat.dtype, s.kv_rank + r, s.kv_rank):
            y = K.latent_attention_mma(q_lat.view(-1, H, s.kv_rank + r), k_table, group.block_table, batch.row_count, batch.entry_ranges(),
                                       batch.entries, batch.longest_portion(), ctx.page_size, s.scale, batch.attention_slots(None),
                                       self.sinks, s.kv_rank)
        else:                   # the 32-bit path, and sizes the tensor-core kernel does not take
            y = K.paged_attention_rows(q_lat.view(-1, H, s.kv_rank + r), k_table, k_table, group.block_table, batch.row_entry,
                                       batch.row_count, ctx.page_size, None, s.scale, None, batch.attention_slots(None),
                                       sinks=self.sinks, value_dim=s.kv_rank)
        o = K.head_linear(y.view(-1, H * s.kv_rank), H, s.kv_rank, 0, self.m_uv, gate=stacked if s.gated else None,
                          g_off=s.q_rank + s.kv_rank + r, pad_to=product_width(ctx, H * s.v_head_dim), transposed=self.turned)
        return linear(ctx, o, self.w_o, keep_split=True)
