"""Sequence-mixing and feed-forward mechanisms for models served as a ragged in-flight batch.

Each class holds one layer's device tensors in the layout its kernels want and has ``forward(x, ctx)``: ``x`` is the
fp32 residual stream [rows, width] of this step's token rows, ``ctx`` (``inflight.StepContext``) carries the batch
description, the paged pools and the state slots.  Every size and constant is a constructor argument, so a model
definition (``models/``) only maps its configuration and tensor names onto them.  The arithmetic is in the CUDA
operators of ``ops`` (include/trtllm_b200_ragged.h); nothing here computes on the host.

Precision: the residual stream, normalisations, softmax, the recurrent state and all that feeds the recurrence are fp32;
projections run in the storage type ``dtype`` (bf16 on tensor cores with fp32 accumulation, or fp32 throughout).
"""
from __future__ import annotations

import torch

from . import ops


class LatentAttention:
    """Attention whose keys and values are up-projections of one cached low-rank latent per position.

    h -> query latent (RMS-normed) -> per-head queries [dim unrotated | rot_dim rotated];
    h -> [lat latent (RMS-normed) | rot_dim rotated key part shared by the heads] = the cache entry.
    score_h(i, j) = scale * (q_h^nope(i) . (W_uk,h c_j) + q_h^rot(i) . k^rot_j), causal softmax, out = W_o concat_h(W_uv,h sum_j p c_j).

    The key up-projection is applied to the QUERY (q_h^nope W_uk,h, a [lat] vector) and the value up-projection to the
    attention-weighted latent, so prefill and decode both run one multi-query kernel over the cache entries and nothing
    per head is ever stored per position.  ``kv_source`` names the layer whose pool is read: the layer itself, or an
    earlier layer with the same latent geometry when this layer has no down-projection of its own."""

    def __init__(self, index, *, heads, dim, rot_dim, vdim, lat, rot_dims, rot_base, scale, eps, w_dq, w_dq_norm, w_uq,
                 w_uk, w_uv, w_o, w_dkv=None, w_dkv_norm=None, kv_source=None):
        self.index, self.heads, self.dim, self.rot_dim, self.vdim, self.lat = index, heads, dim, rot_dim, vdim, lat
        self.rot_dims, self.rot_base, self.scale, self.eps = rot_dims, float(rot_base), float(scale), float(eps)
        self.dtype = w_dq.dtype
        self.w_dq, self.w_dq_norm, self.w_uq, self.w_o = w_dq, w_dq_norm, w_uq, w_o
        # per head: [lat, dim] so that the "output" of the batched product is the absorbed query
        self.w_uk_t = w_uk.view(heads, dim, lat).transpose(1, 2).contiguous()
        self.w_uv = w_uv.view(heads, vdim, lat).contiguous()
        self.w_dkv, self.w_dkv_norm = w_dkv, w_dkv_norm
        self.owns_cache = w_dkv is not None
        self.kv_source = index if self.owns_cache else kv_source
        if not self.owns_cache and (kv_source is None or kv_source >= index):
            raise ValueError(f"layer {index}: a layer without its own latent projection reads an EARLIER layer's cache")
        if rot_dims > rot_dim or rot_dims % 2:
            raise ValueError(f"layer {index}: rotary dims {rot_dims} must be even and at most rot_dim {rot_dim}")

    @property
    def cache_entry(self):
        return self.lat + self.rot_dim

    def forward(self, x, ctx):
        n, H, dn, dr, R = x.shape[0], self.heads, self.dim, self.rot_dim, self.lat
        f32 = torch.float32
        cq = ops.rmsnorm_rows(ops.linear(x, self.w_dq, out_dtype=f32), self.w_dq_norm, self.eps, out_dtype=self.dtype)
        q = ops.linear(cq, self.w_uq, out_dtype=f32)
        table = ctx.rope_table(self.rot_dims, self.rot_base)
        if self.owns_cache:
            kv = ops.linear(x, self.w_dkv, out_dtype=f32)
            ops.latent_kv_append(ctx.pools[self.index], kv, self.w_dkv_norm, self.eps, table, self.rot_dims, ctx.batch,
                                 ctx.page, R, dr)
        qa = torch.empty((n, H, R + dr), dtype=self.dtype, device=x.device)
        ops.linear(q.view(n, H, dn + dr)[:, :, :dn], self.w_uk_t, out=qa[:, :, :R])
        ops.rope_query_tail(qa, q, table, H, dn, dr, self.rot_dims, R)
        lat_out = ops.latent_attention(qa, ctx.pools[self.kv_source], ctx.batch, ctx.page, H, R, dr, self.scale)
        heads_out = torch.empty((n, H, self.vdim), dtype=self.dtype, device=x.device)
        ops.linear(lat_out, self.w_uv, out=heads_out)
        return ops.linear(heads_out.view(n, H * self.vdim), self.w_o, out_dtype=f32)


class GatedLinearRecurrence:
    """Recurrent block with a real-gated linear recurrent unit (De et al., "Griffin: Mixing Gated Linear Recurrences
    with Local Attention for Efficient Language Models", 2024).

    Two branches of ``channels``: y = gelu_tanh(W_y h + b_y); u = causal per-channel conv over ``taps`` inputs of
    (W_x h + b_x).  With u cut into ``blocks`` parts, r = sigmoid(A_b u_b + a_b), i = sigmoid(B_b u_b + b_b),
    a = exp(-decay_scale * r * softplus(lam)), S <- a S + sqrt(1 - a^2) i u, output W_o (S * y).
    Per sequence the layer carries S (fp32 [channels]) and the last taps - 1 convolution inputs in a state slot."""

    def __init__(self, index, *, channels, blocks, taps, w_y, b_y, w_x, b_x, conv_w, conv_b, w_ra, b_ra, w_ri, b_ri, lam,
                 w_o, decay_scale=8.0):
        if channels % blocks:
            raise ValueError(f"layer {index}: {channels} channels do not split into {blocks} blocks")
        self.index, self.channels, self.blocks, self.taps, self.decay_scale = index, channels, blocks, taps, decay_scale
        self.dtype = w_y.dtype
        self.w_y, self.b_y, self.w_x, self.b_x, self.conv_w, self.conv_b = w_y, b_y, w_x, b_x, conv_w.contiguous(), conv_b
        # per block: the recurrence-gate rows, then the input-gate rows -> one batched product gives both logits
        self.w_gates = torch.cat([w_ra, w_ri], dim=1).contiguous()       # [blocks, 2 bw, bw]
        self.b_gates = torch.cat([b_ra, b_ri], dim=1).contiguous()       # [blocks, 2 bw]
        self.lam, self.w_o = lam, w_o

    def forward(self, x, ctx):
        n, f32 = x.shape[0], torch.float32
        bw = self.channels // self.blocks
        y = ops.linear(x, self.w_y, bias=self.b_y, out_dtype=self.dtype, act=ops.ACT_GELU_TANH)
        xb = ops.linear(x, self.w_x, bias=self.b_x, out_dtype=f32)
        conv_state, rec_state = ctx.states[self.index]
        u = ops.causal_conv1d(xb, self.conv_w, self.conv_b, conv_state, ctx.batch)
        gates = torch.empty((n, self.blocks, 2 * bw), dtype=f32, device=x.device)
        ops.linear(u.view(n, self.blocks, bw), self.w_gates, bias=self.b_gates, out=gates, compute=ops.COMPUTE_FMA32)
        s = ops.rglru_scan(u, gates, self.lam, y, rec_state, ctx.batch, self.blocks, self.decay_scale)
        return ops.linear(s, self.w_o, out_dtype=f32)


class ClampedGatedMLP:
    """g = min(W_gate h, limit), u = clamp(W_up h, +-limit), y = g * sigmoid(alpha g) * (u + up_shift), out = W_down y.
    Gate and up rows are stored as one [2 ff, width] matrix (gate rows first), as the other models' fc_gate is."""

    def __init__(self, *, w_gate, w_up, w_down, limit, alpha=1.702, up_shift=1.0):
        self.w_gate_up = torch.cat([w_gate, w_up], dim=0).contiguous()
        self.w_down, self.limit, self.alpha, self.up_shift = w_down, float(limit), float(alpha), float(up_shift)
        self.dtype = w_down.dtype

    def forward(self, x, ctx):
        act = ops.linear_gated(x, self.w_gate_up, self.dtype, self.alpha, self.limit, self.up_shift)    # generation steps
        if act is None:
            gu = ops.linear(x, self.w_gate_up, out_dtype=torch.float32)
            act = ops.gated_act(gu, self.dtype, self.alpha, self.limit, self.up_shift)
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


class LayerStackModel:
    """Embedding, a stack of (mixer, optional feed-forward) layers, output norm and head.

    ``post_norm`` stacks normalise each sublayer's OUTPUT and add it to the residual, x <- x + norm(f(x)), with
    norm weights stored around zero (``norm_offset`` = 1); the sublayers read the residual itself."""

    def __init__(self, *, vocab, width, dtype, embed, embed_scale, layers, final_norm, head, eps, norm_offset=1.0):
        self.vocab, self.width, self.dtype, self.eps, self.norm_offset = vocab, width, dtype, float(eps), float(norm_offset)
        self.embed, self.embed_scale, self.layers, self.final_norm, self.head = embed, float(embed_scale), layers, final_norm, head

    # what the session has to provide
    def cache_layers(self):
        return {l["mixer"].index: l["mixer"].cache_entry for l in self.layers
                if isinstance(l["mixer"], LatentAttention) and l["mixer"].owns_cache}

    def state_layers(self):
        return {l["mixer"].index: (l["mixer"].taps, l["mixer"].channels) for l in self.layers
                if isinstance(l["mixer"], GatedLinearRecurrence)}

    def forward(self, ctx, on_layer=None):
        x = ops.embed_scaled(self.embed, ctx.batch.tok_ids, self.embed_scale)
        for i, l in enumerate(self.layers):
            ops.rmsnorm_rows(l["mixer"].forward(x, ctx), l["norm1"], self.eps, self.norm_offset, out=x, accumulate=True)
            if l["mlp"] is not None:
                ops.rmsnorm_rows(l["mlp"].forward(x, ctx), l["norm2"], self.eps, self.norm_offset, out=x, accumulate=True)
            if on_layer is not None:
                on_layer(i, x)
        return x

    def logits(self, x, rows_idx):
        h = ops.rmsnorm_rows(x, self.final_norm, self.eps, self.norm_offset, out_dtype=self.dtype, rows_idx=rows_idx)
        return ops.linear(h, self.head, out_dtype=torch.float32)
