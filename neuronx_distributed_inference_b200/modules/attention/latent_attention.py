"""Latent attention with a softmax sink and per-head output gates, on ragged rows and the paged cache.

Keys and values of every head are linear images of ONE low-rank row per token, ``c = rms_norm(W_dkv x)``: ``k_h = U_h c``,
``v_h = V_h c``.  Only ``c`` is cached (``kv_rank`` numbers per token and layer instead of ``heads * (dim + vdim)``), and neither
keys nor values are ever materialised: with ``a_h = U_h^T q_h`` the score is ``q_h . k_h = a_h . c`` and the head's output is
``V_h (sum_j p_j c_j)``, so attention runs as multi-query attention over the latent rows, which serve as keys AND values.  There are
no positional rotations.  Constructor parameters, so that other stacks can combine them:

* ``sink``: one learned logit per head joins the softmax denominator (a slot without key or value; not scaled);
* ``head_gate``: head ``h``'s output is multiplied by ``sigmoid(W_g x)_h`` — one factor per head, read from the mixer's input;
* ``scale``: multiplies the scores;
* ``q_rank``: queries pass a latent of their own, ``q = W_uq rms_norm(W_dq x)``, instead of one projection;
* ``rot_dim`` / ``rope``: every query head carries ``rot_dim`` extra channels and every token ONE extra key part of ``rot_dim`` channels
  shared by all heads; both are rotated by position (rotate-half layout; ``rope = (inv_freq fp64, magnitude, tag)``) and their product
  joins the score.  The rotated key part is stored behind the latent in the same cache row, so a row is ``kv_rank + rot_dim`` numbers,
  the key of the multi-query attention is the whole row and its value the first ``kv_rank`` numbers;
* ``window``: position ``i`` sees ``j`` iff ``0 <= i - j < window``;
* ``channel_gate``: the concatenated head outputs are multiplied element by element with ``sigmoid(W_g x)`` (``heads * vdim`` gate
  channels instead of one per head).

Data flow (CUDA: csrc/seqmix.cu for the two middle steps, GEMMs around them):

    p   = W_in x                          q (or its latent) | latent | rotated key part | gates in ONE GEMM
          latent_norm_append(p)           fp32 RMS norm of the latent slice(s), rotation of the shared key part, paged cache write
    a   = q_h U_h                         batched over heads (rotated query channels appended by rope_half_tail)
    l   = paged_window_attention(a)       fp32 softmax (+ sink) over the latent cache, times sigmoid(gate_h)
    y   = W_o [V_h l_h]                   batched over heads, then the output projection

DeepSeek-style caches in this package (models/deepseek) keep expanded keys and values; this module is the compressed-cache form.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...parallel.layers import ColumnParallelLinear, RowParallelLinear
from .conv_window_attention import ragged_rope_tables


class LatentSinkAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, kv_rank: int, *, scale: float, eps: float,
                 sink: bool = True, head_gate: bool = True, layer_idx: int = 0, dtype=torch.bfloat16, device=None, tp_group=None,
                 q_rank: int = 0, rot_dim: int = 0, rope=None, window=None, channel_gate: bool = False):
        super().__init__()
        if tp_group is not None and tp_group.size != 1:
            raise NotImplementedError("latent attention: the latent row is shared by all heads; tensor parallel degree 1")
        if head_gate and channel_gate:
            raise ValueError("one gate per head or one per channel, not both")
        self.n_q, self.head_dim, self.v_head_dim, self.kv_rank = num_heads, head_dim, v_head_dim, kv_rank
        self.scale, self.eps, self.layer_idx = float(scale), float(eps), layer_idx
        self.q_rank, self.rot_dim, self.window, self.channel_gate = int(q_rank or 0), int(rot_dim or 0), (int(window) if window else None), channel_gate
        # the first slice of the input projection: the queries themselves, or their latent
        self.Cq = self.q_rank or num_heads * head_dim
        self.Cg = num_heads * v_head_dim if channel_gate else (num_heads if head_gate else 0)
        self.in_proj = ColumnParallelLinear(hidden_size, self.Cq + kv_rank + self.rot_dim + self.Cg, bias=False, gather_output=False, dtype=dtype,
                                            device=device, tensor_model_parallel_group=tp_group)
        if self.q_rank:
            self.q_up = ColumnParallelLinear(self.q_rank, num_heads * (head_dim + self.rot_dim), bias=False, gather_output=False, dtype=dtype,
                                             device=device, tensor_model_parallel_group=tp_group)
            self.q_norm_weight = nn.Parameter(torch.ones(self.q_rank, dtype=torch.float32, device=device), requires_grad=False)
        if self.rot_dim:
            inv, self.rope_magnitude, self.rope_tag = rope
            self.register_buffer("rope_inv_freq", inv.to(device=device, dtype=torch.float64), persistent=False)
        self.o_proj = RowParallelLinear(num_heads * v_head_dim, hidden_size, bias=False, input_is_parallel=True, dtype=dtype,
                                        device=device, tensor_model_parallel_group=tp_group)
        self.k_up = nn.Parameter(torch.zeros(num_heads, head_dim, kv_rank, dtype=dtype, device=device), requires_grad=False)
        self.v_up = nn.Parameter(torch.zeros(num_heads, v_head_dim, kv_rank, dtype=dtype, device=device), requires_grad=False)
        f32 = dict(dtype=torch.float32, device=device)
        self.latent_norm_weight = nn.Parameter(torch.ones(kv_rank, **f32), requires_grad=False)
        self.sinks = nn.Parameter(torch.zeros(num_heads, **f32), requires_grad=False) if sink else None

    def kv_shape(self):
        """One kv head whose key row is also its value row (with a rotated part: the value is the row's first ``kv_rank`` numbers)."""
        return (1, self.kv_rank + self.rot_dim, None)

    def forward(self, x, meta, kv_mgr, cache_index=None):
        B, T, _ = x.shape
        ex = meta.extras
        ctx, qlen = ex["ctx_len"], ex["q_len"]
        H, R, rot, d = self.n_q, self.kv_rank, self.rot_dim, self.head_dim
        p = self.in_proj(x)
        cache, _ = kv_mgr.get_kv_by_layer_id(self.layer_idx if cache_index is None else cache_index)
        cos, sin = ragged_rope_tables(meta, T, rot, 0.0, self.rope_inv_freq, self.rope_magnitude, self.rope_tag) if rot else (None, None)
        # whole prompts (no row brings earlier context): the new rows are all the keys there are, so attention can read them in token
        # order with the contiguous-key tcgen05 kernel; every other step (portions after a prefix, decoded tokens) reads the paged cache
        whole = (meta.is_prefill and not meta.has_prefix and T >= 16 and not rot and not self.window
                 and ops.latent_prefill_on_tensor_cores(p, R))
        rows = ops.latent_norm_append(p, self.Cq, R, self.latent_norm_weight, self.eps, cache, meta.block_table, ctx, qlen, emit_rows=whole,
                                      rot_dim=rot, cos=cos, sin=sin, q_rank=self.q_rank, q_weight=self.q_norm_weight if self.q_rank else None)
        if self.q_rank:
            rows, cq = rows
            q = self.q_up(cq).view(B * T, H, d + rot)
        else:
            q = p.view(B * T, -1)[:, :self.Cq].unflatten(1, (H, d))
        # batched over heads with strided operands and results: the products land in [B, T, H, .] layout, no transposing copies
        a = torch.empty(B, T, H, R + rot, dtype=p.dtype, device=p.device)
        torch.bmm(q[..., :d].transpose(0, 1), self.k_up, out=a.view(B * T, H, R + rot)[..., :R].transpose(0, 1))
        if rot:
            ops.rope_half_tail(q.view(B, T, H, d + rot), a, rot, cos, sin)
        gate = p[..., self.Cq + R + rot:] if self.Cg else None
        head_gate = gate if not self.channel_gate else None
        if whole:
            lat = ops.attention_prefill(a, rows, rows, self.scale, True, sinks=self.sinks)
            lat = ops.head_gate_mul(lat, head_gate) if head_gate is not None else lat
        else:
            lat = ops.paged_window_attention(a, cache, cache, meta.block_table, ctx, qlen, self.scale, None, self.window, 0, head_gate, self.sinks,
                                             gate_per_head=True, value_dim=R if rot else None)
        o = torch.empty(B, T, H * self.v_head_dim, dtype=p.dtype, device=p.device)
        torch.bmm(lat.view(B * T, H, R).transpose(0, 1), self.v_up.transpose(1, 2), out=o.view(B * T, H, self.v_head_dim).transpose(0, 1))
        if self.channel_gate:
            o = ops.gated_act_mul(o, gate, "sigmoid", act_on_other=True)
        return self.o_proj(o)
