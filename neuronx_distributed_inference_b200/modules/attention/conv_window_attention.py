"""Attention over convolved projections with a kept-prefix sliding window, on ragged rows and the paged cache.

Differences from :class:`AttentionBase`, each a constructor parameter so that other stacks can combine them:

* ``conv_taps``: a depthwise causal convolution over time runs on every channel of the biased q / k / v projections before anything
  else; the last ``taps - 1`` projected rows of a sequence are carried in a state line (``RecurrentStateCache``);
* ``row_norm``: q and k are RMS-normalised over the WHOLE projection row (all heads at once) with one weight per channel;
* ``rot_dims`` / ``rot_base``: rotary positions on the first ``rot_dims`` channels of every head, pairs ``(2i, 2i+1)``;
* ``softcap``: scores pass ``cap * tanh(s / cap)`` before the softmax;
* ``window`` / ``keep_first``: key ``j`` is visible from ``i`` iff ``j <= i and (i - j < window or j < keep_first)``; the kept
  tokens stay in the cache at their true positions, so rotation and distance are unchanged;
* ``out_gate``: the concatenated heads are multiplied by ``sigmoid(W_g x)`` before the output projection;
* ``kv_source``: the layer has no k / v projections and reads the cache another layer wrote (its own q, mask and gate);
* ``chunk``: instead of a window, key ``j`` is visible from ``i`` iff ``j <= i`` and both lie in the same chunk of ``chunk`` positions
  (counted from position 0 of the sequence);
* ``distance_bias``: ``slope_h * (i - j)`` is taken off the score of head ``h``, ``slope_h = 2^(-8 (h + 1) / heads)``; positions enter
  such a layer only through this term (``rot_dims = 0``: no rotation).

``bias`` / ``row_norm`` / ``out_gate`` switch the projection biases, the row norms and the gate off for stacks without them.  A stack
that runs a layer several times per forward passes ``cache_index``: the run's cache and its own line of carried projection rows.

Data flow (CUDA: csrc/seqmix.cu, one kernel per line after the first):

    p     = W_in x + b                  q | k | v | gate in ONE GEMM
    q     = conv_qknorm_rope_append(p)  convolution + row norms + rotation + paged cache write
            short_conv_update(p)        carried projection rows
    o     = paged_window_attention(q)   fp32 softmax over the cache, times sigmoid(gate)
    y     = W_o o
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import ops
from ...parallel.layers import ColumnParallelLinear, RowParallelLinear


def ragged_rope_tables(meta, T: int, rot_dims: int, rot_base: float, inv_freq=None, magnitude: float = 1.0, tag=None):
    """cos / sin ``[B, T, rot_dims / 2]`` fp32 at positions ``ctx_len + t``; the angle is formed in fp64 so that far positions
    lose nothing.  ``inv_freq`` [rot_dims / 2] (fp64, on the device): frequencies that are not the plain ``base^(-2i/dims)`` (scaled
    rotary variants, :func:`modules.rope.compute_inv_freq`), ``magnitude`` multiplies cos and sin; ``tag`` tells such variants apart.
    Cached on the forward's metadata per (dims, base, tag)."""
    key = ("ragged_rope", rot_dims, float(rot_base), tag)
    if key not in meta.extras:
        ctx = meta.extras["ctx_len"]
        pos = ctx.double().view(-1, 1) + torch.arange(T, device=ctx.device, dtype=torch.float64).view(1, T)
        # (scalar ** tensor: no host-to-device copy, so the step stays capturable in a CUDA graph)
        inv = inv_freq if inv_freq is not None else \
            float(rot_base) ** (-torch.arange(0, rot_dims, 2, device=ctx.device, dtype=torch.float64) / rot_dims)
        ang = pos.unsqueeze(-1) * inv
        meta.extras[key] = ((torch.cos(ang) * magnitude).float().contiguous(), (torch.sin(ang) * magnitude).float().contiguous())
    return meta.extras[key]


class ConvWindowAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, *, conv_taps: int,
                 rot_dims: int, rot_base: float, scale: float, softcap: Optional[float], window: Optional[int], keep_first: int,
                 eps: float, layer_idx: int, kv_source: Optional[int] = None, dtype=torch.bfloat16, device=None, tp_group=None,
                 bias: bool = True, row_norm: bool = True, out_gate: bool = True, chunk: Optional[int] = None, distance_bias: bool = False):
        super().__init__()
        self.n_q, self.n_kv, self.head_dim, self.v_head_dim = num_heads, num_kv_heads, head_dim, v_head_dim
        self.taps, self.rot_dims, self.rot_base = conv_taps, rot_dims, rot_base
        self.scale, self.softcap, self.window, self.keep_first, self.eps = scale, softcap, window, keep_first, eps
        self.layer_idx, self.kv_source = layer_idx, kv_source
        self.owns_kv = kv_source is None
        self.chunk = int(chunk) if chunk else None
        if self.chunk and window:
            raise ValueError("a layer masks by window or by chunk, not both")
        if tp_group is not None and tp_group.size != 1:
            raise NotImplementedError("row-wide q/k norms need the whole projection on one rank: tensor parallel degree 1")
        self.Cq = num_heads * head_dim
        self.Ckv = num_kv_heads * (head_dim + v_head_dim) if self.owns_kv else 0
        self.Co = num_heads * v_head_dim
        self.Cg = self.Co if out_gate else 0
        self.in_proj = ColumnParallelLinear(hidden_size, self.Cq + self.Ckv + self.Cg, bias=bias, gather_output=False, dtype=dtype,
                                            device=device, tensor_model_parallel_group=tp_group)
        self.o_proj = RowParallelLinear(self.Co, hidden_size, bias=False, input_is_parallel=True, dtype=dtype, device=device,
                                        tensor_model_parallel_group=tp_group)
        f32 = dict(dtype=torch.float32, device=device)
        self.conv_weight = nn.Parameter(torch.zeros(self.Cq + self.Ckv, conv_taps, **f32), requires_grad=False)
        self.q_norm_weight = nn.Parameter(torch.ones(self.Cq, **f32), requires_grad=False) if row_norm else None
        self.k_norm_weight = nn.Parameter(torch.ones(num_kv_heads * head_dim, **f32), requires_grad=False) if self.owns_kv and row_norm else None
        if distance_bias:
            self.register_buffer("slopes", torch.tensor([2.0 ** (-8.0 * (h + 1) / num_heads) for h in range(num_heads)], **f32), persistent=False)
        else:
            self.slopes = None
        self.state = f"attn_conv{layer_idx}"

    def state_name(self, cache_index=None):
        return self.state if cache_index is None else f"{self.state}.run{cache_index}"

    def state_specs(self, cache_index=None):
        return {self.state_name(cache_index): (self.taps - 1, self.Cq + self.Ckv)}

    def kv_shape(self):
        return (self.n_kv, self.head_dim, self.v_head_dim) if self.owns_kv else None

    def forward(self, x, meta, kv_mgr, cache_index=None):
        B, T, _ = x.shape
        ex = meta.extras
        ctx, qlen, lines = ex["ctx_len"], ex["q_len"], ex["state_lines"]
        p = self.in_proj(x)
        C = self.Cq + self.Ckv
        cos, sin = ragged_rope_tables(meta, T, self.rot_dims, self.rot_base) if self.rot_dims else (None, None)
        k_cache, v_cache = kv_mgr.get_kv_by_layer_id(self.layer_idx if cache_index is None else cache_index)
        st = kv_mgr.states.tensor(self.state_name(cache_index))
        q = ops.conv_qknorm_rope_append(p, self.conv_weight, st, lines, ctx, qlen, self.q_norm_weight, self.k_norm_weight, self.eps,
                                        self.n_q, self.n_kv if self.owns_kv else 0, self.head_dim, self.v_head_dim, cos, sin,
                                        k_cache, v_cache, meta.block_table)
        ops.short_conv_update(p[..., :C], st, lines, ctx, qlen)
        o = ops.paged_window_attention(q, k_cache, v_cache, meta.block_table, ctx, qlen, self.scale, self.softcap, self.window,
                                       self.keep_first, p[..., C:] if self.Cg else None, chunk=self.chunk, slopes=self.slopes)
        return self.o_proj(o)
