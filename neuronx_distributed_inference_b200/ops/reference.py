"""Plain-PyTorch definitions of every op in ``ops``.

Two jobs: (1) the CPU execution path (``on_cpu`` / gloo tests — the role ``to_cpu()`` plays in
the reference, application_base.py:556-628), (2) the fp32 oracle that each CUDA kernel's
numerics test compares against.  Shapes: B batch, T active tokens, S cache length,
Hq/Hkv heads, D head dim.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rmsnorm(x, weight, eps: float, offset: float = 0.0, residual=None):
    """y = x * rsqrt(mean(x^2)+eps) * (offset + weight), statistics in fp32
    (reference custom_calls.py:8-36; Gemma uses offset=1)."""
    if residual is not None:
        x = x + residual
        residual = x
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * (weight.float() + offset)
    y = y.to(x.dtype)
    return y if residual is None else (y, residual)


def _dequant_weight(w, scale):
    if scale is None:
        return w
    wf = w.float()
    s = scale.float()
    if s.dim() == 1:
        s = s.unsqueeze(-1)
    elif s.dim() == 2 and s.shape != wf.shape and s.shape[-1] != 1:
        # blockwise [out/bs0, in/bs1] -> expand
        r0, r1 = wf.shape[0] // s.shape[0], wf.shape[1] // s.shape[1]
        s = s.repeat_interleave(r0, 0).repeat_interleave(r1, 1)
    return wf * s


def linear(x, w, bias=None, norm_weight=None, norm_eps: float = 1e-6, norm_offset: float = 0.0,
           act: Optional[str] = None, scale=None):
    """y = act(norm(x) @ dequant(w)^T + bias)."""
    if norm_weight is not None:
        x = rmsnorm(x, norm_weight, norm_eps, norm_offset)
    if scale is not None:
        w = _dequant_weight(w, scale).to(x.dtype)
    y = F.linear(x, w, bias)
    if act is not None:
        y = activation(y, act)
    return y


def activation(y, act: str):
    if act == "silu_mul":
        g, u = y.chunk(2, -1)
        return F.silu(g.float()).to(y.dtype) * u
    if act == "gelu_mul":
        g, u = y.chunk(2, -1)
        return F.gelu(g.float()).to(y.dtype) * u
    if act == "gelu_tanh_mul":
        g, u = y.chunk(2, -1)
        return F.gelu(g.float(), approximate="tanh").to(y.dtype) * u
    if act == "silu":
        return F.silu(y)
    if act == "gelu":
        return F.gelu(y)
    if act == "gelu_tanh":
        return F.gelu(y, approximate="tanh")
    if act == "relu":
        return F.relu(y)
    if act == "relu2":
        return F.relu(y).square()
    if act == "sigmoid":
        return torch.sigmoid(y)
    raise ValueError(act)


def rotate_half(x):
    x1, x2 = x.chunk(2, -1)
    return torch.cat((-x2, x1), -1)


def apply_rope(x, cos, sin, interleaved: bool = False):
    """x [B,T,H,D]; cos/sin [B,T,R/2] (R = rotary dim <= D).  Half-rotation (HF Llama,
    reference attention/utils.py:233-249) or interleaved pairs (Llama-4 / GPT-J)."""
    R = cos.shape[-1] * 2
    xr, xp = x[..., :R], x[..., R:]
    c = cos.unsqueeze(2).float()
    s = sin.unsqueeze(2).float()
    xf = xr.float()
    if interleaved:
        x1, x2 = xf[..., 0::2], xf[..., 1::2]
        o = torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), -1).flatten(-2)
    else:
        x1, x2 = xf[..., : R // 2], xf[..., R // 2:]
        o = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), -1)
    o = o.to(x.dtype)
    return o if xp.shape[-1] == 0 else torch.cat((o, xp), -1)


def _expand_kv(k, n_rep):
    if n_rep == 1:
        return k
    B, H, S, D = k.shape
    return k[:, :, None].expand(B, H, n_rep, S, D).reshape(B, H * n_rep, S, D)


def attention_with_mask(q, k, v, mask, scale, sinks=None, softcap: Optional[float] = None):
    """q [B,Hq,T,D], k/v [B,Hkv,S,D], boolean mask [B,1|Hq,T,S] (True = attend).  fp32 softmax.
    ``sinks`` [Hq]: learned per-head logit joining the softmax denominator (GPT-OSS,
    reference attention_base.py learned-sink variant)."""
    n_rep = q.shape[1] // k.shape[1]
    k = _expand_kv(k, n_rep)
    v = _expand_kv(v, n_rep)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if softcap:
        s = torch.tanh(s / softcap) * softcap
    s = s.masked_fill(~mask, float("-inf"))
    if sinks is not None:
        sk = sinks.float().view(1, -1, 1, 1).expand(s.shape[0], -1, s.shape[2], 1)
        p = torch.softmax(torch.cat((s, sk), -1), -1)[..., :-1]
    else:
        m = s.amax(-1, keepdim=True)
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        e = torch.exp(s - m)
        p = e / e.sum(-1, keepdim=True).clamp_min(1e-30)
    return torch.matmul(p, v.float()).to(q.dtype)


def build_mask(q_pos, kv_len: int, window: Optional[int] = None, chunk: Optional[int] = None,
               key_valid=None, device=None):
    """Causal / sliding-window / chunked mask.  q_pos [B,T] absolute positions; key j visible iff
    j <= pos (causal), j > pos - window (SWA, reference model_base.py:187-376 mask builders),
    floor(j/chunk) == floor(pos/chunk) (Llama-4 chunked attention).  -> [B,1,T,S] bool."""
    j = torch.arange(kv_len, device=q_pos.device).view(1, 1, -1)
    p = q_pos.unsqueeze(-1)
    m = j <= p
    if window:
        m = m & (j > p - window)
    if chunk:
        m = m & ((j // chunk) == (p // chunk))
    if key_valid is not None:
        m = m & key_valid.bool().unsqueeze(1)
    return m.unsqueeze(1)


def attention_prefill(q, k, v, scale, causal: bool = True, window=None, chunk=None, key_valid=None,
                      q_pos=None, sinks=None, softcap=None):
    """q [B,T,Hq,D], k/v [B,S,Hkv,D] (new tokens, T==S unless prefix) -> [B,T,Hq,D]."""
    B, T = q.shape[:2]
    S = k.shape[1]
    if q_pos is None:
        q_pos = torch.arange(S - T, S, device=q.device).unsqueeze(0).expand(B, T)
    if causal:
        mask = build_mask(q_pos, S, window, chunk, key_valid)
    else:
        mask = torch.ones(B, 1, T, S, dtype=torch.bool, device=q.device)
        if key_valid is not None:
            mask = mask & key_valid.bool().view(B, 1, 1, S)
    o = attention_with_mask(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), mask, scale, sinks, softcap)
    return o.transpose(1, 2)


def kv_append(k_cache, v_cache, k_new, v_new, seq_ids, positions):
    """Write k_new/v_new [B,T,Hkv,D] into caches [L,Hkv,S,D] at (line=seq_ids[b], pos=positions[b,t]).
    Out-of-range lines/positions are skipped (reference K10 OOB-skip semantics)."""
    B, T = positions.shape
    L, H, S, D = k_cache.shape
    line = seq_ids.view(B, 1).expand(B, T).reshape(-1).long()
    pos = positions.reshape(-1).long()
    ok = (line >= 0) & (line < L) & (pos >= 0) & (pos < S)
    line, pos = line[ok], pos[ok]
    kn = k_new.reshape(B * T, H, D)[ok].to(k_cache.dtype)
    vn = v_new.reshape(B * T, H, v_new.shape[-1])[ok].to(v_cache.dtype)   # V may have its own head dim (MLA)
    k_cache[line, :, pos] = kn
    v_cache[line, :, pos] = vn


def attention_decode(q, k_cache, v_cache, seq_ids, positions, scale, window=None, chunk=None,
                     sinks=None, active_mask=None, softcap=None, k_scale=None, v_scale=None, active_base=None):
    """Attend q [B,T,Hq,D] over cache lines (already containing the active tokens).
    Token t of row b sees cache slots j <= positions[b,t] (+window/chunk).  ``active_mask`` [B,T,M] (token-tree
    speculation, M >= T) gives the visibility of the M slots starting at ``active_base`` [B,1] (default: the slot of the
    first active token); slots before the base are fully visible, slots after ``base+M`` are hidden."""
    B, T = positions.shape
    S = k_cache.shape[2]
    lines = seq_ids.long().clamp(0, k_cache.shape[0] - 1)
    k = k_cache[lines]
    v = v_cache[lines]
    if k.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        k = k.to(q.dtype) * (1.0 if k_scale is None else k_scale)
        v = v.to(q.dtype) * (1.0 if v_scale is None else v_scale)
    mask = build_mask(positions, S, window, chunk)
    if active_mask is not None:
        M = active_mask.shape[-1]
        base = (positions[:, :1] if active_base is None else active_base.view(B, 1)).long().unsqueeze(-1)   # [B,1,1]
        j = torch.arange(S, device=q.device).view(1, 1, S)
        prior = (j < base).expand(B, T, S)
        idx = (j - base).clamp(0, M - 1).expand(B, T, S)
        act = torch.gather(active_mask.bool().expand(B, T, M), 2, idx) & (j >= base) & (j < base + M)
        mask = (prior | act).unsqueeze(1)
        if window:
            mask = mask & build_mask(positions, S, window, None)
    o = attention_with_mask(q.transpose(1, 2), k, v, mask, scale, sinks, softcap)
    return o.transpose(1, 2)


def paged_kv_append(k_cache, v_cache, k_new, v_new, slot_mapping):
    """caches [num_blocks, block_size, Hkv, D]; slot = block*block_size+offset, -1 = skip
    (reference block_kv_cache_manager.py:268-328)."""
    nb, bs, H, D = k_cache.shape
    slots = slot_mapping.reshape(-1).long()
    ok = slots >= 0
    kc = k_cache.view(nb * bs, H, D)
    vc = v_cache.view(nb * bs, H, D)
    kc[slots[ok]] = k_new.reshape(-1, H, D)[ok].to(k_cache.dtype)
    vc[slots[ok]] = v_new.reshape(-1, H, D)[ok].to(v_cache.dtype)


def paged_attention_decode(q, k_cache, v_cache, block_table, positions, scale, window=None, sinks=None):
    """q [B,T,Hq,D]; block_table [B, max_blocks]; positions [B,T]."""
    nb, bs, H, D = k_cache.shape
    B = q.shape[0]
    bt = block_table.long().clamp_min(0)
    k = k_cache[bt].reshape(B, -1, H, D).transpose(1, 2)
    v = v_cache[bt].reshape(B, -1, H, D).transpose(1, 2)
    mask = build_mask(positions, k.shape[2], window)
    o = attention_with_mask(q.transpose(1, 2), k, v, mask, scale, sinks)
    return o.transpose(1, 2)


def sample(logits, top_k, top_p, temperature, rand=None, global_topk: int = 256):
    """On-device sampling semantics of the reference (sampling.py:241-464): restrict to the global
    top-k (k<=global_topk), per-row top-k mask, temperature, top-p mask on the cumulative softmax,
    softmax, inverse-CDF draw with ``rand`` [B] uniform (0.5 when deterministic).
    logits [B,V] fp32; top_k [B] int (<=0 => global_topk); top_p, temperature [B]. -> tokens [B]."""
    B, V = logits.shape
    K = min(global_topk, V)
    vals, idx = torch.topk(logits.float(), K, dim=-1)
    k = torch.where(top_k <= 0, torch.full_like(top_k, K), top_k).clamp(max=K).view(B, 1)
    ar = torch.arange(K, device=logits.device).view(1, K)
    vals = vals.masked_fill(ar >= k, float("-inf"))
    t = temperature.float().view(B, 1)
    greedy = (t == 0) | (k == 1)
    vals = vals / torch.where(t == 0, torch.ones_like(t), t)
    probs = torch.softmax(vals, -1)
    cum = torch.cumsum(probs, -1)
    keep = (cum - probs) < top_p.float().view(B, 1)  # always keeps the first token
    probs = torch.where(keep, probs, torch.zeros_like(probs))
    probs = probs / probs.sum(-1, keepdim=True)
    cdf = torch.cumsum(probs, -1)
    if rand is None:
        rand = torch.full((B,), 0.5, device=logits.device)
    r = rand.float().view(B, 1) * cdf[:, -1:]
    choice = (cdf < r).sum(-1).clamp(max=K - 1)
    choice = torch.where(greedy.view(B), torch.zeros_like(choice), choice)
    return idx.gather(1, choice.view(B, 1)).view(B)


def argmax(logits):
    return logits.float().argmax(-1)


def moe_route(router_logits, top_k: int, act: str = "softmax", normalize: bool = True,
              act_over_topk: bool = False, renorm_eps=None, correction=None, groups=None, scale: float = 1.0):
    """-> (weights [N,top_k] fp32, expert ids [N,top_k]).  softmax-then-topk (Mixtral/DBRX/Qwen3),
    sigmoid (Llama-4) or topk-then-softmax (GPT-OSS ``apply_act_fn_over_topk``).

    ``correction`` [E] / ``groups`` (count, keep): the experts are CHOSEN by ``score + correction`` among the ``keep`` groups (of
    ``count`` equal groups of neighbouring experts) whose largest corrected score is largest — every other expert counts as minus
    infinity — while the weights are the uncorrected scores of the chosen ones; ``scale`` multiplies the weights."""
    x = router_logits.float()
    if correction is not None or groups is not None:
        p = torch.softmax(x, -1) if act == "softmax" else torch.sigmoid(x)
        choice = p if correction is None else p + correction.float()
        if groups is not None and groups[0] > 1:
            count, keep = int(groups[0]), int(groups[1])
            best = choice.view(x.shape[0], count, -1).max(-1).values
            kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, torch.topk(best, keep, -1).indices, True)
            choice = choice.masked_fill(~kept.repeat_interleave(x.shape[1] // count, 1), float("-inf"))
        i = torch.topk(choice, top_k, -1).indices
        w = p.gather(1, i)
        if renorm_eps is not None:
            w = w / (w.sum(-1, keepdim=True) + renorm_eps)
        return w * scale, i
    if act_over_topk:
        v, i = torch.topk(x, top_k, -1)
        w = torch.softmax(v, -1) if act == "softmax" else torch.sigmoid(v)
        return w, i
    p = torch.softmax(x, -1) if act == "softmax" else torch.sigmoid(x)
    w, i = torch.topk(p, top_k, -1)
    if renorm_eps is not None:          # chosen scores divided by their sum (+ eps), whatever the activation
        w = w / (w.sum(-1, keepdim=True) + renorm_eps)
    elif normalize and act == "softmax":
        w = w / w.sum(-1, keepdim=True)
    return (w if scale == 1.0 else w * scale), i


def identity_expert_add(y, x, topk_w, topk_i, num_experts: int):
    """Routed slots whose expert id is ``>= num_experts`` are identity experts (no weights: the expert's output is its input):
    ``y + x * sum_j topk_w[:, j] [topk_i[:, j] >= num_experts]``, summed in fp32."""
    coef = (topk_w.float() * (topk_i >= num_experts)).sum(-1, keepdim=True)
    return (y.float() + x.float() * coef).to(y.dtype)


def moe_experts(x, w_gate_up, w_down, topk_w, topk_i, act: str = "silu_mul", expert_offset: int = 0,
                gate_up_bias=None, down_bias=None, act_fn=None, scale_input: bool = False, gate_up_scale=None, down_scale=None):
    """Dropless expert MLPs.  x [N,H]; w_gate_up [E_local, 2I, H] ([gate; up] rows, K-major like nn.Linear — the
    reference stores [E,H,2I]; K-major is what TMA/UMMA and the GEMV kernels stream); w_down
    [E_local, H, I]; experts owned here are [expert_offset, expert_offset+E_local).
    -> partial output [N,H] (sum over owned experts; all-reduce across expert/tensor shards outside)."""
    N, H = x.shape
    E = w_gate_up.shape[0]
    out = torch.zeros(N, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        sel = (topk_i == e + expert_offset)
        tok = sel.any(-1).nonzero().flatten()
        if tok.numel() == 0:
            continue
        wt = (topk_w * sel).sum(-1)[tok]
        xin = x[tok]
        if scale_input:   # Llama-4 "early expert affinity modulation": the affinity scales the expert INPUT
            xin = (xin.float() * wt.unsqueeze(-1)).to(x.dtype)
            wt = torch.ones_like(wt)
        h = F.linear(xin, w_gate_up[e].to(x.dtype))
        if gate_up_scale is not None:      # weight-only 8-bit experts: per-(expert, output channel) scale applied to the GEMM output
            h = (h.float() * gate_up_scale[e].float()).to(x.dtype)
        if gate_up_bias is not None:
            h = h + gate_up_bias[e].to(h.dtype)
        h = act_fn(h) if act_fn is not None else activation(h, act)
        y = F.linear(h, w_down[e].to(x.dtype))
        if down_scale is not None:
            y = (y.float() * down_scale[e].float()).to(x.dtype)
        if down_bias is not None:
            y = y + down_bias[e].to(y.dtype)
        out[tok] += y.float() * wt.unsqueeze(-1)
    return out.to(x.dtype)


def quantize_per_channel(w, dtype=torch.int8, axis: int = 0):
    """Symmetric per-output-channel quantisation.  -> (q, scale fp32 [out])."""
    wf = w.float()
    amax = wf.abs().amax(dim=1 - axis if w.dim() == 2 else -1, keepdim=True).clamp_min(1e-12)
    qmax = 127.0 if dtype == torch.int8 else (448.0 if dtype == torch.float8_e4m3fn else 57344.0)
    scale = amax / qmax
    q = wf / scale
    q = q.round().clamp(-qmax, qmax).to(torch.int8) if dtype == torch.int8 else q.clamp(-qmax, qmax).to(dtype)
    return q, scale.squeeze(-1)


def quantize_per_tensor(w, dtype=torch.int8):
    wf = w.float()
    qmax = 127.0 if dtype == torch.int8 else (448.0 if dtype == torch.float8_e4m3fn else 57344.0)
    scale = wf.abs().max().clamp_min(1e-12) / qmax
    q = wf / scale
    q = q.round().clamp(-qmax, qmax).to(torch.int8) if dtype == torch.int8 else q.clamp(-qmax, qmax).to(dtype)
    return q, scale.reshape(1)


def quantize_blockwise(w, block=(128, 128), dtype=torch.float8_e4m3fn):
    out, inp = w.shape
    b0, b1 = block
    assert out % b0 == 0 and inp % b1 == 0
    wf = w.float().view(out // b0, b0, inp // b1, b1)
    qmax = 448.0 if dtype == torch.float8_e4m3fn else 127.0
    scale = wf.abs().amax((1, 3), keepdim=True).clamp_min(1e-12) / qmax
    q = (wf / scale)
    q = q.round().clamp(-qmax, qmax).to(torch.int8) if dtype == torch.int8 else q.clamp(-qmax, qmax).to(dtype)
    return q.view(out, inp), scale.view(out // b0, inp // b1)


def rmsnorm_quant(x, weight, eps, clamp: float = float("inf")):
    """RMSNorm + dynamic per-row fp8(e4m3) quantisation (reference kernel K6)."""
    y = rmsnorm(x, weight, eps).float()
    if math.isfinite(clamp):
        y = y.clamp(-clamp, clamp)
    amax = y.abs().amax(-1, keepdim=True).clamp_min(1e-12)
    scale = amax / 448.0
    return (y / scale).to(torch.float8_e4m3fn), scale


# ---- sequence mixers on ragged rows -------------------------------------------------------------------------------------
# Shared conventions of the ops below: activations are ``[B, T, ...]`` with row ``b`` holding ``q_len[b] <= T`` new tokens at
# positions ``ctx_len[b] + t`` (the rest of the row is padding and is neither read nor written); per-sequence state lives in line
# ``slots[b]`` of a state tensor and counts as zero for a row whose ``ctx_len`` is 0, so a slot that is handed to a new sequence
# needs no clearing.

def scaled_add_rmsnorm(x, y, weight, alpha: float, eps: float, offset: float = 0.0, lp_dtype=None):
    """``out = rms_unit(alpha * x + y) * (offset + weight)`` in fp32 (``y`` may be None).  Returns ``(out fp32, out cast to lp_dtype
    or None)`` — the second copy feeds the next projection."""
    s = x.float() * alpha
    if y is not None:
        s = s + y.float()
    out = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        out = out * (weight.float() + offset)
    return out, (None if lp_dtype is None or lp_dtype == torch.float32 else out.to(lp_dtype))


def _conv_window(u, state, slots, ctx_len):
    """[B, K-1+T, C] fp32: each row's carried inputs (zeros for a fresh sequence) in front of its new ones."""
    B = u.shape[0]
    prev = state[slots.long()].float()
    prev = torch.where((ctx_len > 0).view(B, 1, 1), prev, torch.zeros_like(prev))
    return torch.cat([prev, u.float()], 1)


def short_conv(u, weight, bias, state, slots, ctx_len, q_len, silu: bool = False):
    """Causal depthwise convolution over time with carried inputs: ``y[b, t, c] = sum_j weight[c, j] * win[b, t + j, c]`` where
    ``win`` is the row's last ``K - 1`` inputs followed by ``u``.  ``u`` [B, T, C], ``weight`` [C, K], ``state`` [lines, K-1, C].
    Returns fp32; the state is NOT advanced (see :func:`short_conv_update`)."""
    T, K = u.shape[1], weight.shape[1]
    win = _conv_window(u, state, slots, ctx_len)
    y = sum(win[:, j:j + T] * weight[:, j].float() for j in range(K))
    if bias is not None:
        y = y + bias.float()
    return F.silu(y) if silu else y


def short_conv_update(u, state, slots, ctx_len, q_len):
    """Advance the carried inputs: line ``slots[b]`` becomes the last ``K - 1`` of (old inputs, ``u[b, :q_len[b]]``)."""
    B, T, C = u.shape
    Km1 = state.shape[1]
    if Km1 == 0:
        return
    win = _conv_window(u, state, slots, ctx_len)
    idx = (q_len.long().view(B, 1) + torch.arange(Km1, device=u.device).view(1, Km1)).unsqueeze(-1).expand(B, Km1, C)
    new = win.gather(1, idx).to(state.dtype)
    keep = (q_len > 0).view(B, 1, 1)
    state[slots.long()] = torch.where(keep, new, state[slots.long()])


def rope_partial_interleaved(x, cos, sin):
    """x [B, T, H, D]; cos/sin [B, T, R/2]: channel pairs (2i, 2i+1), i < R/2, are rotated, the rest pass through."""
    R = 2 * cos.shape[-1]
    xr = x[..., :R].float().reshape(*x.shape[:-1], R // 2, 2)
    c, s = cos.float().unsqueeze(2), sin.float().unsqueeze(2)
    a, b = xr[..., 0], xr[..., 1]
    rot = torch.stack([a * c - b * s, b * c + a * s], -1).reshape(*x.shape[:-1], R)
    return torch.cat([rot, x[..., R:].float()], -1)


def conv_qknorm_rope_append(qkv, conv_w, state, slots, ctx_len, q_len, q_norm_w, k_norm_w, eps: float, n_q: int, n_kv: int,
                            D: int, Dv: int, cos, sin, k_cache, v_cache, block_table, out_dtype=None):
    """Fused front half of a convolved-projection attention layer.  ``qkv`` [B, T, >= n_q*D + n_kv*(D+Dv)] holds the biased q | k | v
    projections (``n_kv = 0``: queries only, for a layer that reads another layer's cache; a norm weight of ``None`` skips that row
    norm, ``cos = None`` skips the rotation).  Steps: short causal convolution of every
    channel (carried inputs in ``state``), RMS norm of the WHOLE q row and of the WHOLE k row (plain weights), rotation of the first
    ``2 * cos.shape[-1]`` channels of every q / k head, and the write of k (normed, rotated) and v (convolved only) into the paged
    caches ``[blocks, page, n_kv, D | Dv]`` at position ``ctx_len + t``.  Returns q [B, T, n_q, D]."""
    B, T = qkv.shape[:2]
    Cq, Ck, Cv = n_q * D, n_kv * D, n_kv * Dv
    C = Cq + Ck + Cv
    y = short_conv(qkv[..., :C], conv_w, None, state, slots, ctx_len, q_len)
    q = y[..., :Cq]
    if q_norm_w is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm_w.float()
    q = q.view(B, T, n_q, D)
    if cos is not None:
        q = rope_partial_interleaved(q, cos, sin)
    if n_kv:
        k = y[..., Cq:Cq + Ck]
        if k_norm_w is not None:
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_norm_w.float()
        k = k.view(B, T, n_kv, D)
        if cos is not None:
            k = rope_partial_interleaved(k, cos, sin)
        v = y[..., Cq + Ck:].view(B, T, n_kv, Dv)
        page = k_cache.shape[1]
        t = torch.arange(T, device=qkv.device).view(1, T)
        pos = ctx_len.long().view(B, 1) + t
        ok = t < q_len.long().view(B, 1)
        blk = torch.gather(block_table.long(), 1, (pos // page).clamp(0, block_table.shape[1] - 1))
        slot = (blk * page + pos % page)[ok]
        k_cache.view(-1, n_kv, D)[slot] = k[ok].to(k_cache.dtype)
        v_cache.view(-1, n_kv, Dv)[slot] = v[ok].to(v_cache.dtype)
    return q.to(out_dtype or qkv.dtype)


def paged_window_attention(q, k_cache, v_cache, block_table, ctx_len, q_len, scale: float, softcap: float, window: int,
                           keep_first: int, gate=None, sinks=None, gate_per_head: bool = False, chunk=None, slopes=None, value_dim=None, head_scale=None):
    """Soft-capped attention of ragged query rows over a paged cache that already holds their own keys.  Query at position
    ``p = ctx_len + t`` sees key ``j`` iff ``j <= p and (p - j < window or j < keep_first)``; ``window <= 0`` means unbounded.
    score = cap * tanh(scale * q.k / cap) (cap <= 0: none), softmax in fp32.  ``gate`` [B, T, Hq * Dv]: the output is multiplied by
    ``sigmoid(gate)`` (``gate_per_head``: gate [B, T, Hq], one factor per head).  ``sinks`` [Hq] fp32: ``exp(sinks[h])`` joins the
    softmax denominator of head ``h`` (a slot without key or value, neither scaled nor capped).  ``chunk`` > 0: key ``j`` is visible only
    from positions of its own chunk, ``j // chunk == p // chunk`` (chunks count from position 0 of the sequence).  ``slopes`` [Hq] fp32:
    ``slopes[h] * (p - j)`` is taken off the score of head ``h`` (after scale and cap).  ``value_dim``: the value of a key is the first
    ``value_dim`` channels of the row in ``v_cache`` (latent caches whose key row is the latent followed by a rotated part).
    ``head_scale`` [Hq] fp32: the score of head ``h`` is multiplied by ``head_scale[h]`` as well (a learned temperature per head).
    q [B, T, Hq, D] -> [B, T, Hq * Dv]."""
    B, T, Hq, D = q.shape
    if value_dim is not None:
        v_cache = v_cache[..., :value_dim]
    page, G, Dv = v_cache.shape[1], v_cache.shape[2], v_cache.shape[3]
    bt = block_table.long().clamp_min(0)
    k = k_cache[bt].reshape(B, -1, G, D).float()
    v = v_cache[bt].reshape(B, -1, G, Dv).float()
    S = k.shape[1]
    p = (ctx_len.long().view(B, 1) + torch.arange(T, device=q.device).view(1, T)).unsqueeze(-1)          # [B, T, 1]
    j = torch.arange(S, device=q.device).view(1, 1, S)
    see = j <= p
    if window and window > 0:
        see = see & ((p - j < window) | (j < keep_first))
    if chunk and chunk > 0:
        see = see & (torch.div(j, chunk, rounding_mode="floor") == torch.div(p, chunk, rounding_mode="floor"))
    rep = Hq // G
    s = torch.einsum("bthd,bshd->bhts", q.float(), k.repeat_interleave(rep, 2)) * scale
    if head_scale is not None:
        s = s * head_scale.float().view(1, Hq, 1, 1)
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    if slopes is not None:
        s = s - slopes.float().view(1, Hq, 1, 1) * (p - j).clamp_min(0).float().unsqueeze(1)
    s = s.masked_fill(~see.unsqueeze(1), float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float().view(1, Hq, 1, 1).expand(B, Hq, T, 1)], -1)
        pr = torch.softmax(s, -1)[..., :-1]
    else:
        pr = torch.softmax(s, -1)
    o = torch.einsum("bhts,bshd->bthd", pr, v.repeat_interleave(rep, 2)).reshape(B, T, Hq * Dv)
    if gate is not None:
        gf = torch.sigmoid(gate.float())
        o = o * (gf.repeat_interleave(Dv, -1) if gate_per_head else gf)
    valid = (torch.arange(T, device=q.device).view(1, T) < q_len.long().view(B, 1)).unsqueeze(-1)
    return torch.where(valid, o, torch.zeros_like(o)).to(q.dtype)


def ssd_scan(xBC, dt_raw, z, A_log, dt_bias, D_skip, state, slots, ctx_len, q_len, n_heads: int, head_dim: int, n_state: int,
             n_groups: int):
    """Mamba-2 recurrence with a carried fp32 state ``[lines, n_heads, n_state, head_dim]``.  ``xBC`` [B, T, inner + 2 G N] is
    x | B | C after convolution and SiLU; per head ``h`` (group ``h // (n_heads / G)``), with ``dt = softplus(dt_raw + dt_bias)``:
    ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D_skip x``.  Returns ``y * silu(z)`` in fp32 [B, T, inner]; padding
    steps leave the state untouched."""
    B, T = xBC.shape[:2]
    nh, P, N, G = n_heads, head_dim, n_state, n_groups
    inner = nh * P
    x = xBC[..., :inner].float().view(B, T, nh, P)
    Bm = xBC[..., inner:inner + G * N].float().view(B, T, G, N).repeat_interleave(nh // G, 2)
    Cm = xBC[..., inner + G * N:inner + 2 * G * N].float().view(B, T, G, N).repeat_interleave(nh // G, 2)
    dt = F.softplus(dt_raw.float() + dt_bias.float(), threshold=1e9)
    dA = torch.exp(-torch.exp(A_log.float()) * dt)
    S = state[slots.long()].float()
    S = torch.where((ctx_len > 0).view(B, 1, 1, 1), S, torch.zeros_like(S))
    ys = []
    for t in range(T):
        live = (t < q_len).view(B, 1, 1, 1)
        S_new = S * dA[:, t, :, None, None] + (dt[:, t, :, None] * Bm[:, t])[..., None] * x[:, t, :, None, :]
        S = torch.where(live, S_new, S)
        ys.append((S * Cm[:, t, :, :, None]).sum(2))
    state[slots.long()] = torch.where((q_len > 0).view(B, 1, 1, 1), S, state[slots.long()].float()).to(state.dtype)
    y = torch.stack(ys, 1) + x * D_skip.float().view(1, 1, nh, 1)
    return y.reshape(B, T, inner) * F.silu(z.float())


def group_rmsnorm(y, weight, groups: int, eps: float, out_dtype=None):
    """RMS norm of ``groups`` equal parts of the last axis, each by its own root mean square, times ``weight``."""
    yf = y.float().reshape(*y.shape[:-1], groups, y.shape[-1] // groups)
    yf = (yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + eps)).reshape(y.shape)
    return (yf * weight.float()).to(out_dtype or y.dtype)


def clamped_glu(gu, limit: float, alpha: float = 1.702):
    """``[gate | up]`` halves -> ``g * sigmoid(alpha * g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``."""
    g, u = gu.float().chunk(2, -1)
    g = g.clamp(max=limit)
    u = u.clamp(-limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gu.dtype)


# ---- fp32 residual stream of pre-norm / parallel blocks, latent KV cache, plain experts ---------------------------------------
def stream_add_rmsnorm(x, adds=(), normed=None, normed_weight=None, vec=None, weight=None, eps: float = 1e-6, lp_dtype=None,
                       emit_stream_lp: bool = False):
    """One update of an fp32 residual stream plus the norm that reads it::

        s = [x] + sum(adds) + [rms_unit(normed) * normed_weight] + [vec]            (fp32; every term optional)
        h = rms_unit(s) * weight                                                   (when ``weight`` is given)

    ``rms_unit(v) = v / sqrt(mean(v^2) + eps)``; ``vec`` is one vector ``[W]`` added to every row.  Returns ``(s fp32, s cast to
    lp_dtype or None, h in lp_dtype (fp32 when lp_dtype is None) or None)``: the casts feed the next projections."""
    s = None if x is None else x.float()
    for y in adds:
        if y is not None:
            s = y.float() if s is None else s + y.float()
    if normed is not None:
        n = normed.float()
        n = n * torch.rsqrt(n.pow(2).mean(-1, keepdim=True) + eps)
        if normed_weight is not None:
            n = n * normed_weight.float()
        s = n if s is None else s + n
    if vec is not None:
        s = s + vec.float()
    lp = None if lp_dtype in (None, torch.float32) else lp_dtype
    h = None
    if weight is not None:
        h = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        h = h if lp is None else h.to(lp)
    return s, (s.to(lp) if (emit_stream_lp and lp is not None) else None), h


def rotate_half_rows(x, cos, sin):
    """x [..., R] with cos / sin broadcastable to [..., R / 2]: channel ``i`` pairs with ``i + R / 2``; the pair ``(u, v)`` becomes
    ``(u cos - v sin, v cos + u sin)``.  fp32."""
    half = x.shape[-1] // 2
    u, v = x[..., :half].float(), x[..., half:].float()
    return torch.cat([u * cos - v * sin, v * cos + u * sin], -1)


def latent_norm_append(p, offset: int, rank: int, weight, eps: float, cache, block_table, ctx_len, q_len, emit_rows: bool = False,
                       rot_dim: int = 0, cos=None, sin=None, q_rank: int = 0, q_weight=None):
    """Channels ``[offset, offset + rank)`` of the projection rows ``p`` [B, T, C] are RMS-normalised (fp32, ``weight`` [rank]) and
    written to the paged latent cache ``[blocks, page, 1, rank + rot_dim]`` at positions ``ctx_len + t`` for ``t < q_len``.

    ``rot_dim`` > 0: the next ``rot_dim`` channels (not normalised) are one rotated key part shared by all heads; they are rotated in
    the rotate-half layout with ``cos`` / ``sin`` [B, T, rot_dim / 2] and stored behind the latent in the same cache row.
    ``q_rank`` > 0: channels ``[0, q_rank)`` are a query latent; its RMS norm times ``q_weight`` is returned as well
    (``(rows, q_latent [B, T, q_rank])`` instead of ``rows``)."""
    B, T = p.shape[:2]
    page = cache.shape[1]
    c = p[..., offset:offset + rank].float()
    c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    if rot_dim:
        c = torch.cat([c, rotate_half_rows(p[..., offset + rank:offset + rank + rot_dim], cos.float(), sin.float())], -1)
    pos = ctx_len.long().view(B, 1) + torch.arange(T, device=p.device).view(1, T)
    live = torch.arange(T, device=p.device).view(1, T) < q_len.long().view(B, 1)
    width = block_table.shape[1]
    blk = torch.gather(block_table.long(), 1, (pos // page).clamp(0, width - 1))
    flat = blk * page + pos % page
    cache.view(-1, rank + rot_dim)[flat[live]] = c[live].to(cache.dtype)
    rows = torch.where(live.unsqueeze(-1), c, torch.zeros_like(c)).to(cache.dtype).view(B, T, 1, rank + rot_dim) if emit_rows else None
    if q_rank:
        cq = p[..., :q_rank].float()
        cq = cq * torch.rsqrt(cq.pow(2).mean(-1, keepdim=True) + eps) * q_weight.float()
        return rows, cq.to(p.dtype)
    return rows


def rope_half_tail(src, dst, rot_dim: int, cos, sin):
    """The last ``rot_dim`` channels of every head of ``src`` [B, T, H, Ds] are rotated (rotate-half layout, ``cos`` / ``sin``
    [B, T, rot_dim / 2], fp32) and written to the last ``rot_dim`` channels of the heads of ``dst`` [B, T, H, Dd]."""
    dst[..., dst.shape[-1] - rot_dim:] = rotate_half_rows(src[..., src.shape[-1] - rot_dim:], cos.float().unsqueeze(2),
                                                          sin.float().unsqueeze(2)).to(dst.dtype)
    return dst


def stream_norm_conv(x, adds, weight, conv_w, state, slots, ctx_len, q_len, eps: float, lp_dtype=None):
    """Update of an fp32 residual stream, the norm that reads it and a short causal convolution over time of the normalised rows::

        s_t = x_t + sum(adds_t)                                         (fp32)
        h_t = rms_unit(s_t) * weight
        y_t = h_t + sum_j conv_w[:, j] * h_(t - taps + 1 + j)           (zeros before the start of the sequence)

    The rows ``s`` of the ``taps - 1`` positions before a portion come from line ``slots[b]`` of ``state`` [lines, taps - 1, W] fp32
    (zero when ``ctx_len`` is 0) and are normalised like the new ones, so a result does not depend on where a prompt was cut.  The
    state is NOT advanced (:func:`short_conv_update` on ``s`` does that).  ``conv_w = None``: no convolution.  Returns
    ``(s fp32, y in lp_dtype (fp32 when None))``."""
    s = x.float()
    for a in adds:
        if a is not None:
            s = s + a.float()
    unit = lambda v: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.float()       # noqa: E731
    h = unit(s)
    if conv_w is not None:
        T, K = s.shape[1], conv_w.shape[1]
        win = unit(_conv_window(s, state, slots, ctx_len)) if K > 1 else h
        h = h + sum(win[:, j:j + T] * conv_w[:, j].float() for j in range(K))
    return s, (h if lp_dtype in (None, torch.float32) else h.to(lp_dtype))


def gated_act_mul(gate, other, act: str = "gelu_tanh", act_on_other: bool = False):
    """``act(gate) * other`` in fp32, cast to the type of ``gate``; ``other`` may be a strided slice of a wider row.
    ``act_on_other``: ``gate * act(other)`` instead (the activation goes on the strided operand)."""
    if act_on_other:
        return (gate.float() * activation(other.float(), act)).to(gate.dtype)
    return (activation(gate.float(), act) * other.float()).to(gate.dtype)


def unary_act(x, act: str):
    return activation(x.float(), act).to(x.dtype)


# ---- sandwich-norm blocks, per-head norms around a rotate-half rotation, the gated delta rule -------------------------------------
def _norm_rows(v, center: bool, eps: float):
    """``v`` over its last axis: minus its mean when ``center``, divided by the root of the mean square (of the deviations) + eps."""
    if center:
        v = v - v.mean(-1, keepdim=True)
    return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def stream_sandwich_norm(x, a=None, b=None, a_weight=None, b_weight=None, a_scale: float = 1.0, b_scale: float = 1.0, post_weight=None,
                         layer_scale=None, mult: float = 1.0, next_weight=None, eps: float = 1e-6, center: bool = True, lp_dtype=None):
    """One update of an fp32 residual stream whose sublayers are normalised on BOTH sides, plus the norm the next sublayer reads::

        y = a_scale * f_a(a) + b_scale * f_b(b)        f(v) = rms_unit(v) * weight when a weight is given, else v   (b optional)
        s = x + mult * layer_scale * norm(y) * post_weight                                        (s = x when a is None)
        h = norm(s) * next_weight                                                                 (when next_weight is given)

    ``norm`` is a layer norm without bias when ``center`` (mean taken off, variance of the deviations), an RMS norm otherwise; all of it
    is fp32, nothing between ``a`` / ``b`` and ``s`` is rounded.  Returns ``(s fp32, h in lp_dtype or None)``."""
    s = x.float()
    if a is not None:
        def side(v, w, sc):
            v = v.float()
            if w is not None:
                v = _norm_rows(v, False, eps) * w.float()
            return v * sc
        y = side(a, a_weight, a_scale)
        if b is not None:
            y = y + side(b, b_weight, b_scale)
        y = _norm_rows(y, center, eps)
        if post_weight is not None:
            y = y * post_weight.float()
        if layer_scale is not None:
            y = y * layer_scale.float()
        s = s + mult * y
    h = None
    if next_weight is not None:
        h = _norm_rows(s, center, eps) * next_weight.float()
        h = h if lp_dtype in (None, torch.float32) else h.to(lp_dtype)
    return s, h


def head_norm_rope_append(p, n_q: int, n_kv: int, D: int, Dv: int, cos, sin, q_norm_w, k_norm_w, norm_at: int, eps: float,
                          value_from_key: bool, k_cache, v_cache, block_table, ctx_len, q_len, out_dtype=None):
    """Front half of a grouped-query attention layer on ragged rows.  ``p`` [B, T, >= n_q D + n_kv D (+ n_kv Dv)] holds q | k | v
    (no v slice when ``value_from_key``: the raw k slice doubles as the value, untouched by norm or rotation, so ``Dv == D``).
    Every q and k head is RMS-normalised over its ``D`` channels (``norm_at`` 1: before the rotation, 2: after it, 0: not at all;
    ``q_norm_w`` / ``k_norm_w`` [D] are shared by the heads, ``None`` = no weight) and its first ``2 * cos.shape[-1]`` channels are
    rotated in the rotate-half layout (channel ``i`` pairs with ``i + R / 2``); ``cos = None`` skips the rotation.  Keys and values go
    to the paged caches ``[blocks, page, n_kv, D | Dv]`` at position ``ctx_len + t``.  Returns q [B, T, n_q, D]."""
    B, T = p.shape[:2]
    Cq, Ck = n_q * D, n_kv * D
    q = p[..., :Cq].float().reshape(B, T, n_q, D)
    k_raw = p[..., Cq:Cq + Ck].float().reshape(B, T, n_kv, D)
    v = k_raw if value_from_key else p[..., Cq + Ck:Cq + Ck + n_kv * Dv].float().reshape(B, T, n_kv, Dv)

    def prep(x, w):
        if norm_at == 1:
            x = _norm_rows(x, False, eps)
            if w is not None:
                x = x * w.float()
        if cos is not None:
            R = 2 * cos.shape[-1]
            x = torch.cat([rotate_half_rows(x[..., :R], cos.float().unsqueeze(2), sin.float().unsqueeze(2)), x[..., R:]], -1)
        if norm_at == 2:
            x = _norm_rows(x, False, eps)
            if w is not None:
                x = x * w.float()
        return x
    q, k = prep(q, q_norm_w), prep(k_raw, k_norm_w)
    page = k_cache.shape[1]
    t = torch.arange(T, device=p.device).view(1, T)
    pos = ctx_len.long().view(B, 1) + t
    ok = t < q_len.long().view(B, 1)
    blk = torch.gather(block_table.long(), 1, (pos // page).clamp(0, block_table.shape[1] - 1))
    slot = (blk * page + pos % page)[ok]
    k_cache.view(-1, n_kv, D)[slot] = k[ok].to(k_cache.dtype)
    v_cache.view(-1, n_kv, Dv)[slot] = v[ok].to(v_cache.dtype)
    return q.to(out_dtype or p.dtype)


def gated_delta_scan(qkv, beta_raw, a_raw, A_log, dt_bias, state, slots, ctx_len, q_len, n_heads: int, n_qk: int, D: int, Dv: int,
                     unit_eps: float = 1e-6):
    """Gated delta rule with a carried fp32 state ``[lines, n_heads, D, Dv]``.  ``qkv`` [B, T, 2 n_qk D + n_heads Dv] is q | k | v after
    their convolutions and activations; head ``h`` reads q / k head ``h // (n_heads / n_qk)``.  q and k are scaled to unit length
    (``unit_eps`` under the root) and q also by ``D^-1/2``; write strength ``b = sigmoid(beta_raw)``, decay with
    ``log decay = -exp(A_log) * softplus(a_raw + dt_bias)`` (both [B, T, n_heads]).  Per head and step the state ``M`` is shrunk,
    ``M *= decay``, corrected along k towards v, ``e = b * (v - M' k)``, ``M += outer(k, e)``, and read AFTER the correction,
    ``y = M' q``.  Returns y fp32 [B, T, n_heads * Dv]; padding steps leave the state untouched."""
    B, T = qkv.shape[:2]
    H, rep = n_heads, n_heads // n_qk
    Cq = n_qk * D
    unit = lambda x: x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + unit_eps)          # noqa: E731
    q = (unit(qkv[..., :Cq].float().reshape(B, T, n_qk, D)) * D ** -0.5).repeat_interleave(rep, 2)
    k = unit(qkv[..., Cq:2 * Cq].float().reshape(B, T, n_qk, D)).repeat_interleave(rep, 2)
    v = qkv[..., 2 * Cq:2 * Cq + H * Dv].float().reshape(B, T, H, Dv)
    beta = torch.sigmoid(beta_raw.float())
    g = torch.exp(-torch.exp(A_log.float()) * F.softplus(a_raw.float() + dt_bias.float(), threshold=1e9))
    S = state[slots.long()].float()
    S = torch.where((ctx_len > 0).view(B, 1, 1, 1), S, torch.zeros_like(S))
    out = []
    for t in range(T):
        live = (t < q_len).view(B, 1, 1, 1)
        Sd = S * g[:, t, :, None, None]
        u = beta[:, t, :, None] * (v[:, t] - torch.einsum("bhdv,bhd->bhv", Sd, k[:, t]))
        Sn = Sd + k[:, t, :, :, None] * u[:, :, None, :]
        S = torch.where(live, Sn, S)
        out.append(torch.einsum("bhdv,bhd->bhv", S, q[:, t]))
    state[slots.long()] = torch.where((q_len > 0).view(B, 1, 1, 1), S, state[slots.long()].float()).to(state.dtype)
    return torch.stack(out, 1).reshape(B, T, H * Dv)


def head_rmsnorm_gate(y, weight, heads: int, eps: float, gate, act: str = "silu", out_dtype=None):
    """``y`` [..., heads * Dv] fp32: every head is divided by its root mean square over ``Dv``, times ``weight`` [Dv] (shared by the
    heads), times ``act(gate)`` (``gate`` [..., heads * Dv], possibly a strided slice of a wider row); the gate comes AFTER the norm."""
    Dv = y.shape[-1] // heads
    yf = _norm_rows(y.float().reshape(*y.shape[:-1], heads, Dv), False, eps) * weight.float()
    return (yf.reshape(y.shape) * activation(gate.float(), act)).to(out_dtype or y.dtype)
