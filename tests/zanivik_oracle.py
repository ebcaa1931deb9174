"""Plain float64 definition of the Zanivik decoder, one function per mechanism, whole sequences only (no cache, no state handed
between calls, no batches).  The tests compare the engine with this file; nothing here is shared with the product path."""
import math

import torch

F64 = torch.float64


def layer_norm(x, w, eps):
    """Centre x over its last axis, divide by the root of (second moment of the centred values + eps), multiply by w; there is no bias."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(x):
    return x * torch.sigmoid(x)


def gelu_erf(x):
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def rotary_frequencies(rot):
    """dims / 2 frequencies on a geometric ladder that starts at 1 and shrinks by base^(-2/dims) per step.  ``scaling`` {factor, low, high,
    original} slows the long wavelengths: shorter than original/high untouched, longer than original/low divided by factor, and a linear
    blend (in original / wavelength) for the band between."""
    d = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / d) for i in range(d // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = []
    for fi in f.tolist():
        wl = 2.0 * math.pi / fi
        if wl < sc["original"] / sc["high"]:
            out.append(fi)
        elif wl > sc["original"] / sc["low"]:
            out.append(fi / sc["factor"])
        else:
            s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * fi / sc["factor"] + s * fi)
    return torch.tensor(out, dtype=F64)


def rotate(x, rot, first_position=0):
    """x [T, H, D]: the first ``dims`` channels split into a low and a high half; with c, s = cos, sin(position * f_i):
    lo' = lo c - hi s, hi' = hi c + lo s; the channels past ``dims`` are copied."""
    d = rot["dims"]
    if not d:
        return x
    f = rotary_frequencies(rot)
    pos = torch.arange(first_position, first_position + x.shape[0], dtype=F64)
    a = pos[:, None] * f[None]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :d // 2], x[..., d // 2:d]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., d:]], -1)


def softmax_rows(s, see, sink=None):
    """Rows of ``s`` [..., n] over the visible entries; ``sink`` [...] adds exp(sink) to the denominator only."""
    s = s.masked_fill(~see, -float("inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.unsqueeze(-1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.unsqueeze(-1) - m)
    return e / den


def window_attention(q, k, v, scale, window, sink=None, temp=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; consecutive runs of H / G query heads share a kv head.  Row i of the score matrix keeps columns
    i - window + 1 .. i (all columns up to i without a window); scores are scaled dot products, times temp[h] when given; ``sink`` [H] enters
    :func:`softmax_rows`."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    see = (i - j >= 0) & ((i - j < window) if window else True)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        if temp is not None:
            s = s * temp[h]
        p = softmax_rows(s, see, None if sink is None else sink[h].expand(T))
        out[:, h] = p @ v[:, g]
    return out


def causal_conv(x, w, bias=None):
    """x [T, C], w [C, K]: y[t] = sum_d w[:, K - 1 - d] * x[t - d] over d < K, inputs before the sequence counting as zero."""
    T, K = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            src = t - (K - 1) + j
            if src >= 0:
                y[t] += w[:, j] * x[src]
    return y if bias is None else y + bias


def gated_delta_rule(q, k, v, beta, decay):
    """q, k [T, H, D], v [T, H, Dv], beta, decay [T, H].  Per step: shrink the state by the decay, correct it along k towards v with
    strength beta, then read it at q (the read comes after the correction)."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=F64)
    out = []
    for t in range(T):
        S = decay[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def ssd_recurrence(x, B, C, dt, A, D):
    """x [T, H, P], B, C [T, H, N], dt [T, H], A, D [H].  Per step the state [N, P] decays by exp(-A dt), takes in dt * outer(B, x), and is read
    along C; D x is a skip path."""
    T, H, P = x.shape
    S = torch.zeros(H, B.shape[-1], P, dtype=F64)
    ys = []
    for t in range(T):
        S = torch.exp(-A * dt[t])[:, None, None] * S + dt[t][:, None, None] * torch.einsum("hn,hp->hnp", B[t], x[t])
        ys.append(torch.einsum("hnp,hn->hp", S, C[t]) + D[:, None] * x[t])
    return torch.stack(ys)


def left_sink_gate(h, m, w, p, eps):
    """Attention half of a ``parallel`` pair."""
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, m["heads"], m["dim"])
    k = (h @ w[p + "k"].T).view(T, m["kv_heads"], m["dim"])
    v = (h @ w[p + "v"].T).view(T, m["kv_heads"], m["vdim"])
    q, k = rms_norm(rotate(q, m["rot"]), eps), rms_norm(rotate(k, m["rot"]), eps)
    o = window_attention(q, k, v, m["scale"], (m.get("mask") or {}).get("size"), sink=w[p + "sink"]).reshape(T, -1)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def right_delta(h, m, w, p, eps):
    """Recurrent half of a ``parallel`` pair."""
    T, H, G, D, Dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, Dv)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)       # noqa: E731
    q, k = (unit(q) * D ** -0.5).repeat_interleave(H // G, 1), unit(k).repeat_interleave(H // G, 1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"], threshold=1e9))
    o = rms_norm(gated_delta_rule(q, k, v, beta, decay), eps, w[p + "norm"]).reshape(T, -1) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def left_key_values(h, m, w, p, eps):
    """Attention half of a ``parallel_2`` pair: no value projection, the raw keys double as values."""
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, m["heads"], m["dim"])
    k = (h @ w[p + "k"].T).view(T, m["kv_heads"], m["dim"])
    qn, kn = rotate(rms_norm(q, eps, w[p + "q.norm"]), m["rot"]), rotate(rms_norm(k, eps, w[p + "k.norm"]), m["rot"])
    o = window_attention(qn, kn, k, m["scale"], (m.get("mask") or {}).get("size"), temp=w[p + "temp"]).reshape(T, -1)
    return o @ w[p + "o"].T


def right_mamba2(h, m, w, p, eps):
    """Recurrent half of a ``parallel_2`` pair."""
    T, H, P, N, G = h.shape[0], m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    I = H * P
    pr = h @ w[p + "in"].T
    z, xBC, dt = pr[:, :I], pr[:, I:2 * I + 2 * G * N], pr[:, 2 * I + 2 * G * N:]
    xBC = silu(causal_conv(xBC, w[p + "conv"], w[p + "conv.b"]))
    x = xBC[:, :I].view(T, H, P)
    B = xBC[:, I:I + G * N].view(T, G, N).repeat_interleave(H // G, 1)
    C = xBC[:, I + G * N:].view(T, G, N).repeat_interleave(H // G, 1)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"], threshold=1e9)
    y = ssd_recurrence(x, B, C, dt, torch.exp(w[p + "A_log"]), w[p + "D"]).reshape(T, I) * silu(z)
    ng = m.get("norm_groups", 1)
    y = rms_norm(y.view(T, ng, I // ng), eps).reshape(T, I) * w[p + "norm"]
    return y @ w[p + "o"].T


def mixer(h, layer, w, p, eps):
    m = layer["mixer"]
    if layer["type"] == "parallel":
        return m["left_scale"] * left_sink_gate(h, m["left"], w, p + "left.", eps) + m["right_scale"] * right_delta(h, m["right"], w, p + "right.", eps)
    a, b = left_key_values(h, m["left"], w, p + "left.", eps), right_mamba2(h, m["right"], w, p + "right.", eps)
    return 0.5 * (rms_norm(a, eps, w[p + "left.out"]) + rms_norm(b, eps, w[p + "right.out"]))


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence; ``streams`` collects the residual stream after every layer."""
    w = {k: v.double() for k, v in w.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + mult * layer_norm(mixer(layer_norm(x, w[p + "norm1"], eps), layer, w, p + "mix.", eps), w[p + "norm1b"], eps) * w[p + "ls1"]
        if layer.get("mlp") is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            y = gelu_erf(h @ w[p + "mlp.up"].T) @ w[p + "mlp.down"].T
            x = x + mult * layer_norm(y, w[p + "norm2b"], eps) * w[p + "ls2"]
        if streams is not None:
            streams.append(x)
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T
