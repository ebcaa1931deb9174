"""Plain definition of the Tusipel decoder, one function per mechanism, float64, whole sequences, no cache.  Shares nothing with the
engine: tests compare the engine (loader, caches per layer run, state lines, ragged batches, kernels) against these functions."""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def block_norm(x, w, eps):
    """Weight stored around zero."""
    return rms(x, eps) * (1.0 + w)


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    return sum(pad[j:j + T] * w[:, j] for j in range(taps))


def canon(h, w):
    """What a sublayer reads; a stack without these convolutions (no taps in its configuration) reads h itself."""
    return h if w is None else h + causal_conv(h, w)


def yarn_tables(T, rot):
    """cos / sin [T, dims / 2] of the rotate-half layout with the scaled frequencies."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        where = lambda t: dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))       # noqa: E731
        lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / sc["factor"] * ramp + f * (1 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    a = torch.arange(T, dtype=torch.float64).unsqueeze(1) * f
    return torch.cos(a) * mag, torch.sin(a) * mag


def rotate_half(x, cos, sin):
    """x [T, ..., dims]; dimension i pairs with i + dims / 2."""
    half = x.shape[-1] // 2
    u, v = x[..., :half], x[..., half:]
    while cos.dim() < u.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([u * cos - v * sin, v * cos + u * sin], -1)


def softmax_rows(s, see):
    s = s.masked_fill(~see, float("-inf"))
    e = torch.exp(s - s.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def latent_attention(h, w, p, m, eps):
    T, H, d, r, dv, R = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    kv = h @ w[p + "dkv"].T
    c = rms(kv[:, :R], eps) * w[p + "dkv.norm"]
    cos, sin = yarn_tables(T, m["rot"])
    k_rot = rotate_half(kv[:, R:], cos, sin)                                  # [T, r], one for all heads
    q_rot = rotate_half(q[..., d:], cos, sin)
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    see = (j <= i)
    if (m.get("mask") or {}).get("size"):
        see = see & (i - j < m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        s = (q[:, a, :d] @ k[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = softmax_rows(s, see) @ v[:, a]
    return (out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def conv_attention(h, w, p, m):
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for n in ("q", "k", "v"):
        u = h @ w[p + n].T
        proj[n] = causal_conv(u, w[p + n + ".conv"]) if p + n + ".conv" in w else u
    q, k, v = proj["q"].view(T, H, d), proj["k"].view(T, G, d), proj["v"].view(T, G, dv)
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    see = (j <= i)
    if (m.get("mask") or {}).get("size"):
        see = see & (i // m["mask"]["size"] == j // m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        s = (q[:, a] @ k[:, g].T) * m["scale"] - slope * (i - j).double()
        out[:, a] = softmax_rows(s, see) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def dense_ff(h, w, p, f):
    L = f["limit"]
    g = (h @ w[p + "gate"].T).clamp(max=L)
    u = (h @ w[p + "up"].T).clamp(-L, L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(z, correction, r):
    """-> (weights [T, top], ids [T, top]); ids >= r['experts'] are identity experts."""
    n, top = r["experts"] + r.get("identity", 0), r["top"]
    s = torch.softmax(z, -1)
    choice = s + correction
    groups = r.get("groups")
    if groups:
        per = n // groups["count"]
        best = choice.view(-1, groups["count"], per).max(-1).values
        keep = torch.zeros_like(best, dtype=torch.bool)
        keep.scatter_(1, best.topk(groups["keep"], -1).indices, True)
        choice = choice.masked_fill(~keep.repeat_interleave(per, 1), float("-inf"))
    idx = choice.topk(top, -1).indices
    return s.gather(1, idx) * r.get("scale", 1.0), idx


def moe_ff(h, w, p, f):
    r = f["router"]
    wt, idx = route(h @ w[p + "router"].T, w[p + "correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            if e >= r["experts"]:
                y = h[t]
            else:
                a = h[t] @ w[f"{p}e{e}.gate"].T
                y = (a * torch.sigmoid(a) * (h[t] @ w[f"{p}e{e}.up"].T)) @ w[f"{p}e{e}.down"].T
            out[t] += wt[t, k] * y
    return out


def layer_order(n, loop):
    """[(layer, first of a later pass)]."""
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] (float64) of one whole sequence; ``streams`` collects the residual stream after every layer run."""
    w = {k: v.double() for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    x = x0
    for i, again in layer_order(len(cfg["layers"]), cfg.get("loop")):
        if again:
            x = x + x0
        spec, p = cfg["layers"][i], f"l{i}."
        h = canon(block_norm(x, w[p + "norm1"], eps), w.get(p + "canon1"))
        if spec["type"] == "latent_attention":
            x = x + latent_attention(h, w, p + "mix.", spec["mixer"], eps)
        else:
            x = x + conv_attention(h, w, p + "mix.", spec["mixer"])
        f = spec.get("mlp")
        if f is not None:
            h = canon(block_norm(x, w[p + "norm2"], eps), w.get(p + "canon2"))
            x = x + (dense_ff(h, w, p + "mlp.", f) if f["kind"] == "dense" else moe_ff(h, w, p + "mlp.", f))
        if streams is not None:
            streams.append(x.clone())
    return block_norm(x, w["final.norm"], eps) @ w["head"].T
