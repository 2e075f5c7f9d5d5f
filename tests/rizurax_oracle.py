"""Plain, slow restatement of the Rizurax design (hybrid decoder: differential attention + gated delta rule) in torch float64.

One function per mechanism, whole sequences only, no cache, no batching: it is the yardstick the engine, its cache / state manager and
its kernels are compared with.  It shares no code with the product package.

Notation: T tokens, W model width, H query heads, G key/value heads, D per-map query/key size, Dv value size.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + w.to(F))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed_tokens(tokens, table, bigram=None, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0):
    """Token embedding plus (if there is a pair table) a hashed (previous, current) pair embedding; a sequence's first token takes the
    table's last row."""
    rows = []
    for i, t in enumerate(tokens):
        x = table[t].to(F)
        if bigram is not None:
            row = buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets
            x = x + bigram[row].to(F)
        rows.append(x)
    return torch.stack(rows)


def rotary_tables(positions, rot: dict):
    """cos / sin [T, dims/2] of the interleaved rotary embedding with the YaRN frequency blend and amplitude factor."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=F)
    f = base ** (-2.0 * i / dims)
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def turn_dim(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        amp = 0.1 * math.log(factor) + 1.0
    ang = torch.as_tensor(positions, dtype=F)[:, None] * f[None, :]
    return torch.cos(ang) * amp, torch.sin(ang) * amp


def rotate_pairs(x, cos, sin, dims: int):
    """x [T, n, D]: pairs (2i, 2i+1) of the first `dims` entries are rotated, the rest pass."""
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def differential_attention(h, w: dict, m: dict, eps: float):
    """h [T, W] -> [T, W].  Two softmax maps per head over shared values, combined as a1 - lambda a2, unit-RMS per head."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].to(F).T).view(T, H * 2, D)
    k = (h @ w["k"].to(F).T).view(T, G * 2, D)
    v = (h @ w["v"].to(F).T).view(T, G, Dv)
    cos, sin = rotary_tables(range(T), m["rot"])
    q = rotate_pairs(q, cos, sin, m["rot"]["dims"]).view(T, H, 2, D)
    k = rotate_pairs(k, cos, sin, m["rot"]["dims"]).view(T, G, 2, D)
    lam = math.exp(float((w["lq1"].to(F) * w["lk1"].to(F)).sum())) - math.exp(float((w["lq2"].to(F) * w["lk2"].to(F)).sum())) + m["diff"]
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        a = []
        for mp in range(2):
            s = (q[:, hd, mp] @ k[:, g, mp].T) * m["scale"]
            s = s.masked_fill(~causal, float("-inf"))
            a.append(torch.softmax(s, -1) @ v[:, g])
        o = a[0] - lam * a[1]
        heads.append(rms_unit(o, eps) * (1.0 - m["diff"]))
    return torch.cat(heads, -1) @ w["o"].to(F).T


def short_conv_silu(x, taps_w):
    """x [T, C], taps_w [C, taps]; the last tap multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x])
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y += pad[j:j + T] * taps_w[:, j].to(F)[None, :]
    return silu(y)


def gated_delta(h, w: dict, m: dict, eps: float):
    """h [T, W] -> [T, W]: per head a [D, Dv] state with decay, delta-rule write and read-out after the write."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w["q"].to(F).T, w["q.conv"]).view(T, G, D)
    k = short_conv_silu(h @ w["k"].to(F).T, w["k.conv"]).view(T, G, D)
    v = short_conv_silu(h @ w["v"].to(F).T, w["v.conv"]).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].to(F).T)
    decay = torch.exp(-torch.exp(w["A_log"].to(F)) * torch.nn.functional.softplus(h @ w["a"].to(F).T + w["dt_bias"].to(F)))
    gate = silu(h @ w["g"].to(F).T).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(D, Dv, dtype=F)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = rms_unit(out, eps) * w["norm"].to(F)[None, None, :] * gate
    return out.reshape(T, H * Dv) @ w["o"].to(F).T


def dense_mlp(h, w: dict):
    return (gelu_tanh(h @ w["gate"].to(F).T) * (h @ w["up"].to(F).T)) @ w["down"].to(F).T


def layer_schedule(cfg: dict):
    """Order in which the layers run, the looped span repeated in a row."""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = lp["start"], lp["stop"], lp["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] (float64) of one whole sequence; optionally the residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = embed_tokens(list(tokens), weights["embed"], weights["bigram"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    else:
        x = embed_tokens(list(tokens), weights["embed"])
    trace = []
    for li in layer_schedule(cfg):
        spec = cfg["layers"][li]
        pre = f"l{li}."
        mw = {k[len(pre) + 4:]: t for k, t in weights.items() if k.startswith(pre + "mix.")}
        fn = differential_attention if spec["type"] == "attention" else gated_delta
        upd = fn(zero_centred_norm(x, weights[pre + "norm1"], eps), mw, spec["mixer"], eps)
        if spec.get("mlp"):
            fw = {k[len(pre) + 4:]: t for k, t in weights.items() if k.startswith(pre + "mlp.")}
            upd = upd + dense_mlp(zero_centred_norm(x, weights[pre + "norm2"], eps), fw)
        x = x + upd
        trace.append(x)
    logits = zero_centred_norm(x, weights["final.norm"], eps) @ weights["head"].to(F).T
    return (logits, torch.stack(trace)) if return_layers else logits
