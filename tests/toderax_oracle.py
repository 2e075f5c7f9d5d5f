"""Plain, slow restatement of the Toderax design in torch float64: a decoder whose layers run their mixer and then their feed-forward on
several residual streams (hyper-connections), with group-wise RMS norms, three sequence mixers (a gated linear recurrence whose forget
gate also sets the write strength; softmax attention within position chunks with a sink; retention with a fixed decay per head, the last
two side by side) and a mixture-of-experts feed-forward with a shared expert.

One function per mechanism, whole sequences only, no cache, no batching: it is the yardstick the engine, its cache / state manager and
its kernels are compared with.  It shares no code with the product package.

Notation: T tokens, W model width, H query heads, G key/value heads, D query/key size, Dv value size, s streams.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, w, groups: int, eps: float):
    """The last axis in `groups` equal consecutive parts, each brought to unit RMS by itself; then the gain over the whole axis."""
    T, W = x.shape
    return unit_rms(x.reshape(T, groups, W // groups), eps).reshape(T, W) * w.to(F)


def silu(z):
    return z * torch.sigmoid(z)


def gate_recurrence(h, w: dict, m: dict, eps: float):
    """h [T, W] -> [T, W].  Per head a [D, Dv] state; row i of it is kept with f_i and takes (1 - f_i) v: S <- diag(f) S + (1 - f) v^T,
    read out as S^T q after the write; f never falls below a learned floor."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w["q"].to(F).T).view(T, H, D)
    v = (h @ w["v"].to(F).T).view(T, H, Dv)
    floor = w["lower"].to(F)
    f = (floor + (1.0 - floor) * torch.sigmoid(h @ w["f"].to(F).T + w["f.b"].to(F))).view(T, H, D)
    out = torch.zeros(T, H, Dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(D, Dv, dtype=F)
        for t in range(T):
            S = f[t, hd][:, None] * S + torch.outer(1.0 - f[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = unit_rms(out, eps) * w["norm"].to(F)[None, None, :]
    return out.reshape(T, H * Dv) @ w["o"].to(F).T


def chunk_sink_attention(h, w: dict, m: dict, eps: float):
    """h [T, W] -> [T, W].  Grouped-query softmax attention without positions in the scores: q and k (with biases) are brought to unit RMS per
    head, scores are q.k * scale * temp_h, a query sees the keys at or before it that lie in its own chunk of `mask.size` positions, and the
    softmax denominator holds one more term exp(sink_h) that carries no value."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ w["q"].to(F).T + w["q.b"].to(F)).view(T, H, D), eps)
    k = unit_rms((h @ w["k"].to(F).T + w["k.b"].to(F)).view(T, G, D), eps)
    v = (h @ w["v"].to(F).T + w["v.b"].to(F)).view(T, G, Dv)
    pos = torch.arange(T)
    see = pos[None, :] <= pos[:, None]
    size = (m.get("mask") or {}).get("size")
    if size:
        see &= (pos[None, :] // size) == (pos[:, None] // size)
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] * float(w["temp"][hd])
        s = s.masked_fill(~see, float("-inf"))
        s = torch.cat([s, torch.full((T, 1), float(w["sink"][hd]), dtype=F)], 1)
        p = torch.softmax(s, -1)[:, :T]
        heads.append(p @ v[:, g])
    return torch.cat(heads, -1) @ w["o"].to(F).T


def half_rotation(x, rot: dict):
    """x [T, n, D]: entry i of the first `dims` is paired with entry i + dims/2 and the pair is turned by position * base^(-2i/dims)."""
    T = x.shape[0]
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    ang = torch.arange(T, dtype=F)[:, None] * base ** (-2.0 * torch.arange(half, dtype=F) / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def retention(h, w: dict, m: dict, eps: float):
    """h [T, W] -> [T, W].  Per head S <- decay_h S + k v^T, o = S^T q (no softmax, no denominator); q and k rotated, k scaled by D^-1/2 after
    the rotation; unit-RMS heads times silu of an output gate."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = half_rotation((h @ w["q"].to(F).T).view(T, H, D), m["rot"])
    k = half_rotation((h @ w["k"].to(F).T).view(T, H, D), m["rot"]) * D ** -0.5
    v = (h @ w["v"].to(F).T).view(T, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(D, Dv, dtype=F)
        for t in range(T):
            S = float(m["decay"][hd]) * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = unit_rms(out, eps).reshape(T, H * Dv) * silu(h @ w["g"].to(F).T)
    return out @ w["o"].to(F).T


def side_by_side(h, w: dict, m: dict, eps: float):
    """Chunked sink attention and retention on the same input; each output is RMS-normed over the width with its own gain, then the mean."""
    sub = lambda side: {k[len(side) + 1:]: t for k, t in w.items() if k.startswith(side + ".") and k != side + ".out"}
    a = unit_rms(chunk_sink_attention(h, sub("left"), m["left"], eps), eps) * w["left.out"].to(F)
    b = unit_rms(retention(h, sub("right"), m["right"], eps), eps) * w["right.out"].to(F)
    return 0.5 * (a + b)


def clamped_expert(h, w: dict, limit: float):
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = (h @ w["gate"].to(F).T).clamp(max=limit)
    u = (h @ w["up"].to(F).T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].to(F).T


def expert_mixture(h, w: dict, mlp: dict):
    """Softmax router over all experts; the `top` best experts of a token run and are weighted by their (not renormalised) scores; a shared
    expert runs for every token."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    score = torch.softmax(h @ w["router"].to(F).T, -1)
    best = torch.topk(score, top, -1).indices
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for e in range(E):
        ew = {n: w[f"e{e}.{n}"] for n in ("gate", "up", "down")}
        use = (best == e).any(-1)
        if use.any():
            out[use] += score[use, e][:, None] * clamped_expert(h[use], ew, mlp["expert"]["limit"])
    if mlp.get("shared"):
        out += clamped_expert(h, {n: w[f"shared.{n}"] for n in ("gate", "up", "down")}, mlp["shared"]["limit"])
    return out


MIXERS = {"hgrn2": gate_recurrence, "parallel": side_by_side}


def forward(cfg: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] (float64) of one whole sequence; optionally the sum of the residual streams after every layer."""
    eps, groups, ns = cfg["norm"]["eps"], cfg["norm"].get("groups", 1), cfg.get("streams", 0)
    x0 = weights["embed"].to(F)[list(tokens)] * float(cfg["embedding"]["scale"])
    xs = [x0.clone() for _ in range(max(ns, 1))]
    trace = []

    def sublayer(pre, q, fn):
        nonlocal xs
        if ns:
            cin, cout, mix = (weights[f"{pre}hc{q}.{n}"].to(F) for n in ("in", "out", "mix"))
            u = sum(cin[s] * xs[s] for s in range(ns))
            y = fn(group_norm(u, weights[f"{pre}norm{q}"], groups, eps))
            xs = [sum(mix[s, t] * xs[s] for s in range(ns)) + cout[t] * y for t in range(ns)]
        else:
            xs = [xs[0] + fn(group_norm(xs[0], weights[f"{pre}norm{q}"], groups, eps))]

    for li, spec in enumerate(cfg["layers"]):
        pre = f"l{li}."
        mw = {k[len(pre) + 4:]: t for k, t in weights.items() if k.startswith(pre + "mix.")}
        sublayer(pre, 1, lambda h: MIXERS[spec["type"]](h, mw, spec["mixer"], eps))
        if spec.get("mlp"):
            fw = {k[len(pre) + 4:]: t for k, t in weights.items() if k.startswith(pre + "mlp.")}
            sublayer(pre, 2, lambda h: expert_mixture(h, fw, spec["mlp"]))
        trace.append(sum(xs))
    logits = group_norm(sum(xs), weights["final.norm"], groups, eps) @ weights["head"].to(F).T
    return (logits, torch.stack(trace)) if return_layers else logits
