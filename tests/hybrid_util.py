"""Helpers of the hybrid-decoder tests: small random Rizurax models (config dict + weights) and error measures."""
import math

import torch


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, scaling=True, diff=0.35, ff=48, base=500.0):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 48, "fast": 16.0, "slow": 2.0}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot,
                                           "scale": 1.0 / math.sqrt(dim), "diff": diff},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=4, ff=48):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(layers, vocab=97, width=40, loop=None, bigram=(53, 31, 5), eps=1e-5):
    cfg = {"architecture": "Rizurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return cfg


def make_weights(cfg, seed=0, gain=1.0):
    """Random weights, rounded to bfloat16 values (held as float32) so that every dtype sees the same numbers."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).to(torch.float32)
    w = {"embed": r(cfg["vocab"], W), "head": r(cfg["vocab"], W, s=W ** -0.5), "final.norm": r(W, s=0.2)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        w["bigram"] = r(bg["buckets"] + 1, W, s=0.5)
    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        w[p + "norm1"] = r(W, s=0.2)
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if ly["type"] == "attention":
            w[p + "mix.q"] = r(H * 2 * D, W, s=gain * 2.0 * W ** -0.5)
            w[p + "mix.k"] = r(G * 2 * D, W, s=gain * 2.0 * W ** -0.5)
            w[p + "mix.v"] = r(G * Dv, W, s=W ** -0.5)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[p + "mix." + n] = r(D, s=0.3)
            w[p + "mix.o"] = r(W, H * Dv, s=(H * Dv) ** -0.5)
        else:
            w[p + "mix.q"] = r(G * D, W, s=W ** -0.5)
            w[p + "mix.k"] = r(G * D, W, s=W ** -0.5)
            w[p + "mix.v"] = r(H * Dv, W, s=W ** -0.5)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                w[p + f"mix.{n}.conv"] = r(c, m["conv"], s=0.6)
            w[p + "mix.b"] = r(H, W, s=W ** -0.5)
            w[p + "mix.a"] = r(H, W, s=W ** -0.5)
            w[p + "mix.A_log"] = r(H, s=0.5)
            w[p + "mix.dt_bias"] = r(H, s=0.5)
            w[p + "mix.norm"] = 1.0 + r(Dv, s=0.2)
            w[p + "mix.g"] = r(H * Dv, W, s=W ** -0.5)
            w[p + "mix.o"] = r(W, H * Dv, s=(H * Dv) ** -0.5)
        if ly["mlp"]:
            ff = ly["mlp"]["ff"]
            w[p + "norm2"] = r(W, s=0.2)
            w[p + "mlp.gate"] = r(ff, W, s=W ** -0.5)
            w[p + "mlp.up"] = r(ff, W, s=W ** -0.5)
            w[p + "mlp.down"] = r(W, ff, s=ff ** -0.5)
    return w


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def row_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest per-row RMS difference, relative to the RMS of the wanted rows."""
    got, want = got.double().cpu(), want.double().cpu()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()).max())


def bf16_close(got: torch.Tensor, want: torch.Tensor) -> bool:
    """bfloat16 engine against the float64 oracle: rows agree to rounding noise on average (a few per cent of the logits' RMS through
    several layers) and no single row is far off."""
    got, want = got.double().cpu(), want.double().cpu()
    e = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    return float(e.mean()) < 0.04 and float(e.max()) < 0.3
