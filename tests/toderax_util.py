"""Helpers of the Toderax tests: small random models (config dict + weights under the design's tensor names)."""
import math

import torch


def moe(experts=6, top=2, ff=24, limit=1.5, shared_ff=20, shared_limit=0.75):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return m


def gate_layer(heads=2, dim=12, vdim=20, mlp="default"):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": moe() if mlp == "default" else mlp}


def pair_layer(heads=4, kv_heads=2, dim=12, vdim=20, chunk=24, scale=None, r_heads=3, r_dim=16, r_vdim=8, rot_dims=8, base=500.0, decay=None,
               mlp="default"):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if chunk:
        left["mask"] = {"size": chunk}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "rot": {"dims": rot_dims, "base": base},
             "decay": list(decay) if decay is not None else [1.0 - 2.0 ** (-3 - i) for i in range(r_heads)]}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": moe() if mlp == "default" else mlp}


def make_config(layers, vocab=89, width=48, streams=3, groups=2, eps=1e-5, embed_scale=3.0):
    cfg = {"architecture": "Toderax", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "embedding": {"scale": embed_scale},
           "layers": layers}
    if streams:
        cfg["streams"] = streams
    return cfg


def make_weights(cfg, seed=0):
    """Random weights, rounded to bfloat16 values (held as float32) so that every dtype sees the same numbers."""
    g = torch.Generator().manual_seed(seed)
    W, ns = cfg["width"], cfg.get("streams", 0)
    bf = lambda t: t.to(torch.bfloat16).to(torch.float32)
    r = lambda *shape, s=1.0: bf(torch.randn(*shape, generator=g) * s)
    w = {"embed": r(cfg["vocab"], W, s=0.5), "head": r(cfg["vocab"], W, s=W ** -0.5), "final.norm": 1.0 + r(W, s=0.2)}

    def experts(p, spec):
        names = [f"e{e}" for e in range(spec["router"]["experts"])] + (["shared"] if spec.get("shared") else [])
        for n in names:
            ff = spec["shared"]["ff"] if n == "shared" else spec["expert"]["ff"]
            w[f"{p}{n}.gate"], w[f"{p}{n}.up"], w[f"{p}{n}.down"] = r(ff, W, s=2.0 * W ** -0.5), r(ff, W, s=2.0 * W ** -0.5), r(W, ff, s=ff ** -0.5)
        w[p + "router"] = r(spec["router"]["experts"], W, s=2.0 * W ** -0.5)

    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        w[p + "norm1"] = 1.0 + r(W, s=0.2)
        for q in (1, 2):
            if ns and (q == 1 or ly["mlp"]):
                w[f"{p}hc{q}.in"] = bf(1.0 / ns + torch.randn(ns, generator=g) * 0.2)
                w[f"{p}hc{q}.out"] = bf(1.0 + torch.randn(ns, generator=g) * 0.3)
                w[f"{p}hc{q}.mix"] = bf(torch.eye(ns) + torch.randn(ns, ns, generator=g) * 0.15)
        if ly["type"] == "hgrn2":
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.f"], w[p + "mix.v"] = r(H * D, W, s=W ** -0.5), r(H * D, W, s=2.0 * W ** -0.5), r(H * Dv, W, s=W ** -0.5)
            w[p + "mix.f.b"] = r(H * D, s=1.0)
            w[p + "mix.lower"] = bf(torch.sigmoid(torch.randn(H * D, generator=g) * 2.0))
            w[p + "mix.norm"] = 1.0 + r(Dv, s=0.2)
            w[p + "mix.o"] = r(W, H * Dv, s=(H * Dv) ** -0.5)
        else:
            a, b = m["left"], m["right"]
            H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            pl, pr = p + "mix.left.", p + "mix.right."
            w[pl + "q"], w[pl + "k"], w[pl + "v"] = r(H * D, W, s=W ** -0.5), r(G * D, W, s=W ** -0.5), r(G * Dv, W, s=W ** -0.5)
            w[pl + "q.b"], w[pl + "k.b"], w[pl + "v.b"] = r(H * D, s=0.3), r(G * D, s=0.3), r(G * Dv, s=0.3)
            w[pl + "temp"] = bf(2.0 + torch.rand(H, generator=g) * 3.0)   # sharp maps: a key that is wrongly seen or missed moves the output
            w[pl + "sink"] = r(H, s=1.0) + 1.0
            w[pl + "o"] = r(W, H * Dv, s=(H * Dv) ** -0.5)
            Hr, Dr, Dvr = b["heads"], b["dim"], b["vdim"]
            w[pr + "q"], w[pr + "k"], w[pr + "v"], w[pr + "g"] = (r(Hr * Dr, W, s=W ** -0.5), r(Hr * Dr, W, s=W ** -0.5), r(Hr * Dvr, W, s=W ** -0.5),
                                                                    r(Hr * Dvr, W, s=W ** -0.5))
            w[pr + "o"] = r(W, Hr * Dvr, s=(Hr * Dvr) ** -0.5)
            w[p + "mix.left.out"], w[p + "mix.right.out"] = 1.0 + r(W, s=0.2), 1.0 + r(W, s=0.2)
        if ly["mlp"]:
            w[p + "norm2"] = 1.0 + r(W, s=0.2)
            experts(p + "mlp.", ly["mlp"])
    return w
