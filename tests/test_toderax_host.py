"""CPU tests of the Toderax family's host side: config parsing through the architecture registry, cache / state storage per mixer, and the
float64 restatement's own mechanisms (chunk mask, sink, streams) on cases that can be worked out by hand."""
import json

import pytest
import torch

from tests import toderax_oracle as O
from tests.toderax_util import gate_layer, make_config, make_weights, moe, pair_layer


def test_registry_parses_a_config_file(tmp_path):
    from qserve_b200.modelcfg import (ARCHITECTURES, AttentionMixerConfig, GateRecurrenceMixerConfig, MoeConfig, ParallelMixerConfig,
                                      RetentionMixerConfig, read_model_config)

    cfg = make_config([gate_layer(mlp=None), pair_layer(chunk=40, rot_dims=6, mlp=moe(experts=5, top=2, ff=12, limit=0.5, shared_ff=0))],
                      streams=5, groups=3, embed_scale=7.5)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = read_model_config(str(tmp_path))
    assert "Toderax" in ARCHITECTURES and c.architecture == "Toderax" and c.block == "sequential"
    assert (c.streams, c.norm_groups, c.embed_scale, c.norm_offset) == (5, 3, 7.5, 0.0) and c.schedule() == [0, 1]
    g, p = c.layers[0].mixer, c.layers[1].mixer
    assert isinstance(g, GateRecurrenceMixerConfig) and c.layers[0].mlp is None
    assert isinstance(p, ParallelMixerConfig) and isinstance(p.left, AttentionMixerConfig) and isinstance(p.right, RetentionMixerConfig)
    assert p.left.chunk == 40 and p.left.rot is None and p.left.sink and p.left.qk_norm and p.left.bias and p.left.head_temp and p.left.maps == 1
    assert p.right.rot.dims == 6 and p.right.rot.layout == "half" and len(p.right.decay) == p.right.heads
    m = c.layers[1].mlp
    assert isinstance(m, MoeConfig) and (m.experts, m.top, m.ff, m.limit, m.shared_ff) == (5, 2, 12, 0.5, 0)


def test_plain_residual_and_no_mask_are_the_defaults():
    from qserve_b200.modelcfg import parse_toderax

    cfg = make_config([pair_layer(chunk=0)], streams=0, groups=1)
    del cfg["norm"]["groups"]
    c = parse_toderax(cfg)
    assert c.streams == 0 and c.norm_groups == 1 and c.layers[0].mixer.left.chunk == 0
    bad = make_config([pair_layer()])
    bad["layers"][0]["mixer"]["right"]["decay"] = [0.5]
    with pytest.raises(ValueError):
        parse_toderax(bad)


def test_cache_storage_per_mixer():
    from qserve_b200.cache import HybridCache
    from qserve_b200.modelcfg import parse_toderax

    c = parse_toderax(make_config([gate_layer(heads=2, dim=12, vdim=20), pair_layer(heads=4, kv_heads=2, dim=12, vdim=20, r_heads=3, r_dim=16, r_vdim=8)]))
    cache = HybridCache(c, torch.float32, torch.device("cpu"), max_tokens=200, max_seqs=3, page_size=64)
    assert cache.num_pages == 4 and tuple(cache.runs[0]["state"].shape) == (3, 2, 12, 20)
    assert tuple(cache.runs[1]["left"]["k"].shape) == (4, 64, 2, 12) and tuple(cache.runs[1]["left"]["v"].shape) == (4, 64, 2, 20)
    assert tuple(cache.runs[1]["right"]["state"].shape) == (3, 3, 16, 8) and cache.runs[1]["right"]["state"].dtype == torch.float32


def test_oracle_chunks_and_sink_by_hand():
    """With q = k (all scores equal within a chunk) the attention is a plain average over the visible keys, the sink counting as one more."""
    T, D, size = 7, 4, 3
    h = torch.eye(T, dtype=torch.float64)
    w = {"q": torch.zeros(D, T), "k": torch.zeros(D, T), "v": torch.eye(T), "q.b": torch.ones(D), "k.b": torch.ones(D), "v.b": torch.zeros(T),
         "temp": torch.tensor([1.0]), "sink": torch.tensor([4.0]), "o": torch.eye(T)}
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": T, "scale": 1.0, "mask": {"size": size}}
    out = O.chunk_sink_attention(h, w, m, 0.0)  # unit-RMS q and k: every score is D * scale = 4 = the sink
    for i in range(T):
        first = i - i % size
        want = torch.zeros(T, dtype=torch.float64)
        want[first:i + 1] = 1.0 / (i - first + 2)
        assert torch.allclose(out[i], want, atol=1e-12)


def test_oracle_streams_reduce_to_the_plain_residual():
    """One stream with coefficients 1 is the plain residual."""
    cfg = make_config([gate_layer(), pair_layer()], streams=1)
    w = make_weights(cfg, 1)
    for k in list(w):
        if ".hc" in k:
            w[k] = torch.ones_like(w[k])
    plain = dict(cfg)
    del plain["streams"]
    toks = list(range(30))
    assert torch.allclose(O.forward(cfg, w, toks), O.forward(plain, w, toks), atol=1e-10)
