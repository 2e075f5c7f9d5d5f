"""GPU tests of the hybrid decoders: the engine (model, cache / state manager, scheduler, kernels) against the plain float64 restatement in
tests/rizurax_oracle.py, on small random models of several shapes."""
import math

import pytest
import torch

from tests import rizurax_oracle as O
from tests.hybrid_util import bf16_close, attention_layer, delta_layer, make_config, make_weights, random_tokens, row_err

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4   # float32 engine vs float64 oracle


def _engine(cfg, w, dtype=torch.float32, max_tokens=1024, **kw):
    from qserve_b200.engine import Engine
    from qserve_b200.hybrid import HybridDecoder
    from qserve_b200.modelcfg import ARCHITECTURES

    model = HybridDecoder(ARCHITECTURES[cfg["architecture"]](cfg), w, dtype, torch.device("cuda:0"))
    return Engine(model, max_tokens=max_tokens, **kw)


def _whole(eng, sid, toks):
    out = eng.step([(sid, toks, list(range(len(toks))))])
    eng.release(sid)
    return out


MIXED = [attention_layer(), delta_layer(), attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=8, scaling=False, ff=0),
         delta_layer(heads=2, kv_heads=2, dim=24, vdim=16, conv=2)]


# ------------------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("bigram", [(53, 31, 5), (1, 3, 2), None])
def test_embedding_pair_table_and_final_norm(dev, bigram):
    cfg = make_config([], bigram=bigram)
    w = make_weights(cfg, 1)
    toks = random_tokens(40, cfg["vocab"], 1)
    got = _whole(_engine(cfg, w), "a", toks)
    assert row_err(got, O.forward(cfg, w, toks)) < F32_TOL


@pytest.mark.parametrize("layer", [
    attention_layer(ff=0), attention_layer(heads=3, kv_heads=1, dim=20, vdim=12, rot_dims=20, scaling=False, ff=0),
    attention_layer(heads=2, kv_heads=2, dim=64, vdim=160, rot_dims=32, ff=0), attention_layer(heads=1, kv_heads=1, dim=8, vdim=8, rot_dims=2, ff=0),
    delta_layer(ff=0), delta_layer(heads=2, kv_heads=2, dim=40, vdim=8, conv=1, ff=0), delta_layer(heads=6, kv_heads=1, dim=8, vdim=72, conv=7, ff=0),
    delta_layer(heads=1, kv_heads=1, dim=128, vdim=32, conv=3, ff=0),
], ids=lambda l: f"{l['type']}-{l['mixer']['heads']}x{l['mixer']['kv_heads']}x{l['mixer']['dim']}x{l['mixer']['vdim']}")
def test_single_mixer_layer(dev, layer):
    cfg = make_config([layer])
    w = make_weights(cfg, 2)
    toks = random_tokens(150, cfg["vocab"], 2)
    eng = _engine(cfg, w)
    taps = []
    got = eng.step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    assert row_err(taps[0], layers[0]) < F32_TOL
    assert row_err(got, want) < F32_TOL


def test_feed_forward_beside_mixer_and_loop(dev):
    cfg = make_config(MIXED, loop=(1, 3, 3))
    w = make_weights(cfg, 3)
    toks = random_tokens(90, cfg["vocab"], 3)
    taps = []
    got = _engine(cfg, w).step([("a", toks, list(range(len(toks))))], tap=lambda r, x: taps.append(x.clone()))
    want, layers = O.forward(cfg, w, toks, return_layers=True)
    assert len(taps) == layers.shape[0] == 8
    for r, t in enumerate(taps):
        assert row_err(t, layers[r]) < F32_TOL, f"layer run {r}"
    assert row_err(got, want) < F32_TOL


def test_bfloat16_engine_stays_within_rounding(dev):
    cfg = make_config(MIXED, loop=(0, 2, 2))
    w = make_weights(cfg, 4)
    toks = random_tokens(200, cfg["vocab"], 4)
    got = _whole(_engine(cfg, w, torch.bfloat16), "a", toks)
    assert bf16_close(got, O.forward(cfg, w, toks))


# ------------------------------------------------------------------------------------------------------------------------
# the same logits however the tokens are cut, batched and placed
# ------------------------------------------------------------------------------------------------------------------------
def _portions(eng, sid, toks, sizes):
    """Feed toks in portions of the given sizes (cycled), wanting every position."""
    outs, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - at)
        outs.append(eng.step([(sid, toks[at:at + n], list(range(n)))]))
        at, i = at + n, i + 1
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_then_token_by_token(dev, dtype):
    close = (lambda a, b: row_err(a, b) < F32_TOL) if dtype == torch.float32 else bf16_close
    cfg = make_config(MIXED, loop=(1, 3, 2))
    w = make_weights(cfg, 5)
    toks = random_tokens(200, cfg["vocab"], 5)
    want = O.forward(cfg, w, toks)
    eng = _engine(cfg, w, dtype)
    got = torch.cat([eng.step([("a", toks[:61], list(range(61)))]), _portions(eng, "a", toks[61:], [1])])
    assert close(got, want)
    eng.release("a")
    got = _portions(eng, "b", toks, [1])  # from the very first token on, one by one
    assert close(got, want)


@pytest.mark.parametrize("sizes", [[2], [3, 2, 64, 5], [63, 1, 65], [128, 7]])
def test_portions_of_a_prompt(dev, sizes):
    cfg = make_config(MIXED, loop=(1, 3, 2))
    w = make_weights(cfg, 6)
    toks = random_tokens(197, cfg["vocab"], 6)
    got = _portions(_engine(cfg, w), "a", toks, sizes)
    assert row_err(got, O.forward(cfg, w, toks)) < F32_TOL


# head sizes that the tensor-core attention kernels and the two-column scan take in bfloat16
FAST = [attention_layer(heads=8, kv_heads=2, dim=32, vdim=64, rot_dims=16), delta_layer(heads=4, kv_heads=2, dim=64, vdim=128, conv=3),
        attention_layer(heads=2, kv_heads=2, dim=16, vdim=32, rot_dims=8, ff=0), delta_layer(heads=2, kv_heads=1, dim=128, vdim=64, conv=2, ff=0)]


@pytest.mark.parametrize("dtype,layers", [(torch.float32, MIXED), (torch.bfloat16, FAST), (torch.float32, FAST)], ids=["f32", "bf16-fast", "f32-fast"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(dev, dtype, layers):
    """Four live sequences at most, a pool that cannot hold all requests at once: pages and slots are handed out again, portions of some
    requests run beside single tokens of others, and every position must equal the request run alone."""
    cfg = make_config(layers, loop=(1, 3, 2), width=64 if layers is FAST else 40)
    w = make_weights(cfg, 7)
    lens = [150, 70, 1, 33, 129, 64, 90]
    reqs = {f"r{i}": random_tokens(n, cfg["vocab"], 10 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, w, v) for k, v in reqs.items()}
    eng = _engine(cfg, w, dtype, max_tokens=6 * 64, max_seqs=4)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting, live = list(reqs), []
    sizes = [2, 17, 1, 64, 5, 1, 1, 40]
    step = 0
    while waiting or live:
        def pages(k):
            return -(-len(reqs[k]) // 64)
        while waiting and len(live) < 4 and sum(pages(k) for k in live) + pages(waiting[0]) <= 6:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for j, k in enumerate(live):
            if (step + j) % 5 == 4 and len(live) > 1:
                continue  # left out of this step
            room = len(reqs[k]) - at[k]
            n = min(sizes[(step + 3 * j) % len(sizes)], room)
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
        out = eng.step(entries)
        r = 0
        for k, t, _ in entries:
            got[k].append(out[r:r + len(t)])
            r += len(t)
            at[k] += len(t)
            if at[k] == len(reqs[k]):
                ends.append(k)
        for k in ends:
            eng.release(k)
            live.remove(k)
        step += 1
    assert eng.cache.free_pages() == 6 and len(eng.cache.slots) == 4
    for k in reqs:
        if dtype == torch.float32:
            assert row_err(torch.cat(got[k]), want[k]) < F32_TOL, k
        else:
            assert bf16_close(torch.cat(got[k]), want[k]), k
            alone = _whole(eng, "alone", reqs[k])  # the same kernels on the whole prompt: the batch changes nothing beyond rounding
            assert row_err(torch.cat(got[k]), alone) < 0.03, k


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_graph_replay_equals_eager_launches(dev, dtype):
    """Decode-only steps replay a CUDA graph captured per batch size; the logits are those of eager launches up to rounding (the vendor
    matrix products may pick another algorithm inside a capture), also when the batch size changes, a sequence ends and its slot and pages
    go to a new one."""
    cfg = make_config(MIXED, loop=(1, 3, 2))
    w = make_weights(cfg, 13)
    reqs = [random_tokens(n, cfg["vocab"], 30 + i) for i, n in enumerate([40, 90, 23, 70])]
    outs = []
    for graphs in (True, False):
        eng = _engine(cfg, w, dtype, max_tokens=5 * 64, max_seqs=3, use_graphs=graphs)
        got = []
        eng.step([(i, reqs[i][:20], []) for i in range(3)])
        for t in range(20, 23):
            got.append(eng.step([(i, reqs[i][t:t + 1], [0]) for i in range(3)]))
        eng.release(2)
        eng.step([(3, reqs[3][:50], [])])
        for t in range(23, 40):
            got.append(eng.step([(0, reqs[0][t:t + 1], [0]), (1, reqs[1][t:t + 1], [0]), (3, reqs[3][t + 27:t + 28], [0])]))
        eng.release(0)
        for t in range(40, 43):
            got.append(eng.step([(1, reqs[1][t:t + 1], []), (3, reqs[3][t + 27:t + 28], [0])]))
        assert bool(eng._graphs) == graphs
        outs.append(torch.cat(got))
    assert row_err(outs[0], outs[1]) < (1e-5 if dtype == torch.float32 else 2e-2)


def test_long_decoding(dev):
    cfg = make_config([delta_layer(conv=3), attention_layer()], loop=(0, 2, 2))
    w = make_weights(cfg, 8)
    toks = random_tokens(330, cfg["vocab"], 8)
    eng = _engine(cfg, w)
    eng.step([("a", toks[:10], [])])
    got = _portions(eng, "a", toks[10:], [1])
    assert row_err(got, O.forward(cfg, w, toks)[10:]) < F32_TOL


# ------------------------------------------------------------------------------------------------------------------------
# one key that matters: far back, at page borders, the first tokens -- in a prompt and when decoding
# ------------------------------------------------------------------------------------------------------------------------
def _needle_model(n_tokens, needle, dim=8, vdim=8):
    """One attention layer, one head, no rotation to speak of (base huge), identity-like projections: the stream carries q | k | v directly.
    The last token's query matches the key at `needle` with a large score on map 1; values are distinct per position."""
    H = G = 1
    width = 2 * dim * 2 + vdim
    layer = attention_layer(heads=H, kv_heads=G, dim=dim, vdim=vdim, rot_dims=2, scaling=False, diff=0.25, ff=0, base=1e30)
    cfg = make_config([layer], vocab=n_tokens + 1, width=width, bigram=None, eps=1e-6)
    w = make_weights(cfg, 9)
    eye = torch.eye(width)
    w["l0.mix.q"], w["l0.mix.k"], w["l0.mix.v"] = eye[: 2 * dim].clone(), eye[2 * dim: 4 * dim].clone(), eye[4 * dim:].clone()
    w["l0.norm1"] = torch.zeros(width)
    emb = torch.randn(n_tokens + 1, width, generator=torch.Generator().manual_seed(3)) * 0.1
    emb[:, 4 * dim:] = torch.randn(n_tokens + 1, vdim, generator=torch.Generator().manual_seed(4))
    emb[n_tokens, 2: dim] = 3.0           # the query of the last token (vocab id n_tokens), map 1, non-rotated dims
    emb[needle, 2 * dim + 2: 3 * dim] = 3.0  # the key of the needle (token id = its position)
    w["embed"] = emb.to(torch.bfloat16).float()
    toks = list(range(n_tokens - 1)) + [n_tokens]
    return cfg, w, toks


@pytest.mark.parametrize("needle", [0, 1, 63, 64, 127, 128, 129, 300, 510])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out(dev, needle, decode):
    n = 512
    cfg, w, toks = _needle_model(n, needle)
    want = O.forward(cfg, w, toks)[-1:]
    # the needle must matter: without it the oracle's answer moves by far more than the tolerance
    w2 = {k: v.clone() for k, v in w.items()}
    w2["embed"][needle, :] = w2["embed"][(needle + 1) % (n - 1), :]
    assert row_err(O.forward(cfg, w2, toks)[-1:], want) > 50 * F32_TOL
    eng = _engine(cfg, w)
    if decode:
        eng.step([("a", toks[:-1], [])])
        got = eng.step([("a", toks[-1:], [0])])
    else:
        got = eng.step([("a", toks, [n - 1])])
    assert row_err(got, want) < F32_TOL


@pytest.mark.parametrize("needle", [0, 63, 64, 128, 300, 510])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out_on_the_fast_kernels(dev, needle, decode):
    """The same in bfloat16 with head sizes the tensor-core prompt and single-token kernels take."""
    n = 512
    cfg, w, toks = _needle_model(n, needle, dim=16, vdim=32)
    want = O.forward(cfg, w, toks)[-1:]
    eng = _engine(cfg, w, torch.bfloat16)
    if decode:
        eng.step([("a", toks[:-1], [])])
        got = eng.step([("a", toks[-1:], [0])])
    else:
        eng.step([("a", toks[:100], [])])
        got = eng.step([("a", toks[100:], [n - 101])])
    assert row_err(got, want) < 0.05


@pytest.mark.parametrize("shape", [(4, 2, 2, 16, 32), (6, 3, 2, 48, 96), (8, 2, 2, 32, 64), (2, 1, 1, 64, 128), (3, 3, 2, 16, 256), (16, 1, 2, 16, 32)],
                         ids=lambda s: "H%d-G%d-maps%d-D%d-Dv%d" % s)
def test_fast_attention_kernels_match_the_plain_kernel(dev, shape):
    """Same bfloat16 inputs and cache through the tensor-core kernels and through the plain kernel: prompt portions with and
    without context, portions that end inside a page, short portions and single tokens in one batch."""
    from qserve_b200.hybrid import MultiMapAttentionMixer, StepBatch
    from qserve_b200.modelcfg import AttentionMixerConfig, RotaryConfig

    H, G, maps, D, Dv = shape
    m = AttentionMixerConfig(H, G, D, Dv, RotaryConfig(8, 100.0), D ** -0.5, maps=maps, diff=0.3 if maps == 2 else 0.0, head_norm=maps == 2)
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g)
    w = {"q": r(H * maps * D, 8), "k": r(G * maps * D, 8), "v": r(G * Dv, 8), "o": r(8, H * Dv)}
    for n in ("lq1", "lk1", "lq2", "lk2"):
        w[n] = r(D) * 0.3
    mixer = MultiMapAttentionMixer(m, w, 1e-5, torch.bfloat16, dev)
    pages, page = 40, 64
    kpool = torch.zeros(pages, page, G, maps * D, dtype=torch.bfloat16, device=dev)
    vpool = torch.zeros(pages, page, G, Dv, dtype=torch.bfloat16, device=dev)
    table = torch.randperm(pages, generator=g).to(torch.int32).view(4, 10).to(dev)
    # step 1: context; step 2: continuation of every sequence with another portion size
    steps = [[(0, 0, -1, [0] * 200), (1, 0, -1, [0] * 70), (2, 0, -1, [0] * 3), (3, 0, -1, [0] * 16)],
             [(0, 200, 0, [0] * 1), (1, 70, 0, [0] * 130), (2, 3, 0, [0] * 15), (3, 16, 0, [0] * 64)],
             [(0, 201, 0, [0] * 90), (1, 200, 0, [0] * 1), (2, 18, 0, [0] * 1), (3, 80, 0, [0] * 17)],
             # many short portions: the single-token kernel gives each block several key tiles, or none
             [(0, 291, 0, [0] * 15), (1, 201, 0, [0] * 15), (2, 19, 0, [0] * 15), (3, 97, 0, [0] * 15)],
             [(0, 306, 0, [0] * 1), (3, 112, 0, [0] * 1)]]
    for entries in steps:
        b = StepBatch.build(entries, table, dev)
        T = b.n_tokens
        proj = (r(T, mixer.in_features) * 1.5).to(torch.bfloat16).to(dev)
        outs = []
        for fast in (True, False):
            p2, out = proj.clone(), torch.zeros(T, H * Dv, dtype=torch.bfloat16, device=dev)
            scratch = torch.empty(mixer.scratch_floats(T), dtype=torch.float32, device=dev) if fast else None
            mixer.run(p2, out, b, {"k": kpool, "v": vpool}, page, scratch, 0, torch.cuda.current_stream().cuda_stream)
            outs.append(out.float())
        torch.cuda.synchronize()
        d = (outs[0] - outs[1]).abs()
        assert float(d.max()) <= 2.0 ** -6 * float(outs[1].abs().max()) and float(d.mean()) < 1e-3 * float(outs[1].abs().mean())


def test_delta_state_remembers_an_early_token(dev):
    """A recurrent layer with decay close to one: what the first token wrote is still read hundreds of tokens later."""
    cfg = make_config([delta_layer(heads=2, kv_heads=1, dim=16, vdim=16, conv=2, ff=0)])
    w = make_weights(cfg, 11)
    w["l0.mix.A_log"] = torch.full((2,), -9.0)
    toks = random_tokens(400, cfg["vocab"], 11)
    want = O.forward(cfg, w, toks)
    other = list(toks)
    other[0] = (toks[0] + 1) % cfg["vocab"]
    assert row_err(O.forward(cfg, w, other)[-1:], want[-1:]) > 20 * F32_TOL
    eng = _engine(cfg, w)
    eng.step([("a", toks[:5], [])])
    eng.step([("a", toks[5:399], [])])
    assert row_err(eng.step([("a", toks[399:], [0])]), want[-1:]) < F32_TOL


# ------------------------------------------------------------------------------------------------------------------------
# generation through the engine's own entry point and scheduler
# ------------------------------------------------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler(dev):
    cfg = make_config(MIXED, loop=(1, 3, 2))
    w = make_weights(cfg, 12)
    prompts = [random_tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate([5, 140, 33, 1, 70, 12])]
    from qserve_b200.engine import SamplingParams

    eng = _engine(cfg, w, max_tokens=7 * 64, max_seqs=3, max_batch_tokens=96, chunk=48)
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=8)] * len(prompts))
    assert eng.cache.free_pages() == 7 and len(eng.cache.slots) == 3
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        seq = list(p)
        for tok in o:  # every chosen token is the oracle's argmax (up to ties within rounding)
            lg = O.forward(cfg, w, seq)[-1]
            assert lg[tok] >= lg.max() - 1e-3 * lg.abs().max(), (len(p), len(seq))
            seq.append(tok)


def test_sampling_is_seeded_and_respects_top_k(dev):
    from qserve_b200.engine import SamplingParams, sample

    logits = torch.randn(5, 50, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    a = sample(logits, [SamplingParams(temperature=0.8, top_k=3, top_p=0.9)] * 5, g)
    g.manual_seed(1)
    b = sample(logits, [SamplingParams(temperature=0.8, top_k=3, top_p=0.9)] * 5, g)
    assert torch.equal(a, b)
    top3 = torch.topk(logits, 3).indices
    assert all(int(a[i]) in top3[i].tolist() for i in range(5))
    assert torch.equal(sample(logits, [SamplingParams()] * 5), logits.argmax(-1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff", [(40, 48), (37, 21), (256, 264), (1030, 12)])
def test_norm_and_activation_kernels_on_aligned_and_odd_rows(dev, dtype, width, ff):
    """The stream's norm (with the previous update added in place, one or two gains) and the gated activation, on widths that take the
    16-byte kernels and on widths that do not, against the formulas in float64."""
    from qserve_b200._lib import check, lib

    g = torch.Generator().manual_seed(width)
    T, dt = 7, 0 if dtype == torch.bfloat16 else 1
    s = torch.cuda.current_stream().cuda_stream
    x = torch.randn(T, width, generator=g).to(dev)
    add = torch.randn(T, width, generator=g).to(dtype).to(dev)
    w1, w2 = (torch.randn(width, generator=g) * 0.3).to(dev), (torch.randn(width, generator=g) * 0.3).to(dev)
    for use_add, two in ((True, True), (False, True), (True, False)):
        xs = x.clone()
        o1, o2 = torch.zeros(T, width, dtype=dtype, device=dev), torch.zeros(T, width, dtype=dtype, device=dev)
        check(lib.qs_hyb_rms_norm(o1.data_ptr(), o2.data_ptr() if two else None, xs.data_ptr(), add.data_ptr() if use_add else None, w1.data_ptr(),
                                  w2.data_ptr() if two else None, 1.0, 1e-5, T, width, dt, s))
        want_x = x.double() + (add.double() if use_add else 0.0)
        n = want_x / (want_x.pow(2).mean(-1, keepdim=True) + 1e-5).sqrt()
        tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8
        assert torch.allclose(xs.double(), want_x, atol=1e-6)
        assert row_err(o1, n * (1.0 + w1.double())) < tol
        if two:
            assert row_err(o2, n * (1.0 + w2.double())) < tol
    gu = (torch.randn(T, 2 * ff, generator=g) * 2.0).to(dtype).to(dev)
    for off in (0, 8, 3):  # the output lands at a column offset of a wider row, as in the concatenated input of the output projection
        out = torch.zeros(T, off + ff, dtype=dtype, device=dev)
        check(lib.qs_hyb_gelu_tanh_mul(out.data_ptr() + off * out.element_size(), out.stride(0), gu.data_ptr(), T, ff, dt, s))
        z, u = gu[:, :ff].double(), gu[:, ff:].double()
        want = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3))) * u
        assert row_err(out[:, off:], want) < (1e-5 if dtype == torch.float32 else 2.0 ** -8)
        assert float(out[:, :off].abs().sum()) == 0.0
