"""CPU tests of the hybrid decoders' host side: config parsing and the architecture registry, the rotary frequency table, the page / slot
manager, the scheduler's batching, the safetensors reader, the command line."""
import json
import math
import os
import struct
import subprocess
import sys

import pytest
import torch

from tests import rizurax_oracle as O
from tests.hybrid_util import attention_layer, delta_layer, make_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_registry_parses_a_config_file(tmp_path):
    from qserve_b200.modelcfg import ARCHITECTURES, AttentionMixerConfig, DeltaMixerConfig, read_model_config

    cfg = make_config([attention_layer(), delta_layer(ff=0), attention_layer(scaling=False)], loop=(1, 3, 3))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = read_model_config(str(tmp_path))
    assert "Rizurax" in ARCHITECTURES and c.architecture == "Rizurax"
    assert c.schedule() == [0, 1, 2, 1, 2, 1, 2] == O.layer_schedule(cfg)
    assert isinstance(c.layers[0].mixer, AttentionMixerConfig) and c.layers[0].mixer.maps == 2 and c.layers[0].mixer.head_norm
    assert isinstance(c.layers[1].mixer, DeltaMixerConfig) and c.layers[1].mlp is None
    assert c.layers[2].mixer.rot.factor is None and c.pair_buckets == 53
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "nope"}))
    with pytest.raises(ValueError):
        read_model_config(str(tmp_path))


def test_no_loop_and_no_pair_table():
    from qserve_b200.modelcfg import parse_rizurax

    c = parse_rizurax(make_config([delta_layer(), attention_layer()], bigram=None))
    assert c.schedule() == [0, 1] and c.pair_buckets == 0


@pytest.mark.parametrize("rot", [{"dims": 24, "base": 20000.0, "scaling": {"factor": 2.0, "original": 512, "fast": 32.0, "slow": 1.0}},
                                 {"dims": 8, "base": 100.0, "scaling": {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 4.0}},
                                 {"dims": 64, "base": 1e6}])
def test_rotary_table_matches_the_oracle(rot):
    from qserve_b200.modelcfg import _parse_rot

    r = _parse_rot(rot)
    cos, sin = O.rotary_tables([1], rot)
    amp = r.amplitude()
    f = torch.tensor(r.inv_freq(), dtype=torch.float64)
    assert torch.allclose(torch.cos(f) * amp, cos[0], rtol=0, atol=1e-12) and torch.allclose(torch.sin(f) * amp, sin[0], rtol=0, atol=1e-12)
    assert amp == (1.0 if "scaling" not in rot else 0.1 * math.log(rot["scaling"]["factor"]) + 1.0)


def _cpu_cache(max_tokens=256, max_seqs=2):
    from qserve_b200.cache import HybridCache
    from qserve_b200.modelcfg import parse_rizurax

    cfg = parse_rizurax(make_config([attention_layer(), delta_layer()], loop=(0, 2, 2)))
    return HybridCache(cfg, torch.float32, torch.device("cpu"), max_tokens, max_seqs, page_size=64)


def test_cache_pages_and_slots_are_handed_out_again():
    from qserve_b200.cache import OutOfPages, OutOfSlots

    c = _cpu_cache()
    assert c.num_pages == 4 and len(c.runs) == 4 and "k" in c.runs[0] and "state" in c.runs[1]
    a = c.admit("a")
    c.reserve("a", 65)
    assert len(a.pages) == 2 and c.free_pages() == 2
    a.length = 65
    c.reserve("a", 63)   # fills the second page exactly
    assert len(a.pages) == 2
    b = c.admit("b")
    with pytest.raises(OutOfSlots):
        c.admit("c")
    c.reserve("b", 128)
    with pytest.raises(OutOfPages):
        c.reserve("a", 64)
    first = list(a.pages)
    c.release("a")
    d = c.admit("d")
    assert d.slot == a.slot
    c.reserve("d", 1)
    assert d.pages[0] in first
    assert c.block_table_host[d.slot, 0] == d.pages[0]
    c.release("b"), c.release("d")
    assert c.free_pages() == 4 and len(c.slots) == 2
    with pytest.raises(KeyError):
        c.release("d")


def test_scheduler_chunks_prompts_and_batches_decodes():
    from qserve_b200.engine import Request, Scheduler

    c = _cpu_cache(max_tokens=512, max_seqs=2)
    s = Scheduler(c, max_batch_tokens=100, chunk=64)
    reqs = [Request("x", list(range(150))), Request("y", list(range(10))), Request("z", list(range(5)))]
    for r in reqs:
        s.add(r)
    seen = []
    for _ in range(6):
        batch = s.schedule()
        seen.append([(r.id, len(t)) for r, t in batch])
        for r, t in batch:
            c.reserve(r.id, len(t))
            c.seqs[r.id].length += len(t)
            r.fed += len(t)
            if r.fed == len(r.prompt) + len(r.output):
                r.output.append(0)
                if len(r.output) == 2:
                    s.retire(r)
    assert seen[0] == [("x", 64), ("y", 10)]          # two slots: z waits
    assert seen[1] == [("x", 64), ("y", 1)]           # a prompt portion beside a decoded token
    assert seen[2][0] == ("x", 22) and ("z", 5) in seen[2]  # y retired, z admitted into its slot
    assert all(sum(n for _, n in b) <= 100 for b in seen)


def test_safetensors_reader(tmp_path):
    from qserve_b200.checkpoint import read_safetensors

    a = torch.randn(3, 5).to(torch.bfloat16)
    b = torch.arange(7, dtype=torch.int32)
    blobs = [a.view(torch.int16).numpy().tobytes(), b.numpy().tobytes()]
    header = {"__metadata__": {"x": "y"}, "a": {"dtype": "BF16", "shape": [3, 5], "data_offsets": [0, len(blobs[0])]},
              "b": {"dtype": "I32", "shape": [7], "data_offsets": [len(blobs[0]), len(blobs[0]) + len(blobs[1])]}}
    hj = json.dumps(header).encode()
    (tmp_path / "m.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    got = read_safetensors(str(tmp_path / "m.safetensors"))
    assert torch.equal(got["a"], a) and torch.equal(got["b"], b) and set(got) == {"a", "b"}


def test_trace_runner_is_an_executable_with_the_documented_flags():
    path = os.path.join(ROOT, "bin", "trace_run")
    assert os.access(path, os.X_OK)
    out = subprocess.run([sys.executable, path, "--help"], capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0
    for flag in ("--model", "--dtype", "--out", "--max-tokens"):
        assert flag in out.stdout
