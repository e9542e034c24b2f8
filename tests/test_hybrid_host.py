"""Host-side pieces of the layered hybrid decoders (no GPU): configuration reader, model registry, state slots, portion
scheduling, and the plain oracle's own consistency."""
import json
import os
import struct
import types

import numpy as np
import pytest
import torch

from oracle import kinetar_plain as plain
from tests.hybrid_helpers import SMALL, attn_scan, delta, model_config


def _write_checkpoint(tmp_path, config, weights):
    hdr, blobs, off = {}, [], 0
    for k, v in weights.items():
        raw = v.view(torch.int16).numpy().tobytes()
        hdr[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    js = json.dumps(hdr).encode()
    with open(tmp_path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(js)) + js + b"".join(blobs))
    with open(tmp_path / "config.json", "w") as f:
        json.dump(config, f)


def test_config_reader_and_registry(tmp_path):
    from jacobiforcing_b200.hybrid_config import FF_NONE, FF_RELU2, HybridConfig, iter_safetensors
    from jacobiforcing_b200.registry import architecture_of, resolve
    w = plain.random_weights(SMALL, 0, low=5)
    _write_checkpoint(tmp_path, SMALL, w)
    assert architecture_of(str(tmp_path)) == "Kinetar"
    fam = resolve(str(tmp_path))
    assert fam.name == "hybrid" and fam.native_config
    hc = fam.load_config(str(tmp_path))
    assert isinstance(hc, HybridConfig) and hc.is_hybrid
    assert [s.mixer for s in hc.layers] == [0, 1, 0, 1]
    assert hc.layers[1].d_low_a == 5 and hc.layers[1].d_low_g == 5           # read from the tensor shapes
    assert hc.layers[3].ff_kind == FF_NONE and hc.layers[0].ff_kind == FF_RELU2 and hc.layers[0].ff == 72
    assert hc.layers[0].a_qt_every == 5 and abs(hc.layers[0].a_qt_coef - 0.4) < 1e-7
    assert hc.layers[2].s_state == 5 and hc.layers[2].s_dt_rank == 2 and hc.layers[2].s_conv == 4
    names = {n for n, _, _, _ in iter_safetensors(str(tmp_path / "model.safetensors"))}
    assert names == set(w)
    # the engine configuration takes the native description and relaxes the page-size rule for it
    from jacobiforcing_b200.config import Config
    c = Config(str(tmp_path), kvcache_block_size=64, num_kvcache_blocks=8, max_num_batched_tokens=128)
    assert c.hf_config.is_hybrid and c.hf_config.vocab == SMALL["vocab"]
    with pytest.raises(AssertionError):
        Config(str(tmp_path), kvcache_block_size=24)


def test_unknown_architecture_and_layer_type(tmp_path):
    from jacobiforcing_b200.hybrid_config import HybridConfig
    from jacobiforcing_b200.registry import resolve
    with open(tmp_path / "config.json", "w") as f:
        json.dump({"architecture": "Nonesuch"}, f)
    with pytest.raises(NotImplementedError):
        resolve(str(tmp_path))
    bad = model_config([attn_scan()])
    bad["layers"][0]["type"] = "mystery"
    with pytest.raises(NotImplementedError):
        HybridConfig.from_dict(bad, {})


def _sched(pages=8, page=16, slots=2, budget=32, max_seqs=4):
    from jacobiforcing_b200.engine.scheduler import Scheduler
    cfg = types.SimpleNamespace(max_num_seqs=max_seqs, max_num_batched_tokens=budget, eos=-1, num_kvcache_blocks=pages,
                                kvcache_block_size=page, num_state_slots=slots, hf_config=types.SimpleNamespace(is_hybrid=True))
    return Scheduler(cfg)


def _seq(n, max_tokens=4):
    from jacobiforcing_b200.engine.sequence import Sequence
    from jacobiforcing_b200.sampling_params import SamplingParams
    return Sequence(list(range(1, n + 1)), SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))


def test_state_slots_are_reused_and_owned():
    from jacobiforcing_b200.engine.state_manager import StateSlotManager
    sm = StateSlotManager(2)
    a, b, c = _seq(3), _seq(3), _seq(3)
    assert sm.allocate(a) == 0 and sm.allocate(b) == 1 and not sm.can_allocate()
    with pytest.raises(RuntimeError):
        sm.allocate(c)
    sm.deallocate(a)
    assert a.state_slot == -1 and sm.allocate(c) == 0
    assert sm.allocate(c) == 0                                       # idempotent for a live request


def test_portion_scheduling_chunks_prompts_beside_decoding():
    s = _sched(pages=8, page=16, slots=2, budget=32)
    assert not s.block_manager.enable_prefix_cache                   # pages of stateful models are never shared
    a, b, c = _seq(50, 3), _seq(10, 3), _seq(5, 3)
    for q in (a, b, c):
        s.add(q)
    p = s.schedule_portions()
    assert [(q.seq_id, n) for q, n in p] == [(a.seq_id, 32)]       # the budget cuts the first prompt
    s.postprocess_portions(p, [None])
    p = s.schedule_portions()
    assert [(q.seq_id, n) for q, n in p] == [(a.seq_id, 18), (b.seq_id, 10)]   # rest of a, all of b; c has no slot
    s.postprocess_portions(p, [7, 8])
    assert len(a) == 51 and len(b) == 11 and a.num_cached_tokens == 50
    p = s.schedule_portions()
    assert [(q.seq_id, n) for q, n in p] == [(a.seq_id, 1), (b.seq_id, 1)]
    s.postprocess_portions(p, [7, 8])
    p = s.schedule_portions()
    s.postprocess_portions(p, [7, 8])                                 # third token: both finish, slots and pages return
    assert a.is_finished and b.is_finished and len(s.state_manager.free_slots) == 2
    assert len(s.block_manager.free_block_ids) == 8
    p = s.schedule_portions()
    assert [(q.seq_id, n) for q, n in p] == [(c.seq_id, 5)] and c.state_slot in (0, 1)


def test_portion_scheduling_preempts_the_youngest_when_pages_run_out():
    s = _sched(pages=3, page=16, slots=2, budget=64)
    a, b = _seq(16, 40), _seq(15, 40)
    s.add(a)
    s.add(b)
    p = s.schedule_portions()
    assert [q.seq_id for q, _ in p] == [a.seq_id, b.seq_id]        # one page each, one page spare
    s.postprocess_portions(p, [3, 3])
    p = s.schedule_portions()                                         # a's 17th token takes the spare page
    assert [q.seq_id for q, _ in p] == [a.seq_id, b.seq_id]
    s.postprocess_portions(p, [3, 3])
    p = s.schedule_portions()                                         # b's 17th token needs a page that is not there
    assert [q.seq_id for q, _ in p] == [a.seq_id]
    assert b.state_slot == -1 and b.num_cached_tokens == 0 and s.waiting[0] is b


def test_oracle_mechanisms_agree_with_direct_formulas():
    """The plain oracle against closed forms on tiny inputs: convolution taps, sink share, scan and delta recurrences."""
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    w = torch.tensor([[10.0, 1.0]], dtype=torch.float64)
    assert plain.short_conv(u, w).flatten().tolist() == [1.0, 12.0, 23.0]
    pe = plain.sinusoid(torch.tensor([3]), 4)
    assert np.allclose(pe.numpy(), [[np.sin(3.0), np.cos(3.0), np.sin(0.03), np.cos(0.03)]])
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert np.allclose(plain.norm_one_plus(x, torch.tensor([0.0, 1.0], dtype=torch.float64), 0.0).numpy(),
                       [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])
    # one head, one token: the softmax is shared between the key itself and the sink
    c = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "q_temp": {"coef": 0.0, "every": 1}, "scale": 1.0}
    eye = torch.eye(2, dtype=torch.float64)
    p = {"q": eye, "k": eye, "q.conv": torch.ones(2, 1, dtype=torch.float64), "k.conv": torch.ones(2, 1, dtype=torch.float64),
         "sink": torch.tensor([0.5], dtype=torch.float64), "g": torch.zeros(2, 2, dtype=torch.float64), "o": eye}
    h = torch.tensor([[1.0, 2.0]], dtype=torch.float64)
    share = np.exp(5.0) / (np.exp(5.0) + np.exp(0.5))
    assert np.allclose(plain.sink_attention(h, p, c).numpy(), [[0.5 * share * 1.0, 0.5 * share * 2.0]])


def test_header_symbols_match_the_binding():
    import re
    from jacobiforcing_b200 import _hybrid_cabi
    src = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "jacobi_hybrid.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    declared = sorted(set(re.findall(r"\b(hy_[a-z_0-9]+)\s*\(", src)))
    assert declared == sorted(_hybrid_cabi.EXPORTS)
    import ctypes
    lib = ctypes.CDLL(_hybrid_cabi.build())
    for name in declared:
        assert hasattr(lib, name), f"{name} declared but not exported"


def test_no_cpu_fallback_for_the_hybrid_engine():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from jacobiforcing_b200.hybrid_config import HybridConfig
    from jacobiforcing_b200.hybrid_runtime import HybridRuntime
    w = plain.random_weights(SMALL, 0)
    hc = HybridConfig.from_dict(SMALL, {k: tuple(v.shape) for k, v in w.items()})
    with pytest.raises(RuntimeError, match="no CUDA device"):
        HybridRuntime(hc)
