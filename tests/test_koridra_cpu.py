"""What needs no GPU of the Koridra design: reading its configuration, the model description and its tensor
names, sizes taken from a checkpoint's shapes, the cache manager's handling of chunks and of mixers with two
needs, and the plain implementation against closed forms."""
import copy
import json
import os

import numpy as np
import pytest

import plain_koridra as plain
from tiny_koridra import CONFIGS, KOR_A, KOR_B
from tuff_b200.cache import CacheManager
from tuff_b200.config import ConfigError, config_from_dict
from tuff_b200.models.model import Model
from tuff_b200.parts.base import CompositeNeed, PagedKVNeed, StateNeed


def test_config_round_trip_and_description():
    for name, (raw, _) in CONFIGS.items():
        arch, cfg = config_from_dict(raw, name)
        assert arch.name == "Koridra" and cfg == arch.parse_config(arch.config_to_dict(cfg), name)
        assert len(cfg.layers) == len(raw["layers"]) and cfg.vocab == raw["vocab"]
    _, cfg = config_from_dict(KOR_A, "a")
    assert cfg.layers[2].ff is None and cfg.layers[0].mixer.left.chunk == 24 and cfg.layers[3].mixer.left.rot_scaling is None
    assert cfg.layers[0].mixer.right.gate_rank == 8 and cfg.layers[1].mixer.decay == (0.5, 0.9, 0.995)


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "decay"), [0.5], "decay"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mixer", "left", "vdim"), 16, "vdim"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 15, "dims"), (("layers", 1, "mlp", "kind"), "experts", "kind"),
    (("norm", "eps"), "x", "eps"), (("width",), None, "width"), (("layers",), [], "layers")])
def test_config_errors_name_the_key(path, value, word):
    raw = copy.deepcopy(KOR_A)
    node = raw
    for p in path[:-1]:
        node = node[p]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw, "cfg")
    assert word in str(e.value)


def test_model_description_and_tensor_names():
    arch, cfg = config_from_dict(KOR_A, "a")
    model = Model(arch.model_spec(cfg))
    exp = model.expected_tensors()
    assert exp["l0.mix.left.q.norm"].shape == (4 * 32,) and exp["l0.mix.left.k"].shape == (2 * 32, 80)
    assert exp["l0.mix.right.a1"].shape == (8, 80) and exp["l0.mix.right.a2.b"].shape == (2 * 24,)
    assert exp["l0.mix.right.norm"].shape == (40,) and exp["l1.mix.norm"].shape == (3 * 40,)
    assert "l2.norm2" not in exp and "l2.mlp.gate" not in exp and "l0.mix.left.v" not in exp
    assert exp["pos"].shape == (400, 80) and exp["head"].shape == (301, 80)
    needs = model.storage_needs()
    assert needs[0] == CompositeNeed((PagedKVNeed(2, 32, chunk=24), StateNeed((2, 40, 24))))
    assert needs[1] == StateNeed((3, 40, 16)) and model.replayable


def test_a_size_that_only_the_checkpoint_gives(tmp_path):
    """The inner width of a decay gate is read from the shape of the gate's first matrix."""
    import torch
    from tuff_b200.config.registry import load_config
    from tuff_b200.weights import write_safetensors
    raw = copy.deepcopy(KOR_B)
    del raw["layers"][2]["mixer"]["right"]["gate_rank"]
    with open(tmp_path / "config.json", "w") as f:
        json.dump(raw, f)
    write_safetensors(str(tmp_path / "model.safetensors"), [("l2.mix.right.a1", torch.zeros(7, 64, dtype=torch.bfloat16))])
    arch, cfg = load_config(str(tmp_path))
    assert cfg.layers[2].mixer.right.gate_rank == 7
    assert Model(arch.model_spec(cfg)).expected_tensors()["l2.mix.right.a2"].shape == (40, 7)


def test_pages_go_back_when_a_chunk_has_passed():
    need = CompositeNeed((PagedKVNeed(1, 8, chunk=10), StateNeed((2, 3))))
    cm = CacheManager([need, StateNeed((4,)), PagedKVNeed(1, 8)], page_size=4, max_tokens=64, max_requests=2)
    assert len(cm.groups) == 2 and len(list(cm.leaf_storages())) == 4
    rc = cm.open("a")
    held = []
    for n in (3, 6, 1, 1, 9, 1, 20):
        cm.reserve(rc, n)
        cm.commit(rc, n)
        cm.check()
        first = rc.n_tokens // 10 * 10                 # the next token's chunk starts here
        table = rc.tables[0]
        assert all((p == -1) == ((b + 1) * 4 <= first) for b, p in enumerate(table)), (rc.n_tokens, table)
        assert all(p != -1 for p in rc.tables[1])       # the group without a chunk keeps everything
        held.append(cm.groups[0].pool.n_held)
    assert max(held) <= 10 // 4 + 2 + 20 // 4
    cm.close(rc)
    cm.check()
    assert cm.groups[0].pool.n_held == 0 and cm.slots.n_held == 0


def test_plain_recurrence_against_its_closed_form():
    rng = np.random.default_rng(0)
    T, H, dk, dv = 12, 2, 3, 4
    q, k, v = rng.normal(size=(T, H, dk)), rng.normal(size=(T, H, dk)), rng.normal(size=(T, H, dv))
    a = rng.uniform(0.3, 1.0, size=(T, H, dk))
    o = plain.decaying_state_scan(q, k, v, a)
    for t in (0, 5, 11):
        ref = np.zeros((H, dv))
        for s in range(t + 1):
            w = np.prod(a[s + 1:t + 1], axis=0)        # decays applied after token s entered
            ref += np.einsum("hk,hk,hv->hv", q[t] * w, k[s], v[s])
        assert np.abs(o[t] - ref).max() < 1e-12


def test_plain_mask_sink_and_rotation():
    ok = plain.chunk_mask(7, 3)
    assert ok[2, 0] and not ok[3, 2] and ok[5, 3] and not ok[5, 6] and plain.chunk_mask(4, None)[3, 0]
    p = plain.sink_softmax(np.zeros((1, 4)), np.array([[True, True, False, False]]))
    assert np.allclose(p, [[1 / 3, 1 / 3, 0, 0]])
    f, amp = plain.yarn_frequencies(8, 100.0, None)
    assert np.allclose(f, 100.0 ** (-np.arange(4) / 4)) and amp == 1.0
    x = np.zeros((1, 1, 6)); x[0, 0, 0] = 1.0; x[0, 0, 5] = 7.0
    y = plain.rotate_interleaved(x, [1], 4, np.array([np.pi / 2, 0.3]), 2.0)
    assert np.allclose(y[0, 0], [0, 2.0, 0, 0, 0, 7.0])
    f2, amp2 = plain.yarn_frequencies(8, 100.0, dict(factor=4.0, original=16, fast=4.0, slow=1.0))
    assert abs(amp2 - (0.1 * np.log(4.0) + 1)) < 1e-12 and f2[0] == f[0] and np.isclose(f2[-1], f[-1] / 4.0)
