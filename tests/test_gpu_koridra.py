"""Koridra on the GPU against the plain implementation (tests/plain_koridra.py): every mechanism alone,
whole models replayed in four ways, pages and slots used again, edges of chunks and pages, long
decoding, and generation through the engine's own entry point."""
import io
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_koridra as plain
import traces
from test_gpu_parts import DT, bind_random, dev, f64, make_ctx, run_part_in_portions
from tiny import random_tokens
from tiny_koridra import CONFIGS, make_folder
from tuff_b200.cache import CacheManager

pytestmark = pytest.mark.gpu

# Root mean square of the difference of a logits row (mean taken off) over that of the row itself.
ROW_TOL = {"float32": 2e-4, "bfloat16": 6e-2}
LENGTHS = {"kor_a": (70, 45, 97, 130, 66), "kor_b": (83, 40, 129, 65, 100), "kor_c": (150, 64, 37, 200, 129),
           "kor_d": (120, 51, 33, 160, 101)}
PAGE = {"kor_a": 16, "kor_b": 4, "kor_c": 64, "kor_d": 16}


def row_error(got, ref):
    d = got - ref
    d = d - d.mean()
    return float(np.sqrt((d * d).mean()) / max(1e-9, np.sqrt(((ref - ref.mean()) ** 2).mean())))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("koridra")
    out = {}
    for name in CONFIGS:
        folder = make_folder(base, name)
        vocab = CONFIGS[name][0]["vocab"]
        reqs = {f"r{i}": random_tokens(vocab, n, 10 * i + len(name)) for i, n in enumerate(LENGTHS[name])}
        p = plain.PlainKoridra(folder)
        out[name] = (folder, reqs, {rid: p.forward(t) for rid, t in reqs.items()})
    return out


def run_trace(folder, dtype, steps, tmp_path, page_size, max_tokens=None):
    from tuff_b200.engine.replay import replay
    from tuff_b200.engine.runner import ModelRunner
    n = max_tokens or traces.tokens_needed(steps, round_to=max(64, page_size))
    runner = ModelRunner(folder, dtype=dtype, max_tokens=n, page_size=page_size, max_requests=4)
    runner.cache.owners = {}
    log = io.StringIO()
    replay(runner, io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), str(tmp_path), report=log)
    assert log.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
    runner.cache.check()
    assert not runner.cache.live
    return runner


def logits_by_place(out_dir, wanted, vocab):
    out = {}
    for step, rows in wanted.items():
        got = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for i, place in enumerate(rows):
            out[place] = got[i].copy()
    return out


def compare(out_dir, wanted, expect, vocab, dtype, what):
    for (rid, pos), got in logits_by_place(out_dir, wanted, vocab).items():
        err = row_error(got, expect[rid][pos])
        assert err <= ROW_TOL[dtype], f"{what} {dtype}: request {rid} position {pos}: error {err:.3g}"


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("mode", ["whole", "tail_decoded", "portions", "mixed"])
def test_replay_modes(models, tmp_path, name, dtype, mode):
    folder, reqs, expect = models[name]
    steps, wanted = getattr(traces, mode)(reqs)
    runner = run_trace(folder, dtype, steps, tmp_path, PAGE[name])
    compare(str(tmp_path), wanted, expect, CONFIGS[name][0]["vocab"], dtype, f"{name} {mode}")
    if mode == "mixed":
        reused = [k for k, who in runner.cache.owners.items() if len(set(who)) > 1]
        assert len(reused) >= 1, runner.cache.owners


@pytest.mark.parametrize("name", list(CONFIGS))
def test_float32_logits_do_not_depend_on_the_cut(models, tmp_path, name):
    """Every sum of the 32-bit path runs in an order that the sizes alone decide: a (request, position) has
    the same logits, bit for bit, whole, with its tail decoded, in portions, and mixed with others."""
    folder, reqs, _ = models[name]
    vocab = CONFIGS[name][0]["vocab"]
    seen = None
    for mode in ("whole", "tail_decoded", "portions", "mixed"):
        steps, wanted = getattr(traces, mode)(reqs)
        out = tmp_path / mode
        run_trace(folder, "float32", steps, out, PAGE[name])
        got = logits_by_place(str(out), wanted, vocab)
        if seen is None:
            seen = got
        else:
            for place, row in got.items():
                assert np.array_equal(row, seen[place]), (mode, place, np.abs(row - seen[place]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_one_by_one(models, dtype):
    """The stream after every layer, against the plain implementation's."""
    from tuff_b200.engine.batch import StepEntry, layout_entries, to_device
    from tuff_b200.engine.runner import ModelRunner
    folder, reqs, _ = models["kor_a"]
    toks = reqs["r1"]
    ref = []
    plain.PlainKoridra(folder).forward(toks, ref)
    runner = ModelRunner(folder, dtype=dtype, max_tokens=128, page_size=8, max_requests=2)
    rc = runner.open("x")
    runner.cache.reserve(rc, len(toks))
    ctx = to_device(layout_entries([StepEntry(rc, toks, [])], runner.cache), runner.device, runner.dtype)
    m = runner.model
    x = m.embedding.forward(ctx)
    for i, e in enumerate(m.schedule):
        layer = m.layers[e.layer]
        layer.block.forward(ctx, x, layer, runner.cache.storages[e.storage], False)
        err = np.abs(f64(x) - ref[i]).max()
        assert err <= (2e-5 if dtype == "float32" else 6e-2) * (i + 1), (i, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_entry_point(models, name, dtype):
    from tuff_b200 import Engine, SamplingParams
    folder = models[name][0]
    vocab = CONFIGS[name][0]["vocab"]
    prompts = [random_tokens(vocab, n, 40 + n) for n in (7, 13, 1, 30, 5)]
    eng = Engine(folder, dtype=dtype, ctx_size=128, max_tokens=256, page_size=8, max_batched_tokens=16, max_running=3)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    assert [len(o) for o in outs] == [12] * 5
    p = plain.PlainKoridra(folder)
    margin = 1e-3 if dtype == "float32" else 0.25
    for prompt, out in zip(prompts, outs):
        ref = p.forward(prompt + out)
        for i, tok in enumerate(out):
            row = ref[len(prompt) + i - 1]
            assert row.max() - row[tok] <= margin, (i, tok, int(row.argmax()), row.max() - row[tok])
    eng.runner.cache.check()
    assert not eng.runner.cache.live
    if dtype == "bfloat16":
        assert eng.runner.graph_replays > 0          # pure decode steps ran as captured graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_chunks(models, tmp_path, dtype):
    """A short prompt, then 250 tokens one by one: the chunk of the softmax branch ends ten times, its pages
    go back to the pool while the request lives, and the states run on."""
    folder = models["kor_a"][0]
    vocab = CONFIGS["kor_a"][0]["vocab"]
    toks = random_tokens(vocab, 253, 5)
    steps, wanted = traces.tail_decoded({"long": toks}, tail=250)
    # chunks of 24 and 40 positions: a request never holds more than 40 + a page of keys
    runner = run_trace(folder, dtype, steps, tmp_path, page_size=8, max_tokens=64)
    compare(str(tmp_path), wanted, {"long": plain.PlainKoridra(folder).forward(toks)}, vocab, dtype, "long decoding")
    assert max(len(set(who)) for who in runner.cache.owners.values()) == 1
    assert sum(len(who) for who in runner.cache.owners.values()) > 2 * 8      # the same pages, handed out again


def test_first_tokens_and_single_token_requests(models, tmp_path):
    folder, _, _ = models["kor_b"]
    vocab = CONFIGS["kor_b"][0]["vocab"]
    reqs = {"one": random_tokens(vocab, 1, 1), "two": random_tokens(vocab, 2, 2), "three": random_tokens(vocab, 3, 3)}
    expect = {rid: plain.PlainKoridra(folder).forward(t) for rid, t in reqs.items()}
    for mode in ("whole", "portions"):
        steps, wanted = getattr(traces, mode)(reqs, *(((1, 1, 1),) if mode == "portions" else ()))
        run_trace(folder, "float32", steps, tmp_path / mode, 4)
        compare(str(tmp_path / mode), wanted, expect, vocab, "float32", f"first tokens {mode}")


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv", [(3, 16, 40), (2, 80, 24), (1, 130, 33), (4, 64, 64)])
def test_lightning_attention_part(dtype, H, dk, dv):
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(H + dk)
    d, eps = 72, 1e-5
    m = dict(heads=H, dim=dk, vdim=dv, decay=list(np.linspace(0.6, 0.999, H)))
    part = MIXERS.build(PartSpec("lightning_attention", dict(d_model=d, norm_eps=eps, **m)))
    w = bind_random(part, dtype, rng, std=0.15)
    cm = CacheManager([part.cache_need()], page_size=4, max_tokens=64, max_requests=3, dtype=DT[dtype], device="cuda:0")
    hs = [f64(dev(rng.normal(size=(n, d)), DT[dtype])) for n in (45, 6, 19)]
    got = run_part_in_portions(part, cm, cm.storages[0], dtype, hs, cuts=(1, 5, 2, 17, 1, 1, 8))
    for g, h in zip(got, hs):
        ref = plain.lightning_mixer(h, w, m, eps)
        assert np.abs(g - ref).max() <= (3e-5 if dtype == "float32" else 4e-2) * max(1, np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv,tau,rank", [(2, 24, 40, 4.0, 8), (3, 16, 16, 1.0, 5), (1, 72, 96, 16.0, 16)])
def test_gated_linear_attention_part(dtype, H, dk, dv, tau, rank):
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(H + dk)
    d, eps = 64, 0.02          # an eps of the size of the read-out's mean square: the scale of q shows through the norm
    m = dict(heads=H, dim=dk, vdim=dv, tau=tau)
    part = MIXERS.build(PartSpec("gated_linear_attention", dict(d_model=d, norm_eps=eps, gate_rank=rank, out_scale=1.3, **m)))
    w = bind_random(part, dtype, rng, std=0.3)
    w["a2.b"] = w.pop("a2_bias")
    cm = CacheManager([part.cache_need()], page_size=4, max_tokens=64, max_requests=3, dtype=DT[dtype], device="cuda:0")
    hs = [f64(dev(rng.normal(size=(n, d)), DT[dtype])) for n in (37, 3, 22)]
    got = run_part_in_portions(part, cm, cm.storages[0], dtype, hs, cuts=(2, 1, 9, 1, 1, 16, 3))
    for g, h in zip(got, hs):
        ref = 1.3 * plain.gated_linear_branch(h, w, m, eps)
        assert np.abs(g - ref).max() <= (3e-5 if dtype == "float32" else 4e-2) * max(1, np.abs(ref).max())


def test_a_far_token_stays_in_the_state():
    """One key and value 300 tokens back, a hundred times larger than the rest, and a query that asks for it
    at the end: what is read out is that value times decay^300, carried through portions of all sizes."""
    from tuff_b200.kernels import ops
    H, dk, dv, T = 2, 32, 48, 320
    rng = np.random.default_rng(3)
    q, k, v = (0.01 * rng.normal(size=(T, H * d)) for d in (dk, dk, dv))
    k[7, :dk] = 0.0; k[7, 5] = 100.0
    v[7, :dv] = np.arange(dv) + 1.0
    q[T - 1, :dk] = 0.0; q[T - 1, 5] = 1.0
    decay = np.array([0.99, 0.5])
    ref = plain.decaying_state_scan(q.reshape(T, H, dk), k.reshape(T, H, dk), v.reshape(T, H, dv), decay[None, :, None])
    assert abs(ref[T - 1, 0, 3] - 100.0 * 4.0 * 0.99 ** (T - 8)) < 0.05 * abs(ref[T - 1, 0, 3])     # the test shows what it says
    state = torch.zeros(3, H, dv, dk, device="cuda")
    out = torch.empty(T, H * dv, device="cuda")
    cuts, p = [5, 2, 1, 33, 64, 2, 100, 17, 1, 95], 0
    for n in cuts:
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        ops.linear_attention(dev(q[p:p + n]), dev(k[p:p + n]), dev(v[p:p + n]), state, torch.tensor([1], dtype=torch.int32, device="cuda"),
                             cu, out[p:p + n], H, dk, dv, head_decay=dev(decay))
        p += n
    assert p == T
    assert np.abs(f64(out).reshape(T, H, dv) - ref).max() <= 1e-4 * np.abs(ref).max()
    assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0      # other slots untouched


def test_a_state_slot_is_clean_when_it_is_used_again():
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(4)
    d = 48
    part = MIXERS.build(PartSpec("lightning_attention", dict(d_model=d, heads=2, dim=16, vdim=24, decay=[1.0, 0.9], norm_eps=1e-5)))
    bind_random(part, "float32", rng, std=0.3)
    cm = CacheManager([part.cache_need()], page_size=4, max_tokens=64, max_requests=1, dtype=torch.float32, device="cuda:0")
    h = f64(dev(rng.normal(size=(9, d))))
    first = run_part_in_portions(part, cm, cm.storages[0], "float32", [10.0 * h], cuts=(9,))[0]
    again = run_part_in_portions(part, cm, cm.storages[0], "float32", [h], cuts=(4, 5))[0]          # the only slot, used again
    fresh = CacheManager([part.cache_need()], page_size=4, max_tokens=64, max_requests=1, dtype=torch.float32, device="cuda:0")
    clean = run_part_in_portions(part, fresh, fresh.storages[0], "float32", [h], cuts=(9,))[0]
    assert np.array_equal(again, clean) and not np.allclose(first, clean)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,page,chunk,rot,yarn", [(4, 2, 32, 4, 24, 16, True), (2, 2, 48, 8, 40, 48, False),
                                                        (6, 1, 16, 16, 17, 0, False), (4, 2, 64, 8, 96, 32, True),
                                                        (3, 3, 20, 4, None, 10, True)])
def test_keys_as_values_attention_part(dtype, H, G, hd, page, chunk, rot, yarn):
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(H + hd)
    d, eps = 64, 1e-5
    scaling = dict(factor=4.0, original=64, fast=16.0, slow=2.0) if yarn else None
    pos = PartSpec("rope_yarn", dict(head_dim=hd, theta=1000.0, rotary_dim=rot, pairing="interleaved", **(scaling or {}))) if rot else None
    part = MIXERS.build(PartSpec("gqa_attention", dict(
        d_model=d, num_heads=H, num_kv_heads=G, head_dim=hd, qk_norm_eps=eps, qk_norm_span="projection", values="keys",
        position_encoding=pos, scale=0.3, chunk=chunk, sink=0.0, out_scale=0.7)))
    w = bind_random(part, dtype, rng, std=0.3)
    m = dict(heads=H, kv_heads=G, dim=hd, scale=0.3, mask=dict(size=chunk) if chunk else None,
             rot=dict(dims=rot, base=1000.0, scaling=scaling))
    cm = CacheManager([part.cache_need()], page_size=page, max_tokens=256, max_requests=3, dtype=DT[dtype], device="cuda:0")
    hs = [f64(dev(rng.normal(size=(n, d)), DT[dtype])) for n in (101, 6, 50)]
    got = run_part_in_portions(part, cm, cm.storages[0], dtype, hs, cuts=(3, 1, 7, 2, 1, 30))
    for g, h in zip(got, hs):
        ref = 0.7 * plain.keys_as_values_attention(h, w["q_proj"], w["k_proj"], w["out_proj"], w["q_layernorm"],
                                                   w["k_layernorm"], m, eps)
        assert np.abs(g - ref).max() <= (3e-5 if dtype == "float32" else 4e-2) * max(1, np.abs(ref).max())
    cm.check()


@pytest.mark.parametrize("mode", ["portion", "decoded"])
@pytest.mark.parametrize("page", [4, 16])
def test_one_key_stands_out_at_the_edges_of_a_chunk(mode, page):
    """One key with a score far above all others: a query whose chunk holds it returns that key's value almost
    alone, the next chunk's first query does not see it.  Keys at the chunk's first and last place, at page
    borders, and hundreds of places back in a wide chunk."""
    from tuff_b200.kernels import ops
    H, G, hd, T = 2, 1, 32, 260
    rng = np.random.default_rng(7)
    for chunk, key_at in ((48, 48), (48, 95), (200, 3), (0, 1), (64, 63), (64, 64)):
        k = 0.1 * rng.normal(size=(T, G * hd))
        v = rng.normal(size=(T, G * hd))
        q = 0.1 * rng.normal(size=(T, H * hd))
        k[key_at] = 0.0; k[key_at, 0] = 30.0
        q[:, 0] = 1.0; q[:, hd] = 1.0                       # every query of both heads asks for it
        kp = torch.zeros(T // page + 1, G, page, hd, device="cuda")
        vp = torch.zeros_like(kp)
        table = torch.arange(T // page + 1, dtype=torch.int32, device="cuda").flip(0).reshape(1, -1).contiguous()
        pages = table[0].long()
        for t in range(T):
            kp[pages[t // page], 0, t % page] = dev(k[t]); vp[pages[t // page], 0, t % page] = dev(v[t])
        positions = torch.arange(T, dtype=torch.int32, device="cuda")
        rows = torch.zeros(T, dtype=torch.int32, device="cuda")
        out = torch.empty(T, H * hd, device="cuda")
        if mode == "portion":
            ops.paged_attention(dev(q), kp, vp, table, positions, rows, out, H, G, hd, 1.0, chunk=chunk, sink=0.0,
                                cu_q=torch.tensor([0, T], dtype=torch.int32, device="cuda"), all_single=False, max_seq_len=T)
        else:
            for t in range(T):
                ops.paged_attention(dev(q[t:t + 1]), kp, vp, table, positions[t:t + 1], rows[:1], out[t:t + 1], H, G, hd, 1.0,
                                    chunk=chunk, sink=0.0, cu_q=None, all_single=True, max_seq_len=T)
        ref = np.zeros((T, H, hd))
        ok = plain.chunk_mask(T, chunk)
        for a in range(H):
            ref[:, a] = plain.sink_softmax(q[:, a * hd:(a + 1) * hd] @ k.T, ok) @ v
        got = f64(out).reshape(T, H, hd)
        assert np.abs(got - ref).max() <= 2e-4, (chunk, key_at, np.abs(got - ref).max())
        last_in = T - 1 if not chunk else min(T - 1, (key_at // chunk + 1) * chunk - 1)
        assert np.abs(got[last_in, 0] - v[key_at]).max() < 1e-3                       # seen at the chunk's last place
        if last_in + 1 < T:
            assert np.abs(got[last_in + 1, 0] - v[key_at]).max() > 0.1                # and not one place later
        if key_at > 0:
            assert np.abs(got[key_at - 1, 0] - v[key_at]).max() > 0.1                 # nor before it exists


@pytest.mark.parametrize("hd,page", [(64, 16), (64, 64), (128, 8), (128, 64)])
def test_chunk_edges_and_sink_in_the_tensor_core_kernels(hd, page):
    """The same question put to the bf16 kernels (tcgen05 for portions of head size 64, TMA + mma.sync for head size
    128 and for single tokens, sliced over the keys): portions of 128 and of 7 tokens and tokens one by one."""
    from tuff_b200.kernels import ops
    H, G, T = 4, 2, 300
    rng = np.random.default_rng(hd + page)
    bf = torch.bfloat16
    for chunk, key_at in ((96, 96), (96, 191), (250, 5), (0, 2), (64, 63)):
        k = f64(dev(0.1 * rng.normal(size=(T, G * hd)), bf)); v = f64(dev(rng.normal(size=(T, G * hd)), bf))
        q = f64(dev(0.1 * rng.normal(size=(T, H * hd)), bf))
        k[key_at, :hd] = 0.0; k[key_at, 0] = 30.0
        q[:, 0] = 1.0; q[:, hd] = 1.0                        # the two heads of group 0 ask for it
        n_pages = (T + page - 1) // page
        kp = torch.zeros(n_pages + 1, G, page, hd, device="cuda", dtype=bf); vp = torch.zeros_like(kp)
        table = torch.arange(n_pages, dtype=torch.int32, device="cuda").flip(0).reshape(1, -1).contiguous()
        pages = table[0].long()
        for t in range(T):
            kp[pages[t // page], :, t % page] = dev(k[t], bf).view(G, hd); vp[pages[t // page], :, t % page] = dev(v[t], bf).view(G, hd)
        positions = torch.arange(T, dtype=torch.int32, device="cuda")
        rows = torch.zeros(T, dtype=torch.int32, device="cuda")
        ok = plain.chunk_mask(T, chunk)
        ref = np.zeros((T, H, hd))
        for a in range(H):
            g = a // (H // G)
            ref[:, a] = 0.5 * plain.sink_softmax(q[:, a * hd:(a + 1) * hd] @ k[:, g * hd:(g + 1) * hd].T, ok) @ v[:, g * hd:(g + 1) * hd]
        qd = dev(q, bf)
        for cuts in ((128, 7, 1, 1, 100, 63), (1,) * 40 + (260,)):
            out = torch.zeros(T, H * hd, device="cuda", dtype=bf)
            p = 0
            for n in cuts:
                n = min(n, T - p)
                single = n == 1
                ops.paged_attention(qd[p:p + n], kp, vp, table, positions[p:p + n], rows[:n], out[p:p + n], H, G, hd, 1.0,
                                    chunk=chunk, sink=0.0, out_scale=0.5, all_single=single, max_seq_len=T,
                                    cu_q=None if single else torch.tensor([0, n], dtype=torch.int32, device="cuda"), single_prefix=0)
                p += n
            got = f64(out).reshape(T, H, hd)
            assert np.abs(got - ref).max() <= 2e-2, (chunk, key_at, cuts[:3], np.abs(got - ref).max())
        last_in = T - 1 if not chunk else min(T - 1, (key_at // chunk + 1) * chunk - 1)
        assert np.abs(got[last_in, 0] - 0.5 * v[key_at, :hd]).max() < 2e-2
        if last_in + 1 < T:
            assert np.abs(got[last_in + 1, 0] - 0.5 * v[key_at, :hd]).max() > 0.05


def test_the_sink_takes_its_share():
    """Scores of zero over n keys and a sink of zero: every weight is 1 / (n + 1), so the first token's
    output is half its value."""
    from tuff_b200.kernels import ops
    H = G = 1; hd = 16; T = 5; page = 4
    v = np.random.default_rng(8).normal(size=(T, hd))
    kp = torch.zeros(2, G, page, hd, device="cuda"); vp = torch.zeros_like(kp)
    for t in range(T):
        vp[t // page, 0, t % page] = dev(v[t])
    table = torch.tensor([[0, 1]], dtype=torch.int32, device="cuda")
    out = torch.empty(T, hd, device="cuda")
    args = (torch.zeros(T, hd, device="cuda"), kp, vp, table, torch.arange(T, dtype=torch.int32, device="cuda"),
            torch.zeros(T, dtype=torch.int32, device="cuda"), out, H, G, hd, 1.0)
    ops.paged_attention_plain(*args, sink=0.0)
    ref = np.cumsum(v, axis=0) / (np.arange(T) + 2.0)[:, None]
    assert np.abs(f64(out) - ref).max() < 1e-5
    ops.paged_attention_plain(*args, sink=math.log(3.0), out_scale=2.0)
    ref = 2.0 * np.cumsum(v, axis=0) / (np.arange(T) + 4.0)[:, None]
    assert np.abs(f64(out) - ref).max() < 1e-5


def test_yarn_tables_and_interleaved_rotation():
    from tuff_b200.kernels import ops
    from tuff_b200.parts import POSITION_ENCODINGS, PartSpec
    for span, hd, base, sc in ((16, 32, 1e4, dict(factor=4.0, original=64, fast=16.0, slow=2.0)), (48, 48, 500.0, None),
                               (10, 20, 1e6, dict(factor=8.0, original=1024, fast=32.0, slow=1.0))):
        pe = POSITION_ENCODINGS.build(PartSpec("rope_yarn", dict(head_dim=hd, theta=base, rotary_dim=span, **(sc or {}))))
        f, amp = plain.yarn_frequencies(span, base, sc)
        inv, rot = pe.fused_tables("cuda:0")
        assert rot == span and np.abs(f64(inv) - f).max() <= 1e-7 * f.max() and abs(pe.amplitude - amp) < 1e-12
        # the kernel, without norm or pages: q and k turned in place at given positions
        H, G, T = 3, 2, 9
        rng = np.random.default_rng(span)
        x = rng.normal(size=(T, (H + G) * hd))
        pos = np.array([0, 1, 2, 50, 51, 300, 7, 1000, 3])
        qk = dev(x).contiguous()
        ops.qk_norm_rope_write(qk, None, None, inv, dev(pos, torch.int32), torch.zeros(T, dtype=torch.int32, device="cuda"), None,
                               None, None, H, G, hd, span, 0.0, write_kv=False, interleaved=True, amplitude=pe.amplitude,
                               v_from_k=True)
        ref = plain.rotate_interleaved(x.reshape(T, H + G, hd), pos, span, f64(inv), amp).reshape(T, -1)
        assert np.abs(f64(qk) - ref).max() < 2e-4          # float32 angles at position 1000


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_after_the_sum_and_position_vectors(dtype):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(9)
    for T, d in ((3, 80), (40, 192), (300, 96)):
        s = rng.normal(size=(T, d)) * 3
        w = 1 + 0.1 * rng.normal(size=d)
        sd = dev(s)
        x = torch.empty_like(sd)
        h = torch.empty(T, d, dtype=DT[dtype], device="cuda") if dtype == "bfloat16" else None
        ops.rmsnorm_fork(sd, dev(w), 1e-5, 2.5, x, h, sd, DT[dtype])
        ref = plain.rms_norm(f64(dev(s)), f64(dev(w)), 1e-5)
        assert np.abs(f64(x) - ref).max() < 1e-5 and np.abs(f64(sd) - 2.5 * ref).max() < 1e-5
        if h is not None:
            assert np.array_equal(f64(h), f64(x.to(torch.bfloat16)))
    V, P, d = 50, 30, 40
    table, ptab = rng.normal(size=(V, d)), rng.normal(size=(P, d))
    toks, pos = rng.integers(0, V, 12), rng.integers(0, P, 12)
    out = torch.empty(12, d, device="cuda")
    ops.embed(dev(toks, torch.int32), dev(table, DT[dtype]), out, dev(pos, torch.int32), dev(ptab, DT[dtype]))
    ref = f64(dev(table, DT[dtype]))[toks] + f64(dev(ptab, DT[dtype]))[pos]
    assert np.abs(f64(out) - ref).max() < 1e-6


def test_gated_group_norm():
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(10)
    for T, width, group in ((7, 96, 24), (33, 640, 640), (5, 120, 40), (2, 300, 300)):
        o, g = rng.normal(size=(T, width)) * 5, rng.normal(size=(T, width + 8))
        w = 1 + 0.1 * rng.normal(size=group)
        out = torch.empty(T, width, device="cuda")
        gd = dev(g)
        ops.gated_group_norm(dev(o), gd[:, 8:], dev(w), 1e-5, group, out, gate_act=ops.GATE_SILU, out_scale=0.5)
        ref = 0.5 * plain.rms_norm(o.reshape(T, width // group, group), f64(dev(w)), 1e-5).reshape(T, width) * plain.silu(g[:, 8:])
        assert np.abs(f64(out) - ref).max() < 2e-5
        ops.gated_group_norm(dev(o), gd[:, 8:], dev(w), 1e-5, group, out, gate_act=ops.GATE_SIGMOID)
        ref = plain.rms_norm(o.reshape(T, width // group, group), f64(dev(w)), 1e-5).reshape(T, width) * plain.sigmoid(g[:, 8:])
        assert np.abs(f64(out) - ref).max() < 2e-5


def test_trace_run_program_and_command_line(models, tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, reqs, expect = models["kor_b"]
    vocab = CONFIGS["kor_b"][0]["vocab"]
    steps, wanted = traces.mixed(reqs)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(tmp_path),
                        "--max-tokens", str(traces.tokens_needed(steps))], input=text, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    compare(str(tmp_path), wanted, expect, vocab, "float32", "trace_run")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "tuff"), "--model", folder, "--prompt-ids", "5 9 200 31", "-n", "6",
                        "--dump-tokens", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [int(t) for t in r.stdout.split()]
    ref = plain.PlainKoridra(folder).forward([5, 9, 200, 31] + ids[-6:])
    for i, tok in enumerate(ids[-6:]):
        assert ref[3 + i].max() - ref[3 + i][tok] < 1e-3
