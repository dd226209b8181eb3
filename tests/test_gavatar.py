"""Gavatar on the step engine against the plain implementation (oracle/gavatar.py): every mechanism alone, whole prompts against
token-by-token decoding, prompts cut into portions down to two tokens, batches of unequal requests, pages and slots that are given
back and taken again, keys just inside and just outside a window (in a prompt and decoded), page borders, the first tokens of a
sequence, long decoding, sizes that happen to be equal or one, both precisions, and greedy generation through the scheduler and the
command line.  Where random weights would hide a fault, the configuration's score scale is raised so that every softmax leans on few
keys, and the test first shows on the oracle itself that a window one token off (or a sink left out) would be noticed.  On the kernel
sources under the CPU emulator and, marked gpu, on the native library."""
import copy
import json

import pytest
import torch

from leopard_b200 import gavatar
from leopard_b200.scheduler import Request, Scheduler, generate
from leopard_b200.seqlm import StepEntry
from oracle import gavatar as O
from gavatar_common import (TOL, attention_layer, backend, emu_lib, latent_layer, make_engine, mixed_model, mlstm_layer, model, moe,  # noqa: F401
                            rel_err)


def _tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _all(n):
    return list(range(n))


def _rows(got, want):
    """relative error of every row"""
    got, want = got.double().cpu(), want.double()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()


def _prompt_then_decode(eng, toks, n_prompt, key="r"):
    got = [eng.step([StepEntry(key, toks[:n_prompt], _all(n_prompt))])]
    for t in toks[n_prompt:]:
        got.append(eng.step([StepEntry(key, [t], [0])]))
    return torch.cat(got, 0)


LAYERS = {
    "attention": attention_layer(),
    "attention, odd sizes, one key head": attention_layer(heads=3, kv_heads=1, dim=5, vdim=7, window=3),
    "attention, six heads a group": attention_layer(heads=6, kv_heads=1, dim=4, vdim=4, window=6),
    "attention, every head its own keys": attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, window=20),
    "attention, four and eight heads a group": attention_layer(heads=8, kv_heads=1, dim=4, vdim=3, window=7),
    "latent": latent_layer(),
    "latent, one head": latent_layer(heads=1, dim=6, vdim=3, q_rank=7, kv_rank=5, window=6),
    "latent + experts": latent_layer(heads=2, dim=4, vdim=4, q_rank=4, kv_rank=4, window=3, mlp=moe()),
    "mlstm": mlstm_layer(),
    "mlstm, two row groups, two column tiles": mlstm_layer(heads=1, dim=36, vdim=33),
    "mlstm, one of each + one expert of one": mlstm_layer(heads=1, dim=1, vdim=1, gate_cap=2.0, mlp=moe(experts=1, top=1, ff=3)),
}


@pytest.mark.parametrize("name", list(LAYERS))
def test_each_mechanism_alone(backend, name):
    """a one-layer model: the whole prompt in one step, and the same tokens with the last ones decoded through cache and state"""
    cfg = model([LAYERS[name]])
    w = O.random_weights(cfg, seed=3)
    toks = _tokens(9, cfg["vocab"], seed=1)
    res = []
    want = O.forward(cfg, w, toks, residuals=res)
    eng = make_engine(cfg, w, backend)
    taps = []
    eng.tap = lambda li, x: taps.append(x.clone())
    got = eng.step([StepEntry("p", toks, _all(9))])
    assert rel_err(taps[0], res[0]) < TOL["float32"]              # the residual stream after the layer
    assert float(_rows(got, want).max()) < 5 * TOL["float32"]
    eng.tap = None
    eng.finish("p")
    assert float(_rows(_prompt_then_decode(eng, toks, 6), want).max()) < 5 * TOL["float32"]


def test_positions_shift_and_loop_vectors(backend):
    """the pieces around the mixers, each shown to matter on the oracle: the position vectors, the shift towards the previous token
    and the vector added before every pass of the loop"""
    cfg = model([mlstm_layer(), latent_layer()], loop=(1, 2, 3))
    w = O.random_weights(cfg, seed=4)
    toks = _tokens(5, cfg["vocab"], seed=5)
    want = O.forward(cfg, w, toks)
    for name in ("l0.shift", "l1.shift", "loop.step"):
        w2 = dict(w)
        w2[name] = torch.zeros_like(w[name])
        assert float(_rows(O.forward(cfg, w2, toks), want).max()) > 1e-2, name
    assert len(O.layer_runs(cfg)) == 4
    res = []
    eng = make_engine(cfg, w, backend)
    eng.tap = lambda li, x: res.append(x.clone())
    got = eng.step([StepEntry("p", toks, _all(5))])
    assert len(res) == 4
    assert float(_rows(got, want).max()) < 5 * TOL["float32"]
    # the same request row by row: every step's shift reads the row that the step before left in the slot
    eng.tap = None
    eng.finish("p")
    assert float(_rows(_prompt_then_decode(eng, toks, 1), want).max()) < 5 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_long_decoding(backend, dtype):
    """a prompt, then tokens one by one: past every window, over many page borders, the recurrent state carried through every step"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=11)
    long = backend[0] == "cuda"      # the emulator spends seconds a step
    toks = _tokens(90 if long else 12 if dtype == "float32" else 7, cfg["vocab"], seed=2)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, dtype, max_tokens=96)
    got = _prompt_then_decode(eng, toks, 21 if long else 3)
    assert rel_err(got, want) < TOL[dtype]
    if dtype == "float32":
        assert float(_rows(got, want).max()) < 5 * TOL[dtype]


@pytest.mark.parametrize("cuts", [(2, 2, 3, 2), (5, 6), (1, 2, 17)])
def test_portions_of_a_prompt(backend, cuts):
    """a prompt fed in portions: windows that reach into earlier portions, states and shifted rows handed from portion to portion,
    portions longer than the recurrence's 16-token stage"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=12)
    toks = _tokens(sum(cuts), cfg["vocab"], seed=3)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend)
    got, at = [], 0
    for n in cuts:
        got.append(eng.step([StepEntry("r", toks[at:at + n], _all(n))]))
        at += n
    assert float(_rows(torch.cat(got, 0), want).max()) < 5 * TOL["float32"]


def test_batch_of_unequal_requests_and_reuse(backend):
    """three requests of different lengths in one batch, decoded together while the short ones end; then a new request takes the
    pages and the slot that were given back (the pools are sized so that it must)"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=13)
    lens = {"a": (1, 2), "b": (5, 3), "c": (8, 1)}            # prompt length, decoded tokens
    toks = {k: _tokens(p + d, cfg["vocab"], seed=30 + i) for i, (k, (p, d)) in enumerate(lens.items())}
    want = {k: O.forward(cfg, w, toks[k]) for k in lens}
    eng = make_engine(cfg, w, backend, max_tokens=8, max_seqs=3)
    got = {k: [] for k in lens}
    out = eng.step([StepEntry(k, toks[k][:p], [p - 1]) for k, (p, d) in lens.items()])
    for i, k in enumerate(lens):
        got[k].append(out[i:i + 1])
    live = list(lens)
    for step in range(3):
        live = [k for k in live if step < lens[k][1]]
        out = eng.step([StepEntry(k, [toks[k][lens[k][0] + step]], [0]) for k in live])
        for i, k in enumerate(live):
            got[k].append(out[i:i + 1])
        for k in live:
            if step + 1 == lens[k][1]:
                eng.finish(k)
    for k, (p, d) in lens.items():
        assert float(_rows(torch.cat(got[k], 0), want[k][p - 1:]).max()) < 5 * TOL["float32"], k
    c = eng.cache
    assert c.pages_in_use() == 0 and len(c.free_slots) == c.n_slots
    before = (c.n_slots, c.n_pages)
    t2 = _tokens(7, cfg["vocab"], seed=77)
    again = eng.step([StepEntry("a", t2, _all(7))])           # the name of an ended request, a used slot, used pages
    assert float(_rows(again, O.forward(cfg, w, t2)).max()) < 5 * TOL["float32"]
    assert (c.n_slots, c.n_pages) == before


def _one_off(cfg, delta):
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        if "mask" in l["mixer"]:
            l["mixer"]["mask"]["size"] += delta
    return c


@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
@pytest.mark.parametrize("mode", ["prompt", "decoded"])
def test_edge_of_the_window(backend, kind, mode):
    """a large score scale makes every softmax lean on few keys: the oracle with a window one token longer or shorter differs by far
    more than the tolerance on many rows past the window, and the engine agrees with the right one — also across page borders (pages of
    4 tokens, windows of 6 and 7) and with the pages before the window given back while the request runs"""
    layer = (attention_layer(heads=4, kv_heads=2, dim=8, vdim=4, window=6, scale=3.0) if kind == "attention"
             else latent_layer(heads=2, dim=4, vdim=6, q_rank=6, kv_rank=8, window=7, scale=0.5))
    cfg = model([layer])
    w = O.random_weights(cfg, seed=21)
    toks = _tokens(19, cfg["vocab"], seed=6)
    want = O.forward(cfg, w, toks)
    size = layer["mixer"]["mask"]["size"]
    for delta in (-1, 1):
        off = _rows(O.forward(_one_off(cfg, delta), w, toks), want)
        assert int((off[size:] > 200 * TOL["float32"]).sum()) >= (len(toks) - size) // 3      # wherever the edge key carries weight
        assert float(off[: size - 1].max()) < 1e-12           # rows that see everything either way
    eng = make_engine(cfg, w, backend, max_tokens=8)
    got = eng.step([StepEntry("r", toks, _all(19))]) if mode == "prompt" else _prompt_then_decode(eng, toks, size - 2)
    assert float(_rows(got, want).max()) < 5 * TOL["float32"]
    assert sum(p >= 0 for p in eng.cache.get("r").pages) <= -(-size // 4) + 1      # only the window's pages are still held


@pytest.mark.gpu
def test_far_keys_among_hundreds():
    """windows of hundreds of keys (several key tiles of the attention kernels, many pages), sharp softmaxes: the key at the far edge
    of the window carries weight on many rows, in prompts cut into portions and in decoding, and the oracle with a window one token
    off is told apart; the rows of a portion's tiles start and end at every offset against the window's edge"""
    layers = [attention_layer(heads=8, kv_heads=2, dim=16, vdim=8, window=150, scale=2.5),
              latent_layer(heads=4, dim=8, vdim=8, q_rank=12, kv_rank=16, window=131, scale=0.45)]
    cfg = model(layers, width=24)
    w = O.random_weights(cfg, seed=31)
    toks = _tokens(330, cfg["vocab"], seed=32)
    want = O.forward(cfg, w, toks)
    for delta in (-1, 1):
        off = _rows(O.forward(_one_off(cfg, delta), w, toks), want)
        assert int((off[150:] > 200 * TOL["float32"]).sum()) >= 40
    eng = make_engine(cfg, w, ("cuda", None), max_tokens=400, page_size=16)
    got, at = [], 0
    for n in (129, 2, 67, 101, 3):
        got.append(eng.step([StepEntry("r", toks[at:at + n], _all(n))]))
        at += n
    for t in toks[at:]:
        got.append(eng.step([StepEntry("r", [t], [0])]))
    assert float(_rows(torch.cat(got, 0), want).max()) < 5 * TOL["float32"]


def test_sink_and_head_mixing_are_there(backend):
    """left out, each would move the rows by far more than the tolerance: a sink of large weight, a mixing matrix far from the unit
    matrix (also negative entries), a gate"""
    cfg = model([latent_layer(window=9), attention_layer(window=9)])
    w = O.random_weights(cfg, seed=22)
    w["l0.mix.sink"] = torch.tensor([3.0, -1.0, 5.0])
    w["l1.mix.talk"] = torch.tensor([[0.5, -0.75, 0.25, 1.0], [1.5, 0.0, -0.5, 0.0], [0.0, 0.0, 0.0, 1.0], [0.25, 0.25, 0.25, 0.25]])
    toks = _tokens(12, cfg["vocab"], seed=7)
    want = O.forward(cfg, w, toks)
    for name, other in (("l0.mix.sink", torch.full((3,), -30.0)), ("l1.mix.talk", torch.eye(4)), ("l1.mix.g", torch.zeros_like(w["l1.mix.g"])),
                        ("l0.mix.g", torch.zeros_like(w["l0.mix.g"]))):
        w2 = dict(w)
        w2[name] = other
        assert float(_rows(O.forward(cfg, w2, toks), want).median()) > 200 * TOL["float32"], name
    eng = make_engine(cfg, w, backend)
    assert float(_rows(_prompt_then_decode(eng, toks, 5), want).max()) < 5 * TOL["float32"]


def test_memory_of_the_recurrence(backend):
    """mLSTM with forget gates near one keeps the first tokens: changing token 0 moves the last row of a 36-token sequence on the
    oracle; the engine carries the state over three 16-token stages, two portions, decoding, and into a slot that was used before"""
    cfg = model([mlstm_layer(heads=2, dim=4, vdim=6, gate_cap=6.0)])
    w = O.random_weights(cfg, seed=23)
    w["l0.mix.f.b"] = torch.tensor([6.0, 5.0])
    toks = _tokens(36, cfg["vocab"], seed=8)
    want = O.forward(cfg, w, toks)
    other = O.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert float(_rows(other[-1:], want[-1:])) > 20 * TOL["float32"]
    eng = make_engine(cfg, w, backend, max_seqs=1)
    eng.step([StepEntry("old", _tokens(5, cfg["vocab"], seed=9), [])])
    eng.finish("old")                                          # its state stays in the slot; the next request must not see it
    got = [eng.step([StepEntry("r", toks[:33], _all(33))]), eng.step([StepEntry("r", toks[33:35], _all(2))]),
           eng.step([StepEntry("r", toks[35:], [0])])]
    assert eng.cache.n_slots == 1
    assert float(_rows(torch.cat(got, 0), want).max()) < 5 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_equal_or_one(backend, dtype):
    """one head everywhere, top 1 of 1 and top = experts, a window of one token, a loop of one pass over everything, no loop at all,
    a loop whose span is empty, a width that is odd"""
    layers = [attention_layer(heads=1, kv_heads=1, dim=4, vdim=4, window=1, mlp=moe(experts=1, top=1, ff=2)),
              latent_layer(heads=1, dim=4, vdim=4, q_rank=4, kv_rank=4, window=1, mlp=moe(experts=4, top=4, ff=4)),
              mlstm_layer(heads=1, dim=4, vdim=4, gate_cap=1.0)]
    toks = _tokens(6, 23, seed=10)
    for loop in ((0, 3, 1), None, (2, 2, 5)) if dtype == "float32" else ((0, 3, 1),):
        cfg = model(layers, width=9, vocab=23, eps=1e-6, embed_scale=1.0, loop=loop)
        w = O.random_weights(cfg, seed=24)
        want = O.forward(cfg, w, toks)
        eng = make_engine(cfg, w, backend, dtype)
        got = _prompt_then_decode(eng, toks, 3)
        assert rel_err(got, want) < TOL[dtype]


def test_greedy_generation_through_the_scheduler(backend):
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=19)
    prompts = [_tokens(n, cfg["vocab"], seed=40 + n) for n in (3, 6, 1)]
    eng = make_engine(cfg, w, backend, max_seqs=2)
    outs = generate(eng, prompts, max_new_tokens=2)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in o:                                   # every generated token is the oracle's arg-max given what came before
            lg = O.forward(cfg, w, seq)[-1]
            top2 = lg.topk(2).values
            assert int(lg.argmax()) == t or float(top2[0] - top2[1]) < 1e-3
            seq.append(t)
        assert len(o) == 2
    assert eng.cache.pages_in_use() == 0
    sched = Scheduler(eng, max_running=1)
    first = outs[0][0]
    sched.add(Request("x", prompts[0], max_new_tokens=2, eos={first}))
    sched.add(Request("y", prompts[1], max_new_tokens=2))
    done = sched.run()
    assert done["x"].output == [first] and done["y"].output == outs[1][:2]


@pytest.mark.gpu
def test_command_line_generate_and_trace(tmp_path):
    """the registry picks the loader from config.json; `generate` and `trace` run the same step engine"""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from leopard_b200.safetensors_io import save_file
    root = Path(__file__).resolve().parents[1]
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=20)
    (tmp_path / "m").mkdir()
    (tmp_path / "m/config.json").write_text(json.dumps(cfg))
    save_file(w, tmp_path / "m/model.safetensors")
    toks = _tokens(12, cfg["vocab"], seed=8)
    r = subprocess.run([sys.executable, "-m", "leopard_b200", "generate", "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt",
                        ",".join(map(str, toks)), "--max-new-tokens", "3"], cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])["output"]
    assert out[0] == int(O.forward(cfg, w, toks)[-1].argmax())
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:9], "want": [0, 8]}, {"id": "s", "tokens": toks[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[9:10], "want": []}, {"id": "s", "tokens": toks[2:3], "want": [0]}],
              "end": ["s"]},
             {"step": 2, "entries": [{"id": "q", "tokens": toks[10:11], "want": [0]}], "end": ["q"]}]
    for dtype in ("float32", "bfloat16"):
        r = subprocess.run([str(root / "bin/trace_run"), "--model", str(tmp_path / "m"), "--dtype", dtype, "--out", str(tmp_path / dtype),
                            "--max-tokens", "64"], input="\n".join(map(json.dumps, steps)) + "\n", cwd=root, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        want = O.forward(cfg, w, toks)
        got = [torch.from_numpy(np.fromfile(tmp_path / dtype / f"{i}.f32", dtype="<f4").reshape(n, -1)) for i, n in ((0, 2), (1, 1), (2, 1))]
        assert rel_err(got[0], want[[0, 8]]) < TOL[dtype] and rel_err(got[1], want[2:3]) < TOL[dtype]
        assert rel_err(got[2], want[10:11]) < TOL[dtype]


def test_registry_and_config_reader():
    from leopard_b200 import registry
    from leopard_b200.seqlm import LatentAttentionConfig, MLSTMConfig, MoEConfig, WindowAttentionConfig
    assert "Gavatar" in registry.architectures()
    cfg, source = gavatar.config_from_dict(mixed_model())
    assert (cfg.norm, cfg.embed_scale, cfg.position_base) == ("sandwich_vector", 3.0, 10000.0)
    assert source == [0, 1, 0, 1, 2] and [l.weights_of for l in cfg.layers] == [None, None, 0, 1, None]
    assert [l.add_before for l in cfg.layers] == [("loop.step", 0), None, ("loop.step", 1), None, None]
    assert all(l.token_shift for l in cfg.layers)
    a, b, _, _, c = cfg.layers
    assert isinstance(a.mixer, LatentAttentionConfig) and (a.mixer.q_rank, a.mixer.rot_dim, a.mixer.sink, a.mixer.head_gate, a.mixer.window) == (5, 0, True, True, 4)
    assert isinstance(a.ff, MoEConfig) and (a.ff.router, a.ff.experts, a.ff.top, a.ff.shared_ff) == ("softmax_top", 5, 2, 0)
    assert isinstance(b.mixer, MLSTMConfig) and b.mixer.gate_cap == 8.0 and b.ff is None
    assert isinstance(c.mixer, WindowAttentionConfig)
    assert (c.mixer.qk_norm, c.mixer.bias, c.mixer.value_norm, c.mixer.talking_heads, c.mixer.out_gate, c.mixer.window) == ("unit", True, True, True, True, 5)
    assert gavatar.tensor_namer(source)(3, "mix.q") == "l1.mix.q" and gavatar.tensor_namer(source)(None, "embed") == "embed"
    assert gavatar.layer_runs(model([mlstm_layer()] * 3, loop=(1, 3, 2))) == [(0, None), (1, 0), (2, None), (1, 1), (2, None)]
    with pytest.raises(ValueError):
        gavatar.config_from_dict({"architecture": "other"})
    with pytest.raises(ValueError):
        gavatar.config_from_dict(model([mlstm_layer()], loop=(0, 2, 1)))
