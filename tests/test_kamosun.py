"""Kamosun on the step engine against the plain implementation (oracle/kamosun.py): every mechanism alone, whole prompts against
token-by-token decoding, prompts cut into portions down to two tokens, batches of unequal requests, pages and slots that are given
back and taken again, keys just inside and just outside a block of the block-local attention (in a prompt and decoded), page borders,
the first tokens of a sequence, long decoding, sizes that happen to be equal or one, both precisions, and greedy generation through
the scheduler and the command line.  Where random weights would hide a fault, the configuration's score scale is raised so that every
softmax leans on few keys, and the test first shows on the oracle itself that a block one token off (or a gate, a cap, a clamp left
out) would be noticed.  On the kernel sources under the CPU emulator and, marked gpu, on the native library."""
import copy
import json

import pytest
import torch

from leopard_b200 import kamosun
from leopard_b200.scheduler import Request, Scheduler, generate
from leopard_b200.seqlm import StepEntry, RotaryConfig, BandScaling, rotary_table
from oracle import kamosun as O
from kamosun_common import (TOL, attention_layer, backend, dense, emu_lib, make_engine, mixed_model, model, moe, parallel_layer,  # noqa: F401
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


MODELS = {
    "attention": [attention_layer()],
    "attention, odd sizes, one key head, all rotated": [attention_layer(heads=3, kv_heads=1, dim=6, vdim=7, chunk=4, rot_dims=6)],
    "attention, every head its own keys, no rotation": [attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, chunk=20, rot_dims=0)],
    "attention + dense": [attention_layer(mlp=dense())],
    "attention + experts": [attention_layer(mlp=moe())],
    "attention + experts, no shared one, top 1": [attention_layer(mlp=moe(experts=4, top=1, shared=0))],
    "two layers, the second on the first one's keys": [attention_layer(), attention_layer(kv_from=0, chunk=3)],
    "parallel": [parallel_layer()],
    "parallel, no rescaling, odd sizes": [parallel_layer(heads=3, kv_heads=3, dim=4, vdim=7, rot_dims=2, scaling=False, r_heads=1, r_dim=5,
                                                       r_vdim=9, decay=(0.9,))],
    "parallel + experts": [parallel_layer(mlp=moe())],
}


@pytest.mark.parametrize("name", list(MODELS))
def test_each_mechanism_alone(backend, name):
    """a small model: the whole prompt in one step, and the same tokens with the last ones decoded through cache and state"""
    cfg = model(MODELS[name])
    w = O.random_weights(cfg, seed=3)
    toks = _tokens(9, cfg["vocab"], seed=1)
    res = []
    want = O.forward(cfg, w, toks, taps=res)
    eng = make_engine(cfg, w, backend)
    taps = []
    eng.tap = lambda li, x: taps.append(x.clone())
    got = eng.step([StepEntry("p", toks, _all(9))])
    for a, b in zip(taps, res):                                   # the stream after every layer
        assert rel_err(a, b) < TOL["float32"]
    assert float(_rows(got, want).max()) < 5 * TOL["float32"]
    eng.tap = None
    eng.finish("p")
    assert float(_rows(_prompt_then_decode(eng, toks, 6), want).max()) < 5 * TOL["float32"]


def test_every_piece_matters_on_the_oracle():
    """the pieces around the mixers, each shown to move the logits when it is left out or changed: the norm's shift and slope, the
    residual gates, the depth average's weights, the cap, the clamp, the router's weight on the input, the output bias, the branch
    gains, the decay"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=4)
    toks = _tokens(8, cfg["vocab"], seed=5)
    want = O.forward(cfg, w, toks)
    changes = {"l0.norm1.b": 0.0, "l0.norm2.alpha": 0.1, "l1.rg1.b": 8.0, "l0.rg2": 0.0, "l2.dwa": 0.25, "l0.mix.o.b": 0.0,
               "l2.mix.left.out": 0.0, "l2.mix.right.norm": 0.1, "l1.mlp.router": 0.0, "l3.mix.q.norm": 0.3, "final.norm.b": 0.0}
    for name, value in changes.items():
        w2 = dict(w)
        w2[name] = torch.full_like(w[name], value)
        assert float(_rows(O.forward(cfg, w2, toks), want).median()) > 200 * TOL["float32"], name
    for path, value in ((("layers", 2, "mixer", "left", "softcap"), 0.3), (("layers", 0, "mlp", "limit"), 0.1),
                        (("layers", 1, "mlp", "expert", "limit"), 0.1), (("layers", 1, "mlp", "shared", "limit"), 0.05),
                        (("layers", 2, "mixer", "right", "decay"), [0.1, 0.2]), (("residual_mult",), 0.3),
                        (("layers", 2, "mixer", "left", "rot", "scaling", "factor"), 64.0)):
        c2 = copy.deepcopy(cfg)
        node = c2
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        assert float(_rows(O.forward(c2, w, toks), want).median()) > 50 * TOL["float32"], path


def test_band_rescaled_frequencies():
    """the three bands on a table whose wavelengths fall into each of them, against the oracle's loop"""
    rot = {"base": 300.0, "dims": 12, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}}
    want = O.frequencies(rot)
    plain = O.frequencies({"base": 300.0, "dims": 12})
    kinds = {"kept": 0, "divided": 0, "blended": 0}
    for f, g in zip(want, plain):
        kinds["kept" if f == g else "divided" if abs(f - g / 8.0) < 1e-15 else "blended"] += 1
    assert all(kinds.values()), kinds
    got, mag = rotary_table(RotaryConfig(dims=12, base=300.0, layout="interleaved", scaling=BandScaling(factor=8.0, original=256.0, low=1.0, high=4.0)))
    assert mag == 1.0
    assert torch.allclose(got.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-7, atol=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_then_long_decoding(backend, dtype):
    """a prompt, then tokens one by one: over many block and page borders, the lightning state carried through every step"""
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


@pytest.mark.parametrize("cuts", [(2, 2, 3, 2), (5, 6), (1, 2, 36)])
def test_portions_of_a_prompt(backend, cuts):
    """a prompt fed in portions: blocks that began in earlier portions, the lightning state handed from portion to portion, a portion
    longer than the recurrence's 32-token chunk"""
    cfg = mixed_model()
    w = O.random_weights(cfg, seed=12)
    toks = _tokens(sum(cuts), cfg["vocab"], seed=3)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, max_tokens=48)
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


@pytest.mark.parametrize("shared", [False, True])
@pytest.mark.parametrize("mode", ["prompt", "decoded"])
def test_edge_of_the_block(backend, shared, mode):
    """a large score scale makes every softmax lean on few keys: the oracle with blocks one token longer or shorter differs by far
    more than the tolerance on many rows, and the engine agrees with the right one — in a layer with keys of its own and in one that
    reads another layer's, whose blocks are of another size; across page borders (pages of 4 tokens, blocks of 6 and 5), with the pages
    before the block given back while the request runs"""
    layers = [attention_layer(heads=4, kv_heads=2, dim=8, vdim=4, chunk=6, scale=3.0)]
    if shared:
        layers.append(attention_layer(heads=4, kv_heads=2, dim=8, vdim=4, chunk=5, scale=3.0, kv_from=0))
    cfg = model(layers)
    w = O.random_weights(cfg, seed=21)
    toks = _tokens(19, cfg["vocab"], seed=6)
    want = O.forward(cfg, w, toks)
    for delta in (-1, 1):
        off = _rows(O.forward(_one_off(cfg, delta), w, toks), want)
        assert int((off[5:] > 200 * TOL["float32"]).sum()) >= 7      # wherever a block's first key carries weight
        assert float(off[:4].max()) < 1e-12                         # rows that see the same either way
    eng = make_engine(cfg, w, backend, max_tokens=8)
    got = eng.step([StepEntry("r", toks, _all(19))]) if mode == "prompt" else _prompt_then_decode(eng, toks, 4)
    assert float(_rows(got, want).max()) < 5 * TOL["float32"]
    assert sum(p >= 0 for p in eng.cache.get("r").pages) <= 3      # only the block's pages are still held


@pytest.mark.gpu
def test_far_keys_among_hundreds():
    """blocks of hundreds of keys (several key tiles of the attention kernels, many pages) beside causal attention over everything,
    sharp softmaxes: the first key of a block and of the sequence carry weight on many rows, in prompts cut into portions and in
    decoding, and the oracle with blocks one token off is told apart; a portion's tiles start and end at every offset against a
    block's edge"""
    layers = [attention_layer(heads=8, kv_heads=2, dim=16, vdim=8, chunk=150, scale=2.5, rot_dims=8),
              attention_layer(heads=8, kv_heads=2, dim=16, vdim=8, chunk=131, scale=2.5, rot_dims=8, kv_from=0),
              parallel_layer(heads=4, kv_heads=2, dim=8, vdim=8, scale=2.0, softcap=30.0, rot_dims=8, r_heads=2, r_dim=8, r_vdim=8,
                             decay=(0.99, 0.999))]
    cfg = model(layers, width=24)
    w = O.random_weights(cfg, seed=31)
    toks = _tokens(330, cfg["vocab"], seed=32)
    want = O.forward(cfg, w, toks)
    for delta in (-1, 1):
        off = _rows(O.forward(_one_off(cfg, delta), w, toks), want)
        assert int((off[130:] > 200 * TOL["float32"]).sum()) >= 40
    first = O.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])      # the causal branch and the state remember token 0
    assert float(_rows(first[-20:], want[-20:]).median()) > 20 * TOL["float32"]
    eng = make_engine(cfg, w, ("cuda", None), max_tokens=400, page_size=16)
    got, at = [], 0
    for n in (129, 2, 67, 101, 3):
        got.append(eng.step([StepEntry("r", toks[at:at + n], _all(n))]))
        at += n
    for t in toks[at:]:
        got.append(eng.step([StepEntry("r", [t], [0])]))
    assert float(_rows(torch.cat(got, 0), want).max()) < 5 * TOL["float32"]


def test_memory_of_the_lightning_state(backend):
    """decays near one keep the first tokens: changing token 0 moves the last row of a 36-token sequence on the oracle; the engine
    carries the state over two 32-token chunks, two portions, decoding, and into a slot that was used before"""
    cfg = model([parallel_layer(decay=(0.999, 0.98))])
    w = O.random_weights(cfg, seed=23)
    w["l0.mix.left.out"] = torch.zeros_like(w["l0.mix.left.out"])      # only the recurrent branch speaks
    toks = _tokens(36, cfg["vocab"], seed=8)
    want = O.forward(cfg, w, toks)
    other = O.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert float(_rows(other[-1:], want[-1:])) > 20 * TOL["float32"]
    eng = make_engine(cfg, w, backend, max_seqs=1, max_tokens=40)
    eng.step([StepEntry("old", _tokens(5, cfg["vocab"], seed=9), [])])
    eng.finish("old")                                          # its state stays in the slot; the next request must not see it
    got = [eng.step([StepEntry("r", toks[:33], _all(33))]), eng.step([StepEntry("r", toks[33:35], _all(2))]),
           eng.step([StepEntry("r", toks[35:], [0])])]
    assert eng.cache.n_slots == 1
    assert float(_rows(torch.cat(got, 0), want).max()) < 5 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_equal_or_one(backend, dtype):
    """one head everywhere, top 1 of 1 and top = experts, blocks of one token, a residual multiplier of one, a width that is odd, no
    feed-forward at all"""
    layers = [attention_layer(heads=1, kv_heads=1, dim=4, vdim=4, chunk=1, rot_dims=4, mlp=moe(experts=1, top=1, ff=2, shared=1)),
              attention_layer(heads=1, kv_heads=1, dim=4, vdim=4, chunk=2, rot_dims=4, kv_from=0, mlp=moe(experts=4, top=4, ff=4, shared=0)),
              parallel_layer(heads=1, kv_heads=1, dim=4, vdim=4, rot_dims=4, r_heads=1, r_dim=4, r_vdim=4, decay=(1.0,))]
    toks = _tokens(6, 23, seed=10)
    cfg = model(layers, width=9, vocab=23, eps=1e-6, mult=1.0)
    w = O.random_weights(cfg, seed=24)
    want = O.forward(cfg, w, toks)
    eng = make_engine(cfg, w, backend, dtype)
    got = _prompt_then_decode(eng, toks, 3)
    assert rel_err(got, want) < TOL[dtype]


@pytest.mark.gpu
def test_wide_layers_on_the_tensor_cores():
    """sizes at which the serving precision sends its products to the tcgen05 GEMM (rows, widths and expert segments of tile size):
    the bias of the gate product, the clamped unit after the product, the row scale of sorted expert rows (every token takes both
    experts, so that no row of the 16-bit run rests on a close call of the router)"""
    layers = [attention_layer(heads=4, kv_heads=2, dim=32, vdim=32, chunk=100, rot_dims=16, mlp=dense(ff=256)),
              parallel_layer(heads=4, kv_heads=4, dim=32, vdim=32, rot_dims=32, r_heads=2, r_dim=32, r_vdim=64, decay=(0.9, 0.99),
                             mlp=moe(experts=2, top=2, ff=128, shared=128))]
    cfg = model(layers, width=128, vocab=300)
    w = O.random_weights(cfg, seed=41)
    toks = _tokens(300, cfg["vocab"], seed=42)
    want = O.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfg, w, ("cuda", None), dtype, max_tokens=512, page_size=64)
        got = eng.step([StepEntry("r", toks[:280], _all(280))])
        assert rel_err(got, want[:280]) < TOL[dtype], dtype
        more = torch.cat([eng.step([StepEntry("r", [t], [0])]) for t in toks[280:]], 0)
        assert rel_err(more, want[280:]) < TOL[dtype], dtype


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
    from leopard_b200.seqlm import DenseFFConfig, MoEConfig, ParallelMixerConfig, RetentionConfig, WindowAttentionConfig
    assert "Kamosun" in registry.architectures()
    cfg = kamosun.config_from_dict(mixed_model())
    assert (cfg.norm, cfg.residual_mult, cfg.residual_gate, cfg.depth_average) == ("parallel_dyt", 0.7, True, True)
    a, b, c, d = cfg.layers
    assert isinstance(a.mixer, WindowAttentionConfig)
    assert (a.mixer.qk_norm, a.mixer.bias, a.mixer.out_bias, a.mixer.chunk, a.mixer.window, a.mixer.kv_from, a.mixer.rot.layout) == \
        ("head", True, True, 5, None, None, "half")
    assert isinstance(a.ff, DenseFFConfig) and (a.ff.act, a.ff.ff, a.ff.limit) == ("clamp_glu", 10, 1.5)
    assert (b.mixer.kv_from, b.mixer.chunk) == (0, 3)
    assert isinstance(b.ff, MoEConfig) and (b.ff.router, b.ff.act, b.ff.experts, b.ff.top, b.ff.shared_ff, b.ff.shared_gate) == \
        ("sigmoid_input", "clamp_glu", 5, 2, 7, False)
    assert (b.ff.limit, b.ff.shared_limit) == (1.2, 0.8)
    assert isinstance(c.mixer, ParallelMixerConfig) and c.ff is None
    left, right = c.mixer.left, c.mixer.right
    assert isinstance(left, WindowAttentionConfig) and (left.bias, left.chunk, left.softcap, left.rot.layout) == (False, None, 3.0, "interleaved")
    assert left.rot.scaling == BandScaling(factor=4.0, original=64.0, low=1.0, high=4.0)
    assert isinstance(right, RetentionConfig) and (right.form, right.decay, right.k_scale, right.rot.dims) == ("lightning", (0.8, 0.97), 1.0, 0)
    assert d.ff.shared_ff == 0
    assert kamosun.tensor_name(3, "mix.q") == "l3.mix.q" and kamosun.tensor_name(None, "embed") == "embed"
    with pytest.raises(ValueError):
        kamosun.config_from_dict({"architecture": "other"})
    bad = mixed_model()
    bad["layers"][1]["mixer"]["kv_from"] = 2                  # not an earlier attention layer with keys of its own
    with pytest.raises(ValueError):
        make_engine(bad, O.random_weights(mixed_model(), seed=1), ("cpu", object()))


@pytest.mark.parametrize("rows", [3, 70])
def test_linear_with_bias_row_scale_and_gate(backend, rows):
    """the product's options one by one against torch, on the weight-streaming kernel (few rows) and the tile kernel: a bias per
    weight row, a scale per output row applied before it, the clamped gated unit, and the gated accumulate form"""
    from leopard_b200 import _lib
    eng = make_engine(model([attention_layer()]), O.random_weights(model([attention_layer()]), seed=1), backend)
    dev = eng.device
    g = torch.Generator().manual_seed(rows)
    K, N = 20, 14
    a = torch.randn(rows, K, generator=g)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    bias, scale = torch.randn(N, generator=g), torch.rand(rows, generator=g) + 0.5
    gate, x0 = torch.randn(rows, N // 2, generator=g), torch.randn(rows, N // 2, generator=g)
    z = (a.double() @ w.double().T) * scale.double()[:, None] + bias.double()
    got = eng.linear(a.to(dev), w.to(dev), torch.float32, bias=bias.to(dev), row_scale=scale.to(dev))
    assert rel_err(got, z) < TOL["float32"]
    lim = 0.8
    gg, uu = z[:, : N // 2].clamp(max=lim), z[:, N // 2:].clamp(-lim, lim)
    unit = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    got = eng.linear(a.to(dev), w.to(dev), torch.float32, _lib.EPI_CLAMP_GLU, lim, 1.702, bias=bias.to(dev), row_scale=scale.to(dev))
    assert rel_err(got, unit) < TOL["float32"]
    x = x0.clone().to(dev)
    eng.linear(a.to(dev), w.to(dev), torch.float32, _lib.EPI_CLAMP_GLU, lim, 1.702, bias=bias.to(dev), row_scale=scale.to(dev),
               into=(x, 0.3, gate.to(dev)))
    assert rel_err(x, x0.double() + 0.3 * unit * torch.sigmoid(gate.double())) < TOL["float32"]


@pytest.mark.parametrize("width", [12, 10])
def test_elementwise_kernels(backend, width):
    """Dynamic Tanh (one and two parameter sets, both operand precisions), the gated add, the depth average with its copy and the
    gated RMS norm against torch, on widths that take the four-columns-a-thread path and the one-column path, on strided rows"""
    from leopard_b200 import _lib
    eng = make_engine(model([attention_layer()]), O.random_weights(model([attention_layer()]), seed=1), backend)
    dev, L, st = eng.device, eng.L, eng._stream()
    g = torch.Generator().manual_seed(width)
    M = 5
    wide = torch.randn(M, 3 * width + 4, generator=g).to(dev)
    x = wide[:, width:2 * width]                                  # strided rows, base off the start
    gain, shift = torch.randn(2, width, generator=g).to(dev), torch.randn(2, width, generator=g).to(dev)
    for dtype in ("float32", "bfloat16"):
        eng.act = torch.float32 if dtype == "float32" else torch.bfloat16
        y1, y2 = eng.dyt(x * 3.0, (0.7, gain[0], shift[0]), (1.9, gain[1], shift[1]))
        for y, al, k in ((y1, 0.7, 0), (y2, 1.9, 1)):
            want = torch.tanh(al * 3.0 * x.double()) * gain[k].double() + shift[k].double()
            assert rel_err(y.float(), want) < (TOL["float32"] if dtype == "float32" else 4e-3)
    eng.act = torch.float32
    acc0, y = torch.randn(M, width, generator=g).to(dev), wide[:, :width]
    gt, yb, gb = wide[:, 2 * width:3 * width], shift[0], shift[1]
    acc = acc0.clone()
    eng._check(L.lp_gated_axpy_f32(_lib.ptr(acc), acc.stride(0), _lib.ptr(y), y.stride(0), _lib.ptr(yb), _lib.ptr(gt), gt.stride(0),
                                   _lib.ptr(gb), 0.6, M, width, st), "lp_gated_axpy_f32")
    assert rel_err(acc, acc0.double() + 0.6 * (y.double() + yb.double()) * torch.sigmoid(gt.double() + gb.double())) < TOL["float32"]
    hist = torch.randn(4, M, width, generator=g).to(dev)
    coef = torch.tensor([0.5, -1.25, 2.0], device=dev)
    out, copy = torch.zeros(M, width, device=dev), hist[3]
    eng._check(L.lp_depth_average_f32(_lib.ptr(hist), hist.stride(0), hist.stride(1), _lib.ptr(coef), 3, _lib.ptr(out), out.stride(0),
                                      _lib.ptr(copy), copy.stride(0), M, width, st), "lp_depth_average_f32")
    want = sum(float(coef[j]) * hist[j].double() for j in range(3))
    assert rel_err(out, want) < TOL["float32"] and torch.equal(hist[3], out)
    normed = torch.zeros(M, width, device=dev)
    eng._check(L.lp_rmsnorm_gated_f32(_lib.ptr(x), x.stride(0), M, width, _lib.ptr(gain[0]), 1e-5, _lib.ptr(gt), gt.stride(0),
                                      _lib.ptr(normed), normed.stride(0), 1, st), "lp_rmsnorm_gated_f32")
    want = O.unit_rms(x.double(), 1e-5) * gain[0].double() * torch.sigmoid(gt.double())
    assert rel_err(normed, want) < TOL["float32"]
