"""Derosun without a GPU: the config reader and its refusals, the declared tensor names, the
plain statement's pieces against values worked out by hand, and the engine's host side (cache
groups, state rows, packing, portions, mixed batches, reused pages and slots) with torch
stand-ins for the kernels, against the plain statement."""
import copy
import math

import numpy as np
import pytest
import torch

import derosun_tiny as dt
import emulated_kernels
import plain_derosun as plain
import tiny


def test_reader_builds_the_layers_the_file_lists():
    from tgo_b200.registry import model_spec_from_config
    spec = model_spec_from_config(dt.D1)
    assert spec.architecture == "Derosun" and not spec.tied_head and len(spec.layers) == 4
    assert [ls.block for ls in spec.layers] == ["postnorm_residual"] * 4
    assert all(ls.residual_scale == 2.0 for ls in spec.layers) and spec.embedding_scale == 0.5
    mem = spec.layers[0].mixer
    assert (mem.kind, mem.num_heads, mem.head_dim, mem.value_dim, mem.gate_cap) == ("mlstm", 3, 8, 12, 10.0)
    att = spec.layers[1].mixer
    assert (att.kind, att.num_heads, att.num_kv_heads, att.head_dim, att.value_dim) == \
        ("sink_attention", 4, 2, 12, 20)
    assert att.qk_norm and att.qk_norm_scope == "row" and att.softcap == 5.0 and att.scale == 0.3
    assert not att.sink and not att.bias and att.window is None
    assert att.position.kind == "rope_banded" and att.position.scaling == (8.0, 1.0, 4.0, 64)
    lat = spec.layers[2].mixer
    assert (lat.kind, lat.num_heads, lat.head_dim, lat.rope_dim, lat.value_dim, lat.latent_rank,
            lat.query_rank) == ("latent_attention", 3, 12, 8, 10, 20, 28)
    assert lat.position.kind == "rope_stretched_interleaved"
    assert lat.position.scaling == (4.0, 32, 8.0, 1.0)
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.bias
    assert spec.layers[0].feed_forward.activation == "silu"
    plain_spec = model_spec_from_config(dt.D2)
    assert plain_spec.embedding_scale == 1.0 and plain_spec.layers[0].residual_scale == 1.0
    assert plain_spec.layers[0].mixer.softcap is None and plain_spec.layers[3].mixer.position is None
    assert plain_spec.layers[0].mixer.position.scaling is None


def _changed(path, value):
    cfg = copy.deepcopy(dt.D1)
    at = cfg
    for key in path[:-1]:
        at = at[key]
    if value is ...:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,word", [
    (("width",), 0, "width"), (("vocab",), ..., "vocab"), (("norm", "eps"), -1.0, "norm.eps"),
    (("postln_alpha",), "two", "postln_alpha"), (("embedding", "scale"), float("inf"), "embedding.scale"),
    (("layers", 0, "type"), "conv", "layers[0].type"),
    (("layers", 0, "mixer", "gate_cap"), 0.0, "gate_cap"),
    (("layers", 0, "mixer", "heads"), ..., "heads"),
    (("layers", 1, "mixer", "heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "mixer", "rot", "scaling", "low"), ..., "rot.scaling.low"),
    (("layers", 1, "mixer", "softcap"), -2.0, "softcap"),
    (("layers", 2, "mixer", "rot", "dims"), 10, "rot.dims"),
    (("layers", 2, "mixer", "kv_rank"), ..., "kv_rank"),
    (("layers", 2, "mixer", "rot", "scaling", "fast"), 0.0, "rot.scaling.fast"),
    (("layers", 0, "mlp", "kind"), "moe", "mlp.kind"),
    (("layers", 0, "mlp", "ff"), ..., "mlp.ff"),
])
def test_reader_refuses_by_key(path, value, word):
    from tgo_b200.config.qwen3 import ConfigError
    from tgo_b200.registry import model_spec_from_config
    with pytest.raises(ConfigError) as err:
        model_spec_from_config(_changed(path, value))
    assert word in str(err.value)


@pytest.mark.parametrize("name", sorted(dt.CONFIGS))
def test_declared_tensors_are_the_weights_the_tests_make(name):
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    cfg, _ = dt.CONFIGS[name]
    W = dt.make_weights(cfg, 1)
    model = Model(model_spec_from_config(cfg), torch.float32, "cpu")
    declared = {w.name: tuple(w.shape) for w in model.weight_specs() if not w.optional}
    assert declared == {k: tuple(v.shape) for k, v in W.items()}


def test_a_written_folder_loads(tmp_path):
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    from tgo_b200.weights.binder import WeightError, load_weights
    from tgo_b200.weights.safetensors import SafetensorsRepo
    W = dt.make_weights(dt.D1, 2)
    d = dt.write_model_dir(str(tmp_path / "m"), dt.D1, W)
    model = Model(model_spec_from_config(dt.D1), torch.bfloat16, "cpu")
    weights = load_weights(model.weight_specs(), SafetensorsRepo(d), torch.bfloat16, "cpu", None, log=None)
    assert weights["l0.mix.i.b"].dtype == torch.float32 and weights["l0.mlp.down.b"].dtype == torch.float32
    assert weights["l1.mix.q.norm"].shape == (4 * 12,) and weights["l2.mix.dkv"].shape == (28, 48)
    model.bind(dict(weights))
    # the expansion matrices are held per head: W_uk^T [rank, dim] and W_uv [vdim, rank]
    lat = model.blocks[2].mixer
    assert lat.w_uk_t.shape == (3, 20, 12) and lat.w_uv.shape == (3, 10, 20)
    assert torch.equal(lat.w_uk_t[1].float(), torch.from_numpy(W["l2.mix.uk"][12:24].T.copy()).float())
    # a layer without a feed-forward ships no second norm
    W2 = dict(W)
    W2["l1.norm2"] = W["l0.norm2"]
    d2 = dt.write_model_dir(str(tmp_path / "m2"), dt.D1, W2)
    with pytest.raises(WeightError):
        load_weights(model.weight_specs(), SafetensorsRepo(d2), torch.bfloat16, "cpu", None, log=None)


def test_plain_pieces_by_hand():
    # the norm: x / sqrt(mean x^2 + eps) * w, a plain weight
    assert np.allclose(plain.rms_norm(np.array([[3.0, 4.0]]), np.array([1.0, 2.0]), 0.0),
                       [[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]])
    # half-split pairs (i, i + dims/2) and neighbouring pairs (2i, 2i + 1); the rest passes
    v = np.array([1.0, 2.0, 0.0, 0.0, 7.0])
    f = np.array([math.pi / 2, math.pi])
    assert np.allclose(plain.rotate(v, 1, f, 4, False), [0, -2, 1, 0, 7], atol=1e-12)
    assert np.allclose(plain.rotate(v, 1, f, 4, True), [-2, 1, 0, 0, 7], atol=1e-12)
    assert np.allclose(plain.rotate(v, 1, f, 4, True, 3.0), [-6, 3, 0, 0, 7], atol=1e-12)
    # wavelength bands: base 1 gives wavelength 2 pi for every pair
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 100}
    assert np.allclose(plain.banded_frequencies(4, 1.0, sc), [1.0, 1.0])                 # 6.28 < 25
    assert np.allclose(plain.banded_frequencies(4, 1.0, dict(sc, original=5)), [0.25, 0.25])   # > 5
    mid = plain.banded_frequencies(4, 1.0, dict(sc, original=4 * math.pi))     # original / l = 2
    s = (2.0 - 1.0) / 3.0
    assert np.allclose(mid, [(1 - s) * 0.25 + s] * 2)
    # the ramp: turns(t) = dims ln(original / (2 pi t)) / (2 ln base)
    f, mag = plain.stretched_frequencies(8, 100.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})
    b = plain.base_frequencies(8, 100.0)
    assert np.allclose(f, [b[0], b[1] * (0.5 / 4 + 0.5), b[2] / 4, b[3] / 4])
    assert math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    # the memory with one head of one channel, no projections to speak of: by hand
    W = {"p.q": np.array([[1.0]]), "p.k": np.array([[1.0]]), "p.v": np.array([[1.0]]),
         "p.g": np.array([[0.0]]), "p.o": np.array([[1.0]]), "p.norm": np.array([1.0]),
         "p.i": np.array([[0.0]]), "p.i.b": np.array([0.0]), "p.f": np.array([[0.0]]),
         "p.f.b": np.array([0.0])}
    m = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 100.0}
    h = np.array([[2.0], [3.0]])
    _, (S, n, mx) = plain.mlstm(h, W, m, 0.0, "p.")
    lf = math.log(0.5)                     # forget gate logsigmoid(0), input gate 0
    # m_1 = max(lf + 0, 0) = 0: S_1 = 0.5 * 0 + 1 * 2 * 2 = 4; m_2 = 0: S_2 = 0.5 * 4 + 9 = 11
    assert np.allclose(S, [[[11.0]]]) and np.allclose(n, [[0.5 * 2 + 3]]) and np.allclose(mx, [0.0])
    assert math.isclose(lf, plain.log_sigmoid(0.0))
    # a large input gate moves the maximum and everything is scaled by exp(-m)
    W["p.i.b"] = np.array([5.0])
    _, (S, n, mx) = plain.mlstm(h[:1], W, m, 0.0, "p.")
    i_gate = 100.0 * math.tanh(0.05)
    assert np.allclose(mx, [i_gate]) and np.allclose(S, [[[4.0]]]) and np.allclose(n, [[2.0]])
    # the feed-forward's biases
    F = {"f.gate": np.array([[0.0]]), "f.gate.b": np.array([30.0]), "f.up": np.array([[2.0]]),
         "f.up.b": np.array([1.0]), "f.down": np.array([[0.1]]), "f.down.b": np.array([-1.0])}
    assert np.allclose(plain.feed_forward(np.array([[1.0]]), F, "f."), [[30.0 * 3.0 * 0.1 - 1.0]])


# ---------------------------------------------------- the engine's host side on the CPU
@pytest.fixture()
def emulated(monkeypatch):
    emulated_kernels.install(monkeypatch)


def _engine(cfg, W, page_size, max_tokens, slots=4):
    from tgo_b200.engine.step import Engine
    model = dt.bind_model(cfg, W, torch.float32, "cpu")
    return Engine(model, page_size=page_size, max_tokens=max_tokens, num_slots=slots, graphs=False)


def _check(got, cfg, W, requests, tol=2e-4):
    for rid, toks in requests.items():
        want = plain.forward(cfg, W, toks)
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[p]).max() <= tol * max(1.0, np.abs(want[p]).max()), \
                (rid, p)


@pytest.mark.parametrize("name", ["D1", "D2", "D3", "D4"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_engine_host_side_against_plain(emulated, name, family):
    cfg, page = dt.CONFIGS[name]
    W = dt.make_weights(cfg, 3)
    requests = tiny.random_requests(cfg["vocab"], [37, 9, 1, 50, 18, 26], seed=5)
    trace = {"whole": tiny.trace_whole, "tail": lambda r: tiny.trace_tail(r, 6),
             "portions": tiny.trace_portions,
             "mixed": lambda r: tiny.trace_mixed(r, seed=2, max_live=3, tail=5)}[family](requests)
    # a pool for what is live at once, three state slots: pages and slots come back and go out again
    eng = _engine(cfg, W, page, tiny.max_tokens_of(trace, page), slots=3)
    owners = [dict() for _ in eng.cache.groups]
    got = tiny.run_trace_engine(eng, trace, poison=True, owners=owners)
    _check(got, cfg, W, requests)
    if family == "mixed" and eng.cache.groups:
        assert any(len(ids) > 1 for g in owners for ids in g.values())      # a page was reused


def test_the_cache_holds_one_latent_row_per_token(emulated):
    cfg, page = dt.CONFIGS["D1"]
    eng = _engine(cfg, dt.make_weights(cfg, 3), page, 64)
    shapes = sorted((g.planes, g.row_shape) for g in eng.cache.groups)
    assert shapes == [(1, (1, 20 + 8)), (2, (2, 12))]           # the latent row; keys [2 kv heads, 12]
    assert eng.model.state_shapes == {0: (3 * 8 * 12 + 3 * 8 + 3,), 3: (2 * 16 * 4 + 2 * 16 + 2,)}


def test_a_reused_state_slot_starts_from_zero(emulated):
    from tgo_b200.engine.step import StepEntry
    cfg, page = dt.CONFIGS["D3"]
    W = dt.make_weights(cfg, 4)
    eng = _engine(cfg, W, page, 64, slots=1)
    first, second = [3, 7, 11, 2, 9, 30, 1], [5, 1, 8, 40]
    for rid, toks in (("a", first), ("b", second)):
        eng.admit(rid)
        got = eng.step([StepEntry(rid, toks, list(range(len(toks))))]).numpy()
        want = plain.forward(cfg, W, toks)
        assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
        eng.finish(rid)


def test_a_failing_step_leaves_the_state_alone(emulated, monkeypatch):
    from tgo_b200.engine.step import StepEntry
    from tgo_b200.kernels import ops
    cfg, page = dt.CONFIGS["D1"]
    W = dt.make_weights(cfg, 5)
    eng = _engine(cfg, W, page, 64, slots=2)
    toks = [4, 9, 60, 33, 2, 17, 5, 80, 41]
    eng.admit("a")
    eng.step([StepEntry("a", toks[:4], [])])
    good = ops.mlstm_chunked
    calls = []

    def failing(*a, **k):
        calls.append(1)
        good(*a, **k)
        if len(calls) == 2:              # the last layer's memory: the first has moved already
            raise RuntimeError("no")
    monkeypatch.setattr(ops, "mlstm_chunked", failing)
    with pytest.raises(RuntimeError):
        eng.step([StepEntry("a", toks[4:], [])])
    assert len(calls) == 2
    monkeypatch.setattr(ops, "mlstm_chunked", good)
    assert eng.length("a") == 4
    got = eng.step([StepEntry("a", toks[4:], list(range(5)))]).numpy()
    want = plain.forward(cfg, W, toks)[4:]
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
