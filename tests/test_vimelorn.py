"""Vimelorn without a GPU: the config reader and its refusals, the declared tensor names, the
plain statement's pieces against values worked out by hand, and the engine's host side (cache
groups with kept first pages, the convolution's state rows, packing, portions, mixed batches,
reused pages and slots) with torch stand-ins for the kernels, against the plain statement."""
import copy
import math

import numpy as np
import pytest
import torch

import emulated_kernels
import plain_vimelorn as plain
import tiny
import vimelorn_tiny as vt


def test_reader_builds_the_layers_the_file_lists():
    from tgo_b200.registry import model_spec_from_config
    spec = model_spec_from_config(vt.V1)
    assert spec.architecture == "Vimelorn" and not spec.tied_head and len(spec.layers) == 3
    assert [ls.block for ls in spec.layers] == ["hyper_connections"] * 3
    assert all(ls.streams == 3 for ls in spec.layers) and spec.embedding_scale == 3.0
    win = spec.layers[0].mixer
    assert (win.kind, win.num_heads, win.num_kv_heads, win.head_dim, win.value_dim) == \
        ("sink_attention", 4, 2, 12, 20)
    assert (win.window, win.keep_first, win.conv_taps, win.qk_unit_norm, win.scale) == (7, 2, 3, True, 0.3)
    assert win.position.kind == "rope_half_split" and win.position.rotary_dim == 8
    assert win.position.theta == 500.0 and not win.qk_norm and win.distance_bias_max is None
    cau = spec.layers[1].mixer
    assert cau.qk_norm and cau.qk_norm_scope == "row" and cau.position is None and cau.window is None
    assert cau.query_temperature == (0.4, 5) and cau.distance_bias_max == 30 and not cau.qk_unit_norm
    ff = spec.layers[1].feed_forward
    assert (ff.kind, ff.experts, ff.identity_experts, ff.top, ff.intermediate_size) == \
        ("routed_experts", 5, 1, 2, 24)
    assert not ff.gated and ff.router_scores == "all" and ff.router_correction and ff.shared_gate
    assert ff.activation == "relu_squared" and ff.shared.kind == "plain_dense"
    assert ff.shared.intermediate_size == 28 and ff.shared.activation == "relu_squared"
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.kind == "gated_dense"
    assert spec.layers[2].mixer.keep_first == 0
    bare = model_spec_from_config(vt.V5)
    assert [ls.block for ls in bare.layers] == ["prenorm_residual"] * 2 and bare.embedding_scale == 1.0
    assert bare.layers[0].mixer.position is None
    lone = model_spec_from_config(vt.V2)
    assert lone.layers[0].streams == 1 and lone.layers[0].feed_forward.shared is None
    assert not lone.layers[0].feed_forward.shared_gate and lone.layers[0].feed_forward.identity_experts == 0


def _changed(path, value, base=None):
    cfg = copy.deepcopy(base or vt.V1)
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
    (("streams",), 9, "streams"), (("streams",), 0, "streams"),
    (("embedding", "scale"), float("inf"), "embedding.scale"),
    (("layers", 0, "type"), "mamba", "layers[0].type"),
    (("layers", 0, "mixer", "heads"), ..., "heads"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 14, "rot.dims"),
    (("layers", 0, "mixer", "rot", "base"), ..., "rot.base"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mixer", "mask", "keep_first"), -1, "mask.keep_first"),
    (("layers", 0, "mixer", "conv"), 65, "conv"), (("layers", 0, "mixer", "scale"), ..., "scale"),
    (("layers", 1, "mixer", "bias_max"), ..., "bias_max"),
    (("layers", 1, "mixer", "q_temp", "every"), 0, "q_temp.every"),
    (("layers", 1, "mixer", "q_temp", "coef"), "big", "q_temp.coef"),
    (("layers", 1, "mlp", "kind"), "sparse", "mlp.kind"),
    (("layers", 1, "mlp", "router", "top"), 7, "router.top"),
    (("layers", 1, "mlp", "router", "identity"), -2, "router.identity"),
    (("layers", 1, "mlp", "expert"), ..., "mlp.expert"), (("layers", 0, "mlp", "ff"), ..., "mlp.ff"),
])
def test_reader_refuses_by_key(path, value, word):
    from tgo_b200.config.qwen3 import ConfigError
    from tgo_b200.registry import model_spec_from_config
    with pytest.raises(ConfigError) as err:
        model_spec_from_config(_changed(path, value))
    assert word in str(err.value)


@pytest.mark.parametrize("name", sorted(vt.CONFIGS))
def test_declared_tensors_are_the_weights_the_tests_make(name):
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    cfg, _ = vt.CONFIGS[name]
    W = vt.make_weights(cfg, 1, vt.REL_ROWS[name])
    model = Model(model_spec_from_config(cfg), torch.float32, "cpu")
    declared = {w.name: tuple(w.shape) for w in model.weight_specs() if not w.optional}
    assert set(declared) == set(W)
    for k, shape in declared.items():                       # -1: the tensor's own shape gives it
        assert len(shape) == W[k].ndim and all(a in (-1, b) for a, b in zip(shape, W[k].shape)), k


def test_a_written_folder_loads(tmp_path):
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    from tgo_b200.weights.binder import WeightError, load_weights
    from tgo_b200.weights.safetensors import SafetensorsRepo
    W = vt.make_weights(vt.V1, 2, 10)
    d = vt.write_model_dir(str(tmp_path / "m"), vt.V1, W)
    model = Model(model_spec_from_config(vt.V1), torch.bfloat16, "cpu")
    weights = load_weights(model.weight_specs(), SafetensorsRepo(d), torch.bfloat16, "cpu", None, log=None)
    assert weights["l0.hc1.mix"].dtype == torch.float32 and weights["l0.hc1.mix"].shape == (3, 3)
    assert weights["l1.mix.rel"].dtype == torch.float32 and weights["l1.mlp.correction"].dtype == torch.float32
    assert weights["l0.mix.q.conv"].dtype == torch.float32 and weights["l0.mix.q"].dtype == torch.bfloat16
    model.bind(dict(weights))
    att = model.blocks[1].mixer
    # the distance table is laid out by distance: row n is the table's bucket of n, the last
    # row stands for everything farther
    assert att.dist_bias.shape[1] == 3 and att.dist_bias.shape[0] <= 31
    for n in range(att.dist_bias.shape[0]):
        assert torch.equal(att.dist_bias[n], torch.from_numpy(
            W["l1.mix.rel"][plain.distance_bucket(n, 10, 30)]).float())
    assert plain.distance_bucket(att.dist_bias.shape[0] - 1, 10, 30) == 9
    ff = model.blocks[1].feed_forward
    assert ff.w_router.shape == (5 + 1 + 1, 48) and ff.w_gate is None and ff.w_up.shape == (5, 24, 48)
    assert torch.equal(ff.w_router[6], torch.from_numpy(W["l1.mlp.shared.sg"][0]).float())
    # the three convolutions lie side by side in the order of the joined projection's rows
    conv = model.blocks[0].mixer.conv
    assert conv.shape == (4 * 12 + 2 * 12 + 2 * 20, 3)
    assert torch.equal(conv[48:72], torch.from_numpy(W["l0.mix.k.conv"]).float())
    # a layer without a feed-forward ships no second norm and no second set of coefficients
    W2 = dict(W)
    W2["l2.hc2.in"] = W["l0.hc2.in"]
    d2 = vt.write_model_dir(str(tmp_path / "m2"), vt.V1, W2)
    with pytest.raises(WeightError):
        load_weights(model.weight_specs(), SafetensorsRepo(d2), torch.bfloat16, "cpu", None, log=None)
    # a distance table of the wrong width is refused, one of another length is taken
    W3 = dict(W)
    W3["l1.mix.rel"] = W["l1.mix.rel"][:, :2]
    with pytest.raises(WeightError):
        load_weights(model.weight_specs(), SafetensorsRepo(vt.write_model_dir(str(tmp_path / "m3"), vt.V1, W3)),
                     torch.bfloat16, "cpu", None, log=None)
    W4 = dict(W)
    W4["l1.mix.rel"] = np.concatenate([W["l1.mix.rel"], W["l1.mix.rel"][:4]])
    load_weights(model.weight_specs(), SafetensorsRepo(vt.write_model_dir(str(tmp_path / "m4"), vt.V1, W4)),
                 torch.bfloat16, "cpu", None, log=None)


def test_plain_pieces_by_hand():
    assert np.allclose(plain.rmsnorm(np.array([[3.0, 4.0]]), np.array([1.0, 2.0]), 0.0),
                       [[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]])
    # the convolution: the last tap meets the current token, zeros before the start
    u = np.array([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]])
    w = np.array([[100.0, 10.0, 1.0], [0.0, 0.0, 2.0]])
    assert np.allclose(plain.short_conv(u, w), [[1, 20], [12, 40], [123, 60]])
    # half-split pairs (i, i + dims/2); the rest passes
    x = np.array([[[1.0, 2.0, 0.0, 0.0, 7.0]]])
    assert np.allclose(plain.rotate_half_split(np.repeat(x, 2, 0), [0, 1], 4, 1.0)[0], x[0])
    got = plain.rotate_half_split(np.repeat(x, 2, 0), [0, math.pi / 2], 4, 1.0)[1, 0]
    assert np.allclose(got, [0, 0, 1, 2, 7], atol=1e-12)      # base 1: both pairs turn by the position
    # the window and the kept first tokens
    vis = plain.visible_window_keep(8, 3, 2)
    assert vis[7].tolist() == [True, True, False, False, False, True, True, True]
    assert vis[3].tolist() == [True, True, True, True, False, False, False, False]
    assert plain.visible_window_keep(4, 1, 0)[3].tolist() == [False, False, False, True]
    # the buckets of a table of 8 rows up to distance 64: exact below 4, then four logarithmic
    # steps of 64/4 = 16 -> a factor of 2 each
    assert [plain.distance_bucket(n, 8, 64) for n in (0, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == \
        [0, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]
    # the temperature: 1 until position every - 1 has passed
    assert np.allclose(plain.query_temperature([0, 2, 3, 7], 0.5, 4), [1, 1, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3)])
    # routing: scores 0.5, 0.3, 0.2 (the last an identity expert); a correction of 0.25 on the
    # third makes it second choice, its weight stays 0.2 / (0.5 + 0.2)
    W = {"router": np.log(np.array([[0.5], [0.3], [0.2]])), "correction": np.array([0.0, 0.0, 0.25]),
         "e0.up": np.array([[2.0]]), "e0.down": np.array([[3.0]]), "e1.up": np.array([[1.0]]),
         "e1.down": np.array([[1.0]])}
    mlp = {"router": {"experts": 2, "identity": 1, "top": 2}}
    chosen, wts = plain.route(np.array([[1.0]]), W, "", mlp["router"])
    assert chosen.tolist() == [[0, 2]] and np.allclose(wts, [[0.5 / 0.7, 0.2 / 0.7]])
    out = plain.routed_feed_forward(np.array([[1.0]]), W, "", mlp)
    assert np.allclose(out, [[0.5 / 0.7 * 12.0 + 0.2 / 0.7 * 1.0]])          # down relu(up)^2, and x itself
    # streams: with in = (1, 0), out = (0, 1) and the identity mix, stream 2 collects the sublayers
    cfg = {"norm": {"eps": 0.0}, "streams": 2, "width": 1, "vocab": 2, "layers": []}
    W = {"embed": np.array([[2.0], [4.0]]), "final.norm": np.array([1.0]), "head": np.array([[1.0], [0.0]])}
    assert np.allclose(plain.forward(cfg, W, [1]), [[1.0, 0.0]])            # the norm of 4 + 4 is 1


# ---------------------------------------------------- the engine's host side on the CPU
@pytest.fixture()
def emulated(monkeypatch):
    emulated_kernels.install(monkeypatch)


def _engine(cfg, W, page_size, max_tokens, slots=4):
    from tgo_b200.engine.step import Engine
    model = vt.bind_model(cfg, W, torch.float32, "cpu")
    return Engine(model, page_size=page_size, max_tokens=max_tokens, num_slots=slots, graphs=False)


def _check(got, cfg, W, requests, tol=2e-4):
    for rid, toks in requests.items():
        want = plain.forward(cfg, W, toks)
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[p]).max() <= tol * max(1.0, np.abs(want[p]).max()), \
                (rid, p)


@pytest.mark.parametrize("name", sorted(vt.CONFIGS))
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_engine_host_side_against_plain(emulated, name, family):
    cfg, page = vt.CONFIGS[name]
    W = vt.make_weights(cfg, 3, vt.REL_ROWS[name])
    requests = tiny.random_requests(cfg["vocab"], [37, 9, 1, 50, 18, 26], seed=5)
    trace = {"whole": tiny.trace_whole, "tail": lambda r: tiny.trace_tail(r, 6),
             "portions": tiny.trace_portions,
             "mixed": lambda r: tiny.trace_mixed(r, seed=2, max_live=3, tail=5)}[family](requests)
    # a pool for what is live at once, three state slots: pages and slots come back and go out again
    eng = _engine(cfg, W, page, tiny.max_tokens_of(trace, page), slots=3)
    owners = [dict() for _ in eng.cache.groups]
    got = tiny.run_trace_engine(eng, trace, poison=True, owners=owners)
    _check(got, cfg, W, requests)
    if family == "mixed":
        assert any(len(ids) > 1 for g in owners for ids in g.values())      # a page was reused


def test_cache_groups_and_state_rows(emulated):
    cfg, page = vt.CONFIGS["V1"]
    eng = _engine(cfg, vt.make_weights(cfg, 3, 10), page, 64)
    kinds = sorted((g.kind, g.window, g.keep_first, g.plane_shapes or g.row_shape) for g in eng.cache.groups)
    assert kinds == [("full", None, 0, ((1, 8), (1, 16))), ("window", 5, 0, ((1, 16), (1, 10))),
                     ("window", 7, 2, ((2, 12), (2, 20)))]
    # the convolutions keep taps - 1 rows of q, k and v side by side
    assert eng.model.state_shapes == {0: (2 * (48 + 24 + 40),), 2: (1 * (32 + 16 + 10),)}


def test_a_reused_state_slot_starts_from_zero(emulated):
    from tgo_b200.engine.step import StepEntry
    cfg, page = vt.CONFIGS["V4"]
    W = vt.make_weights(cfg, 4, 7)
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
    cfg, page = vt.CONFIGS["V1"]
    W = vt.make_weights(cfg, 5, 10)
    eng = _engine(cfg, W, page, 64, slots=2)
    toks = [4, 9, 60, 33, 2, 17, 5, 80, 41]
    eng.admit("a")
    eng.step([StepEntry("a", toks[:4], [])])
    good = ops.qkv_conv_rope_norm_cache
    calls = []

    def failing(*a, **k):
        calls.append(1)
        good(*a, **k)
        if len(calls) == 2:              # the last layer's convolution: the first has moved already
            raise RuntimeError("no")
    monkeypatch.setattr(ops, "qkv_conv_rope_norm_cache", failing)
    with pytest.raises(RuntimeError):
        eng.step([StepEntry("a", toks[4:], [])])
    assert len(calls) == 2
    monkeypatch.setattr(ops, "qkv_conv_rope_norm_cache", good)
    assert eng.length("a") == 4
    got = eng.step([StepEntry("a", toks[4:], list(range(5)))]).numpy()
    want = plain.forward(cfg, W, toks)[4:]
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
