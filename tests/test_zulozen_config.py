"""The Zulozen decoder without a device: its configuration and plan against the tensor naming rule, refusals,
what the cache keeps for a mixer that sees blocks of positions, and the plain implementation (tests/plain_zulozen.py)
against closed forms."""
import copy

import numpy as np
import pytest

import plain_zulozen as pz
from zulozen_models import CONFIGS, tensor_shapes


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes_follow_the_naming_rule(name):
    from camelid_b200.engine.model import DecoderModel
    model = DecoderModel.from_config(CONFIGS[name], device="cpu")
    specs = {n: tuple(s.shape) for n, s in model.tensor_specs().items()}
    assert specs == {n: tuple(shape) for n, (shape, _) in tensor_shapes(CONFIGS[name]).items()}
    assert model.use_graphs and model.capture_steps           # every part runs inside captured graphs
    assert model.memory_plan(256).total > 0


def test_the_plan_reads_every_size_from_the_configuration():
    from camelid_b200.config.registry import load_config
    arch, cfg, plan = load_config(CONFIGS["mixed"])
    assert arch.name == "Zulozen" and cfg.residual_mult == 0.4 and len(plan.layers) == 4
    l0, l1, l2, l3 = plan.layers
    assert l0.arrangement == "sandwich" and l0.residual_scale == 0.4
    assert l0.mixer.params["chunk"] == 9 and l0.mixer.params["position"].params == {
        "rotary_dim": 8, "theta": 100.0, "scaling": None, "pairing": "interleaved"}
    assert l0.ffn.kind == "dense" and l0.ffn.params["activation"] == "relu_squared" and l0.ffn.params["bias"]
    assert l1.ffn.kind == "routed_experts" and l1.ffn.params["top"] == 2 and l1.ffn.params["shared_size"] == 40
    assert l2.ffn is None and l2.norm2 is None and l2.post_norm2 is None and l2.post_norm1.params["tensor"] == "l2.norm1b"
    assert l3.ffn.params["shared_size"] is None and l3.ffn.params["weight_on"] == "input"
    _, _, open_plan = load_config(CONFIGS["open"])
    assert open_plan.layers[0].mixer.params["chunk"] is None and open_plan.layers[1].mixer.params["position"] is None


@pytest.mark.parametrize("path,value,key", [
    (("layers", 0, "type"), "recurrent", "layers[0].type"),
    (("layers", 0, "mixer", "kv_heads"), 4, "layers[0].mixer.kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "layers[0].mixer.rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 26, "layers[0].mixer.rot.dims"),
    (("layers", 0, "mixer", "mask", "size"), 0, "layers[0].mixer.mask.size"),
    (("layers", 1, "mlp", "router", "top"), 6, "layers[1].mlp.router.top"),
    (("layers", 1, "mlp", "kind"), "sparse", "layers[1].mlp.kind"),
    (("width",), -3, "width"),
])
def test_refusals_name_the_key(path, value, key):
    from camelid_b200.config.registry import load_config
    from camelid_b200.errors import ConfigError
    cfg = copy.deepcopy(CONFIGS["mixed"])
    d = cfg
    for p in path[:-1]:
        d = d[p]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        load_config(cfg)
    assert key in str(e.value)


def test_a_missing_key_is_named():
    from camelid_b200.config.registry import load_config
    from camelid_b200.errors import ConfigError
    cfg = copy.deepcopy(CONFIGS["odd"])
    del cfg["layers"][0]["mixer"]["scale"]
    with pytest.raises(ConfigError) as e:
        load_config(cfg)
    assert "layers[0].mixer.scale" in str(e.value)


def test_the_cache_gives_back_the_pages_before_the_running_block():
    """Blocks of 100 positions over pages of 64: once a sequence is 200 long, nothing before position 200 is read again."""
    from camelid_b200.cache.book import CacheBook, KVSpec
    spec = KVSpec(2, 16, None, None, 100)
    assert spec.forgets and spec.first_visible(0) == 0 and spec.first_visible(99) == 0 and spec.first_visible(100) == 100
    assert spec.first_visible(250) == 200 and KVSpec(2, 16, 30, None, 100).first_visible(250) == 221
    book = CacheBook([spec, KVSpec(2, 16)], n_pages=8, n_slots=2, max_position=10_000)
    s = book.alloc_slot()
    book.check_extend([(s, 199)])
    book.extend(s, 199)
    book.commit(s, 199)
    assert book.pages[0][s][:2] == [-1, 1] and book.pools[0].n_held == 3       # position 199 may still ask for 100..199
    book.check_extend([(s, 1)])
    book.extend(s, 1)
    book.commit(s, 1)                                                            # 200 long: queries from 200 on see 200..
    assert book.pages[0][s][:3] == [-1, -1, -1] and book.pools[0].n_held == 1
    assert book.pools[1].n_held == 4                                             # the group that keeps everything
    book.audit()
    book.free_slot(s)
    assert book.pools[0].n_free == 8 and book.pools[1].n_free == 8


# ---- the plain implementation against closed forms ----

def test_plain_rotation_pairs_neighbours_and_leaves_the_rest():
    x = np.zeros((3, 1, 6))
    x[:, 0, 0], x[:, 0, 2], x[:, 0, 5] = 1.0, 1.0, 7.0
    y = pz.rotate_interleaved(x, [0, 1, 2], 4, 100.0)
    for p in range(3):
        assert np.allclose(y[p, 0, :2], [np.cos(p), np.sin(p)])                 # frequency 1
        assert np.allclose(y[p, 0, 2:4], [np.cos(p * 0.1), np.sin(p * 0.1)])    # frequency 100^(-2/4)
        assert y[p, 0, 4] == 0.0 and y[p, 0, 5] == 7.0


def test_plain_block_mask_and_sink():
    m = pz.block_mask(7, 3)
    assert m[2].tolist() == [True, True, True, False, False, False, False]
    assert m[3].tolist() == [False, False, False, True, False, False, False]
    assert m[5].tolist() == [False, False, False, True, True, True, False]
    assert pz.block_mask(4, None)[3].all()
    w = pz.sink_softmax(np.zeros((2, 2)), pz.block_mask(2, None), np.log(2.0))
    assert np.allclose(w[0], [1 / 3, 0]) and np.allclose(w[1], [1 / 4, 1 / 4])   # the sink counts as two keys of score 0


def test_plain_routing_scales_the_input_not_the_output():
    rng = np.random.default_rng(0)
    W, ff = 6, 4
    t = {"router": np.array([[5.0] + [0.0] * 5, [0.0] * 6, [-5.0] + [0.0] * 5])}
    for n in ("e0", "e1", "e2", "shared"):
        t[n + ".gate"], t[n + ".up"], t[n + ".down"] = rng.normal(size=(ff, W)), rng.normal(size=(ff, W)), rng.normal(size=(W, ff))
    h = np.zeros((1, W))
    h[0, 0], h[0, 1] = 1.0, 0.5
    cfg = {"router": {"experts": 3, "top": 1}, "shared": {"ff": ff}}
    margins = []
    got = pz.routed_ff(h, t, cfg, margins)
    s = 1 / (1 + np.exp(-5.0))
    assert np.allclose(got, pz.gated_expert(s * h, t, "e0") + pz.gated_expert(h, t, "shared"))
    assert not np.allclose(got, s * pz.gated_expert(h, t, "e0") + pz.gated_expert(h, t, "shared"))
    assert np.allclose(margins[0], 5.0)
    assert np.allclose(pz.dense_ff(h, {"up": np.eye(W), "up.b": np.full(W, -0.25), "down": np.eye(W), "down.b": np.ones(W)})[0, :3],
                       [0.75 ** 2 + 1, 0.25 ** 2 + 1, 1.0])
