"""Fomatar without a device: the configuration's keys and refusals, the plan (schedule of a looped
stretch, cache needs, tensor names against the naming rule), and the plain implementation's own
mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import plain_fomatar as pf
from fomatar_models import CONFIGS, MIXED, PLAIN, FROM_START, random_weights, as_float64, tensor_shapes


def _model(cfg):
    from camelid_b200.engine.model import DecoderModel
    return DecoderModel.from_config(cfg, dtype="float32", device="cpu")


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_follow_the_naming_rule(name):
    cfg = CONFIGS[name]
    specs = _model(cfg).tensor_specs()
    want = tensor_shapes(cfg, ranks=(8, 8))
    assert set(specs) == set(want)
    for n, (shape, _) in want.items():
        free = specs[n].free_dims
        assert all(a == b for i, (a, b) in enumerate(zip(specs[n].shape, shape)) if i not in free), n


def test_schedule_writes_the_looped_stretch_out():
    from camelid_b200.config import load_config
    _, _, plan = load_config(MIXED)
    assert [(e.layer, e.pass_number) for e in plan.schedule] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2),
                                                                 (2, None), (3, None)]
    _, _, plan = load_config(FROM_START)
    assert [(e.layer, e.pass_number) for e in plan.schedule] == [(0, 0), (1, None), (0, 1), (1, None)]
    _, _, plan = load_config(PLAIN)
    assert plan.pass_input is None and [e.layer for e in plan.schedule] == [0, 1]
    assert pf.layer_runs(MIXED) == [(e.layer, e.pass_number) for e in load_config(MIXED)[2].schedule]


def test_every_pass_has_its_own_cache_and_state():
    from camelid_b200.cache import KVSpec, StateSpec, flatten_specs
    m = _model(MIXED)
    needs = [flatten_specs(s) for s in m.entry_cache_specs()]
    assert len(needs) == len(m.schedule) + 1                      # the embedding's previous token comes last
    assert needs[-1] == [StateSpec((1,), "int32", "previous_token")]
    first = needs[0]
    assert KVSpec(2, 24, 9, 40) in first and StateSpec((3, 25, 20), "float32", "memory") in first and StateSpec((3, 25), "float32", "maximum") in first
    assert StateSpec((1, 64), "float32", "shift") in first
    assert needs[1] == needs[3] == needs[5]                       # the same layer, three passes: three entries
    assert StateSpec((4, 20, 12), "float32", "memory") in needs[1] and StateSpec((2, 2 * 24 + 80), "float32", "conv") in needs[1]
    plan = m.memory_plan(256, 4)
    assert plan.cache > 0 and plan.weights == sum(math.prod(s.shape) * 4 for s in m.tensor_specs().values())


def test_configuration_refusals():
    from camelid_b200.config import load_config
    from camelid_b200.errors import ConfigError
    bad = copy.deepcopy(MIXED)
    bad["layers"][1]["type"] = "other"
    with pytest.raises(ConfigError, match=r"layers\[1\].type"):
        load_config(bad)
    bad = copy.deepcopy(MIXED)
    del bad["layers"][0]["mixer"]["left"]["mask"]
    with pytest.raises(ConfigError, match="mask"):
        load_config(bad)
    bad = copy.deepcopy(MIXED)
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        load_config(bad)
    bad = copy.deepcopy(MIXED)
    bad["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="kv_heads"):
        load_config(bad)
    bad = copy.deepcopy(MIXED)
    bad["layers"][0]["mlp"]["kind"] = "routed"
    with pytest.raises(ConfigError, match="mlp.kind"):
        load_config(bad)


def test_low_rank_width_is_the_tensors_own():
    from camelid_b200.weights.loader import check_tensors
    from camelid_b200.errors import WeightsError
    specs = _model(PLAIN).tensor_specs()
    found = {n: (tuple(t.shape), t.dtype) for n, t in random_weights(PLAIN, 0, ranks=(5, 11)).items()}
    check_tensors(specs, found)
    found["l0.mix.q"] = ((1, 72), torch.bfloat16)
    with pytest.raises(WeightsError, match="l0.mix.q"):
        check_tensors(specs, found)


# ---- the plain implementation against closed forms ------------------------------------------------

def test_plain_bigram_rows_and_shift():
    assert pf.bigram_rows([5, 9, 9], {"buckets": 7, "mul_prev": 3, "mul_cur": 2}) == [7, (15 + 18) % 7, (27 + 18) % 7]
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, 0.0]], dtype=torch.float64)
    out = pf.token_shift(h, torch.tensor([0.5, 1.0], dtype=torch.float64))
    assert torch.equal(out, torch.tensor([[0.5, 0.0], [2.0, 2.0], [4.0, 6.0]], dtype=torch.float64))


def test_plain_window_sees_exactly_its_window():
    T, D = 12, 4
    q = torch.zeros(T, 1, D, dtype=torch.float64)
    k = torch.zeros(T, 1, D, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1)
    zero = torch.zeros(1, dtype=torch.float64)
    out = pf.window_scores_core(q, k, v, 1.0, 3, zero, zero)          # equal scores: the mean of the visible values
    assert torch.allclose(out.view(-1)[5:], torch.arange(5, T, dtype=torch.float64) - 1.0)
    assert float(out[0, 0, 0]) == 0.0 and float(out[1, 0, 0]) == 0.5
    # the penalty alone: weights proportional to (1 + r2 d)^(-r1)
    out = pf.window_scores_core(q, k, v, 1.0, 2, torch.tensor([2.0], dtype=torch.float64), torch.tensor([1.0], dtype=torch.float64))
    w_near, w_far = 1.0, 2.0 ** -2.0
    assert math.isclose(float(out[7, 0, 0]), (7 * w_near + 6 * w_far) / (w_near + w_far))


def test_plain_matrix_memory_first_token_and_delta_rule_overwrite():
    q = torch.tensor([[[1.0, 0.0]]], dtype=torch.float64)
    k = torch.tensor([[[2.0, 0.0]]], dtype=torch.float64)
    v = torch.tensor([[[3.0, 5.0]]], dtype=torch.float64)
    # i = -1, f = -2, m0 = 0: m1 = max(-2, -1) = -1; S = e^0 k v^T; n . q = 2; e^(-m1) = e > 2
    out = pf.matrix_memory_core(q, k, v, torch.tensor([[-1.0]], dtype=torch.float64), torch.tensor([[-2.0]], dtype=torch.float64))
    assert torch.allclose(out[0, 0], torch.tensor([6.0, 10.0], dtype=torch.float64) / (math.e + 1e-6))
    # delta rule with beta = 1, no decay: writing (k, v2) after (k, v1) leaves exactly v2 under k
    kk = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]]], dtype=torch.float64)
    vv = torch.tensor([[[1.0, 2.0]], [[7.0, -3.0]]], dtype=torch.float64)
    out = pf.delta_core(kk, kk, vv, torch.ones(2, 1, dtype=torch.float64), torch.ones(2, 1, 2, dtype=torch.float64))
    assert torch.allclose(out[1, 0], vv[1, 0])


def test_plain_forward_is_causal_and_loops():
    P = as_float64(random_weights(MIXED, 3))
    toks = [int(t) for t in torch.randint(0, MIXED["vocab"], (14,), generator=torch.Generator().manual_seed(1))]
    full, layers = pf.forward(toks, P, MIXED, keep_layers=True)
    assert layers.shape[0] == 8 and torch.isfinite(full).all()
    assert torch.allclose(pf.forward(toks[:9], P, MIXED), full[:9], atol=1e-9)
    assert float(full.abs().max()) <= MIXED["logit_softcap"]


def test_random_weights_folder_of_the_library(tmp_path):
    """``write_random_model`` draws every tensor of the design by its init rule: gates, rates and fractions in
    their working ranges, so the plain implementation stays finite on them."""
    import json
    from camelid_b200.weights.random_init import write_random_model
    from camelid_b200.weights.safetensors_io import ModelFiles
    folder = write_random_model(str(tmp_path / "m"), MIXED, seed=3)
    files = ModelFiles(folder)
    P = {n: files.tensor(n).to(torch.float64) for n in files.names()}
    files.close()
    assert set(P) == set(tensor_shapes(MIXED, ranks=(8, 8)))
    assert float(P["l0.mix.left.r2"].min()) > 0 and float(P["l0.shift"].min()) > 0
    with open(tmp_path / "m" / "config.json") as f:
        cfg = json.load(f)
    out = pf.forward([1, 5, 9, 2, 7, 7, 3], P, cfg)
    assert torch.isfinite(out).all() and float(out.abs().max()) > 1e-3
