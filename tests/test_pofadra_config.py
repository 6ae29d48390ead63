"""Pofadra without a GPU: the configuration and its errors, the plan's tensors and cache requests, sizes that a tensor's
shape gives, and the plain implementation's own mechanisms on cases small enough to work out by hand."""

import copy
import math

import pytest
import torch

from tests.plain import pofadra as plain
from tests.pofadra_configs import POF_A, POF_B, POF_CONFIGS


def _model(raw, dtype=torch.float32):
    from gtar_kimik3_public_b200.models.model import Model
    from gtar_kimik3_public_b200.registry import architecture, config_from_dict

    config = config_from_dict(raw)
    return Model(architecture("Pofadra").build_plan(config), config, dtype, "cpu")


@pytest.mark.parametrize("tag", sorted(POF_CONFIGS))
def test_configurations_are_read_and_give_their_tensors(tag):
    raw = POF_CONFIGS[tag]
    model = _model(raw)
    specs = model.tensor_specs()
    assert specs["embed"].shape == (raw["vocab"], raw["width"]) and specs["head"].shape == (raw["vocab"], raw["width"])
    assert specs["final.norm"].shape == (raw["width"],)
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        assert specs[f"l{i}.norm1"].shape == (raw["width"],)
        if layer["type"] == "channel_delta":
            assert specs[f"l{i}.mix.q"].shape == (m["kv_heads"] * m["dim"], raw["width"])
            assert specs[f"l{i}.mix.v.conv"].shape == (m["heads"] * m["vdim"], m["conv"])
            assert specs[f"l{i}.mix.dt_bias"].shape == (m["heads"] * m["dim"],)
            assert specs[f"l{i}.mix.a1"].free == (0,) and specs[f"l{i}.mix.g2"].free == (1,)
        else:
            assert specs[f"l{i}.mix.k.norm"].shape == (m["kv_heads"] * m["dim"],)
            assert f"l{i}.mix.v" not in specs
        if layer["mlp"] is None:
            assert not any(name.startswith(f"l{i}.mlp.") for name in specs)
        else:
            r = layer["mlp"]["router"]
            assert specs[f"l{i}.mlp.e{r['experts'] - 1}.down"].shape == (raw["width"], layer["mlp"]["expert"]["ff"])
            assert specs[f"l{i}.mlp.correction"].shape == (r["experts"],)
    assert model.graph_safe()


def test_cache_requests_follow_the_layers():
    from gtar_kimik3_public_b200.parts.base import KVRequest, StateRequest

    requests = _model(POF_A).cache_layout().requests
    assert requests[0] == [StateRequest((4, 24, 40), torch.float32), StateRequest((2, 2 * 2 * 24 + 4 * 40), torch.float32)]
    assert requests[1] == KVRequest(2, 16, 17)
    assert requests[2] == [StateRequest((2, 64, 16), torch.float32)]  # one tap: the convolution keeps nothing
    assert _model(POF_B).cache_layout().requests[4] == KVRequest(1, 32, None)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="rnn"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "cannot be chosen"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "cannot be chosen"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not a feed-forward"),
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "missing keys"),
    (lambda c: c["layers"][1]["mixer"].update(bias=True), "unknown keys"),
    (lambda c: c["norm"].pop("eps"), "missing keys"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_configuration_errors_name_the_key(change, message):
    from gtar_kimik3_public_b200.config.base import ConfigError
    from gtar_kimik3_public_b200.registry import config_from_dict

    raw = copy.deepcopy(POF_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_a_file_chooses_the_low_rank_sizes(tmp_path):
    """The inner sizes of the delta rule's low-rank paths stand in no config: a folder whose tensors have other sizes
    than the random-weights mode's default passes the loader's check, and halves that do not meet are refused."""
    from gtar_kimik3_public_b200.weights.loader import WeightsError, check_tensors

    model = _model(POF_A)
    specs = model.tensor_specs()
    shapes = {name: spec.shape for name, spec in specs.items()}
    dtypes = {name: torch.bfloat16 for name in specs}
    shapes["l0.mix.a1"], shapes["l0.mix.a2"] = (7, 96), (4 * 24, 7)
    check_tensors(tmp_path, specs, shapes, dtypes)
    shapes["l0.mix.a1"] = (7, 95)
    with pytest.raises(WeightsError):
        check_tensors(tmp_path, specs, shapes, dtypes)
    mixer = model.plan.layers[0].mixer
    tensors = {name: torch.zeros(spec.shape) for name, spec in mixer.tensor_specs().items()}
    tensors["a1"], tensors["a2"] = torch.zeros(7, 96), torch.zeros(96, 9)
    with pytest.raises(ValueError, match="do not meet"):
        mixer.load(tensors)
    tensors["a2"] = torch.zeros(96, 7)
    mixer.load(tensors)
    assert mixer.decay_rank == 7 and mixer.w_low2.shape == (4 * 24 + 4 * 40, mixer.w_low1.shape[0])


def test_plain_delta_recurrence_by_hand():
    """d = 1, dv = 1: S_t = g S + k beta (v - g S k), o = S q."""
    q = torch.tensor([[1.0], [2.0]], dtype=torch.float64)
    k = torch.tensor([[1.0], [0.5]], dtype=torch.float64)
    v = torch.tensor([[3.0], [-1.0]], dtype=torch.float64)
    g = torch.tensor([[0.5], [0.25]], dtype=torch.float64)
    beta = torch.tensor([0.5, 1.0], dtype=torch.float64)
    s1 = 0.5 * 3.0
    s2 = 0.25 * s1 + 0.5 * (-1.0 - 0.25 * s1 * 0.5)
    out = plain.delta_recurrence(q, k, v, g, beta)
    assert torch.allclose(out, torch.tensor([[s1], [2.0 * s2]], dtype=torch.float64))


def test_plain_route_by_hand():
    """Two groups of two; the group whose two choice scores add up higher is kept, although the single best expert sits in
    the other; the weights are the scores without the correction, times the constant."""
    w = {"r.router": torch.eye(4, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, 0.3, 0.3], dtype=torch.float64)}
    h = torch.tensor([[2.0, -3.0, 0.5, 0.4]], dtype=torch.float64)
    chosen, weight = plain.route(h, w, "r.", {"experts": 4, "top": 1, "scale": 2.0, "groups": {"count": 2, "keep": 1}})
    s = torch.sigmoid(h[0])
    assert (s[0] + s[1]) < (s[2] + s[3] + 0.6)
    assert chosen.tolist() == [[2]] and math.isclose(weight.item(), 2.0 * s[2].item())
    chosen, weight = plain.route(h, w, "r.", {"experts": 4, "top": 2, "scale": 1.0})  # no groups: the corrected scores decide
    assert chosen[0].tolist() == [2, 3] and torch.allclose(weight[0], s[2:4])


def test_plain_window_attention_sink_and_window():
    """With one head of size 8, weights that pass the input through and a zero gate weight (sigmoid = 1/2), the output of
    token i is half the softmax-with-sink average of the visible keys as projected."""
    T, d = 6, 8
    w = {"m.q": torch.eye(d, dtype=torch.float64), "m.k": torch.eye(d, dtype=torch.float64), "m.g": torch.zeros(d, d, dtype=torch.float64),
         "m.o": torch.eye(d, dtype=torch.float64), "m.q.norm": torch.ones(d, dtype=torch.float64), "m.k.norm": torch.ones(d, dtype=torch.float64)}
    h = torch.randn(T, d, generator=torch.Generator().manual_seed(0), dtype=torch.float64)
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 0.7, "mask": {"size": 3}}
    out = plain.window_attention(h, w, "m.", m, 1e-6)
    n = plain.rms(h, 1e-6)
    for i in range(T):
        seen = list(range(max(0, i - 2), i + 1))
        e = torch.tensor([math.exp(0.7 * float(n[i] @ n[j])) for j in seen], dtype=torch.float64)
        want = 0.5 * sum((e[a] / (1.0 + e.sum())) * h[j] for a, j in enumerate(seen))
        assert torch.allclose(out[i], want, atol=1e-12)
