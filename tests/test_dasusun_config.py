"""Host-side pieces of the Dasusun decoder: its configuration and registry entry, the tensors its plan asks for, the
random-weights mode and the loader's repacking, the stretched rotation's frequencies, and the cache's row pages with
windows and convolution states."""

import copy
import json

import pytest
import torch

from gtar_kimik3_public_b200.cache import Cache
from gtar_kimik3_public_b200.config import ConfigError
from gtar_kimik3_public_b200.models.model import Model
from gtar_kimik3_public_b200.parts.base import RowsRequest, StateRequest, build_part
from gtar_kimik3_public_b200.registry import architecture, config_from_dict, config_from_file
from gtar_kimik3_public_b200.weights import load_weights, write_random_model
from tests.dasusun_configs import DAS_A, DAS_B, DAS_C, DAS_D
from tests.plain import dasusun as plain
from tests.plain.weights import read_safetensors


def _model(raw, dtype=torch.float32):
    config = config_from_dict(raw)
    return Model(architecture(config.ARCH_NAMES[0]).build_plan(config), config, dtype, "cpu")


def test_config_is_chosen_by_its_architecture_key_and_read_whole(tmp_path):
    config = config_from_dict(DAS_A)
    assert type(config).__name__ == "DasusunConfig" and config.vocab == 320 and config.width == 96
    assert config.eps == 1e-5 and config.taps == 4 and len(config.layers) == 3
    assert config_from_dict(DAS_D).taps == 0
    (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
    assert config_from_file(tmp_path) == config


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].__setitem__("type", "sliding_sum"), "mixer"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "feed-forward"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c.__setitem__("depth", 3), "depth"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = copy.deepcopy(DAS_A)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_plan_asks_for_the_files_tensors():
    specs = _model(DAS_A).tensor_specs()
    assert specs["embed"].shape == (320, 96) and specs["final.norm"].shape == (96,)
    assert specs["l0.mix.dkv"].shape == (56 + 8, 96) and specs["l0.mix.uq"].shape == (3 * 32, 48)
    assert specs["l0.mix.uk"].shape == (3 * 24, 56) and specs["l0.mix.uv"].shape == (3 * 40, 56)
    assert specs["l0.mix.o"].shape == (96, 120) and specs["l0.mix.dq.norm"].shape == (48,)
    assert specs["l0.canon1"].shape == (96, 4) and specs["l2.dwa"].shape == (4,) and specs["l0.dwa"].shape == (2,)
    assert specs["l0.mlp.up"].shape == (160, 96) and specs["l0.ls2"].shape == (96,)
    assert not any(name.startswith("l1.mlp") or name in ("l1.norm2", "l1.norm2b", "l1.ls2") for name in specs)  # no feed-forward
    assert "l0.canon1" not in _model(DAS_D).tensor_specs()
    assert [n for n, s in specs.items() if s.optional] == ["lm_head.weight"]  # logits go through the embedding table


def test_random_folder_loads_and_norm_weights_are_offsets(tmp_path):
    config = config_from_dict(DAS_B)
    write_random_model(tmp_path, config, seed=3, std=0.05)
    stored = read_safetensors(tmp_path / "model.safetensors")
    model = _model(DAS_B)
    load_weights(model, tmp_path)
    block = model.plan.layers[0]
    assert torch.allclose(block.norm_in.weight, 1.0 + stored["l0.norm1"].float())
    assert torch.allclose(model.plan.final_norm.weight, 1.0 + stored["final.norm"].float())
    assert torch.equal(block.mixer.q_norm, stored["l0.mix.dq.norm"].float())  # the latents' norms: plain weights
    m = DAS_B["layers"][0]["mixer"]
    assert block.mixer.w_down.shape == (m["q_rank"] + m["kv_rank"] + m["rot_dim"], 72)
    uk = stored["l0.mix.uk"].float().view(m["heads"], m["dim"], m["kv_rank"])
    assert torch.equal(block.mixer.w_uk_t.float(), uk.transpose(1, 2))
    assert model.plan.head.weight is model.plan.embedding.weight
    assert model.plan.layers[2].feed_forward is None and model.plan.layers[2].mixer.window == 1


def test_layers_with_the_same_rotation_share_tables():
    plan = _model(DAS_B).plan
    assert len(plan.positions) == 4
    plan = _model(DAS_A).plan
    assert plan.layers[0].mixer.position is plan.layers[2].mixer.position and len(plan.positions) == 2


@pytest.mark.parametrize("dims,base,scaling", [
    (16, 200000.0, {"factor": 3.0, "original": 1024, "fast": 20.0, "slow": 1.5}),
    (8, 10000.0, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}),
    (24, 100.0, {"factor": 1.5, "original": 256, "fast": 24.0, "slow": 0.5}),
])
def test_stretched_frequencies(dims, base, scaling):
    part = build_part("position", "rope_scaled", dim=dims, base=base, **scaling)
    f, mag = plain.rotary_frequencies(dims, base, scaling)
    assert torch.allclose(part.inv_freq().double(), f, rtol=1e-5, atol=0)
    assert abs(part.magnitude() - mag) < 1e-12
    part.prepare(50, torch.device("cpu"))
    angle = torch.arange(51, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(part.cos[:51].double(), angle.cos() * mag, atol=1e-4)


def test_cache_rows_windows_and_states():
    layout = _model(DAS_A).cache_layout()
    assert layout.requests[0] == [RowsRequest(64, 17), StateRequest((3, 96), torch.float32)]
    assert layout.requests[1][0] == RowsRequest(48, None)
    assert _model(DAS_C).cache_layout().requests[0] == RowsRequest(64, 17)  # one tap keeps no state
    cache = Cache(layout, max_tokens=512, dtype=torch.float32, device="cpu", max_seqs=3)
    a = cache.open()
    cache.grow(a, 200)
    windowed = next(g for g in cache.kv_groups if g.request.window == 17)
    full = next(g for g in cache.kv_groups if g.request.window is None)
    assert windowed.pages.n_used == 4 and full.pages.n_used == 4
    cache.grow(a, 1)  # the next step: pages wholly before the window go back
    assert windowed.pages.n_used == 2 and full.pages.n_used == 4  # positions 184 to 200 lie in two pages
    rows, state = cache.view(0)
    assert rows.rows.shape[1:] == (64, 64) and state.shape == (3, 3, 96)
    state[a].fill_(5.0)
    cache.close(a)
    b = cache.open()
    assert b == a and torch.count_nonzero(cache.view(0)[1][b]) == 0  # a slot used again starts from zero state
    cache.check_invariants()
    assert cache.kv_bytes_per_token() == 4 * (64 + 48 + 48)
