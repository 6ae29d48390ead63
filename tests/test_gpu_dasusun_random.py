"""Dasusun configurations drawn from seeds: sizes, head counts, windows, rotation constants, taps, the order of layers with
and without feed-forward all differ from draw to draw (latents of 64 and 128, which take the tensor-core attention kernel in
bfloat16, are drawn often).  Each runs a schedule of unequal prompts, decoding together, early enders and a second batch in
the first one's slots, every page NaN before, against the plain implementation."""

import tempfile

import pytest
import torch

from tests.plain import dasusun as plain
from tests.plain.weights import read_safetensors

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    gen = torch.Generator().manual_seed(1000 + seed)

    def pick(options):
        return options[int(torch.randint(0, len(options), (1,), generator=gen))]

    width = pick([72, 128, 160, 256, 320])
    layers = []
    for _ in range(pick([2, 3, 5, 7])):
        rot_dim = pick([8, 16, 16, 32, 48])
        dims = pick([d for d in (4, 8, 16, 32, 48) if d <= rot_dim])
        mixer = {"heads": pick([1, 2, 4, 6, 8, 17]), "dim": pick([16, 24, 32, 64, 96]), "rot_dim": rot_dim, "vdim": pick([8, 16, 40, 64]),
                 "q_rank": pick([32, 48, 96, 128]), "kv_rank": pick([24, 64, 64, 128, 128, 192]),
                 "rot": {"base": pick([100.0, 10000.0, 500000.0]), "dims": dims}}
        mixer["scale"] = pick([0.05, 0.125, 0.2, (mixer["dim"] + rot_dim) ** -0.5])
        if pick([True, True, False]):
            mixer["rot"]["scaling"] = {"factor": pick([1.5, 2.0, 8.0]), "original": pick([32, 128, 4096]), "fast": pick([8.0, 32.0]),
                                       "slow": pick([0.5, 1.0, 2.0])}
        window = pick([None, 1, 2, 31, 63, 64, 65, 100, 129])
        if window:
            mixer["mask"] = {"size": window}
        ff = pick([None, 64, 200, 384])
        layers.append({"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None})
    config = {"architecture": "Dasusun", "vocab": pick([97, 300, 1000]), "width": width, "norm": {"eps": pick([1e-6, 1e-5, 1e-3])},
              "layers": layers}
    taps = pick([None, 1, 2, 3, 5])
    if taps:
        config["canon"] = {"taps": taps}
    return config


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_drawn_configuration(seed, dtype):
    from gtar_kimik3_public_b200.engine import Engine, StepEntry
    from gtar_kimik3_public_b200.generate import load
    from gtar_kimik3_public_b200.registry import config_from_dict
    from gtar_kimik3_public_b200.weights import write_random_model

    config = draw_config(seed)
    gen = torch.Generator().manual_seed(seed)
    with tempfile.TemporaryDirectory(prefix="gtar_test_drawn_") as folder:
        write_random_model(folder, config_from_dict(config), seed, std=0.08)
        weights = read_safetensors(folder + "/model.safetensors")
        engine = Engine(load(folder, dtype, "cuda:0"), 1024, max_seqs=3)
    lengths = [int(torch.randint(1, 200, (1,), generator=gen)) for _ in range(6)]
    decoded = [int(torch.randint(0, 70, (1,), generator=gen)) for _ in range(6)]
    requests = [torch.randint(0, config["vocab"], (n + d,), generator=gen).tolist() for n, d in zip(lengths, decoded)]
    for batch in ([0, 1, 2], [3, 4, 5]):
        for group in engine.cache.kv_groups:
            group.k.fill_(float("nan"))
        got = {i: [] for i in batch}
        first = engine.step([StepEntry(i, requests[i][:lengths[i]], list(range(lengths[i]))) for i in batch])
        at = 0
        for i in batch:
            got[i].append(first[at:at + lengths[i]])
            at += lengths[i]
        done = {i: lengths[i] for i in batch}
        engine.end([i for i in batch if done[i] == len(requests[i])])
        while any(done[i] < len(requests[i]) for i in batch):
            live = [i for i in batch if done[i] < len(requests[i])]
            out = engine.step([StepEntry(i, [requests[i][done[i]]], [0]) for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1])
                done[i] += 1
            engine.end([i for i in live if done[i] == len(requests[i])])
        engine.cache.check_invariants()
        for i in batch:
            ids = torch.tensor(requests[i])
            oracle = plain.forward(ids, weights, config, torch.float64)
            mine = torch.cat(got[i]).double().cpu()
            assert torch.isfinite(mine).all(), f"seed {seed} request {i}: logits are not finite"
            err = (mine - oracle).abs().max().item()
            if dtype == "float32":
                assert err < 3e-4, f"seed {seed} request {i}: float32 logits differ from the oracle by {err:.3e}"
            else:
                plain.LOWP = torch.bfloat16
                try:
                    yard = (plain.forward(ids, weights, config, torch.float32).double() - oracle).abs().max().item()
                finally:
                    plain.LOWP = None
                assert err <= 2 * yard + 1e-3, f"seed {seed} request {i}: bfloat16 error {err:.3e} exceeds twice the yardstick {yard:.3e}"
    engine.check()
