"""Small Dasusun configurations for the tests.  They differ from one another in every size and option: heads (also
one), unrotated / rotated / value sizes that are all different, latent sizes, windows (none, 1, shorter than a page,
a page exactly, a page and one, several pages), rotation with and without stretching and over fewer entries than the
rotated part holds, layers without feed-forward, convolutions of 1, 2 and 4 taps and none, widths that are no power of
two."""

import copy

_SCALING_A = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}
_SCALING_B = {"factor": 1.5, "original": 256, "fast": 24.0, "slow": 0.5}


def _mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, rot_dims, base, scaling, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    return m


def _layer(mixer, ff):
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


DAS_A = {
    "architecture": "Dasusun", "vocab": 320, "width": 96, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
    "layers": [
        _layer(_mixer(3, 24, 8, 40, 48, 56, 17, 8, 10000.0, _SCALING_A), 160),
        _layer(_mixer(2, 16, 16, 8, 64, 32, None, 8, 500.0, None, scale=0.3), None),
        _layer(_mixer(1, 32, 8, 16, 24, 40, 70, 8, 10000.0, _SCALING_A), 104),
    ],
}

DAS_B = {
    "architecture": "Dasusun", "vocab": 200, "width": 72, "norm": {"eps": 1e-6}, "canon": {"taps": 2},
    "layers": [
        _layer(_mixer(4, 8, 24, 16, 40, 24, 64, 24, 150000.0, _SCALING_B), 96),
        _layer(_mixer(2, 40, 8, 24, 16, 48, 65, 4, 100.0, None), 200),
        _layer(_mixer(2, 16, 8, 16, 32, 32, 1, 8, 10000.0, None), None),
        _layer(_mixer(5, 8, 8, 8, 56, 16, 200, 8, 10000.0, _SCALING_B), 64),
    ],
}

DAS_C = copy.deepcopy(DAS_A)  # one tap: the convolution only scales its input and keeps no state
DAS_C["canon"] = {"taps": 1}
DAS_C["norm"] = {"eps": 1e-3}

DAS_D = copy.deepcopy(DAS_B)  # no convolution at all
del DAS_D["canon"]
DAS_D["layers"] = DAS_D["layers"][:2]

# Sizes the tensor-core attention kernel takes in bfloat16 (latents of 64 and 128, rotated parts of 16 and 32), with head
# counts that do not divide its sixteen-row tiles and one above sixteen.
DAS_E = {
    "architecture": "Dasusun", "vocab": 256, "width": 128, "norm": {"eps": 1e-6}, "canon": {"taps": 3},
    "layers": [
        _layer(_mixer(3, 16, 16, 24, 64, 64, 44, 16, 300000.0, _SCALING_B), 256),
        _layer(_mixer(20, 8, 32, 8, 32, 128, 130, 16, 10000.0, None), 128),
        _layer(_mixer(5, 24, 16, 16, 48, 64, None, 16, 10000.0, _SCALING_A), None),
        _layer(_mixer(16, 16, 16, 16, 64, 64, 64, 8, 1000.0, None), 192),
    ],
}

DAS_CONFIGS = {"das_e": DAS_E, "das_a": DAS_A, "das_b": DAS_B, "das_c": DAS_C, "das_d": DAS_D}
