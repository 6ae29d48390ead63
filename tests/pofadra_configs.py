"""Small Pofadra configurations for the tests.  They differ from one another in every size and option: layer orders,
head counts (value heads that share key heads, and one of each), key and value sizes that differ and are no power of
two, convolutions of 1 to 4 taps, windows (1, shorter than a page, a page exactly, a page and one, several pages, none),
rotation over part of a head and over all of it and none, experts in one, two and three groups with one or more kept,
one or several experts a token, layers without feed-forward, widths that are no power of two, embedding scales and
logit caps of several sizes and none."""


def _delta(heads, kv_heads, dim, vdim, conv, **ranks):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, **ranks}


def _attention(heads, kv_heads, dim, scale, window=None, rot_dims=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if window:
        m["mask"] = {"size": window}
    return m


def _moe(ff, experts, top, scale, count=None, keep=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


POF_A = {
    "architecture": "Pofadra", "vocab": 320, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.7}, "logit_softcap": 12.0,
    "layers": [
        _layer("channel_delta", _delta(4, 2, 24, 40, 3, decay_rank=12, gate_rank=20), _moe(48, 6, 2, 2.5, 3, 2)),
        _layer("attention", _attention(6, 2, 16, 0.3, window=17, rot_dims=8, base=100.0), _moe(40, 4, 1, 1.0)),
        _layer("channel_delta", _delta(2, 2, 64, 16, 1), None),
        _layer("attention", _attention(2, 2, 40, 0.2, window=70, rot_dims=40), _moe(56, 10, 3, 0.7, 5, 2)),
    ],
}

POF_B = {
    "architecture": "Pofadra", "vocab": 200, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.25},
    "layers": [
        _layer("attention", _attention(3, 1, 24, 0.25, window=64, rot_dims=4, base=500000.0), _moe(32, 9, 4, 1.2, 3, 2)),
        _layer("channel_delta", _delta(3, 1, 132, 36, 4), _moe(24, 5, 5, 0.5)),
        _layer("attention", _attention(4, 4, 8, 0.5, window=1, rot_dims=8), None),
        _layer("channel_delta", _delta(5, 5, 8, 8, 2), _moe(64, 2, 1, 3.0, 2, 2)),
        _layer("attention", _attention(2, 1, 32, 0.18, window=None, rot_dims=None), _moe(16, 12, 2, 1.0, 4, 1)),
    ],
}

# Sizes the tensor-core attention kernels take in bfloat16 (heads of 64 and 128), windows around page borders.
POF_C = {
    "architecture": "Pofadra", "vocab": 256, "width": 128, "norm": {"eps": 1e-6}, "logit_softcap": 50.0,
    "layers": [
        _layer("attention", _attention(4, 2, 64, 0.125, window=65, rot_dims=32), _moe(64, 4, 2, 1.0)),
        _layer("channel_delta", _delta(2, 1, 128, 128, 4), _moe(128, 4, 2, 1.0, 2, 1)),
        _layer("attention", _attention(2, 1, 128, 0.09, window=130, rot_dims=64, base=1000.0), None),
        _layer("attention", _attention(8, 1, 64, 0.125, window=200, rot_dims=16), _moe(32, 16, 4, 2.0, 4, 2)),
    ],
}

# One layer of each kind alone, without feed-forward: a mixer's fault cannot hide behind another's
POF_DELTA = {
    "architecture": "Pofadra", "vocab": 128, "width": 64, "norm": {"eps": 1e-6},
    "layers": [_layer("channel_delta", _delta(3, 3, 20, 28, 4), None)],
}
POF_ATTN = {
    "architecture": "Pofadra", "vocab": 128, "width": 64, "norm": {"eps": 1e-6},
    "layers": [_layer("attention", _attention(4, 2, 24, 0.2, window=33, rot_dims=12), None)],
}

POF_CONFIGS = {"pof_a": POF_A, "pof_b": POF_B, "pof_c": POF_C, "pof_delta": POF_DELTA, "pof_attn": POF_ATTN}


def _every_expert(config):
    """The same model with every expert chosen for every token (all groups kept).  Which experts a token uses is then no
    close call that 16-bit products could settle either way, while the scores still weigh the experts token by token: the
    bfloat16 runs use these, the float32 runs and the router's own tests cover the choice."""
    import copy

    out = copy.deepcopy(config)
    for layer in out["layers"]:
        if layer["mlp"] is not None:
            router = layer["mlp"]["router"]
            router["top"] = router["experts"]
            if "groups" in router:
                router["groups"]["keep"] = router["groups"]["count"]
    return out


POF_CONFIGS.update({tag + "_all": _every_expert(config) for tag, config in list(POF_CONFIGS.items())})
