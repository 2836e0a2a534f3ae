"""Divitar's configuration, its tensor declarations, the rotations' frequencies and the plain implementation's own
consistency (no GPU)."""
import copy
import math

import numpy as np
import pytest

import plain_divitar as pd
from divitar_helpers import MIXED, ODD, ONE_LAYER, WIDE, as_numpy, make_weights, tokens_of


def test_round_trip_and_registry():
    import cbis_b200 as cb
    for cfgd in (MIXED, ODD, WIDE, *ONE_LAYER.values()):
        c = cb.config_from_dict(cfgd)
        assert type(c).__name__ == "DivitarConfig" and cb.config_from_dict(c.to_dict()) == c
        spec = c.model_spec()
        assert [l.arrangement for l in spec.layers] == ["pre_norm_scaled"] * len(cfgd["layers"])
        assert all(l.residual_scale == cfgd.get("residual_mult", 1.0) for l in spec.layers)
        assert all((l.side is None) == ("token_side" not in cfgd) for l in spec.layers)
        assert spec.max_positions == 0 and spec.vocab_size == cfgd["vocab"]
        assert spec.head_spec().params["tensor"] == "head"
        assert spec.head_spec().params["logit_scale"] == cfgd.get("logit_scale", 1.0)
    assert cb.config_from_dict(WIDE).to_dict()["layers"][0] == WIDE["layers"][0]


def test_parts_and_their_constants():
    import cbis_b200 as cb
    layers = cb.config_from_dict(MIXED).model_spec().layers
    assert [l.mixer.kind for l in layers] == ["latent_attention", "rotary_attention", "latent_attention", "rotary_attention",
                                              "latent_attention", "latent_attention"]
    assert [l.cache_source for l in layers] == [None, None, None, None, 0, 2]
    a = layers[1].mixer.params
    assert a["block"] == 23 and a["values_from_keys"] and a["bias"] and a["head_gate"] and a["rot_divide"] == 4.0
    assert a["rot_dims"] == 8 and a["v_head_dim"] == a["head_dim"] == 16
    m = layers[4].mixer.params
    assert m["window"] == 41 and not m["own_latent"] and m["rot_pairs"] == "neighbours" and m["gate"] is None and m["sinks"]
    assert m["rot_blend"] == (4.0, 40, 4.0, 1.0) and layers[2].mixer.params["rot_blend"] is None
    f = layers[1].feed_forward.params
    assert (f["renormalize"], f["renorm_eps"], f["weight_scale"], f["weight_on"], f["shared_inner"]) == (True, 1e-20, 2.5, "output", 40)
    assert layers[2].feed_forward.params["shared_inner"] == 0 and layers[3].feed_forward.kind == "nothing"
    assert layers[0].feed_forward.params["activation"] == "relu2"
    assert [l.side.params["col0"] for l in layers] == [0, 8, 16, 24, 32, 40] and layers[0].side.params["table_width"] == 48
    odd = cb.config_from_dict(ODD).model_spec().layers
    assert odd[2].mixer.params["block"] == 0 and odd[2].mixer.params["rot_dims"] == 0 and odd[3].mixer.params["window"] == 0
    assert odd[3].mixer.params["rot_dim"] == 0 and odd[0].feed_forward.params["weight_scale"] == 1.0


def test_declared_tensors_follow_the_sizes():
    import cbis_b200 as cb
    from cbis_b200.models import Model
    decl = {d.name: tuple(d.shape) for d in Model(cb.config_from_dict(MIXED).model_spec()).declared()}
    assert decl["embed"] == (96, 64) and decl["head"] == (96, 64) and decl["final.norm"] == (64,)
    assert decl["side.embed"] == (96, 48) and decl["l3.side.gate"] == (8, 64) and decl["l3.side.proj"] == (64, 8)
    assert decl["l0.mix.q"] == (2 * 24, 64) and decl["l0.mix.dkv"] == (40, 64) and decl["l0.mix.dkv.norm"] == (32,)
    assert decl["l0.mix.uk"] == (32, 32) and decl["l0.mix.uv"] == (48, 32) and decl["l0.mix.sink"] == (2,)
    assert decl["l0.mix.o"] == (64, 48) and "l0.mix.g" not in decl and decl["l0.mlp.up"] == (80, 64)
    assert decl["l1.mix.q"] == (64, 64) and decl["l1.mix.q.b"] == (64,) and decl["l1.mix.k"] == (32, 64)
    assert decl["l1.mix.k.b"] == (32,) and decl["l1.mix.g"] == (4, 64) and "l1.mix.v" not in decl and "l1.mix.g.b" not in decl
    assert decl["l1.mlp.router"] == (5, 64) and decl["l1.mlp.e4.down"] == (64, 24) and decl["l1.mlp.shared.up"] == (40, 64)
    assert "l2.mlp.shared.up" not in decl and "l3.norm2" not in decl and "l3.mlp.up" not in decl
    assert "l4.mix.dkv" not in decl and decl["l4.mix.uk"] == (32, 32) and decl["l5.mix.uv"] == (72, 24)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "is not one of"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "the values are the keys"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "'scale' is missing"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=3), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "'slow' is missing"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=1), "keeps no latent"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=4), "earlier layer"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=4), "keeps no latent"),
    (lambda c: c["layers"][4]["mixer"].update(kv_rank=16), "differs from layer 0"),
    (lambda c: c["layers"][4]["mixer"]["rot"].update(base=7.0), "differs from layer 0"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "is not one of"),
    (lambda c: c.update(token_side={"dim": 0}), "integer >= 1"),
    (lambda c: c.pop("norm"), "'norm' is missing"),
])
def test_what_a_configuration_refuses(change, message):
    import cbis_b200 as cb
    cfgd = copy.deepcopy(MIXED)
    change(cfgd)
    with pytest.raises(cb.ConfigError, match=message):
        cb.config_from_dict(cfgd)


def test_frequencies_of_both_rotations():
    from cbis_b200.parts.rotation import blended_frequencies, rotary_frequencies
    for base, dims, factor in ((10000.0, 24, 2.0), (50.0, 8, 4.0), (9.0, 2, 1.0)):
        got = rotary_frequencies(base, dims, divide=factor).double().numpy()
        assert np.allclose(got, pd.divided_frequencies(base, dims, factor), rtol=1e-7)
    for base, dims, factor, original, fast, slow in ((5e5, 48, 3.0, 2048, 16.0, 2.0), (100.0, 8, 4.0, 40, 4.0, 1.0),
                                                     (9.0, 6, 1.5, 16, 3.0, 0.5), (1000.0, 64, 8.0, 64, 16.0, 2.0)):
        table, length = blended_frequencies(base, dims, factor, original, fast, slow)
        ref, ref_length = pd.blended_frequencies(base, dims, factor, original, fast, slow)
        assert np.allclose(table.double().numpy(), ref, rtol=1e-7) and length == pytest.approx(ref_length)
        plain = pd.plain_frequencies(base, dims)
        assert np.all(ref <= plain * (1 + 1e-12)) and np.all(ref >= plain / factor * (1 - 1e-12))
    # fast pairs keep their frequency, slow pairs are divided, at least one pair lies between
    ref, _ = pd.blended_frequencies(100.0, 16, 4.0, 40, 4.0, 0.25)
    plain = pd.plain_frequencies(100.0, 16)
    ratio = ref / plain
    assert ratio[0] == 1.0 and ratio[-1] == pytest.approx(0.25) and ((ratio < 1.0) & (ratio > 0.25)).any()


def test_the_plain_implementation_agrees_with_itself():
    """Rows of a prompt do not depend on what follows; a block's first row sees only itself; a window of one token
    gives the token's own value; the residual constant and the logit scale act as plain factors."""
    w = as_numpy(make_weights(MIXED, 3))
    toks = tokens_of(MIXED, 50, 1)
    full, streams, _ = pd.forward(MIXED, w, toks)
    part, _, _ = pd.forward(MIXED, w, toks[:31])
    assert np.abs(full[:31] - part).max() < 1e-9 and streams.shape == (6, 50, 64)
    twice = copy.deepcopy(MIXED)
    twice["logit_scale"] = 2 * MIXED["logit_scale"]
    assert np.allclose(pd.forward(twice, w, toks)[0], 2 * full)
    g = np.random.default_rng(0)
    q, k, v = g.normal(size=(30, 2, 4)), g.normal(size=(30, 1, 4)), g.normal(size=(30, 1, 4))
    out = pd.attention_rows(q, k, v, 0.5, lambda i, j: pd.sees_block(i, j, 7))
    assert np.allclose(out[[0, 7, 14, 28], 0], v[[0, 7, 14, 28], 0])
    out = pd.attention_rows(q, k, v, 0.5, lambda i, j: pd.sees_window(i, j, 1))
    assert np.allclose(out[:, 1], v[:, 0])
    with_sink = pd.attention_rows(q, k, v, 0.5, lambda i, j: pd.sees_window(i, j, 1), sinks=[0.0, math.log(3.0)])
    assert np.allclose(with_sink[:, 1], v[:, 0] * (np.exp(0.5 * (q[:, 1] * k[:, 0]).sum(-1)) /
                                                  (np.exp(0.5 * (q[:, 1] * k[:, 0]).sum(-1)) + 3.0))[:, None])
