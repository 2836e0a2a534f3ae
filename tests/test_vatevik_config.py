"""Vatevik's configuration, its tensor declarations, the rotation's frequencies and the plain implementation's own
consistency (no GPU)."""
import copy
import math

import numpy as np
import pytest

import plain_vatevik as pv
from vatevik_helpers import MIXED, ODD, WIDE, as_numpy, attn, config, dense, make_weights, ret, stretch


def test_round_trip_and_registry():
    import cbis_b200 as cb
    for cfgd in (MIXED, ODD, WIDE):
        c = cb.config_from_dict(cfgd)
        assert type(c).__name__ == "VatevikConfig" and c.to_dict() == cfgd
        spec = c.model_spec()
        assert [l.arrangement for l in spec.layers] == ["sandwich"] * len(cfgd["layers"])
        assert all(l.norm_mixer.kind == "none" and l.post_norm_mixer.kind == "rmsnorm" for l in spec.layers)
        assert spec.max_positions == 0 and spec.vocab_size == cfgd["vocab"]
        assert spec.embedding_spec().params["multiplier"] == cfgd["embedding"]["scale"]
        assert spec.head_spec().params["tensor"] is None                              # the token table again
        assert spec.head_spec().params["soft_cap"] == cfgd.get("logit_softcap", 0.0)


def test_which_layer_gives_its_values_and_which_blend():
    import cbis_b200 as cb
    kinds = [l.mixer.params.get("value_blend") for l in cb.config_from_dict(MIXED).model_spec().layers]
    assert kinds == [None, None, "source", None, "blend", "blend"]
    kinds = [l.mixer.params.get("value_blend") for l in cb.config_from_dict(ODD).model_spec().layers]
    assert kinds == [None, "source", "blend", None, None]


def test_declared_tensors_follow_the_sizes():
    import cbis_b200 as cb
    from cbis_b200.models import Model
    decl = {d.name: tuple(d.shape) for d in Model(cb.config_from_dict(ODD).model_spec()).declared()}
    assert decl["embed"] == (61, 40) and "head" not in decl and decl["final.norm"] == (40,)
    assert decl["l0.mix.q"] == (12, 40) and decl["l0.mix.v"] == (20, 40) and decl["l0.mix.g"] == (20, 40)
    assert decl["l0.mix.o"] == (40, 20) and decl["l0.norm1"] == (40,) and decl["l0.norm2"] == (40,)
    assert decl["l1.mix.q"] == (36, 40) and decl["l1.mix.k"] == (12, 40) and decl["l1.mix.v"] == (20, 40)
    assert decl["l1.mix.q.norm"] == (36,) and decl["l1.mix.k.norm"] == (12,) and decl["l1.mix.vmix"] == ()
    assert decl["l1.mix.o"] == (40, 60) and "l1.norm2" not in decl and "l1.mlp.gate" not in decl      # no feed-forward
    assert decl["l3.mix.q"] == (60, 40) and decl["l3.mix.v"] == (132, 40) and decl["l3.mix.o"] == (40, 132)
    assert "l4.mix.vmix" not in decl and decl["l4.mix.o"] == (40, 50) and decl["l4.mlp.down"] == (40, 56)
    assert not any(n.startswith(("l0.pre", "l1.pre")) for n in decl)                  # no norm before a part


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "is not one of"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "'scale' is missing"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=1.0), "must differ"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "one per head"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 1.5]), "between 0 and 1"),
    (lambda c: c["layers"][4]["mixer"].update(vdim=16), "blends its values"),
    (lambda c: c["layers"][2]["mixer"].update(v_mix=1), "true or false"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "is not one of"),
    (lambda c: c.pop("norm"), "'norm' is missing"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_bad_configurations_are_refused(change, message):
    import cbis_b200 as cb
    cfgd = copy.deepcopy(MIXED)
    change(cfgd)
    with pytest.raises(cb.ConfigError, match=message):
        cb.config_from_dict(cfgd)


def test_mixers_refuse_sizes_no_kernel_takes():
    import cbis_b200 as cb
    from cbis_b200.models import Model
    for layer in (attn(2, 2, 600, 16, 0.1), ret(2, 600, 16, [0.9, 0.9])):
        with pytest.raises(ValueError, match="outside"):
            Model(cb.config_from_dict(config(32, 40, [layer])).model_spec())


def test_frequencies_kept_blended_and_slowed_down():
    from cbis_b200.parts import rotary_frequencies
    plainf = rotary_frequencies(1000.0, 8).double().numpy()
    assert np.allclose(plainf, [1000.0 ** (-2 * i / 8) for i in range(4)], rtol=1e-7)
    st = (8.0, 1.0, 4.0, 64.0)
    f = rotary_frequencies(1000.0, 8, st).double().numpy()
    ref = pv.frequencies(1000.0, 8, stretch(*st))
    assert np.allclose(f, ref, rtol=1e-7)
    wave = 2 * math.pi / plainf                                    # 6.3, 35, 199, 1117 against the edges 16 and 64
    assert wave[0] < 16 < wave[1] < 64 < wave[2]
    assert f[0] == np.float32(plainf[0]) and np.allclose(f[2:], plainf[2:] / 8, rtol=1e-7)
    s = (64 / wave[1] - 1.0) / 3.0
    assert 0 < s < 1 and np.isclose(f[1], (1 - s) * plainf[1] / 8 + s * plainf[1], rtol=1e-7)
    assert rotary_frequencies(10.0, 0).numel() == 0
    with pytest.raises(ValueError):
        rotary_frequencies(10.0, 3)


def test_plain_retention_carries_its_state():
    """The plain recurrence from a state equals the recurrence over the whole sequence, and equals the sum over the
    earlier tokens written out: o_t = sum_j decay^(t-j) (q_t . k_j) v_j."""
    g = np.random.default_rng(3)
    T, H, D, V = 23, 2, 5, 7
    q, k, v = g.normal(size=(T, H, D)), g.normal(size=(T, H, D)), g.normal(size=(T, H, V))
    decays = [0.9, 1.0]
    whole, end = pv.retention_rows(q, k, v, decays)
    first, mid = pv.retention_rows(q[:9], k[:9], v[:9], decays)
    rest, end2 = pv.retention_rows(q[9:], k[9:], v[9:], decays, mid)
    assert np.abs(np.concatenate([first, rest]) - whole).max() < 1e-12 and np.abs(end - end2).max() < 1e-12
    t, h = 17, 0
    direct = sum(decays[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
    assert np.abs(direct - whole[t, h]).max() < 1e-12


def test_plain_attention_pieces():
    g = np.random.default_rng(4)
    s = g.normal(size=6)
    w = pv.softmax_plus_one(s)
    assert abs(w.sum() + 1.0 / (1.0 + np.exp(s).sum()) - 1) < 1e-12
    assert abs(pv.softmax_plus_one(np.array([0.0]))[0] - 0.5) < 1e-12                  # one key of score 0 shares with the 1
    assert pv.softmax_plus_one(np.array([800.0]))[0] > 0.999                          # no overflow
    x = g.normal(size=(3, 2, 8))
    f = pv.frequencies(100.0, 4)
    r = pv.rotate(x, [0, 1, 5], f, 4)
    assert np.allclose(r[0], x[0]) and np.allclose(r[..., 4:], x[..., 4:])            # position 0 and the tail pass unchanged
    assert np.allclose((r[..., :4] ** 2).sum(-1), (x[..., :4] ** 2).sum(-1))          # a rotation keeps the length
    a = 5 * 100.0 ** (-2 * 1 / 4)
    assert np.allclose(r[2, 0, 1], x[2, 0, 1] * np.cos(a) - x[2, 0, 3] * np.sin(a))
    assert np.allclose(r[2, 0, 3], x[2, 0, 3] * np.cos(a) + x[2, 0, 1] * np.sin(a))
    q, k, v = g.normal(size=(6, 4, 3)), g.normal(size=(6, 2, 3)), g.normal(size=(6, 2, 5))
    out = pv.attention_rows(q, k, v, 0.5)
    e = math.exp(0.5 * q[0, 3] @ k[0, 1])
    assert np.allclose(out[0, 3], e / (1 + e) * v[0, 1])                               # the first token: itself and the 1; head 3 reads group 1
    k2, v2 = k.copy(), v.copy()
    k2[4:] += 9.0
    v2[4:] -= 3.0
    assert np.allclose(pv.attention_rows(q, k2, v2, 0.5)[:4], out[:4])                 # nobody sees a later token


def test_one_norm_over_the_whole_projection():
    g = np.random.default_rng(5)
    x, w = g.normal(size=(3, 12)), g.normal(size=12)
    y = pv.rms_norm(x, w, 1e-3)
    assert np.allclose(y, x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-3) * w)
    per_head = pv.rms_norm(x.reshape(3, 3, 4), 1.0, 1e-3).reshape(3, 12) * w
    assert not np.allclose(y, per_head)


def test_random_weights_keep_activations_in_range():
    w = make_weights(MIXED, 3)
    logits, stream = pv.forward(MIXED, as_numpy(w), list(range(20)))
    assert np.isfinite(logits).all() and 0.1 < np.abs(stream[-1]).mean() < 50
    assert np.abs(logits).max() < MIXED["logit_softcap"]


def test_where_long_retention_segments_are_cut_into_pieces():
    """The piece size of a step: none for short segments or where the uncut step fills the SMs, a multiple of 32 that
    gives at least two pieces otherwise; a prompt beside decoding rows counts as the one long walk it is; the table of
    decays holds decay^(32 (i + 1)), rounded once from 64-bit."""
    import torch
    from cbis_b200.kernels import ops
    assert ops.retention_piece_rows(100, 1, 8, 128, 256) == 0                   # short
    assert ops.retention_piece_rows(4096, 64, 8, 128, 256) == 0                 # many long segments: whole
    for longest, segs in ((128, 1), (500, 1), (3000, 1), (700, 4), (100000, 1)):
        rows = ops.retention_piece_rows(longest, segs, 8, 128, 256)
        assert rows > 0 and rows % 32 == 0 and rows <= 32 * ops.RETENTION_PIECE_SIZES and -(-longest // rows) >= 2
    assert ops.retention_piece_rows(3000, 40, 8, 128, 256) == 0
    assert ops.retention_piece_rows(3000, 40, 8, 128, 256, total_rows=3039) > 0      # one prompt beside 39 decoding rows
    assert ops.retention_piece_rows(3000, 40, 8, 128, 256, total_rows=40 * 3000) == 0
    assert ops.retention_piece_rows(3000, 1, 4, 512, 512) == 0 or \
        -(-3000 // ops.retention_piece_rows(3000, 1, 4, 512, 512)) * 4 * 512 * 512 * 4 <= ops.RETENTION_PIECES_MAX_BYTES
    decays = [1.0, 0.5, 0.9873046875]
    table = ops.retention_piece_decays(decays)
    assert table.shape == (ops.RETENTION_PIECE_SIZES, 3) and table.dtype == torch.float32
    for i in (0, 3, ops.RETENTION_PIECE_SIZES - 1):
        for h, d in enumerate(decays):
            assert table[i, h].item() == torch.tensor(d ** (32 * (i + 1)), dtype=torch.float64).float().item()
