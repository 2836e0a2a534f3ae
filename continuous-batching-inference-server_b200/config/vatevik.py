"""Typed configuration of Vatevik folders.

A Vatevik model is a list of unlike layers.  A layer's parts read the residual stream as it is; only a part's RESULT
is normalised before it is added (x += norm1(mixer(x)), then x += norm2(feed_forward(x)); root-mean-square norms with
plain weights).  The mixer is retention (linear attention with a fixed decay per head, rotated queries and keys, a
gate; "retention") or causal attention with grouped key/value heads, a norm over the whole query and key projections,
a rotation whose slow frequencies may be stretched, a softmax with one added to its denominator, and values blended
with those of the first such layer ("attention").  The feed-forward is a gated one (silu) or absent.  Token rows are
multiplied by a constant; the head is the token table again, a scale and a tanh cap.  Every size and every constant
that may differ between two models comes from ``config.json``; the tensor names are the format's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec
from .vekedra import _get, _int, _num, _only

MIXERS = ("attention", "retention")


def _parse_rot(m: Dict[str, Any], where: str, dim: int) -> Dict[str, Any]:
    """``rot``: base and dims, and optionally ``scaling`` (factor, low, high, original); absent: no rotation."""
    rot = m.get("rot")
    if rot is None:
        return {"rot_base": 10000.0, "rot_dims": 0, "rot_stretch": None}
    where += "rot."
    _only(rot, ("base", "dims", "scaling"), where)
    out = {"rot_base": _num(rot, "base", where), "rot_dims": _int(rot, "dims", where, 0), "rot_stretch": None}
    if out["rot_dims"] % 2 or out["rot_dims"] > dim:
        raise ConfigError(f"config.json: {where}dims={out['rot_dims']} must be even and at most dim={dim}")
    sc = rot.get("scaling")
    if sc is not None:
        _only(sc, ("factor", "low", "high", "original"), where + "scaling.")
        st = tuple(_num(sc, k, where + "scaling.") for k in ("factor", "low", "high", "original"))
        if st[2] == st[1]:
            raise ConfigError(f"config.json: {where}scaling.high and .low must differ")
        out["rot_stretch"] = st
    return out


def _parse_mixer(kind: str, m: Dict[str, Any], i: int) -> Dict[str, Any]:
    where = f"layers[{i}].mixer."
    if kind == "retention":
        _only(m, ("decay", "dim", "heads", "rot", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "vdim")}
        decay = _get(m, "decay", where)
        if (not isinstance(decay, list) or len(decay) != out["heads"]
                or not all(isinstance(d, (int, float)) and not isinstance(d, bool) and 0.0 <= d <= 1.0 for d in decay)):
            raise ConfigError(f"config.json: {where}'decay' must list {out['heads']} numbers between 0 and 1, one per head, "
                              f"got {decay!r}")
        out["decay"] = tuple(float(d) for d in decay)
        out.update(_parse_rot(m, where, out["dim"]))
        return out
    if kind == "attention":
        _only(m, ("dim", "heads", "kv_heads", "rot", "scale", "v_mix", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "kv_heads", "vdim")}
        out["scale"] = _num(m, "scale", where)
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {where}heads={out['heads']} is not a multiple of kv_heads={out['kv_heads']}")
        v_mix = m.get("v_mix", False)
        if not isinstance(v_mix, bool):
            raise ConfigError(f"config.json: {where}'v_mix' must be true or false, got {v_mix!r}")
        out["v_mix"] = v_mix
        out.update(_parse_rot(m, where, out["dim"]))
        return out
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not one of {sorted(MIXERS)}")


def _parse_mlp(f: Optional[Dict[str, Any]], i: int) -> Optional[Dict[str, Any]]:
    if f is None:
        return None
    where = f"layers[{i}].mlp."
    kind = _get(f, "kind", where)
    if kind != "dense":
        raise ConfigError(f"config.json: {where}'kind' {kind!r} is not one of ['dense']")
    _only(f, ("kind", "ff"), where)
    return {"kind": "dense", "ff": _int(f, "ff", where)}


@dataclass(frozen=True)
class VatevikLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's sizes and constants, as sorted items
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def mixer_dict(self) -> Dict[str, Any]:
        return dict(self.mixer)

    def mlp_dict(self) -> Optional[Dict[str, Any]]:
        return None if self.mlp is None else dict(self.mlp)


@dataclass(frozen=True)
class VatevikConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float            # 0: no cap
    layers: Tuple[VatevikLayer, ...]
    architecture: str = "Vatevik"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VatevikConfig":
        _only(d, ("architecture", "architectures", "model_type", "embedding", "layers", "logit_scale", "logit_softcap",
                  "norm", "vocab", "width"), "")
        norm = _get(d, "norm", "")
        _only(norm, ("eps",), "norm.")
        emb = d.get("embedding")
        scale = 1.0
        if emb is not None:
            _only(emb, ("scale",), "embedding.")
            scale = _num(emb, "scale", "embedding.", False) if emb.get("scale") is not None else 1.0
        raw = _get(d, "layers", "")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers, source = [], None
        for i, entry in enumerate(raw):
            _only(entry, ("type", "mixer", "mlp"), f"layers[{i}].")
            kind = _get(entry, "type", f"layers[{i}].")
            mixer = _parse_mixer(kind, _get(entry, "mixer", f"layers[{i}]."), i)
            if kind == "attention" and mixer["v_mix"]:
                shape = (mixer["kv_heads"], mixer["vdim"])
                if source is None:
                    source = shape
                elif shape != source:
                    raise ConfigError(f"config.json: layers[{i}].mixer blends its values with those of the first layer with "
                                      f"'v_mix', whose kv_heads x vdim is {source}; its own is {shape}")
            mlp = _parse_mlp(entry.get("mlp"), i)
            layers.append(VatevikLayer(kind, tuple(sorted(mixer.items(), key=lambda kv: kv[0])),
                                       None if mlp is None else tuple(sorted(mlp.items()))))
        cap = d.get("logit_softcap")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), norm_eps=_num(norm, "eps", "norm."),
                   embedding_scale=scale,
                   logit_scale=_num(d, "logit_scale", "") if d.get("logit_scale") is not None else 1.0,
                   logit_softcap=_num(d, "logit_softcap", "") if cap else 0.0, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for layer in self.layers:
            m = layer.mixer_dict()
            base, dims, stretch = m.pop("rot_base"), m.pop("rot_dims"), m.pop("rot_stretch")
            m["rot"] = {"base": base, "dims": dims}
            if stretch is not None:
                m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), stretch))
            if "decay" in m:
                m["decay"] = list(m["decay"])
            out.append({"type": layer.type, "mixer": m, "mlp": layer.mlp_dict()})
        d = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": out,
             "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = PartSpec("rmsnorm", {"width": W, "eps": eps, "offset": 0.0, "name": ""})
        none = PartSpec("none", {"width": W})
        specs, ignored, blending = [], [], False
        for i, layer in enumerate(self.layers):
            m = layer.mixer_dict()
            rot = {k: m[k] for k in ("rot_base", "rot_dims", "rot_stretch")}
            if layer.type == "retention":
                mixer = PartSpec("retention", {"width": W, "heads": m["heads"], "dim": m["dim"], "v_dim": m["vdim"],
                                               "decays": m["decay"], "eps": eps, **rot})
            else:
                blend = None
                if m["v_mix"]:
                    blend = "blend" if blending else "source"
                    blending = True
                mixer = PartSpec("rotary_attention", {"width": W, "n_head": m["heads"], "n_kv_head": m["kv_heads"],
                                                      "head_dim": m["dim"], "v_head_dim": m["vdim"], "scale": m["scale"],
                                                      "window": 0, "qk_norm": True, "eps": eps, "unit_sink": True,
                                                      "value_blend": blend, **rot})
                if blend is None:
                    ignored.append(rf"^l{i}\.mix\.vmix$")
            f = layer.mlp_dict()
            if f is None:
                ff = PartSpec("nothing", {"width": W})
                ignored.append(rf"^l{i}\.norm2$")       # a folder may still carry the norm of the part that is absent
            else:
                ff = PartSpec("gated", {"width": W, "inner": f["ff"], "activation": "silu"})
            # a sandwich whose norms BEFORE the parts are none: the parts read the stream itself
            specs.append(LayerSpec(prefix=f"l{i}.", arrangement="sandwich", mixer=mixer, feed_forward=ff,
                                   norm_mixer=none, norm_feed_forward=none, norm_prefixes=("pre1", "pre2"),
                                   post_norm_mixer=norm, post_norm_feed_forward=norm if f is not None else None,
                                   post_norm_prefixes=("norm1", "norm2")))
        return ModelSpec(width=W, vocab_size=self.vocab, max_positions=0,      # 0: the design sets no limit; the engine's holds
                         token_embedding=PartSpec("token_table", {"vocab_size": self.vocab, "width": W, "tensor": "embed",
                                                                  "multiplier": self.embedding_scale}),
                         position=PartSpec("none", {"width": W}),
                         layers=tuple(specs), schedule=tuple(range(len(specs))),
                         final_norm=norm, final_norm_prefix="final.norm",
                         head=PartSpec("linear", {"vocab_size": self.vocab, "width": W, "tensor": None,
                                                  "logit_scale": self.logit_scale, "soft_cap": self.logit_softcap}),
                         ignored_tensors=tuple(ignored))
