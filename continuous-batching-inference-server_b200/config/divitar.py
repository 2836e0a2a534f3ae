"""Typed configuration of Divitar folders.

A Divitar model is a list of unlike pre-norm layers with root-mean-square norms (plain weights) whose parts' results
are multiplied by one constant m before they join the stream: x += m mixer(norm1(x)), x += m ff(norm2(x)), and, in a
model with a second token table, x += m unit_rms(proj(gelu_tanh(gate x) * e_token)) * w with the layer's own columns
of the token's row.  The mixer is attention over grouped heads whose values are its keys before the rotation, seen
inside blocks of positions, with a gate per head ("attention"), or attention over a cached latent with one rotated
key part per token, a sliding window and a learned number per head in the softmax's denominator ("latent_attention",
which may read the latent of an earlier layer).  The feed-forward is down(relu(up h)^2), a routed mixture of gated
ones with an expert every token uses, or absent.  Every size and every constant that may differ between two models
comes from ``config.json``; the tensor names are the format's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec
from .vekedra import _get, _int, _num, _only

MIXERS = ("attention", "latent_attention")


def _freeze(v):
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    return v


def _thaw(v):
    if isinstance(v, tuple) and all(isinstance(x, tuple) and len(x) == 2 and isinstance(x[0], str) for x in v):
        return {k: _thaw(x) for k, x in v}
    return v


def _mask(m: Dict[str, Any], where: str) -> int:
    mask = m.get("mask")
    if mask is None:
        return 0
    _only(mask, ("size",), where + "mask.")
    return _int(mask, "size", where + "mask.")


def _rot(m: Dict[str, Any], where: str, width: int, scaling_keys) -> Optional[Dict[str, Any]]:
    """``rot``: base, dims and optionally ``scaling`` with the keys the mixer's scheme has; absent: nothing is rotated."""
    rot = m.get("rot")
    if rot is None:
        return None
    where += "rot."
    _only(rot, ("base", "dims", "scaling"), where)
    out = {"base": _num(rot, "base", where), "dims": _int(rot, "dims", where, 0)}
    if out["dims"] % 2 or out["dims"] > width:
        raise ConfigError(f"config.json: {where}dims={out['dims']} must be even and at most {width}")
    sc = rot.get("scaling")
    if sc is not None:
        _only(sc, scaling_keys, where + "scaling.")
        out["scaling"] = {k: _num(sc, k, where + "scaling.") for k in scaling_keys}
    return out


def _parse_mixer(kind: str, m: Dict[str, Any], i: int, before) -> Dict[str, Any]:
    where = f"layers[{i}].mixer."
    if kind == "attention":
        _only(m, ("dim", "heads", "kv_heads", "mask", "rot", "scale", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "kv_heads")}
        out["vdim"] = _int(m, "vdim", where) if m.get("vdim") is not None else out["dim"]
        if out["vdim"] != out["dim"]:
            raise ConfigError(f"config.json: {where}vdim={out['vdim']} differs from dim={out['dim']}: the values are the keys")
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {where}heads={out['heads']} is not a multiple of kv_heads={out['kv_heads']}")
        out["scale"] = _num(m, "scale", where)
        out["block"] = _mask(m, where)
        out["rot"] = _rot(m, where, out["dim"], ("factor",))
        return out
    if kind == "latent_attention":
        _only(m, ("dim", "heads", "kv_from", "kv_rank", "mask", "rot", "rot_dim", "scale", "vdim"), where)
        out = {k: _int(m, k, where) for k in ("dim", "heads", "kv_rank", "vdim")}
        out["rot_dim"] = _int(m, "rot_dim", where, 0) if m.get("rot_dim") is not None else 0
        out["scale"] = _num(m, "scale", where)
        out["window"] = _mask(m, where)
        out["rot"] = _rot(m, where, max(out["rot_dim"], 0), ("factor", "original", "fast", "slow"))
        if out["rot_dim"] and out["rot"] is None:
            raise ConfigError(f"config.json: {where}rot_dim={out['rot_dim']} needs 'rot' (base, dims)")
        src = m.get("kv_from")
        if src is not None:
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"config.json: {where}'kv_from' must name an earlier layer, got {src!r}")
            other = before[src]
            o = other.mixer_dict()
            if other.type != "latent_attention" or o.get("kv_from") is not None:
                raise ConfigError(f"config.json: {where}'kv_from'={src}: that layer keeps no latent of its own")
            for k in ("kv_rank", "rot_dim", "rot"):
                if o[k] != out[k]:
                    raise ConfigError(f"config.json: {where}{k}={out[k]!r} differs from layer {src}'s {o[k]!r}")
            out["kv_from"] = src
        return out
    raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not one of {sorted(MIXERS)}")


def _parse_mlp(f: Optional[Dict[str, Any]], i: int) -> Optional[Dict[str, Any]]:
    if f is None:
        return None
    where = f"layers[{i}].mlp."
    kind = _get(f, "kind", where)
    if kind == "dense":
        _only(f, ("kind", "ff"), where)
        return {"kind": "dense", "ff": _int(f, "ff", where)}
    if kind == "moe":
        _only(f, ("kind", "expert", "router", "shared"), where)
        expert, router = _get(f, "expert", where), _get(f, "router", where)
        _only(expert, ("ff",), where + "expert.")
        _only(router, ("experts", "scale", "top"), where + "router.")
        out = {"kind": "moe", "ff": _int(expert, "ff", where + "expert."),
               "experts": _int(router, "experts", where + "router."), "top": _int(router, "top", where + "router."),
               "scale": _num(router, "scale", where + "router.") if router.get("scale") is not None else 1.0,
               "shared_ff": 0}
        if out["top"] > out["experts"]:
            raise ConfigError(f"config.json: {where}router.top={out['top']} exceeds experts={out['experts']}")
        shared = f.get("shared")
        if shared is not None:
            _only(shared, ("ff",), where + "shared.")
            out["shared_ff"] = _int(shared, "ff", where + "shared.")
        return out
    raise ConfigError(f"config.json: {where}'kind' {kind!r} is not one of ['dense', 'moe']")


@dataclass(frozen=True)
class DivitarLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's sizes and constants, as sorted items (nested ones too)
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def mixer_dict(self) -> Dict[str, Any]:
        return {k: _thaw(v) for k, v in self.mixer}

    def mlp_dict(self) -> Optional[Dict[str, Any]]:
        return None if self.mlp is None else dict(self.mlp)


@dataclass(frozen=True)
class DivitarConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    side_dim: int                   # 0: the model has no second token table
    layers: Tuple[DivitarLayer, ...]
    architecture: str = "Divitar"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DivitarConfig":
        _only(d, ("architecture", "architectures", "model_type", "layers", "logit_scale", "norm", "residual_mult",
                  "token_side", "vocab", "width"), "")
        norm = _get(d, "norm", "")
        _only(norm, ("eps",), "norm.")
        side = d.get("token_side")
        side_dim = 0
        if side is not None:
            _only(side, ("dim",), "token_side.")
            side_dim = _int(side, "dim", "token_side.")
        raw = _get(d, "layers", "")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            _only(entry, ("type", "mixer", "mlp"), f"layers[{i}].")
            kind = _get(entry, "type", f"layers[{i}].")
            mixer = _parse_mixer(kind, _get(entry, "mixer", f"layers[{i}]."), i, layers)
            mlp = _parse_mlp(entry.get("mlp"), i)
            layers.append(DivitarLayer(kind, _freeze(mixer), None if mlp is None else tuple(sorted(mlp.items()))))
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), norm_eps=_num(norm, "eps", "norm."),
                   residual_mult=_num(d, "residual_mult", "", False) if d.get("residual_mult") is not None else 1.0,
                   logit_scale=_num(d, "logit_scale", "", False) if d.get("logit_scale") is not None else 1.0,
                   side_dim=side_dim, layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out = []
        for layer in self.layers:
            m = layer.mixer_dict()
            size = m.pop("block") if layer.type == "attention" else m.pop("window")
            if size:
                m["mask"] = {"size": size}
            if m.get("rot") is None:
                m.pop("rot", None)
            if layer.type == "latent_attention" and not m["rot_dim"]:
                m.pop("rot_dim")
            f = layer.mlp_dict()
            if f is not None and f["kind"] == "moe":
                g = {"kind": "moe", "expert": {"ff": f["ff"]},
                     "router": {"experts": f["experts"], "scale": f["scale"], "top": f["top"]}}
                if f["shared_ff"]:
                    g["shared"] = {"ff": f["shared_ff"]}
                f = g
            out.append({"type": layer.type, "mixer": m, "mlp": f})
        d = {"architecture": self.architecture, "layers": out, "logit_scale": self.logit_scale,
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d

    def model_spec(self) -> ModelSpec:
        W, eps, L = self.width, self.norm_eps, len(self.layers)
        norm = PartSpec("rmsnorm", {"width": W, "eps": eps, "offset": 0.0, "name": ""})
        none = PartSpec("none", {"width": W})
        specs, ignored = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer_dict()
            rot = m.get("rot")
            source = None
            if layer.type == "attention":
                mixer = PartSpec("rotary_attention", {
                    "width": W, "n_head": m["heads"], "n_kv_head": m["kv_heads"], "head_dim": m["dim"],
                    "v_head_dim": m["dim"], "scale": m["scale"], "block": m["block"], "bias": True,
                    "values_from_keys": True, "head_gate": True,
                    "rot_base": rot["base"] if rot else 10000.0, "rot_dims": rot["dims"] if rot else 0,
                    "rot_divide": (rot.get("scaling") or {}).get("factor", 1.0) if rot else 1.0})
            else:
                source = m.get("kv_from")
                sc = (rot or {}).get("scaling")
                mixer = PartSpec("latent_attention", {
                    "width": W, "n_head": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"], "rank": m["kv_rank"],
                    "scale": m["scale"], "window": m["window"], "eps": eps, "own_latent": source is None,
                    "rot_dim": m["rot_dim"], "rot_base": rot["base"] if rot else 10000.0,
                    "rot_dims": rot["dims"] if rot else 0, "rot_pairs": "neighbours",
                    "rot_blend": None if sc is None else (sc["factor"], sc["original"], sc["fast"], sc["slow"]),
                    "sinks": True, "gate": None})
            f = layer.mlp_dict()
            if f is None:
                ff = PartSpec("nothing", {"width": W})
                ignored.append(rf"^l{i}\.norm2$")       # a folder may still carry the norm of the part that is absent
            elif f["kind"] == "dense":
                ff = PartSpec("dense", {"width": W, "inner": f["ff"], "activation": "relu2", "names": ("mlp.up", "mlp.down"),
                                        "plain": True})
            else:
                ff = PartSpec("routed", {"width": W, "inner": f["ff"], "experts": f["experts"], "top": f["top"],
                                         "activation": "silu", "score": "sigmoid", "renormalize": True,
                                         "renorm_eps": 1e-20, "weight_scale": f["scale"], "weight_on": "output",
                                         "shared_inner": f["shared_ff"]})
            side = None
            if self.side_dim:
                side = PartSpec("token_gated", {"width": W, "dim": self.side_dim, "vocab_size": self.vocab,
                                                "table_width": L * self.side_dim, "col0": i * self.side_dim, "eps": eps,
                                                "activation": "gelu_tanh"})
            specs.append(LayerSpec(prefix=f"l{i}.", arrangement="pre_norm_scaled", mixer=mixer, feed_forward=ff,
                                   norm_mixer=norm, norm_feed_forward=norm if f is not None else none,
                                   cache_source=source, norm_prefixes=("norm1", "norm2"),
                                   residual_scale=self.residual_mult, side=side))
        return ModelSpec(width=W, vocab_size=self.vocab, max_positions=0,      # 0: the design sets no limit; the engine's holds
                         token_embedding=PartSpec("token_table", {"vocab_size": self.vocab, "width": W, "tensor": "embed"}),
                         position=PartSpec("none", {"width": W}),
                         layers=tuple(specs), schedule=tuple(range(len(specs))),
                         final_norm=norm, final_norm_prefix="final.norm",
                         head=PartSpec("linear", {"vocab_size": self.vocab, "width": W, "tensor": "head",
                                                  "logit_scale": self.logit_scale}),
                         ignored_tensors=tuple(ignored))
