"""Typed configuration of the Daronex decoder (config.json ``"architecture": "Daronex"``).

A stack of layers around a 32-bit residual stream in which the norm sits on each sublayer's OUTPUT:
``x += norm1(mixer(x))`` then ``x += norm2(ff(x))``, the sublayers reading ``x`` itself; the norms are RMS norms whose
stored weight is the gain's distance from one (``norm.eps``).  config.json lists the layers (``layers[i]``: ``type``,
``mixer``, ``mlp``), and every layer may differ:

* ``type: "latent_attention"``: attention through a latent (``heads``, per head ``dim`` unrotated and ``rot_dim`` rotated
  query/key elements, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``, ``rot.base``, ``rot.dims``), rotation of the interleaved
  pairs ``(2j, 2j + 1)``, every earlier key visible, no gate; with ``kv_from: j`` the layer has no key/value projection and
  reads the cache of layer ``j``.
* ``type: "latent_attention_2"``: the same with rotation of the pairs ``(j, j + dims / 2)``, a sliding window of
  ``mask.size`` positions (the query's own included) and a sigmoid output gate.
* ``type: "gla"``: gated linear attention with a decay per key channel (``heads``, ``dim``, ``vdim``, ``tau``); the inner size
  of its decay projection is the shape of the tensor ``a1`` (``decay_rank`` in config.json where a model is made without
  a checkpoint).
* ``mlp``: null, or ``{"kind": "dense", "ff": n}``: ``down(relu(up h)^2)``.

``logits = head(norm(x)) * logit_scale``.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.{up,down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .model_config import ArchitectureConfig, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_POSITION = 1 << 20      # the design sets no limit of its own; the engine's max_model_len is the one that counts

LATENT_TYPES = {
    # type -> (pairing of the rotation, windowed, gated)
    "latent_attention": ("rotary_interleaved", False, False),
    "latent_attention_2": ("rotary_half", True, True),
}


def _int(d, key, where, least=1):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, int) or isinstance(v, bool) or v < least:
        raise ConfigError(f"Daronex config.json: {where}.{key} must be an integer of at least {least}, found {v!r}")
    return v


def _num(d, key, where, positive=False):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, (int, float)) or isinstance(v, bool) or (positive and not v > 0):
        raise ConfigError(f"Daronex config.json: {where}.{key} must be a{' positive' if positive else ''} number, found {v!r}")
    return float(v)


def _check_latent(kind, m, where, layers, i):
    for k in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
        _int(m, k, where)
    rd = _int(m, "rot_dim", where, least=0)
    if m.get("scale") is None:
        m["scale"] = float(m["dim"] + rd) ** -0.5          # not given: one over the root of a head's query/key size
    _num(m, "scale", where, positive=True)
    if m["kv_rank"] + rd > 1024:
        raise ConfigError(f"Daronex config.json: {where}: kv_rank + rot_dim = {m['kv_rank'] + rd} exceeds the attention kernels' 1024")
    rot = m.get("rot")
    if rd > 0:
        dims = _int(rot, "dims", where + ".rot", least=2)
        if dims % 2 or dims > rd:
            raise ConfigError(f"Daronex config.json: {where}.rot.dims {dims} must be even and at most rot_dim ({rd})")
        _num(rot, "base", where + ".rot", positive=True)
    if LATENT_TYPES[kind][1]:
        _int(m.get("mask"), "size", where + ".mask")
    src = m.get("kv_from")
    if src is not None:
        if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i:
            raise ConfigError(f"Daronex config.json: {where}.kv_from {src!r} must name an earlier layer")
        other, om = layers[src], layers[src].get("mixer")
        if other.get("type") != kind or om.get("kv_from") is not None:
            raise ConfigError(f"Daronex config.json: {where}.kv_from names layer {src}, which is no {kind} layer with a key/value projection of its own")
        window = lambda x: (x.get("mask") or {}).get("size") if LATENT_TYPES[kind][1] else None
        rotation = lambda x: (float(x["rot"]["base"]), int(x["rot"]["dims"])) if x.get("rot_dim") else None
        if (om.get("kv_rank"), om.get("rot_dim"), rotation(om), window(om)) != (m["kv_rank"], rd, rotation(m), window(m)):
            raise ConfigError(f"Daronex config.json: {where}.kv_from: layer {src}'s kv_rank, rot_dim, rotation or window differ from this layer's")


@register_architecture("Daronex", model_type="daronex")
@dataclass
class DaronexConfig(ArchitectureConfig):
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: List[Dict[str, Any]]
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "DaronexConfig":
        vocab, width = _int(data, "vocab", "config"), _int(data, "width", "config")
        eps = _num(data.get("norm"), "eps", "norm", positive=True)
        logit_scale = _num(data, "logit_scale", "config") if data.get("logit_scale") is not None else 1.0
        layers = copy.deepcopy(data.get("layers"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Daronex config.json: 'layers' must list at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind, m = layer.get("type"), layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Daronex config.json: {where}.mixer must be an object")
            if kind in LATENT_TYPES:
                _check_latent(kind, m, where + ".mixer", layers, i)
            elif kind == "gla":
                for k in ("heads", "dim", "vdim"):
                    _int(m, k, where + ".mixer")
                _num(m, "tau", where + ".mixer", positive=True)
                if m.get("decay_rank") is not None:
                    _int(m, "decay_rank", where + ".mixer")
            else:
                raise ConfigError(f"Daronex config.json: {where}.type {kind!r} is not a known layer type ({', '.join(list(LATENT_TYPES) + ['gla'])})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"Daronex config.json: {where}.mlp.kind {mlp.get('kind')!r} is not implemented (only \"dense\")")
                _int(mlp, "ff", where + ".mlp")
        known = {"architecture", "architectures", "model_type", "vocab", "width", "norm", "logit_scale", "layers"}
        return cls(vocab=vocab, width=width, norm_eps=eps, logit_scale=logit_scale, layers=layers, extra={k: v for k, v in data.items() if k not in known})

    def sizes_from_tensors(self, shape_of) -> None:
        for i, layer in enumerate(self.layers):
            if layer["type"] == "gla" and layer["mixer"].get("decay_rank") is None:
                shape = shape_of(f"l{i}.mix.a1")
                if shape is not None and len(shape) == 2:
                    layer["mixer"]["decay_rank"] = int(shape[0])

    def to_json(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "logit_scale": self.logit_scale, "layers": copy.deepcopy(self.layers)}
        for k, v in self.extra.items():
            d.setdefault(k, v)
        return d

    def _mixer(self, i: int, layer: Dict[str, Any]) -> PartSpec:
        W, m = self.width, layer["mixer"]
        if layer["type"] == "gla":
            if m.get("decay_rank") is None:
                raise ConfigError(f"Daronex config.json: layers[{i}].mixer has no decay_rank, and no checkpoint tensor l{i}.mix.a1 gives it")
            return PartSpec("gated_linear_attention", {"hidden_size": W, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "tau": float(m["tau"]),
                                                       "decay_rank": m["decay_rank"], "eps": self.norm_eps, "prefix": "mix."})
        pairing, windowed, gated = LATENT_TYPES[layer["type"]]
        position = None
        if m["rot_dim"] > 0:
            position = PartSpec(pairing, {"theta": float(m["rot"]["base"]), "rotary_dim": int(m["rot"]["dims"])})
        return PartSpec("latent_attention", {
            "hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"], "q_rank": m["q_rank"],
            "kv_rank": m["kv_rank"], "eps": self.norm_eps, "scale": float(m["scale"]), "window": int(m["mask"]["size"]) if windowed else None,
            "position": position, "gate": gated, "shares_cache": m.get("kv_from") is not None, "prefix": "mix."})

    def to_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = lambda name: PartSpec("rms_norm", {"size": W, "eps": eps, "weight": name, "weight_offset": 1.0})
        layers, ignorable = [], []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            layers.append(LayerSpec(
                block="post_norm", mixer_norm=norm("norm1"), mixer=self._mixer(i, layer),
                ffn_norm=norm("norm2") if mlp is not None else None,
                feed_forward=PartSpec("mlp", {"hidden_size": W, "intermediate_size": mlp["ff"], "activation": "relu2", "prefix": "mlp.",
                                              "names": {"up": "up", "down": "down"}}) if mlp is not None else None,
                weight_prefix=f"l{i}."))
            if mlp is None:
                ignorable.append(f"l{i}.norm2")
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=W, vocab_size=self.vocab,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": W, "weight": "embed"}),
            layers=layers, run_order=[RunEntry(i, cache_of=layer["mixer"].get("kv_from")) for i, layer in enumerate(self.layers)],
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": False, "weight": "head", "tied_to": "embed", "scale": self.logit_scale}),
            max_position=MAX_POSITION, ignorable=ignorable)
        spec.validate()
        return spec
