"""Typed configuration of the Nezolorn decoder (config.json ``"architecture": "Nezolorn"``).

A stack of pre-norm layers around a 32-bit residual stream, ``x += m * mixer(norm1(x))`` then
``x += m * ff(norm2(x))`` with one multiplier ``m`` (``residual_mult``) and layer norms that have a weight and no bias
(``norm.eps``).  config.json lists the layers (``layers[i]``: ``type``, ``mixer``, ``mlp``), and every layer may differ:

* ``type: "parallel"``: two mixers on the same input, ``left_scale * left + right_scale * right``.  ``left`` is
  grouped-query attention (``heads``, ``kv_heads``, ``dim``, ``vdim``) without a value projection (a token's value is its
  key before rotation, so ``vdim`` equals ``dim``), rotary positions on the first ``rot.dims`` elements of a head
  (``rot.base``, optional ``rot.scaling`` by wavelength bands), scores times ``scale``, and a mask of the last
  ``mask.size`` tokens plus one pooled entry for every block of ``mask.pool`` tokens wholly before them.  ``right`` is a
  gated matrix memory (``heads``, ``dim``, ``vdim``, ``gate_cap``).
* ``type: "general_delta"``: the generalised delta rule (``heads``, ``dim``); the inner size of its decay projection is
  the shape of the tensor ``w1`` (``decay_rank`` in config.json where a model is made without a checkpoint).
* ``mlp``: null, or ``{"kind": "dense", "ff": n}``: ``down(silu(gate h) * up h)``.

The embedding is ``embed[token] * embedding.scale`` plus, with ``embedding.bigram`` (``buckets``, ``mul_prev``,
``mul_cur``), a row of the table ``bigram`` chosen by the pair (previous token, token).  Tensor names: ``embed``,
``bigram``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .model_config import ArchitectureConfig, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_POSITION = 1 << 20      # the design sets no limit of its own; the engine's max_model_len is the one that counts


def _int(d, key, where, least=1):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, int) or isinstance(v, bool) or v < least:
        raise ConfigError(f"Nezolorn config.json: {where}.{key} must be an integer of at least {least}, found {v!r}")
    return v


def _num(d, key, where, positive=False):
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, (int, float)) or isinstance(v, bool) or (positive and not v > 0):
        raise ConfigError(f"Nezolorn config.json: {where}.{key} must be a{' positive' if positive else ''} number, found {v!r}")
    return float(v)


def _check_left(m, where):
    heads, kv, dim = _int(m, "heads", where), _int(m, "kv_heads", where), _int(m, "dim", where)
    if heads % kv:
        raise ConfigError(f"Nezolorn config.json: {where}: {heads} heads do not group over {kv} key/value heads")
    if m.get("vdim", dim) != dim:
        raise ConfigError(f"Nezolorn config.json: {where}: the values are the keys, so vdim ({m.get('vdim')!r}) must equal dim ({dim})")
    if dim % 4 or dim > 512:
        raise ConfigError(f"Nezolorn config.json: {where}.dim {dim} must be a multiple of 4, at most 512")
    _num(m, "scale", where, positive=True)
    mask = m.get("mask")
    _int(mask, "size", where + ".mask")
    if mask.get("pool") is not None:
        _int(mask, "pool", where + ".mask", least=0)
    rot = m.get("rot")
    if rot is not None:
        dims = _int(rot, "dims", where + ".rot", least=2)
        if dims % 2 or dims > dim:
            raise ConfigError(f"Nezolorn config.json: {where}.rot.dims {dims} must be even and at most dim ({dim})")
        _num(rot, "base", where + ".rot", positive=True)
        sc = rot.get("scaling")
        if sc is not None:
            for k in ("factor", "low", "high", "original"):
                _num(sc, k, where + ".rot.scaling", positive=True)
            if not sc["high"] > sc["low"]:
                raise ConfigError(f"Nezolorn config.json: {where}.rot.scaling: high must exceed low")


def _check_right(m, where):
    for k in ("heads", "dim", "vdim"):
        _int(m, k, where)
    _num(m, "gate_cap", where, positive=True)


@register_architecture("Nezolorn", model_type="nezolorn")
@dataclass
class NezolornConfig(ArchitectureConfig):
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    embedding: Dict[str, Any]
    layers: List[Dict[str, Any]]
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "NezolornConfig":
        vocab, width = _int(data, "vocab", "config"), _int(data, "width", "config")
        mult = _num(data, "residual_mult", "config")
        eps = _num(data.get("norm"), "eps", "norm", positive=True)
        emb = copy.deepcopy(data.get("embedding") or {})
        emb.setdefault("scale", 1.0)
        _num(emb, "scale", "embedding")
        if emb.get("bigram") is not None:
            _int(emb["bigram"], "buckets", "embedding.bigram")
            _int(emb["bigram"], "mul_prev", "embedding.bigram", least=0)
            _int(emb["bigram"], "mul_cur", "embedding.bigram", least=0)
        layers = copy.deepcopy(data.get("layers"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Nezolorn config.json: 'layers' must list at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind, m = layer.get("type"), layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Nezolorn config.json: {where}.mixer must be an object")
            if kind == "parallel":
                _check_left(m.get("left"), where + ".mixer.left")
                _check_right(m.get("right"), where + ".mixer.right")
                m.setdefault("left_scale", 1.0)
                m.setdefault("right_scale", 1.0)
                _num(m, "left_scale", where + ".mixer")
                _num(m, "right_scale", where + ".mixer")
            elif kind == "general_delta":
                _int(m, "heads", where + ".mixer")
                _int(m, "dim", where + ".mixer")
                if m.get("decay_rank") is not None:
                    _int(m, "decay_rank", where + ".mixer")
            else:
                raise ConfigError(f"Nezolorn config.json: {where}.type {kind!r} is not a known layer type (parallel, general_delta)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"Nezolorn config.json: {where}.mlp.kind {mlp.get('kind')!r} is not implemented (only \"dense\")")
                _int(mlp, "ff", where + ".mlp")
        known = {"architecture", "architectures", "model_type", "vocab", "width", "residual_mult", "norm", "embedding", "layers"}
        return cls(vocab=vocab, width=width, residual_mult=mult, norm_eps=eps, embedding=emb, layers=layers,
                   extra={k: v for k, v in data.items() if k not in known})

    def sizes_from_tensors(self, shape_of) -> None:
        for i, layer in enumerate(self.layers):
            if layer["type"] == "general_delta" and layer["mixer"].get("decay_rank") is None:
                shape = shape_of(f"l{i}.mix.w1")
                if shape is not None and len(shape) == 2:
                    layer["mixer"]["decay_rank"] = int(shape[0])

    def to_json(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "residual_mult": self.residual_mult,
             "norm": {"eps": self.norm_eps}, "embedding": copy.deepcopy(self.embedding), "layers": copy.deepcopy(self.layers)}
        for k, v in self.extra.items():
            d.setdefault(k, v)
        return d

    def _mixer(self, i: int, layer: Dict[str, Any]) -> PartSpec:
        W, m = self.width, layer["mixer"]
        if layer["type"] == "general_delta":
            if m.get("decay_rank") is None:
                raise ConfigError(f"Nezolorn config.json: layers[{i}].mixer has no decay_rank, and no checkpoint tensor l{i}.mix.w1 gives it")
            return PartSpec("delta_rule", {"hidden_size": W, "heads": m["heads"], "dim": m["dim"], "decay_rank": m["decay_rank"], "eps": self.norm_eps,
                                           "prefix": "mix."})
        left, right = m["left"], m["right"]
        position = None
        if left.get("rot") is not None:
            rot = left["rot"]
            params = {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"])}
            if rot.get("scaling") is not None:
                params["wavelength_scaling"] = {k: float(rot["scaling"][k]) for k in ("factor", "low", "high", "original")}
            position = PartSpec("rotary_half", params)
        attention = PartSpec("pooled_window_attention", {
            "hidden_size": W, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"], "position": position,
            "window": left["mask"]["size"], "pool": left["mask"].get("pool") or 0, "scale": float(left["scale"]), "values_are_keys": True,
            "names": {"q": "q", "k": "k", "o": "o"}})
        memory = PartSpec("matrix_memory", {"hidden_size": W, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"],
                                            "gate_cap": float(right["gate_cap"]), "eps": self.norm_eps})
        return PartSpec("parallel_mixers", {"left": attention, "right": memory, "left_scale": float(m["left_scale"]),
                                            "right_scale": float(m["right_scale"]), "prefix": "mix."})

    def to_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        layers, ignorable = [], []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            layers.append(LayerSpec(
                block="pre_norm_scaled", block_params={"residual_scale": self.residual_mult},
                mixer_norm=PartSpec("layer_norm", {"size": W, "eps": eps, "weight": "norm1"}),
                mixer=self._mixer(i, layer),
                ffn_norm=PartSpec("layer_norm", {"size": W, "eps": eps, "weight": "norm2"}) if mlp is not None else None,
                feed_forward=PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": mlp["ff"], "activation": "silu", "prefix": "mlp.",
                                                    "names": {"gate": "gate", "up": "up", "down": "down"}}) if mlp is not None else None,
                weight_prefix=f"l{i}."))
            if mlp is None:
                ignorable.append(f"l{i}.norm2")
        emb = {"vocab_size": self.vocab, "hidden_size": W, "weight": "embed", "scale": float(self.embedding.get("scale", 1.0))}
        if self.embedding.get("bigram") is not None:
            b = self.embedding["bigram"]
            emb["pairs"] = {"weight": "bigram", "buckets": b["buckets"], "mul_prev": b["mul_prev"], "mul_cur": b["mul_cur"]}
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=W, vocab_size=self.vocab, embedding=PartSpec("token_embedding", emb),
            layers=layers, run_order=[RunEntry(i) for i in range(len(layers))],
            final_norm=PartSpec("layer_norm", {"size": W, "eps": eps, "weight": "final.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": False, "weight": "head", "tied_to": "embed"}),
            max_position=MAX_POSITION, ignorable=ignorable)
        spec.validate()
        return spec
