"""Lenuzen: a decoder-only model with the norm on the sublayers' outputs and two kinds of shaped attention.

config.json (``"architecture": "Lenuzen"``) gives ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``logit_scale`` and ``layers``: a list whose entries name the layer's mixer (``type``), the mixer's sizes
(``mixer``) and its feed-forward (``mlp``, or null for none).

A layer is h += N1(mixer(h)); h += N2(feed_forward(h)): the sublayers read the float32 residual stream itself,
the layer norms (a weight, no bias) sit on their outputs.  The output is the same norm of h, then the embedding
table as the head, times ``logit_scale``.

Mixers, by ``type`` (both: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, interleaved
rotary pairs on the first ``rot.dims`` channels with ``rot.base`` and the frequency scaling ``rot.scaling``
(``factor``, ``original``, ``fast``, ``slow``), all through ``parts/modulated_attention.py``):
  ``attention``    biases on q, k, v; every q and k head divided by its root mean square after the rotation and
                   every value head by its own; a number a head on the scores (``temp``); a sliding window of
                   ``mask.size``; softmax; a sigmoid gate a head on the output (``g``)
  ``attention_2``  no biases; an RMS norm with weights over the whole q and the whole k projection before the
                   rotation (``q.norm``, ``k.norm``); the heads' scores mixed by ``talk`` [heads, heads]; chunks
                   of ``mask.size`` positions; a softmax whose denominator gains a 1
Feed-forward, by ``mlp.kind``: ``dense``: down(gelu_tanh(up x)) of width ``ff``.

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``final.norm``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Tuple

from ..config.base import ConfigError, ModelConfig, _require, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("attention", "attention_2")
# positions are float32 inside the rotation: every position below 2^24 is exact
MAX_POSITIONS = 1 << 24


def _sub(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"Lenuzen: {where} lacks the section {key!r}")
    return v


@dataclass(frozen=True)
class LenuzenConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_scale: float
    layers: Tuple[Mapping[str, Any], ...]      # as in config.json (validated)
    eos_token_id: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    architecture = "Lenuzen"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LenuzenConfig":
        a = cls.architecture
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError(f"{a}: config.json lacks the list 'layers'")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(vocab=_require(d, "vocab", int, a), width=_require(d, "width", int, a),
                  embedding_scale=float(_require(_sub(d, "embedding", "config.json"), "scale", float, a)),
                  norm_eps=float(_require(_sub(d, "norm", "config.json"), "eps", float, a)),
                  logit_scale=float(d.get("logit_scale", 1.0)),
                  layers=tuple(copy.deepcopy(dict(l)) for l in layers), eos_token_id=eos_ids,
                  initializer_range=float(d.get("initializer_range", 0.05)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        a = self.architecture
        if self.vocab <= 0 or self.width <= 0 or self.norm_eps <= 0:
            raise ConfigError(f"{a}: vocab, width and norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layer {i}"
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{a}: {where} has the type {kind!r}; built: {', '.join(MIXER_TYPES)}")
            m = _sub(layer, "mixer", where)
            for key in ("heads", "kv_heads", "dim", "vdim"):
                if int(_require(m, key, int, f"{a} {where} mixer")) <= 0:
                    raise ConfigError(f"{a}: {where}: {key} must be positive")
            _require(m, "scale", float, f"{a} {where} mixer")
            if int(m["heads"]) % int(m["kv_heads"]):
                raise ConfigError(f"{a}: {where}: heads is not a multiple of kv_heads")
            mask = m.get("mask")
            if mask is not None and int(_require(mask, "size", int, f"{a} {where} mask")) <= 0:
                raise ConfigError(f"{a}: {where}: mask.size must be positive")
            rot = m.get("rot")
            if rot is not None:
                _require(rot, "base", float, f"{a} {where} rot")
                dims = int(_require(rot, "dims", int, f"{a} {where} rot"))
                if dims > int(m["dim"]) or dims % 2 or dims < 0:
                    raise ConfigError(f"{a}: {where}: rot.dims must be even and at most dim")
                sc = rot.get("scaling")
                if sc is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _require(sc, key, float, f"{a} {where} rot.scaling")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{a}: {where} has a feed-forward of kind {mlp.get('kind')!r}; built: 'dense'")
                _require(mlp, "ff", int, f"{a} {where} mlp")

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [copy.deepcopy(dict(l)) for l in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
            # (read by this package's own tools: the tests' trace helper and the random-weights writer)
            "vocab_size": self.vocab,
            "initializer_range": self.initializer_range,
        }
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def init_scales(self) -> Dict[str, float]:
        s = self.initializer_range
        return {"matrix": s, "bias": s, "norm": s}

    # ------------------------------------------------------------------
    def _mixer_spec(self, i: int, layer: Mapping[str, Any]) -> PartSpec:
        m, kind = layer["mixer"], layer["type"]
        size = (m.get("mask") or {}).get("size")
        params: Dict[str, Any] = {
            "hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
            "head_dim": int(m["dim"]), "value_head_dim": int(m["vdim"]), "scale": float(m["scale"]),
            "eps": self.norm_eps, "mask_size": None if size is None else int(size)}
        rot = m.get("rot")
        if rot is not None and int(rot["dims"]) > 0:
            params["position"] = PartSpec("rope_computed", {
                "rotary_dim": int(rot["dims"]), "theta": float(rot["base"]), "layout": "interleaved",
                "scaling": None if rot.get("scaling") is None else dict(rot["scaling"])})
        if kind == "attention":
            params.update(qkv_bias=True, qk_norm="head_unit", value_norm=True, head_temperature=True,
                          mask="causal" if size is None else "window", head_gate=True)
        else:
            params.update(qk_norm="projection", head_mix=True, mask="causal" if size is None else "chunk", sink=True)
        return PartSpec("modulated_attention", params, f"l{i}.mix.")

    def model_spec(self) -> ModelSpec:
        norm = {"hidden_size": self.width, "eps": self.norm_eps, "tensor": ""}
        layers: List[LayerSpec] = []
        for i, layer in enumerate(self.layers):
            parts = {"mixer": self._mixer_spec(i, layer), "mixer_norm": PartSpec("layer_norm_out", norm, f"l{i}.norm1")}
            mlp = layer.get("mlp")
            if mlp is None:
                layers.append(LayerSpec("output_norm_mixer_only", parts))
                continue
            parts["feed_forward"] = PartSpec("dense_mlp", {
                "hidden_size": self.width, "intermediate_size": int(mlp["ff"]), "activation": "gelu_tanh",
                "tensor_names": ("up", "down")}, f"l{i}.mlp.")
            parts["feed_forward_norm"] = PartSpec("layer_norm_out", norm, f"l{i}.norm2")
            layers.append(LayerSpec("output_norm", parts))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "scale": self.embedding_scale, "residual": "float32",
                                                   "tensor": ""}, "embed"),
            layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(layers))),
            final_norm=PartSpec("layer_norm_f32", norm, "final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": "embed",
                                      "tensor": "", "scale": self.logit_scale}, "head"),
            eos_token_ids=self.eos_token_id)


register_architecture(LenuzenConfig.architecture, LenuzenConfig)
