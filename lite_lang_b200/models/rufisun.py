"""Rufisun: a pre-norm decoder over a float32 residual with dynamic-tanh norms, three kinds of mixer and dense or
routed feed-forwards.

config.json (``"architecture": "Rufisun"``) gives ``vocab``, ``width``, ``norm.eps`` and ``layers``: a list whose
entries name the layer's mixer (``type``), the mixer's sizes and constants (``mixer``) and its feed-forward
(``mlp``, or null for none).  Every size and constant is read from there (or, for the distance-bias table, off
the tensor); nothing is fixed by this file but what the design itself fixes.

A layer is h += mixer(N1(h)); h += feed_forward(N2(h)) with N(u) = tanh(alpha u) w + b (a scalar alpha).  The
output is the same norm of h, then the embedding table as the head.

Mixers, by ``type``:
  ``attention``         grouped-query attention without rotation (``heads``, ``kv_heads``, ``dim``, ``vdim``,
                        ``scale``): a learned bias by distance (table ``rel``, logarithmic buckets up to
                        ``bias_max``), a sliding window of ``mask.size`` that also keeps the request's first
                        ``mask.keep_first`` tokens visible, a learned sink a head in the softmax's denominator
                        (``sink``), a sigmoid gate a channel on the heads' outputs (``g``)
  ``latent_attention``  keys and values expanded from one cached latent (``kv_rank``) and one rotated key part
                        (``rot_dim``) a token; the queries go through a latent of their own (``q_rank``); rotary
                        pairs with stretched slow frequencies (``rot``); causal; a learned sink
  ``parallel``          two mixers on the same input, ``left_scale`` * left + ``right_scale`` * right: left is
                        grouped-query attention without rotation whose queries grow with the position
                        (``q_temp``), whose scores are capped (``softcap``), causal, with a learned sink; right is a
                        state-space layer with a scalar decay a head and token (``heads``, ``vdim``, ``state``,
                        ``groups``, ``conv``, ``norm_groups``)
Feed-forward, by ``mlp.kind``: ``dense``: down(relu(up x)^2) of width ``ff``; ``moe``: ``router.experts`` experts
down(gelu(up x)) of width ``expert.ff``, sigmoid scores, the ``router.top`` best chosen and weighted by their
scores as they are, the weight multiplying the expert's input; ``shared`` (optional, ``ff``) adds an expert that
every token uses.

Tensor names: ``embed``, ``l<i>.norm1|norm2`` (+ ``.b``, ``.alpha``), ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm`` (+ ``.b``, ``.alpha``).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Tuple

from ..config.base import ConfigError, ModelConfig, _require, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

LAYER_TYPES = ("attention", "latent_attention", "parallel")
MLP_KINDS = ("dense", "moe")
# positions are float32 inside the rotation: every position below 2^24 is exact
MAX_POSITIONS = 1 << 24


def _sub(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"Rufisun: {where} lacks the section {key!r}")
    return v


def _heads(m: Mapping[str, Any], where: str, a: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        if int(_require(m, key, int, f"{a} {where}")) <= 0:
            raise ConfigError(f"{a}: {where}: {key} must be positive")
    _require(m, "scale", float, f"{a} {where}")
    if int(m["heads"]) % int(m["kv_heads"]):
        raise ConfigError(f"{a}: {where}: heads is not a multiple of kv_heads")


@dataclass(frozen=True)
class RufisunConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]      # as in config.json (validated)
    eos_token_id: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    architecture = "Rufisun"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RufisunConfig":
        a = cls.architecture
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError(f"{a}: config.json lacks the list 'layers'")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(vocab=_require(d, "vocab", int, a), width=_require(d, "width", int, a),
                  norm_eps=float(_require(_sub(d, "norm", "config.json"), "eps", float, a)),
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
            if kind not in LAYER_TYPES:
                raise ConfigError(f"{a}: {where} has the type {kind!r}; built: {', '.join(LAYER_TYPES)}")
            m = _sub(layer, "mixer", where)
            if kind == "attention":
                _heads(m, where, a)
                _require(m, "bias_max", float, f"{a} {where}")
                mask = m.get("mask")
                if mask is not None and mask.get("size") is not None and int(mask["size"]) <= 0:
                    raise ConfigError(f"{a}: {where}: mask.size must be positive")
            elif kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
                    if int(_require(m, key, int, f"{a} {where}")) <= 0:
                        raise ConfigError(f"{a}: {where}: {key} must be positive")
                _require(m, "scale", float, f"{a} {where}")
                rot = _sub(m, "rot", where)
                _require(rot, "base", float, f"{a} {where} rot")
                dims = int(_require(rot, "dims", int, f"{a} {where} rot"))
                if dims > int(m["rot_dim"]) or dims % 2 or dims < 0:
                    raise ConfigError(f"{a}: {where}: rot.dims must be even and at most rot_dim")
                if rot.get("scaling"):
                    for key in ("factor", "original", "fast", "slow"):
                        _require(rot["scaling"], key, float, f"{a} {where} rot.scaling")
            else:
                left, right = _sub(m, "left", where), _sub(m, "right", where)
                _heads(left, where + " left", a)
                if left.get("q_temp"):
                    _require(left["q_temp"], "coef", float, f"{a} {where} q_temp")
                    if int(_require(left["q_temp"], "every", int, f"{a} {where} q_temp")) <= 0:
                        raise ConfigError(f"{a}: {where}: q_temp.every must be positive")
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    if int(_require(right, key, int, f"{a} {where} right")) <= 0:
                        raise ConfigError(f"{a}: {where}: right.{key} must be positive")
                _require(m, "left_scale", float, f"{a} {where}")
                _require(m, "right_scale", float, f"{a} {where}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _require(mlp, "ff", int, f"{a} {where} mlp")
            elif mlp.get("kind") == "moe":
                r = _sub(mlp, "router", where)
                _require(r, "experts", int, f"{a} {where} router")
                _require(r, "top", int, f"{a} {where} router")
                _require(_sub(mlp, "expert", where), "ff", int, f"{a} {where} expert")
                if mlp.get("shared") is not None:
                    _require(mlp["shared"], "ff", int, f"{a} {where} shared")
            else:
                raise ConfigError(f"{a}: {where} has a feed-forward of kind {mlp.get('kind')!r}; "
                                  f"built: {', '.join(MLP_KINDS)}")

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [copy.deepcopy(dict(l)) for l in self.layers],
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
    def _attention(self, m: Mapping[str, Any]) -> Dict[str, Any]:
        return {"hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                "head_dim": int(m["dim"]), "value_head_dim": int(m["vdim"]), "scale": float(m["scale"]),
                "eps": self.norm_eps, "sink": "learned"}

    def _mixer_spec(self, i: int, layer: Mapping[str, Any]) -> PartSpec:
        m, kind, prefix = layer["mixer"], layer["type"], f"l{i}.mix."
        if kind == "attention":
            p = self._attention(m)
            mask = m.get("mask") or {}
            size = mask.get("size")
            p.update(mask="causal" if size is None else "window", mask_size=None if size is None else int(size),
                     keep_first=0 if size is None else int(mask.get("keep_first") or 0), channel_gate=True,
                     distance_bias={"max": float(m["bias_max"]), "buckets": m.get("bias_buckets")})
            return PartSpec("modulated_attention", p, prefix)
        if kind == "latent_attention":
            rot = m["rot"]
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "heads": int(m["heads"]), "dim": int(m["dim"]),
                "rot_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]),
                "q_rank": int(m["q_rank"]), "window": None, "scale": float(m["scale"]),
                "rot_base": float(rot["base"]), "rot_dims": int(rot["dims"]),
                "rot_scaling": None if not rot.get("scaling") else dict(rot["scaling"]), "sink": True,
                "eps": self.norm_eps}, prefix)
        left, right = m["left"], m["right"]
        lp = self._attention(left)
        lp.update(mask="causal", softcap=None if not left.get("softcap") else float(left["softcap"]),
                  query_temperature=None if not left.get("q_temp") else dict(left["q_temp"]))
        rp = {"hidden_size": self.width, "heads": int(right["heads"]), "head_dim": int(right["vdim"]),
              "state": int(right["state"]), "groups": int(right["groups"]), "conv_taps": int(right["conv"]),
              "norm_groups": int(right["norm_groups"]), "eps": self.norm_eps}
        return PartSpec("side_by_side", {
            "hidden_size": self.width, "join": "sum", "left_scale": float(m["left_scale"]),
            "right_scale": float(m["right_scale"]),
            "left": {"kind": "modulated_attention", "params": lp},
            "right": {"kind": "state_space_duality", "params": rp}}, prefix)

    def _mlp_spec(self, i: int, mlp: Mapping[str, Any]) -> PartSpec:
        prefix = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return PartSpec("dense_mlp", {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                                          "activation": "relu2", "tensor_names": ("up", "down")}, prefix)
        shared = mlp.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]),
            "expert_ff": int(mlp["expert"]["ff"]), "shared_ff": 0 if shared is None else int(shared["ff"]),
            "activation": "gelu", "score": "sigmoid", "renormalize": False, "weight_on": "input"}, prefix)

    def model_spec(self) -> ModelSpec:
        norm = {"hidden_size": self.width, "streams": 1, "tensor": ""}
        layers: List[LayerSpec] = []
        for i, layer in enumerate(self.layers):
            parts = {"mixer_norm": PartSpec("dynamic_tanh", norm, f"l{i}.norm1"), "mixer": self._mixer_spec(i, layer)}
            mlp = layer.get("mlp")
            if mlp is None:
                layers.append(LayerSpec("pre_norm_mixer_only", parts))
                continue
            parts["feed_forward_norm"] = PartSpec("dynamic_tanh", norm, f"l{i}.norm2")
            parts["feed_forward"] = self._mlp_spec(i, mlp)
            layers.append(LayerSpec("pre_norm", parts))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "residual": "float32", "tensor": ""}, "embed"),
            layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(layers))),
            final_norm=PartSpec("dynamic_tanh", norm, "final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": "embed",
                                      "tensor": ""}, "head"),
            eos_token_ids=self.eos_token_id)


register_architecture(RufisunConfig.architecture, RufisunConfig)
