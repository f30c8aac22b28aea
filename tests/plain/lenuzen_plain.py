"""Plain, slow Lenuzen forward pass: the oracle of the Lenuzen tests.

Whole sequences, no cache, no batching, one function for each mechanism, float64
throughout.  It shares no code with ``lite_lang_b200``: it reads ``config.json``
and ``model.safetensors`` itself and works on torch tensors on the CPU.

The design in this file's notation (x: residual row of a token, p: its position
from 0, E: embedding table, n = width).

*Residual.*  x = s_e E[token].  A layer is x += L1(mixer(x)); x += L2(ff(x)): the
sublayers read x unnormalised, the norm sits on their output.  L(u) = (u - mean u)
/ sqrt(mean (u - mean u)^2 + eps) * w.  Logits = s_l E L_f(x).

*Rotation* R_p on the first r channels of a head: channels (2i, 2i+1) are turned by
the angle p f_i and both cos and sin carry the factor c = 0.1 ln(F) + 1.  With
b_i = base^(-2i/r), d(t) = r ln(orig / (2 pi t)) / (2 ln base), lo = max(floor
d(fast), 0), hi = min(ceil d(slow), r - 1), g_i = clamp((i - lo) / max(hi - lo,
0.001), 0, 1): f_i = (b_i / F) g_i + b_i (1 - g_i).

*Mixer A* ("attention").  q = Wq x + bq, k, v alike; q, k <- U(R_p q), U(R_p k) per
head, v <- U(v) per head, U(u) = u / sqrt(mean u^2 + eps); query head a reads
key/value head a // (H/G); s_ij = scale tau_a q_i . k_j for 0 <= i - j < W;
softmax over j; o_a <- sigmoid((Wg x)_a) o_a; out = Wo [o_0 .. o_(H-1)].

*Mixer B* ("attention_2").  q = Wq x, k, v alike, no biases; q <- wq * q / sqrt(mean
over all H d channels of q^2 + eps), k alike over its G d channels; R_p on both;
s_ij^a = scale q_i^a . k_j^a; t^a = sum_b T[a, b] s^b; j is visible from i if j <= i
and i // C == j // C; weights e^t_j / (1 + sum_j' e^t_j'); out = Wo [o_0 ..].

*Feed-forward.*  D gelu_tanh(U x).
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional

import torch
from safetensors import safe_open

F = torch.float64


def read_model_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as fh:
        for name in fh.keys():
            t = fh.get_tensor(name)
            tensors[name] = t.to(F) if t.is_floating_point() else t
    return cfg, tensors


# --------------------------------------------------------------------------
# small pieces
# --------------------------------------------------------------------------

def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def layer_norm(u: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    c = u - u.mean(-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w


def unit_rms(u: torch.Tensor, eps: float) -> torch.Tensor:
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def scaled_frequencies(rot: Mapping) -> (torch.Tensor, float):
    """f_i for i < r/2, and the factor on cos and sin."""
    r, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(r // 2, dtype=F)
    b = base ** (-2.0 * i / r)
    sc = rot.get("scaling")
    if not sc:
        return b, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def d(t):
        return r * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(sc["fast"]))), 0)
    hi = min(math.ceil(d(float(sc["slow"]))), r - 1)
    g = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return b / factor * g + b * (1.0 - g), 0.1 * math.log(factor) + 1.0


def rotate(u: torch.Tensor, pos: torch.Tensor, rot: Optional[Mapping]) -> torch.Tensor:
    """u [T, heads, d]; pairs (2i, 2i+1) of the first r channels turned, the rest kept."""
    if not rot:
        return u
    r = int(rot["dims"])
    if r == 0:
        return u
    f, c = scaled_frequencies(rot)
    ang = pos.to(F)[:, None] * f[None, :]
    cs, sn = (torch.cos(ang) * c)[:, None, :], (torch.sin(ang) * c)[:, None, :]
    a, b = u[..., 0:r:2], u[..., 1:r:2]
    out = u.clone()
    out[..., 0:r:2] = a * cs - b * sn
    out[..., 1:r:2] = b * cs + a * sn
    return out


def visible_window(T: int, W: int) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < W)


def visible_chunk(T: int, C: int) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // C == j // C)


def softmax_masked(s: torch.Tensor, vis: torch.Tensor) -> torch.Tensor:
    s = s.masked_fill(~vis, -math.inf)
    e = torch.exp(s - s.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def softmax_with_sink(s: torch.Tensor, vis: torch.Tensor) -> torch.Tensor:
    """e^s_j / (1 + sum e^s_j'): a further key of score 0 that carries no value."""
    s = s.masked_fill(~vis, -math.inf)
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def shaped_attention(q, k, v, scale, vis, temp=None, mix=None, sink=False, gate=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv], vis [T, T] -> [T, H, dv].  temp [H]: a factor a head on the
    scores; mix [H, H]: the heads' scores of a (query, key) pair mixed; gate [T, H]: a factor on the outputs."""
    H, G = q.shape[1], k.shape[1]
    s = torch.stack([(q[:, a] @ k[:, a // (H // G)].T) * scale * (1.0 if temp is None else temp[a]) for a in range(H)])
    if mix is not None:
        s = torch.einsum("ab,bij->aij", mix, s)
    soft = softmax_with_sink if sink else softmax_masked
    o = torch.stack([soft(s[a], vis) @ v[:, a // (H // G)] for a in range(H)], dim=1)
    return o if gate is None else o * gate[:, :, None]


# --------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------

def mixer_a(x: torch.Tensor, pos: torch.Tensor, m: Mapping, w: Mapping[str, torch.Tensor], p: str, eps: float):
    T = x.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (x @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (x @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (x @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q = unit_rms(rotate(q, pos, m.get("rot")), eps)
    k = unit_rms(rotate(k, pos, m.get("rot")), eps)
    v = unit_rms(v, eps)
    gate = sigmoid(x @ w[p + "g"].T)                  # [T, H]
    size = (m.get("mask") or {}).get("size")
    vis = visible_window(T, int(size) if size else T)
    o = shaped_attention(q, k, v, float(m["scale"]), vis, temp=w[p + "temp"], gate=gate)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def mixer_b(x: torch.Tensor, pos: torch.Tensor, m: Mapping, w: Mapping[str, torch.Tensor], p: str, eps: float):
    T = x.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = unit_rms(x @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = unit_rms(x @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = (x @ w[p + "v"].T).view(T, G, dv)
    q = rotate(q.view(T, H, d), pos, m.get("rot"))
    k = rotate(k.view(T, G, d), pos, m.get("rot"))
    size = (m.get("mask") or {}).get("size")
    vis = visible_chunk(T, int(size) if size else T)
    o = shaped_attention(q, k, v, float(m["scale"]), vis, mix=w[p + "talk"], sink=True)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def feed_forward(x: torch.Tensor, w: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_tanh(x @ w[p + "up"].T) @ w[p + "down"].T


MIXERS = {"attention": mixer_a, "attention_2": mixer_b}


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------

def forward(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: receives the residual after every layer."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = w["embed"][ids] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](x, pos, layer["mixer"], w, p + "mix.", eps)
        x = x + layer_norm(y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(feed_forward(x, w, p + "mlp."), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["embed"].T * float(cfg.get("logit_scale", 1.0))
