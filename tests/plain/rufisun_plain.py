"""Plain, slow Rufisun forward pass: the oracle of the Rufisun tests.

Whole sequences, no cache, no batching, one function for each mechanism, float64
throughout.  It shares no code with ``lite_lang_b200``: it reads ``config.json``
and ``model.safetensors`` itself and works on torch tensors on the CPU.

The design in this file's notation (x: residual row of a token, p: its position
from 0, E: embedding table).

*Residual.*  x = E[token].  A layer is x += mixer(N1(x)); x += ff(N2(x)) (the second
only if the layer has a feed-forward).  N(u) = tanh(a u) * w + b with a scalar a.
Logits = E N_f(x).

*Mixer "attention".*  q = Wq u, k = Wk u, v = Wv u; query head a reads key/value head
a // (H/G).  s_ij = scale q_i . k_j + T[bucket(i - j), a]; with B rows in T, h = B // 2
and D = bias_max: bucket(n) = n for n < h, else min(B - 1, h + floor(ln(n / h) /
ln(D / h) * (B - h))).  j is visible from i if j <= i and (i - j < W or j < K).
Weights e^s_ij / (e^sink_a + sum_j' e^s_ij').  The heads side by side are multiplied
by sigmoid(Wg u), then Wo.

*Mixer "latent_attention".*  c_q = R(W_dq u) w_dq, q = W_uq c_q, per head [d plain | r
rotated]; W_dkv u = [c' | k_r]: c = R(c') w_dkv, k_r one rotated key part for all heads;
plain key of head a: (W_uk c)_a, value (W_uv c)_a; s_ij = scale (q_plain . k_plain +
rot(q_r) . rot(k_r)); causal; weights with a sink as above; Wo.  R(u) = u / sqrt(mean
u^2 + eps).  Rotation: channels (2i, 2i+1) turned by p f_i, cos and sin times c_m.  With
b_i = base^(-2i/r), d(t) = r ln(orig / (2 pi t)) / (2 ln base), lo = max(floor d(fast),
0), hi = min(ceil d(slow), r - 1), g_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):
f_i = (b_i / F) g_i + b_i (1 - g_i), c_m = 0.1 ln F + 1.

*Mixer "parallel".*  out = s_l left(u) + s_r right(u).
Left: attention as the first, without bias table, window and gate; q_i is multiplied by
1 + coef ln(floor((i + 1) / every) + 1); s <- cap tanh(s / cap); causal; sink.
Right: W_in u = [z | x | B | C | dt]; [x | B | C] through a causal convolution per
channel (taps weights, the last for the current token, and a bias) and silu;
dt = softplus(dt + dt_bias); per head a (group a // (heads / groups)):
S_t = exp(-exp(A_log_a) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D_a x_t;
y silu(z), then R over each of norm_groups equal parts, times w, then Wo.

*Feed-forward.*  dense: D relu(U u)^2.  moe: z = W_r u, s = sigmoid(z), the top largest
chosen; out = sum over chosen e of D_e gelu(U_e (s_e u)) + D_s gelu(U_s u), gelu the erf
form.
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


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def tanh_norm(u, w, prefix: str):
    return torch.tanh(w[prefix + ".alpha"] * u) * w[prefix] + w[prefix + ".b"]


def unit_rms(u: torch.Tensor, eps: float) -> torch.Tensor:
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def distance_bucket(n: int, B: int, D: float) -> int:
    h = B // 2
    if n < h:
        return n
    return min(B - 1, h + int(math.floor(math.log(n / h) / math.log(D / h) * (B - h))))


def distance_bias(table: torch.Tensor, T: int, D: float) -> torch.Tensor:
    """table [B, H] -> [H, T, T]: entry (a, i, j) = table[bucket(i - j), a] for j <= i (0 elsewhere)."""
    B = table.shape[0]
    by_distance = torch.stack([table[distance_bucket(n, B, D)] for n in range(T)])       # [T, H]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return by_distance[(i - j).clamp(min=0)].permute(2, 0, 1)


def visible_window_keep(T: int, W: Optional[int], keep: int) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    inside = (i - j < W) if W is not None else torch.ones((T, T), dtype=torch.bool)
    return (j <= i) & (inside | (j < keep))


def softmax_with_sink(s: torch.Tensor, vis: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """s [T, T], sink a number: e^s_j / (e^sink + sum e^s_j')."""
    s = s.masked_fill(~vis, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - m)
    return e / (torch.exp(sink - m) + e.sum(-1, keepdim=True))


def sink_attention(q, k, v, scale, vis, sink, bias=None, cap=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv], vis [T, T], sink [H], bias [H, T, T] -> [T, H, dv]."""
    H, G = q.shape[1], k.shape[1]
    out = []
    for a in range(H):
        s = (q[:, a] @ k[:, a // (H // G)].T) * scale
        if cap is not None:
            s = cap * torch.tanh(s / cap)
        if bias is not None:
            s = s + bias[a]
        out.append(softmax_with_sink(s, vis, sink[a]) @ v[:, a // (H // G)])
    return torch.stack(out, dim=1)


def scaled_frequencies(rot: Mapping):
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


def rotate(u: torch.Tensor, pos: torch.Tensor, rot: Mapping) -> torch.Tensor:
    """u [T, heads, width]; pairs (2i, 2i+1) of the first rot.dims channels turned, the rest kept."""
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


# --------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------

def mixer_attention(u, pos, m, w, p, eps):
    T = u.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (u @ w[p + "q"].T).view(T, H, d)
    k = (u @ w[p + "k"].T).view(T, G, d)
    v = (u @ w[p + "v"].T).view(T, G, dv)
    mask = m.get("mask") or {}
    vis = visible_window_keep(T, None if mask.get("size") is None else int(mask["size"]), int(mask.get("keep_first") or 0))
    bias = distance_bias(w[p + "rel"], T, float(m["bias_max"]))
    o = sink_attention(q, k, v, float(m["scale"]), vis, w[p + "sink"], bias=bias)
    return (o.reshape(T, H * dv) * sigmoid(u @ w[p + "g"].T)) @ w[p + "o"].T


def mixer_latent_attention(u, pos, m, w, p, eps):
    T = u.shape[0]
    H, d, r, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = unit_rms(u @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    ckv = u @ w[p + "dkv"].T
    c = unit_rms(ckv[:, :R], eps) * w[p + "dkv.norm"]
    k_rot = rotate(ckv[:, None, R:], pos, m["rot"])                       # [T, 1, r]
    q_rot = rotate(q[:, :, d:], pos, m["rot"])
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    qq = torch.cat([q[:, :, :d], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, r)], dim=-1)
    vis = visible_window_keep(T, None, 0)
    o = sink_attention(qq, kk, v, float(m["scale"]), vis, w[p + "sink"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def capped_attention(u, pos, m, w, p):
    T = u.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (u @ w[p + "q"].T).view(T, H, d)
    k = (u @ w[p + "k"].T).view(T, G, d)
    v = (u @ w[p + "v"].T).view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        f = 1.0 + float(qt["coef"]) * torch.log(torch.floor((pos.to(F) + 1.0) / int(qt["every"])) + 1.0)
        q = q * f[:, None, None]
    cap = m.get("softcap")
    o = sink_attention(q, k, v, float(m["scale"]), visible_window_keep(T, None, 0), w[p + "sink"],
                       cap=None if cap is None else float(cap))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def causal_convolution(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], weight [C, taps] (the last column is the current token's), zeros before the start."""
    T, taps = x.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, x.shape[1]), dtype=x.dtype), x], dim=0)
    out = bias.expand(T, -1).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * weight[:, j]
    return out


def state_space(u, m, w, p, eps):
    T = u.shape[0]
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * P
    proj = u @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    Bm = xbc[:, inner:inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                                  # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros((T, H, P), dtype=F)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros((N, P), dtype=F)
        for t in range(T):
            S = decay[t, a] * S + dt[t, a] * torch.outer(Bm[t, g], x[t, a])
            y[t, a] = S.T @ Cm[t, g] + w[p + "D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def mixer_parallel(u, pos, m, w, p, eps):
    left = capped_attention(u, pos, m["left"], w, p + "left.")
    right = state_space(u, m["right"], w, p + "right.", eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


MIXERS = {"attention": mixer_attention, "latent_attention": mixer_latent_attention, "parallel": mixer_parallel}


# --------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------

def dense_ff(u, w, p):
    return torch.relu(u @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def routed_ff(u, mlp, w, p, margins=None):
    """``margins`` (a list) receives, a token, how far the last chosen expert's score is above the first one not
    chosen (infinite if all are chosen): where that is tiny, rounding may choose otherwise."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    s = sigmoid(u @ w[p + "router"].T)                                    # [T, E]
    if margins is not None:
        ordered = torch.sort(s, dim=-1, descending=True).values
        margins.append(ordered[:, top - 1] - ordered[:, top] if top < E else torch.full((u.shape[0],), math.inf, dtype=F))
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            out[t] += gelu_erf((s[t, e] * u[t]) @ w[f"{p}e{e}.up"].T) @ w[f"{p}e{e}.down"].T
    if mlp.get("shared"):
        out = out + gelu_erf(u @ w[p + "shared.up"].T) @ w[p + "shared.down"].T
    return out


def feed_forward(u, mlp, w, p, margins=None):
    return dense_ff(u, w, p) if mlp["kind"] == "dense" else routed_ff(u, mlp, w, p, margins)


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------

def forward(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None,
            margins: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: receives the residual after every layer;
    ``margins``: every routed layer's margins (see ``routed_ff``)."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = w["embed"][ids]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](tanh_norm(x, w, p + "norm1"), pos, layer["mixer"], w, p + "mix.", eps)
        if layer.get("mlp") is not None:
            x = x + feed_forward(tanh_norm(x, w, p + "norm2"), layer["mlp"], w, p + "mlp.", margins)
        if layers_out is not None:
            layers_out.append(x.clone())
    return tanh_norm(x, w, "final.norm") @ w["embed"].T
