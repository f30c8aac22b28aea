"""Small Rufisun configurations for the tests, and a helper that writes them as model folders."""

from __future__ import annotations

import os
import tempfile
from typing import Optional


def _attention(heads, kv_heads, dim, vdim, scale, bias_max, buckets, size=None, keep=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max,
         "bias_buckets": buckets}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep or 0}
    return m


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None, dims=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "scale": scale, "rot": rot}


def _parallel(left, right, left_scale, right_scale):
    heads, kv_heads, dim, vdim, scale, q_temp, cap = left
    l = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp is not None:
        l["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if cap is not None:
        l["softcap"] = cap
    r = dict(zip(("heads", "vdim", "state", "groups", "conv", "norm_groups"), right))
    return {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}


def _moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


def _dense(ff):
    return {"kind": "dense", "ff": ff}


# what write_folder multiplies the embedding table and the query and key matrices by
EMBED_UP, QK_UP = 5.0, 1.3

CASES = {
    # odd sizes: no width or head size a power of two, values wider and narrower than keys, a window that is no
    # multiple of the page and shorter than the kernels' key tiles, kept first tokens that end inside a page,
    # rotation on a part of the rotated channels with a ramp over a few pairs, groups of two state-space heads,
    # a layer without a feed-forward, experts with and without a shared one
    "P": {
        "config": {"architecture": "Rufisun", "vocab": 211, "width": 88, "norm": {"eps": 3e-6},
                   "layers": [
                       {"type": "attention", "mixer": _attention(6, 2, 24, 40, 0.9, 50, 12, 23, 5), "mlp": _dense(50)},
                       {"type": "latent_attention",
                        "mixer": _latent(3, 20, 6, 12, 37, 19, 1.1, 10000.0, (4.0, 64, 32.0, 1.0), dims=4),
                        "mlp": _moe(5, 2, 20, 12)},
                       {"type": "parallel",
                        "mixer": _parallel((4, 1, 20, 28, 1.2, (0.4, 7), 5.0), (6, 12, 20, 3, 3, 2), 0.7, 1.3),
                        "mlp": None},
                       {"type": "attention", "mixer": _attention(1, 1, 36, 20, 0.7, 30, 7, 9, 0), "mlp": _moe(3, 1, 44)},
                   ]},
        "seed": 5, "page_size": 4},
    # heads of 64 and 128 with values as wide as keys (the tensor-core kernels in bfloat16), pages of 16, windows
    # longer than a key tile, kept tokens of exactly one page and of a few tokens, the layers in another order
    "Q": {
        "config": {"architecture": "Rufisun", "vocab": 300, "width": 128, "norm": {"eps": 2e-5},
                   "layers": [
                       {"type": "parallel",
                        "mixer": _parallel((8, 2, 64, 64, 0.3, (0.25, 16), 30.0), (4, 64, 64, 1, 4, 1), 1.1, 0.8),
                        "mlp": _moe(8, 2, 64, 64)},
                       {"type": "attention", "mixer": _attention(8, 2, 64, 64, 0.25, 40, 16, 44, 16), "mlp": _dense(96)},
                       {"type": "latent_attention", "mixer": _latent(2, 48, 16, 32, 64, 48, 0.35, 30000.0), "mlp": None},
                       {"type": "attention", "mixer": _attention(2, 1, 128, 128, 0.15, 100, 32, 77, 3),
                        "mlp": _moe(4, 1, 32, 40)},
                   ]},
        "seed": 6, "page_size": 16},
    # values that other models make equal or 1: a width that is no multiple of 4, nine query heads on one key
    # head, a window longer than any request of the tests (nothing is ever masked or given back) with kept
    # tokens, an attention without a mask section, a convolution of one tap and one of two, every state-space
    # head a group of its own, every expert chosen, no query temperature and no cap, a table of two buckets
    "R": {
        "config": {"architecture": "Rufisun", "vocab": 97, "width": 90, "norm": {"eps": 1e-6},
                   "layers": [
                       {"type": "attention", "mixer": _attention(9, 1, 20, 28, 1.0, 1000, 2, 1000, 7), "mlp": _moe(3, 3, 20, 8)},
                       {"type": "parallel",
                        "mixer": _parallel((5, 5, 12, 20, 1.3, None, None), (4, 8, 16, 4, 1, 4), 1.0, 1.0),
                        "mlp": _dense(33)},
                       {"type": "attention", "mixer": _attention(4, 2, 32, 32, 0.8, 64, 9), "mlp": _dense(20)},
                       {"type": "parallel",
                        "mixer": _parallel((2, 1, 16, 16, 1.1, (1.0, 1), 2.0), (1, 24, 12, 1, 2, 1), 2.0, 0.5),
                        "mlp": _moe(2, 1, 16)},
                       {"type": "latent_attention", "mixer": _latent(1, 8, 4, 8, 16, 8, 1.5, 77.0, (2.0, 16, 2.0, 1.0)),
                        "mlp": _dense(24)},
                   ]},
        "seed": 7, "page_size": 8},
    # every layer an attention with a window: a request holds a bounded number of pages however long it grows,
    # the pages of its kept first tokens among them (they end inside the second page)
    "W": {
        "config": {"architecture": "Rufisun", "vocab": 120, "width": 64, "norm": {"eps": 1e-5},
                   "layers": [
                       {"type": "attention", "mixer": _attention(4, 2, 16, 16, 1.0, 24, 8, 20, 6), "mlp": _dense(40)},
                       {"type": "attention", "mixer": _attention(2, 2, 32, 24, 0.8, 24, 8, 20, 6), "mlp": _moe(4, 2, 16, 8)},
                   ]},
        "seed": 8, "page_size": 4},
}


def write_folder(name: str, folder: Optional[str] = None, strip: bool = True) -> str:
    """Write the case as a model folder with random weights.  The embedding table and the query and key matrices
    are multiplied up afterwards so that the attention is peaked on few keys (a wrong key, bias or mask shows in
    the logits), and the sinks are raised so that they weigh about as much as the keys together.  ``strip`` takes
    the keys that only size random weights out of config.json, so that the number of buckets has to be read off
    the tensor."""
    import json

    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model

    case = CASES[name]
    cfg = config_from_dict(case["config"])
    folder = folder or tempfile.mkdtemp(prefix=f"ll_rufisun_{name}_")
    write_random_model(folder, cfg, case["seed"], {"matrix": 0.12, "bias": 0.1, "norm": 0.1})
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    for k in list(t):
        if k == "embed":
            t[k] = (t[k].float() * EMBED_UP).to(t[k].dtype)
        elif k.rsplit(".", 1)[-1] in ("q", "k", "uq", "uk"):
            t[k] = (t[k].float() * QK_UP).to(t[k].dtype)
        elif k.endswith(".sink"):
            t[k] = (t[k].float() + 2.5).to(t[k].dtype)
    save_file(t, path, metadata={"format": "pt"})
    if strip:
        path = os.path.join(folder, "config.json")
        d = json.load(open(path))
        for layer in d["layers"]:
            layer["mixer"].pop("bias_buckets", None)
        for k in ("vocab_size", "initializer_range"):
            d.pop(k, None)
        json.dump(d, open(path, "w"))
    return folder
