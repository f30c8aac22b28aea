"""Small Lenuzen configurations for the tests, and a helper that writes them as model folders."""

from __future__ import annotations

import tempfile
from typing import Optional


def _rot(dims, base, scaling=None):
    d = {"base": base, "dims": dims}
    if scaling is not None:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def _mixer(heads, kv_heads, dim, vdim, scale, mask, rot):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": None if mask is None else {"size": mask}, "rot": rot}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CASES = {
    # odd sizes: no width or head size a power of two, values wider and narrower than keys, rotation on a part of
    # the channels, a window and chunks that are no multiple of the page (and smaller than the kernels' key tiles),
    # every query head with a key head of its own in one layer, one head in another, a layer without a
    # feed-forward, the frequency scaling with a ramp over a few pairs, scales that are not dim^-1/2
    "P": {
        "config": {"architecture": "Lenuzen", "vocab": 211, "width": 88, "embedding": {"scale": 3.5},
                   "norm": {"eps": 3e-6}, "logit_scale": 0.7,
                   "layers": [
                       _layer("attention", _mixer(3, 3, 24, 40, 0.33, 7, _rot(10, 10000.0, (4.0, 64, 32.0, 1.0))), 50),
                       _layer("attention_2", _mixer(6, 2, 16, 8, 0.4, 10, _rot(16, 500.0, (3.0, 40, 16.0, 2.0))), 24),
                       _layer("attention", _mixer(1, 1, 36, 20, 0.25, 23, _rot(36, 77.0, (1.5, 30, 8.0, 1.0))), None),
                       _layer("attention_2", _mixer(1, 1, 20, 44, 0.35, 3, _rot(6, 9000.0, (6.0, 1500, 24.0, 1.0))), 33),
                   ]},
        "seed": 5, "page_size": 4},
    # heads of 64 and 128 with values as wide as keys (the tensor-core kernels in bfloat16), pages of 16, a window
    # and chunks longer than a key tile, a chunk that is no multiple of anything, a logit scale of 1
    "Q": {
        "config": {"architecture": "Lenuzen", "vocab": 300, "width": 128, "embedding": {"scale": 11.3},
                   "norm": {"eps": 2e-5}, "logit_scale": 1.0,
                   "layers": [
                       _layer("attention_2", _mixer(4, 4, 128, 128, 0.13, 48, _rot(128, 10000.0, (2.0, 64, 32.0, 1.0))), 96),
                       _layer("attention", _mixer(8, 2, 64, 64, 0.19, 44, _rot(32, 1e6, (8.0, 100, 32.0, 1.0))), 64),
                       _layer("attention_2", _mixer(8, 2, 64, 64, 0.19, 33, _rot(64, 50000.0, (4.0, 50, 4.0, 0.5))), None),
                       _layer("attention", _mixer(2, 1, 128, 128, 0.13, 77, _rot(64, 10000.0, (16.0, 32, 32.0, 1.0))), 40),
                   ]},
        "seed": 6, "page_size": 16},
    # a width that is no multiple of 4, nine query heads on one key head, a window and chunks longer than any
    # request of the tests (nothing is ever masked or given back), a rotation without scaling and a layer
    # without any rotation, no mask at all in one layer
    "R": {
        "config": {"architecture": "Lenuzen", "vocab": 97, "width": 90, "embedding": {"scale": 1.0},
                   "norm": {"eps": 1e-6}, "logit_scale": 2.5,
                   "layers": [
                       _layer("attention", _mixer(9, 1, 20, 28, 0.4, 1000, _rot(6, 77.0)), 33),
                       _layer("attention_2", _mixer(5, 5, 12, 20, 0.5, 400, None), 20),
                       _layer("attention_2", _mixer(4, 2, 32, 32, 0.3, None, _rot(32, 10000.0, (2.0, 16, 2.0, 1.0))), 20),
                   ]},
        "seed": 7, "page_size": 8},
}


def write_folder(name: str, folder: Optional[str] = None) -> str:
    """Write the case as a model folder with random weights.  The cases' score scales are chosen so that the
    attention is peaked on few keys (queries and keys are normalised, so the scale alone sets the spread)."""
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model

    case = CASES[name]
    cfg = config_from_dict(case["config"])
    folder = folder or tempfile.mkdtemp(prefix=f"ll_lenuzen_{name}_")
    write_random_model(folder, cfg, case["seed"], {"matrix": 0.12, "bias": 0.1, "norm": 0.1})
    return folder
