"""Lenuzen through the engine against the plain implementation (tests/plain/lenuzen_plain.py).

CPU: configuration, registry, cache groups (a window and chunks give pages back), the scaled rotary frequencies,
the plain implementation's own properties.  GPU: each mechanism's kernels alone (with inputs made so that a fault
at an edge shows), whole prompts, token-by-token decoding through captured steps, portions down to two tokens,
mixed batches with pages and slots used again, the command-line replay tool and greedy generation through the
scheduler.
"""
import json
import math
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

from helpers import TraceRun, rel_err
from lenuzen_cases import CASES, write_folder
from plain import lenuzen_plain as P

TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
gpu = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def row_errors(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    return np.abs(got - ref).max(axis=-1) / np.abs(ref).max(axis=-1)


def close(got, ref, dtype) -> bool:
    """Every row of logits within the tolerance of its dtype: the design has nothing that decides (no router,
    no top-k), so no row is excused."""
    e = row_errors(got, ref)
    return bool(e.max() <= TOL[torch.float32 if dtype in (torch.float32, "float32") else torch.bfloat16])


def kernel_tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.6e-2


# ---------------------------------------------------------------------------------------------------------
# CPU
# ---------------------------------------------------------------------------------------------------------

def test_config_registry_and_round_trip():
    from lite_lang_b200.config import ConfigError, config_from_dict, known_architectures
    assert "Lenuzen" in known_architectures()
    cfg = config_from_dict(CASES["P"]["config"])
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert [l.block for l in spec.layers] == ["output_norm", "output_norm", "output_norm_mixer_only", "output_norm"]
    a, b = spec.layers[0].parts["mixer"].params, spec.layers[1].parts["mixer"].params
    assert a["mask"] == "window" and a["mask_size"] == 7 and a["qk_norm"] == "head_unit" and a["value_norm"]
    assert a["head_gate"] and a["head_temperature"] and not a.get("sink") and not a.get("head_mix")
    assert b["mask"] == "chunk" and b["mask_size"] == 10 and b["qk_norm"] == "projection" and b["sink"] and b["head_mix"]
    assert a["value_head_dim"] == 40 and a["scale"] == 0.33 and a["position"].params["rotary_dim"] == 10
    assert spec.head.params["scale"] == 0.7 and spec.embedding.params["scale"] == 3.5
    # no mask section: plain causal attention; no rotation section: no position part
    r = config_from_dict(CASES["R"]["config"]).model_spec()
    assert r.layers[2].parts["mixer"].params["mask"] == "causal"
    assert "position" not in r.layers[1].parts["mixer"].params
    for path, value in ((("layers", 0, "type"), "attention_3"), (("layers", 1, "mixer", "kv_heads"), 4),
                        (("layers", 0, "mixer", "rot", "dims"), 11), (("layers", 0, "mlp", "kind"), "gated"),
                        (("layers", 1, "mixer", "mask", "size"), 0)):
        bad = cfg.to_dict()
        d = bad
        for key in path[:-1]:
            d = d[key]
        d[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(bad)
    bad = cfg.to_dict()
    del bad["norm"]
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_cache_groups_and_declared_tensors():
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.engine.model import CausalLM
    model = CausalLM(config_from_dict(CASES["P"]["config"]).model_spec())
    groups = sorted((g.head_dim, g.value_dim, g.window, g.chunk, g.planes) for g in model.cache_groups)
    assert groups == [(16, 8, None, 10, 1), (20, 44, None, 3, 1), (24, 40, 7, None, 1), (36, 20, 23, None, 1)]
    assert all(g.releases for g in model.cache_groups)
    names = model.declared_tensors()
    for n, shape in (("embed", (211, 88)), ("final.norm", (88,)), ("l0.norm1", (88,)), ("l0.norm2", (88,)),
                     ("l0.mix.q.b", (72,)), ("l0.mix.v.b", (120,)), ("l0.mix.temp", (3,)), ("l0.mix.g", (3, 88)),
                     ("l0.mix.o", (88, 120)), ("l1.mix.talk", (6, 6)), ("l1.mix.q.norm", (96,)),
                     ("l1.mix.k.norm", (32,)), ("l1.mlp.up", (24, 88)), ("l1.mlp.down", (88, 24))):
        assert tuple(names[n].shape) == shape, n
    assert names["head"].optional                                     # the head is the embedding table
    for n in ("l2.norm2", "l2.mlp.up", "l1.mix.q.b", "l1.mix.g", "l1.mix.temp", "l0.mix.talk", "l0.mix.q.norm"):
        assert n not in names, n
    # no mask: the group keeps every page
    r = CausalLM(config_from_dict(CASES["R"]["config"]).model_spec())
    assert sorted(g.releases for g in r.cache_groups) == [False, True, True]


def test_pages_go_back_behind_a_window_and_at_a_chunks_end():
    from lite_lang_b200.cache.manager import CacheManager, PagedGroupSpec
    ps = 4
    groups = [PagedGroupSpec(1, 8, 6, 1, 8), PagedGroupSpec(1, 8, None, 1, 8, 10)]
    assert groups[0].first_needed(20) == 15 and groups[1].first_needed(20) == 20 and groups[1].first_needed(19) == 10
    mgr = CacheManager(groups, [4, 4], ps, 2, 64)      # four pages a group: 16 positions for a request of 40
    s = mgr.open()
    for n in range(1, 41):
        assert mgr.reserve(s, n), n
        mgr.advance(s, n)
        mgr.check_invariants()
        held = [[lp for lp, p in enumerate(mgr.pages_of(g, s)) if p >= 0] for g in (0, 1)]
        # the next token (position n) reads from position n - 5, or from its chunk's start: no page before that
        # one's is held, and that page is (unless it is the one not yet asked for)
        for g in (0, 1):
            first = groups[g].first_needed(n) // ps
            assert all(lp >= first for lp in held[g]), (n, g)
            assert first in held[g] or first * ps >= n, (n, g)
    # position 20 opens a chunk: at length 20 the chunked group holds nothing of positions 10..19
    mgr.close(s)
    s = mgr.open()
    for n in (12, 20):
        assert mgr.reserve(s, n)
        mgr.advance(s, n)
    assert all(p < 0 for p in mgr.pages_of(1, s)) and mgr.num_free_pages(1) == 4
    assert [p >= 0 for p in mgr.pages_of(0, s)] == [False, False, False, True, True]     # positions 15.. are read
    mgr.close(s)
    mgr.check_invariants()


def test_scaled_frequencies_of_the_position_part_are_the_plain_ones():
    from lite_lang_b200.config.spec import PartSpec
    from lite_lang_b200.parts import build_part
    for dims, base, sc in ((10, 10000.0, (4.0, 64, 32.0, 1.0)), (16, 500.0, (3.0, 40, 16.0, 2.0)),
                           (64, 1e6, (8.0, 100, 32.0, 1.0)), (128, 10000.0, (40.0, 4096, 32.0, 1.0)),
                           (36, 77.0, None), (6, 10000.0, (8.0, 2048, 32.0, 1.0))):
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        part = build_part("position", PartSpec("rope_computed", {"rotary_dim": dims, "theta": base,
                                                                  "layout": "interleaved", "scaling": rot.get("scaling")}))
        f, c = P.scaled_frequencies(rot)
        assert torch.allclose(part.frequencies(), f, rtol=1e-14, atol=0)
        assert abs(part.amplitude - c) < 1e-15
    # the ramp really has three regimes in one of the cases: untouched, blended, divided by the factor
    f, _ = P.scaled_frequencies({"dims": 64, "base": 1e6, "scaling": {"factor": 8.0, "original": 100, "fast": 32.0, "slow": 1.0}})
    b = 1e6 ** (-2.0 * torch.arange(32, dtype=P.F) / 64)
    ratio = (f / b).numpy()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8.0) < 1e-12 and ((ratio < 0.999) & (ratio > 0.126)).any()


def test_plain_pieces_against_closed_forms():
    g = torch.Generator().manual_seed(0)
    # a sink: weights sum to less than one, and with no visible key of weight the output vanishes
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=P.F)
    vis = torch.tensor([[True, True, False]])
    w = P.softmax_with_sink(s, vis)
    e = torch.exp(s[0, :2])
    assert torch.allclose(w[0, :2], e / (1 + e.sum())) and float(w[0, 2]) == 0.0
    assert torch.allclose(P.softmax_masked(s, vis)[0, :2], e / e.sum())
    # windows and chunks
    assert P.visible_window(6, 3).int().tolist()[5] == [0, 0, 0, 1, 1, 1]
    assert P.visible_chunk(6, 4).int().tolist()[5] == [0, 0, 0, 0, 1, 1]
    assert P.visible_chunk(6, 4).int().tolist()[3] == [1, 1, 1, 1, 0, 0]
    # mixing with the identity is no mixing; a temperature is a factor on the scale
    q, k, v = torch.randn(5, 4, 6, generator=g, dtype=P.F), torch.randn(5, 2, 6, generator=g, dtype=P.F), torch.randn(5, 2, 3, generator=g, dtype=P.F)
    vis = P.visible_window(5, 5)
    a = P.shaped_attention(q, k, v, 0.5, vis)
    assert torch.allclose(a, P.shaped_attention(q, k, v, 0.5, vis, mix=torch.eye(4, dtype=P.F)))
    assert torch.allclose(a, P.shaped_attention(q, k, v, 0.25, vis, temp=torch.full((4,), 2.0, dtype=P.F)))
    # mixing two heads: head 0 takes head 1's scores
    swap = torch.eye(4, dtype=P.F)
    swap[0, 0], swap[0, 1] = 0.0, 1.0
    got = P.shaped_attention(q, k, v, 0.5, vis, mix=swap)
    assert torch.allclose(got[:, 0], a[:, 1]) and torch.allclose(got[:, 2], a[:, 2])
    # the layer norm has no bias and takes the mean off
    u = torch.randn(3, 7, generator=g, dtype=P.F)
    n = P.layer_norm(u + 5.0, torch.ones(7, dtype=P.F), 1e-9)
    assert torch.allclose(n, P.layer_norm(u, torch.ones(7, dtype=P.F), 1e-9)) and float(n.mean(-1).abs().max()) < 1e-12
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=P.F))) - 0.8411919906082768) < 1e-12


# ---------------------------------------------------------------------------------------------------------
# GPU: kernels alone
# ---------------------------------------------------------------------------------------------------------

def _step(entries, ctx, slots):
    """The device arrays of a step whose entries bring ``entries[i]`` tokens after ``ctx[i]`` cached ones."""
    s = types.SimpleNamespace()
    s.req_slot = torch.tensor(slots, dtype=torch.int32, device=dev())
    s.token_req = torch.tensor(np.repeat(np.arange(len(entries)), entries), dtype=torch.int32, device=dev())
    s.positions = torch.tensor(np.concatenate([np.arange(c, c + n) for n, c in zip(entries, ctx)]), dtype=torch.int32,
                               device=dev())
    s.status = torch.zeros(1, dtype=torch.int32, device=dev())
    return s


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,T", [(88, 5), (90, 3), (37, 4), (1536, 9), (5000, 2)])
def test_norm_of_a_sublayers_output_into_the_residual(dtype, hidden, T):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    res = torch.randn(T, hidden, generator=g) * 3
    y = (torch.randn(T, hidden, generator=g) * 20 + 7).to(dtype)          # a mean that is not small
    w = 1 + 0.2 * torch.randn(hidden, generator=g)
    want = res.double() + P.layer_norm(y.double(), w.double(), 3e-6)
    r = res.to(dev()).clone()
    copy = torch.empty(T, hidden, dtype=dtype, device=dev())
    ops.layernorm_into_residual(r, y.to(dev()), w.to(dev()), 3e-6, copy)
    assert rel_err(r.cpu().numpy(), want.numpy()) <= 2e-6                 # the residual is float32 in both
    assert torch.equal(copy, r.to(dtype))
    # float32 partial sums of a split product, added up unrounded; no copy asked for
    parts = torch.randn(3, T, hidden, generator=g) * 5
    want = res.double() + P.layer_norm(parts.double().sum(0), w.double(), 3e-6)
    r = res.to(dev()).clone()
    ops.layernorm_into_residual(r, parts.to(dev()), w.to(dev()), 3e-6, None)
    assert rel_err(r.cpu().numpy(), want.numpy()) <= 2e-6
    assert torch.equal(ops.round_rows(r, dtype), r.to(dtype))


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activation_of_a_plain_feed_forward_and_scaled_logits(dtype):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(7, 50, generator=g) * 3).to(dtype)
    xd = x.to(dev()).clone()
    ops.act_rows(xd, "gelu_tanh")
    assert rel_err(xd.float().cpu().numpy(), P.gelu_tanh(x.double()).numpy()) <= kernel_tol(dtype)
    z = torch.randn(3, 41, generator=g).to(dev())
    want = z.double().cpu() * 0.37
    ops.scale_logits(z, 0.37)
    assert torch.allclose(z.double().cpu(), want, rtol=1e-6)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,rot,mode,vnorm,bias", [
    (3, 3, 24, 40, 10, "head_unit", True, True), (6, 2, 16, 8, 16, "projection", False, False),
    (1, 1, 36, 20, 36, "head_unit", True, True), (9, 1, 20, 28, 0, "projection", False, False),
    (8, 2, 64, 64, 32, "head_unit", True, True), (4, 4, 128, 128, 128, "projection", False, False),
    (2, 2, 32, 48, 32, None, False, True)])
def test_bias_norms_scaled_rotation_and_cache_write(dtype, nh, nkv, hd, vd, rot, mode, vnorm, bias):
    """The order of the steps differs with the kind of norm (over the whole projection before the rotation, a head
    after it); positions far beyond a few turns; extra columns behind q | k | v are left alone; k and v land,
    normalised, in the pages the slot map names and nowhere else."""
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(hd + nh)
    T, ps, pages, extra = 9, 4, 7, 5
    width = (nh + nkv) * hd + nkv * vd
    qkv = (torch.randn(T, width + extra, generator=g) * 2).to(dtype)
    b = torch.randn(width, generator=g) if bias else None
    qw, kw = 1 + 0.3 * torch.randn(nh * hd, generator=g), 1 + 0.3 * torch.randn(nkv * hd, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 250, 4000, 70001, 5, 6], dtype=torch.int32)
    rotd = {"dims": rot, "base": 500.0, "scaling": {"factor": 3.0, "original": 40, "fast": 16.0, "slow": 2.0}}
    freq, amp = None, 1.0
    if rot:
        f, amp = P.scaled_frequencies(rotd)
        freq = f.float().to(dev())
    eps = 3e-6
    slot_map = torch.tensor([5, 6, 7, 12, 0, 27, -1, 1, 2], dtype=torch.int32, device=dev())
    kc = torch.full((pages, nkv, ps, hd), float("nan"), dtype=dtype, device=dev())
    vc = torch.full((pages, nkv, ps, vd), float("nan"), dtype=dtype, device=dev())
    x = qkv.to(dev()).clone()
    ops.qkv_norm_rotate_store(x, None if b is None else b.to(dev()), pos.to(dev()), freq, amp, True, nh, nkv, hd, vd,
                              mode, qw.to(dev()) if mode == "projection" else None,
                              kw.to(dev()) if mode == "projection" else None, vnorm, eps, slot_map, kc, vc, ps, None)
    full = qkv.double()[:, :width] + (0 if b is None else b.double())
    q, k = full[:, :nh * hd], full[:, nh * hd:(nh + nkv) * hd]
    v = full[:, (nh + nkv) * hd:].view(T, nkv, vd)
    if mode == "projection":
        q, k = P.unit_rms(q, eps) * qw.double(), P.unit_rms(k, eps) * kw.double()
    q, k = P.rotate(q.reshape(T, nh, hd), pos, rotd if rot else None), P.rotate(k.reshape(T, nkv, hd), pos, rotd if rot else None)
    if mode == "head_unit":
        q, k = P.unit_rms(q, eps), P.unit_rms(k, eps)
    if vnorm:
        v = P.unit_rms(v, eps)
    want = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1)
    # q comes back in place; k and v go to the token's cache slot only (the row of a token without a slot keeps them)
    got = x.double().cpu()
    qn, kn = nh * hd, nkv * hd
    for t in range(T):
        s = int(slot_map[t])
        if s >= 0:
            got[t, qn:qn + kn] = kc[s // ps, :, s % ps, :].reshape(-1).double().cpu()
            got[t, qn + kn:width] = vc[s // ps, :, s % ps, :].reshape(-1).double().cpu()
        else:
            assert torch.equal(x[t, qn:width].cpu(), qkv[t, qn:width])
            got[t, qn:width] = want[t, qn:]
    # float32 angles at position 70001 carry 70001 * 2^-24 rad of rounding on the fastest pair
    tol = (3e-5 if dtype == torch.float32 else 1.6e-2) * (200 if rot else 1)
    assert float((got[:, :width] - want).abs().max()) <= tol * float(want.abs().max())
    near = [0, 1, 2, 3, 7, 8]                                  # small positions: the plain tolerance
    assert float((got[near, :width] - want[near]).abs().max()) <= kernel_tol(dtype) * float(want.abs().max())
    assert torch.equal(x[:, width:].cpu(), qkv[:, width:])
    written = {int(s) for s in slot_map if s >= 0}
    for s in range(pages * ps):
        if s not in written:
            assert bool(torch.isnan(kc[s // ps, :, s % ps]).all()) and bool(torch.isnan(vc[s // ps, :, s % ps]).all())


def _paged(dtype, seqs_k, seqs_v, ps, nkv, hd, vd, rng, first_live):
    """Keys/values of several requests scattered over a pool whose other slots hold NaN.  Pages that lie wholly
    before ``first_live[r]`` are not there (-1 in the table), as when a window or a chunk has given them back."""
    n_pages = sum((len(k) + ps - 1) // ps for k in seqs_k) + 3
    order = rng.permutation(n_pages)
    kc = torch.full((n_pages, nkv, ps, hd), float("nan"), dtype=dtype)
    vc = torch.full((n_pages, nkv, ps, vd), float("nan"), dtype=dtype)
    max_blocks = max((len(k) + ps - 1) // ps for k in seqs_k)
    bt = torch.full((len(seqs_k), max_blocks), -1, dtype=torch.int32)
    at = 0
    for r, (k, v) in enumerate(zip(seqs_k, seqs_v)):
        for j in range(len(k)):
            if (j // ps + 1) * ps <= first_live[r]:
                continue
            if bt[r, j // ps] < 0:
                bt[r, j // ps] = int(order[at])
                at += 1
            kc[bt[r, j // ps], :, j % ps] = k[j].to(dtype)
            vc[bt[r, j // ps], :, j % ps] = v[j].to(dtype)
    return kc.to(dev()), vc.to(dev()), bt.to(dev())


def _visible(mask, size, T):
    if mask == "window":
        return P.visible_window(T, size)
    if mask == "chunk":
        return P.visible_chunk(T, size)
    return P.visible_window(T, T)


def _first_read(mask, size, p):
    return max(0, p - size + 1) if mask == "window" else (p // size) * size if mask == "chunk" else 0


def _attention_case(dtype, nh, nkv, hd, vd, ps, mask, size, temp, mix, sink, gate, lens, new, seed=0, kernel="blocks"):
    """Prompt portions and single tokens of several requests in one launch, pages of earlier positions given back.
    The last queries of every request are aimed (a large dot product with one key) at the keys on both sides of
    the edge of what they may read, and at the very first key they may read.  ``kernel``: "blocks" (a block a
    token, any sizes), "shaped" (tensor cores; single tokens first, as the batch builder orders a step) or "tc" (as
    "shaped", but the temperature goes onto the queries where the model normalises them and the prompt portions
    to the plain attention's tcgen05 kernel with the gate in its epilogue)."""
    from lite_lang_b200 import ops
    if kernel in ("shaped", "tc"):
        order = sorted(range(len(lens)), key=lambda r: new[r] != 1)
        lens, new = [lens[r] for r in order], [new[r] for r in order]
    rng = np.random.default_rng(hd + seed)
    g = torch.Generator().manual_seed(hd + seed)
    R, group = len(lens), nh // nkv
    ks = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    ks = [k / k.norm(dim=-1, keepdim=True) * math.sqrt(hd) for k in ks]           # unit root mean square
    vs = [torch.randn(n, nkv, vd, generator=g) for n in lens]
    qs = [torch.randn(c, nh, hd, generator=g) for c in new]
    aimed = []
    for r in range(R):
        for back, which in ((0, "outside"), (1, "inside"), (2, "first")):
            if new[r] - 1 - back < 0:
                continue
            p = lens[r] - 1 - back
            lo = _first_read(mask, size, p)
            j = {"outside": lo - 1, "inside": lo, "first": min(lo + 1, p)}[which]
            if j < 0:
                continue
            for h in range(nh):
                qs[r][new[r] - 1 - back, h] = 6.0 * ks[r][j, h // group]
            aimed.append((r, new[r] - 1 - back, j, which))
    ks, vs, qs = ([t.to(dtype).float() for t in ts] for ts in (ks, vs, qs))
    first_live = [_first_read(mask, size, lens[r] - new[r]) for r in range(R)]
    kc, vc, bt = _paged(dtype, ks, vs, ps, nkv, hd, vd, rng, first_live)
    step = _step(new, [n - c for n, c in zip(lens, new)], list(range(R)))
    n_tok = sum(new)
    gate_w = 1 + (torch.randn(n_tok, nh, generator=g) * 2).to(dtype).float() if gate else None
    extra = nh if gate else 0
    pad = (-(nh * hd + 3 + extra)) % 8 if kernel in ("shaped", "tc") else 0      # rows on 16-byte boundaries
    proj = torch.zeros(n_tok, nh * hd + 3 + extra + pad, dtype=dtype)            # q, three other columns, the gate
    proj[:, :nh * hd] = torch.cat([x.reshape(x.shape[0], -1) for x in qs]).to(dtype)
    if gate:
        proj[:, nh * hd + 3:nh * hd + 3 + nh] = gate_w.to(dtype)
    proj = proj.to(dev())
    tv = (1 + 0.5 * torch.randn(nh, generator=g)) if temp else None
    mv = (torch.eye(nh) + 0.3 * torch.randn(nh, nh, generator=g)) if mix else None
    out = torch.full((n_tok, nh * vd), float("nan"), dtype=dtype, device=dev())
    scale = 0.9 / math.sqrt(hd)
    gate_view = proj[:, nh * hd + 3:nh * hd + 3 + nh] if gate else None
    tvd, mvd = None if tv is None else tv.to(dev()), None if mv is None else mv.to(dev())
    if kernel == "blocks":
        ops.attention_modulated(out, proj, proj.stride(0), gate_view, kc, vc, bt, step.token_req, step.req_slot,
                                step.positions, n_tok, nh, nkv, hd, vd, ps, mask, size, sink, scale, tvd, mvd,
                                step.status)
    else:
        q = proj
        if mix:       # the wider queries, made where the model makes them
            rows = torch.zeros(n_tok, (nh + nkv) * hd + nkv * vd, dtype=dtype, device=dev())
            rows[:, :nh * hd] = proj[:, :nh * hd]
            q = torch.full((n_tok, nh * nkv * hd), float("nan"), dtype=dtype, device=dev())
            ops.qkv_norm_rotate_store(rows, None, step.positions, None, 1.0, True, nh, nkv, hd, vd, None, None, None,
                                      False, 1e-6, None, None, None, ps, None, head_mix=mvd, mix_temperature=tvd,
                                      mixed_q=q)
            assert torch.equal(rows[:, :nh * hd], proj[:, :nh * hd])
        if kernel == "tc" and temp:
            rows = torch.zeros(n_tok, (nh + nkv) * hd + nkv * vd, dtype=dtype, device=dev())
            rows[:, :nh * hd] = proj[:, :nh * hd]
            ops.qkv_norm_rotate_store(rows, None, step.positions, None, 1.0, True, nh, nkv, hd, vd, None, None, None,
                                      False, 1e-6, None, None, None, ps, None, mix_temperature=tvd)
            proj[:, :nh * hd] = rows[:, :nh * hd]
            tvd = None
        cu = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32, device=dev())
        ctx = torch.tensor([n - c for n, c in zip(lens, new)], dtype=torch.int32, device=dev())
        n_single = sum(1 for c in new if c == 1)
        tail = (nh, nkv, hd, vd, ps, mask, size, sink, scale, step.status)
        head = (out, q, q.stride(0), bool(mix), gate_view, tvd, kc, vc, bt)
        if n_single:
            stages = (max(lens) + 63) // 64 + 1 if mask == "causal" else (size + 62) // 64 + 1
            span = (stages + 31) // 32
            ops.attn_shaped(*head, cu, ctx, step.req_slot, n_single, n_single * ((group + 127) // 128), *tail,
                            nsplit=(stages + span - 1) // span, span=span)
        if R > n_single and kernel == "tc":
            entries = [(lens[r] - new[r], new[r]) for r in range(n_single, R)]
            blocks, nsplit, split_len = ops.attn_prefill_tc_plan(entries, group, size if mask == "window" else None, nkv,
                                                                 2 * ops.sm_count(dev()))
            ops.attn_prefill_tc(out, q, q.stride(0), kc, vc, bt, cu[n_single:], ctx[n_single:], step.req_slot[n_single:],
                                R - n_single, blocks, nh, nkv, hd, ps, size if mask == "window" else None, scale,
                                step.status, nsplit=nsplit, split_len=split_len, gate=gate_view)
        elif R > n_single:
            ops.attn_shaped(*head, cu[n_single:], ctx[n_single:], step.req_slot[n_single:], R - n_single,
                            ops.attn_shaped_blocks(new[n_single:], group), *tail)
    assert int(step.status.item()) == 0
    want, at = [], 0
    for r in range(R):
        T, c = lens[r], new[r]
        qfull = torch.cat([torch.zeros(T - c, nh, hd, dtype=P.F), qs[r].double()])
        o = P.shaped_attention(qfull, ks[r].double(), vs[r].double(), scale, _visible(mask, size, T),
                               temp=None if tv is None else tv.double(), mix=None if mv is None else mv.double(),
                               sink=sink, gate=None if not gate else
                               torch.cat([torch.zeros(T - c, nh, dtype=P.F), P.sigmoid(gate_w[at:at + c].double())]))
        want.append(o[-c:].reshape(c, nh * vd))
        at += c
    want = torch.cat(want)
    assert not bool(torch.isnan(out).any())
    got = out.float().cpu()
    # (the wider queries of mixed heads are sums of queries rounded once more to bfloat16: with sixteen heads aimed
    # at one key that rounding shows in the scores of the other keys)
    tol = kernel_tol(dtype) * (2 if kernel in ("shaped", "tc") and (mix or (kernel == "tc" and temp)) else 1)
    assert rel_err(got.numpy(), want.numpy()) <= tol, (mask, size)
    return got, want, aimed, vs, new


ATTN_SHAPES = [  # nh, nkv, hd, vd, page size
    (3, 3, 24, 40, 4), (6, 2, 16, 8, 16), (9, 1, 20, 28, 8), (1, 1, 36, 20, 4), (8, 2, 64, 64, 16), (4, 4, 128, 128, 16),
    (2, 1, 128, 128, 64), (5, 5, 12, 20, 8)]


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,ps", ATTN_SHAPES)
def test_window_temperature_and_gate(dtype, nh, nkv, hd, vd, ps):
    for size in (7, 40, 33, 1, 1000):
        got, want, aimed, vs, new = _attention_case(dtype, nh, nkv, hd, vd, ps, "window", size, True, False, False, True,
                                                    [300, 47, 130, 3], [150, 1, 1, 3], seed=size)
        assert any(a[3] == "outside" for a in aimed) or size == 1000
    # without a temperature and a gate the same kernel is a plain windowed attention
    _attention_case(dtype, nh, nkv, hd, vd, ps, "window", 23, False, False, False, False, [100, 70], [100, 1])


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,ps", ATTN_SHAPES)
def test_chunks_mixed_heads_and_sink(dtype, nh, nkv, hd, vd, ps):
    for size in (10, 48, 33, 3, 1, 1000):
        _attention_case(dtype, nh, nkv, hd, vd, ps, "chunk", size, False, True, True, False,
                        [300, 47, 130, 3, 97], [150, 1, 1, 3, 2], seed=size)
    # each mechanism alone, and all of both kinds together on one mask
    _attention_case(dtype, nh, nkv, hd, vd, ps, "chunk", 16, False, False, True, False, [100, 33], [100, 1])
    _attention_case(dtype, nh, nkv, hd, vd, ps, "chunk", 16, False, True, False, False, [100, 33], [100, 1])
    _attention_case(dtype, nh, nkv, hd, vd, ps, "causal", None, True, True, True, True, [260, 65], [200, 1])
    _attention_case(dtype, nh, nkv, hd, vd, ps, "causal", None, False, False, False, False, [260, 65], [200, 1])


SHAPED_SHAPES = [  # nh, nkv, hd, vd, page size
    (8, 2, 64, 64, 16), (4, 4, 128, 128, 16), (2, 1, 128, 128, 64), (6, 2, 64, 128, 16), (4, 2, 128, 64, 32),
    (16, 8, 64, 64, 16), (7, 1, 128, 128, 16)]


@gpu
@pytest.mark.parametrize("nh,nkv,hd,vd,ps", SHAPED_SHAPES)
def test_shaped_scores_on_tensor_cores(nh, nkv, hd, vd, ps):
    """The same cases through the tensor-core kernels: prompt portions 128 rows a CTA beside single tokens whose
    keys are split over CTAs (windows and chunks below, at and above a stage of 64 keys and a part of several)."""
    dt = torch.bfloat16
    for size in (7, 64, 65, 33, 1, 129, 1000):
        _attention_case(dt, nh, nkv, hd, vd, ps, "window", size, True, False, False, True,
                        [300, 47, 130, 3, 260], [150, 1, 1, 3, 1], seed=size, kernel="shaped")
        _attention_case(dt, nh, nkv, hd, vd, ps, "chunk", size, False, True, True, False,
                        [300, 47, 130, 3, 97, 193], [150, 1, 1, 3, 2, 1], seed=size, kernel="shaped")
    _attention_case(dt, nh, nkv, hd, vd, ps, "chunk", 16, False, False, True, False, [100, 33], [100, 1], kernel="shaped")
    _attention_case(dt, nh, nkv, hd, vd, ps, "chunk", 16, True, True, False, True, [100, 33], [100, 1], kernel="shaped")
    _attention_case(dt, nh, nkv, hd, vd, ps, "causal", None, True, True, True, True, [260, 65], [200, 1], kernel="shaped")
    _attention_case(dt, nh, nkv, hd, vd, ps, "causal", None, False, False, False, False, [2300, 2200], [200, 1],
                    kernel="shaped")
    _attention_case(dt, nh, nkv, hd, vd, ps, "window", 48, False, False, False, False, [5, 70, 9], [1, 1, 1],
                    kernel="shaped")


@gpu
@pytest.mark.parametrize("nh,nkv,hd,ps", [(8, 2, 64, 16), (4, 4, 128, 16), (2, 1, 128, 64), (16, 8, 64, 32), (7, 1, 128, 16)])
def test_plain_scores_with_temperature_and_gate_on_the_tcgen05_kernel(nh, nkv, hd, ps):
    """Without mixed heads and sink the prompt portions run on the plain attention's tcgen05 kernel: the
    temperature on the queries, the gate in the epilogue, windows below, at and above a block of 64 keys, row
    blocks whose keys are split over CTAs."""
    dt = torch.bfloat16
    for size in (7, 64, 65, 33, 1, 129, 1000):
        _attention_case(dt, nh, nkv, hd, hd, ps, "window", size, True, False, False, True,
                        [300, 47, 130, 3, 260], [150, 1, 1, 3, 1], seed=size, kernel="tc")
    _attention_case(dt, nh, nkv, hd, hd, ps, "causal", None, True, False, False, True, [2300, 2200], [200, 1], kernel="tc")
    _attention_case(dt, nh, nkv, hd, hd, ps, "causal", None, False, False, False, True, [700, 65], [700, 2], kernel="tc")
    _attention_case(dt, nh, nkv, hd, hd, ps, "window", 200, True, False, False, False, [900], [900], kernel="tc")


@gpu
@pytest.mark.parametrize("M,K,N", [(5, 128, 200), (32, 384, 72), (9, 256, 8192), (200, 96, 136), (300, 200, 333),
                                   (66, 1536, 520), (3, 90, 33)])
def test_activation_in_the_epilogue_of_the_product(M, K, N):
    """act(x W^T) of a feed-forward without a gate: a few tokens through the weight-streaming product, many
    through the two-SM tcgen05 one, both with the activation on the accumulator; other shapes product, then
    kernel.  All against the plain gelu of the product rounded to bfloat16."""
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(M + N)
    x = (torch.randn(M, K, generator=g)).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * (2.0 / math.sqrt(K))).to(torch.bfloat16)
    got = ops.linear_act(x.to(dev()), w.to(dev()), "gelu_tanh")
    z = (x.double() @ w.double().t()).to(torch.bfloat16).double()
    assert tuple(got.shape) == (M, N) and got.dtype == torch.bfloat16
    assert rel_err(got.float().cpu().numpy(), P.gelu_tanh(z).numpy()) <= kernel_tol(torch.bfloat16)
    for act, f in (("relu", lambda t: t.clamp(min=0)), ("silu", lambda t: t * torch.sigmoid(t))):
        got = ops.linear_act(x.to(dev()), w.to(dev()), act)
        assert rel_err(got.float().cpu().numpy(), f(z).numpy()) <= kernel_tol(torch.bfloat16)


@gpu
def test_an_aimed_query_reads_its_key_inside_the_edge_and_not_the_one_outside():
    """The plain formulas agree with the kernel above; here the statement itself: a query aimed at the first key of
    its window (or chunk) returns that key's value, and one aimed at the key before it does not; with a sink a
    query that no key answers returns almost nothing."""
    nh, nkv, hd, vd, ps = 2, 1, 32, 16, 8
    for mask, size in (("window", 24), ("chunk", 24), ("window", 64), ("chunk", 64)):
        got, want, aimed, vs, new = _attention_case(torch.float32, nh, nkv, hd, vd, ps, mask, size, False, False, False,
                                                    False, [200, 131], [40, 1], seed=1)
        offs = np.concatenate([[0], np.cumsum(new)])
        seen = set()
        for r, row, j, which in aimed:
            o = got[offs[r] + row].view(nh, vd)[0]
            hit = float((o - vs[r][j, 0]).abs().max()) < 0.05 * float(vs[r][j, 0].abs().max())
            assert hit == (which != "outside"), (mask, size, r, row, j, which)
            seen.add(which)
        assert seen == {"outside", "inside", "first"}
    from lite_lang_b200 import ops
    # a sink: all keys opposite to the query
    T = 50
    k = torch.ones(T, 1, hd)
    v = torch.randn(T, 1, vd)
    kc = torch.zeros(8, 1, ps, hd)
    vc = torch.zeros(8, 1, ps, vd)
    kc.view(-1, hd)[:T], vc.view(-1, vd)[:T] = k[:, 0], v[:, 0]            # (one kv head: pages are rows of slots)
    bt = torch.arange(8, dtype=torch.int32).view(1, 8)
    q = -torch.ones(1, 2 * hd)
    step = _step([1], [T - 1], [0])
    out = torch.empty(1, 2 * vd, device=dev())
    for sink, small in ((True, True), (False, False)):
        ops.attention_modulated(out, q.to(dev()), 2 * hd, None, kc.to(dev()), vc.to(dev()), bt.to(dev()), step.token_req,
                                step.req_slot, step.positions, 1, 2, 1, hd, vd, ps, "causal", None, sink, 0.5, None, None,
                                step.status)
        assert (float(out.abs().max()) < 1e-4) == small


# ---------------------------------------------------------------------------------------------------------
# GPU: the whole model through the runner, the cache manager, the replay tool and the scheduler
# ---------------------------------------------------------------------------------------------------------
_FOLDERS = {}


def _case(name):
    if name not in _FOLDERS:
        folder = write_folder(name)
        cfg, w = P.read_model_folder(folder)
        rng = np.random.default_rng(CASES[name]["seed"])
        seqs = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (150, 61, 97, 1, 34, 120)]
        refs = [P.forward(cfg, w, s).numpy() for s in seqs]
        _FOLDERS[name] = (folder, seqs, refs)
    return _FOLDERS[name]


def _runner(folder, dtype, page_size, num_pages, slots=4, graphs=True, max_len=256):
    from lite_lang_b200.cache.manager import CacheManager
    from lite_lang_b200.config.base import load_config
    from lite_lang_b200.engine.model import CausalLM
    from lite_lang_b200.engine.runner import ModelRunner
    from lite_lang_b200.weights.loader import load_weights
    model = CausalLM(load_config(folder).model_spec())
    load_weights(model, folder, dtype, dev())
    n_paged = sum(1 for g in model.cache_groups if g.kind == "paged")
    mgr = CacheManager(model.cache_groups, [num_pages] * n_paged, page_size, slots, max_len)
    return mgr, ModelRunner(model, mgr, dev(), 512, cuda_graphs=graphs)


def _feed(runner, mgr, slot, toks, want=None):
    from lite_lang_b200.engine.batch import StepEntry
    assert runner.reserve(slot, len(toks))
    want = tuple(range(len(toks))) if want is None else want
    return runner.step([StepEntry(slot, toks, want)]).float().cpu().numpy().copy()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_whole_decode_and_portions(name, dtype):
    folder, seqs, refs = _case(name)
    mgr, runner = _runner(folder, dtype, CASES[name]["page_size"], 256 // CASES[name]["page_size"])
    for i in (0, 3, 4):                                     # whole prompts (one of them a single token)
        s = mgr.open()
        assert close(_feed(runner, mgr, s, seqs[i]), refs[i], dtype), f"{name} whole {i}"
        mgr.close(s)
    for i, tail in ((0, 120), (2, 40)):                     # a prompt, then many tokens one by one (captured steps):
        s, n = mgr.open(), len(seqs[i])                     # every window and chunk passes over decoded tokens
        head = n - tail
        got = [_feed(runner, mgr, s, seqs[i][:head])] + [_feed(runner, mgr, s, seqs[i][t:t + 1]) for t in range(head, n)]
        assert close(np.concatenate(got), refs[i], dtype), f"{name} decode {i}"
        mgr.close(s)
    s, n = mgr.open(), len(seqs[1])                         # from the very first token on, one by one
    got = [_feed(runner, mgr, s, seqs[1][t:t + 1]) for t in range(n)]
    assert close(np.concatenate(got), refs[1], dtype), f"{name} token by token"
    mgr.close(s)
    sizes = [7, 2, 13, 2, 5, 31, 2, 3, 17, 2, 64, 2, 9]
    for i in (0, 5):                                        # portions of changing size, down to two tokens
        s, n, t, k, got = mgr.open(), len(seqs[i]), 0, 0, []
        while t < n:
            c = min(sizes[k % len(sizes)], n - t)
            got.append(_feed(runner, mgr, s, seqs[i][t:t + c]))
            t, k = t + c, k + 1
        assert close(np.concatenate(got), refs[i], dtype), f"{name} portions {i}"
        mgr.close(s)
    runner.check_status()
    assert runner.graph_replays > 0


@gpu
@pytest.mark.parametrize("name", ["P", "Q"])
def test_a_pool_smaller_than_the_prompt_serves_it_through_the_pages_given_back(name):
    """Every layer of these cases has a window or chunks, so a request holds a bounded number of pages however
    long it grows: a prompt of several times the pool, fed in portions, and the logits are the whole prompt's."""
    folder, seqs, refs = _case(name)
    ps = CASES[name]["page_size"]
    cfg, w = P.read_model_folder(folder)
    toks = [int(t) for t in np.random.default_rng(21).integers(0, cfg["vocab"], 400)]
    ref = P.forward(cfg, w, toks).numpy()
    biggest = max(int(l["mixer"]["mask"]["size"]) for l in cfg["layers"])
    portion = 24
    pages = (biggest + portion + ps - 1) // ps + 3
    assert pages * ps < len(toks) // 2
    mgr, runner = _runner(folder, torch.float32, ps, pages, slots=2, max_len=512)
    s, got = mgr.open(), []
    for t in range(0, 360, portion):
        got.append(_feed(runner, mgr, s, toks[t:t + portion]))
    got += [_feed(runner, mgr, s, toks[t:t + 1]) for t in range(360, 400)]
    assert close(np.concatenate(got), ref, torch.float32)
    mgr.close(s)
    mgr.check_invariants()
    runner.check_status()
    assert mgr.pages_reused > 0


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype, monkeypatch):
    from lite_lang_b200.engine.batch import StepEntry
    monkeypatch.setenv("LITE_LANG_B200_CACHE_FILL", "nan")
    folder, seqs, refs = _case(name)
    ps = CASES[name]["page_size"]
    order = [0, 1, 2, 3, 4, 5, 1, 2, 0]
    need = sorted(((len(seqs[i]) + ps - 1) // ps for i in order), reverse=True)[:3]
    mgr, runner = _runner(folder, dtype, ps, sum(need) + 1, slots=3)
    rng = np.random.default_rng(3)
    waiting, live, all_got, all_ref = list(enumerate(order)), {}, [], []
    while waiting or live:
        while waiting and len(live) < 3:
            k, i = waiting.pop(0)
            live[k] = [i, 0, mgr.open()]
        entries, expect, done = [], [], []
        for k, (i, t, slot) in list(live.items()):
            n = len(seqs[i])
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step, goes on later
            c = min(int(rng.integers(2, 23)) if n - t > 20 else 1, n - t)
            assert runner.reserve(slot, c)
            want = tuple(range(c)) if rng.random() < 0.7 else (c - 1,)
            entries.append(StepEntry(slot, seqs[i][t:t + c], want))
            expect.append(refs[i][[t + w for w in want]])
            live[k][1] = t + c
            if t + c == n:
                done.append(k)
        if not entries:
            continue
        got = runner.step(entries).float().cpu().numpy()
        all_got.append(got.copy())
        all_ref.append(np.concatenate(expect))
        for k in done:
            mgr.close(live.pop(k)[2])
        mgr.check_invariants()
    runner.check_status()
    assert close(np.concatenate(all_got), np.concatenate(all_ref), dtype), name
    assert mgr.pages_reused > 0


@gpu
def test_a_batch_gives_each_request_what_it_gets_alone():
    """In the attention the order of every sum depends on the token's position only; what is left between a
    request alone and the same request beside others, in other pages and slots and cut otherwise, is the
    rounding of the matrix products, whose shapes differ (float32, where nothing else rounds)."""
    from lite_lang_b200.engine.batch import StepEntry
    folder, seqs, refs = _case("P")
    ps = CASES["P"]["page_size"]
    mgr, runner = _runner(folder, torch.float32, ps, 200, graphs=False)
    s = mgr.open()
    alone = _feed(runner, mgr, s, seqs[2])
    mgr.close(s)
    a, b, c = mgr.open(), mgr.open(), mgr.open()
    for slot, toks in ((a, seqs[1][:33]), (c, seqs[4][:9])):
        _feed(runner, mgr, slot, toks)
    got, t = [], 0
    for n in (5, 40, 2, 50):
        entries = [StepEntry(a, seqs[1][33 + len(got):34 + len(got)], (0,)), StepEntry(b, seqs[2][t:t + n], tuple(range(n)))]
        for e in entries:
            assert runner.reserve(e.slot, len(e.tokens))
        got.append(runner.step(entries).float().cpu().numpy()[1:].copy())
        t += n
    got = np.concatenate(got)
    assert float(np.abs(got - alone).max()) <= 2e-5 * float(np.abs(alone).max())


@gpu
def test_replay_tool_and_a_prompt_of_many_tokens_in_one_step():
    """The command-line replay on a folder: a prompt long enough for the prompt attention kernels, cut into three
    steps beside a short request that ends early."""
    folder = write_folder("Q")
    cfg, w = P.read_model_folder(folder)
    toks = [int(t) for t in np.random.default_rng(9).integers(0, cfg["vocab"], 260)]
    ref = P.forward(cfg, w, toks).numpy()
    for dtype in ("float32", "bfloat16"):
        tr = TraceRun(folder, dtype, max_tokens=384, page_size=16)
        try:
            a = tr.step([{"id": "a", "tokens": toks[:200], "want": list(range(0, 200, 7))}])
            b = tr.step([{"id": "a", "tokens": toks[200:259], "want": list(range(59))},
                         {"id": "b", "tokens": toks[:5], "want": [4]}], end=["b"])
            c = tr.step([{"id": "a", "tokens": toks[259:], "want": [0]}], end=["a"])
        finally:
            assert tr.close() == 0
        want = np.concatenate([ref[0:200:7], ref[200:259], ref[259:], ref[4:5]])
        assert close(np.concatenate([a, b[:59], c, b[59:]]), want, dtype)


def _greedy_matches(cfg, w, prompt, out):
    seq = list(prompt)
    for tok in out:
        logits = P.forward(cfg, w, seq)[-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) < 1e-3:              # a near-tie: either token is right, stop comparing
            return
        assert int(torch.argmax(logits)) == tok, (len(prompt), len(seq))
        seq.append(tok)


@gpu
def test_greedy_generation_through_the_scheduler():
    """Engine.generate with more prompts than request slots: the tokens are the plain implementation's greedy
    continuation (float32, so that no near-tie decides)."""
    from lite_lang_b200 import Engine, EngineConfig, SamplingParams
    folder = write_folder("R")
    cfg, w = P.read_model_folder(folder)
    rng = np.random.default_rng(4)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (9, 30, 1, 17, 44)]
    new = 12
    engine = Engine(folder, EngineConfig(dtype="float32", page_size=8, num_pages=40, max_batch_size=3,
                                         max_input_length=64, max_output_length=new, max_tokens_per_step=48))
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=new, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert len(o) == new
        _greedy_matches(cfg, w, p, o)
    assert engine.stats()["graph_replays"] > 0


@gpu
def test_command_line_picks_the_model_by_its_configuration():
    folder = write_folder("P")
    cfg, w = P.read_model_folder(folder)
    prompt = [int(t) for t in np.random.default_rng(8).integers(0, cfg["vocab"], 11)]
    ids = os.path.join(folder, "prompt.json")
    with open(ids, "w") as fh:
        json.dump([prompt], fh)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "lite_lang_b200.cli", "--model_path", folder, "--prompt_ids", ids, "--dtype", "fp32",
           "--max_output_length", "6", "--page_size", "4", "--num_pages", "32", "--max_batch_size", "2",
           "--temperature", "0", "--ignore_eos"]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=root, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = json.loads(res.stdout.strip().splitlines()[-1])["outputs"][0]
    assert len(out) == 6
    _greedy_matches(cfg, w, prompt, out)
