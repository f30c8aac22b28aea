"""Rufisun through the engine against the plain implementation (tests/plain/rufisun_plain.py).

CPU: configuration, registry, cache groups (a window gives pages back, the pages of kept first tokens stay), the
distance buckets and scaled rotary frequencies, the plain implementation's own properties.  GPU: each mechanism's
kernels alone (with inputs made so that a fault at an edge shows), whole prompts, token-by-token decoding through
captured steps, portions down to two tokens, mixed batches with pages and slots used again, the command-line
replay tool and greedy generation through the scheduler.
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
from plain import rufisun_plain as P
from rufisun_cases import CASES, write_folder

TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
gpu = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def row_errors(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    return np.abs(got - ref).max(axis=-1) / np.abs(ref).max(axis=-1)


# a router's margin (the last chosen expert's score less the first one's that is not chosen) below which
# bfloat16 rounding may choose the other expert
UNDECIDED = 0.002


def decided_rows(margins) -> int:
    """How many leading tokens of a sequence have every router's choice safely decided."""
    if not margins:
        return 1 << 30
    low = (torch.stack(margins).min(0).values < UNDECIDED).nonzero()
    return int(low[0]) if low.numel() else 1 << 30


def close(got, ref, dtype, strict=None) -> bool:
    """float32: every row within the tolerance.  bfloat16: random weights give a router a near-tie every few
    dozen tokens (``decided_rows`` finds them in the plain implementation's routers), which bfloat16 rounding may
    decide the other way; that moves the token's row, and through the peaked attention and the recurrent state
    some of the rows after it, by far more than rounding does.  So in bfloat16 the rows must be finite, three in
    four of them within the tolerance and the median row well inside it; a wrong key, mask or state would move
    nearly all rows.  ``strict`` (a mask) names the rows before a sequence's first near-tie: of those, nine in
    ten must be within the tolerance.  The float32 runs, on the same kernels and cache, excuse no row."""
    e = row_errors(got, ref)
    if dtype in (torch.float32, "float32"):
        return bool(e.max() <= TOL[torch.float32])
    if not np.isfinite(np.asarray(got)).all():
        return False
    strict = np.ones(len(e), dtype=bool) if strict is None else np.asarray(strict, dtype=bool)
    tol = TOL[torch.bfloat16]
    return bool(int((e[strict] > tol).sum()) <= 0.1 * max(1, int(strict.sum())) and int((e > tol).sum()) <= 0.25 * len(e)
                and float(np.median(e)) <= 0.5 * tol)


def kernel_tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.6e-2


# ---------------------------------------------------------------------------------------------------------
# CPU
# ---------------------------------------------------------------------------------------------------------

def test_config_registry_and_round_trip():
    from lite_lang_b200.config import ConfigError, config_from_dict, known_architectures
    assert "Rufisun" in known_architectures()
    cfg = config_from_dict(CASES["P"]["config"])
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert [l.block for l in spec.layers] == ["pre_norm", "pre_norm", "pre_norm_mixer_only", "pre_norm"]
    assert [l.parts["mixer"].kind for l in spec.layers] == ["modulated_attention", "latent_attention", "side_by_side",
                                                             "modulated_attention"]
    a = spec.layers[0].parts["mixer"].params
    assert a["mask"] == "window" and a["mask_size"] == 23 and a["keep_first"] == 5 and a["sink"] == "learned"
    assert a["channel_gate"] and a["distance_bias"]["max"] == 50 and a["value_head_dim"] == 40 and a["scale"] == 0.9
    lat = spec.layers[1].parts["mixer"].params
    assert lat["q_rank"] == 19 and lat["kv_rank"] == 37 and lat["window"] is None and lat["sink"]
    assert lat["rot_dims"] == 4 and lat["rot_scaling"]["factor"] == 4.0
    par = spec.layers[2].parts["mixer"].params
    assert par["join"] == "sum" and par["left_scale"] == 0.7 and par["right_scale"] == 1.3
    assert par["left"]["params"]["softcap"] == 5.0 and par["left"]["params"]["query_temperature"] == {"coef": 0.4, "every": 7}
    assert par["right"]["params"]["groups"] == 3 and par["right"]["params"]["conv_taps"] == 3
    moe = spec.layers[1].parts["feed_forward"].params
    assert (moe["experts"], moe["top"], moe["expert_ff"], moe["shared_ff"]) == (5, 2, 20, 12)
    assert moe["weight_on"] == "input" and moe["score"] == "sigmoid" and moe["activation"] == "gelu"
    assert spec.layers[3].parts["feed_forward"].params["shared_ff"] == 0
    assert spec.layers[0].parts["feed_forward"].params["activation"] == "relu2"
    assert spec.head.params["tied_to"] == "embed"
    # no mask section: plain causal attention, nothing kept; no q_temp and no cap: neither mechanism
    r = config_from_dict(CASES["R"]["config"]).model_spec()
    assert r.layers[2].parts["mixer"].params["mask"] == "causal" and r.layers[2].parts["mixer"].params["keep_first"] == 0
    left = r.layers[1].parts["mixer"].params["left"]["params"]
    assert left["softcap"] is None and left["query_temperature"] is None
    for path, value in ((("layers", 0, "type"), "attention_9"), (("layers", 0, "mixer", "kv_heads"), 4),
                        (("layers", 1, "mixer", "rot", "dims"), 7), (("layers", 0, "mlp", "kind"), "gated"),
                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 2, "mixer", "right", "groups"), 0),
                        (("layers", 2, "mixer", "left", "q_temp", "every"), 0)):
        bad = cfg.to_dict()
        d = bad
        for key in path[:-1]:
            d = d[key]
        d[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(bad)
    for key, sub in (("norm", None), ("bias_max", 0), ("left_scale", 2), ("q_rank", 1)):
        bad = cfg.to_dict()
        del (bad if sub is None else bad["layers"][sub]["mixer"])[key]
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_cache_groups_and_declared_tensors():
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.engine.model import CausalLM
    model = CausalLM(config_from_dict(CASES["P"]["config"]).model_spec())
    paged = sorted((g.num_kv_heads, g.head_dim, g.value_dim, g.window, g.keep_first, g.planes)
                   for g in model.cache_groups if g.kind == "paged")
    assert paged == [(1, 20, 28, None, 0, 1), (1, 36, 20, 9, 0, 1), (1, 43, 0, None, 0, 1), (2, 24, 40, 23, 5, 1)]
    state = [g for g in model.cache_groups if g.kind == "state"]
    # the state-space layer's record: heads x vdim x state numbers and the convolution's last two inputs
    assert len(state) == 1 and state[0].shape == (6 * 12 * 20 + 2 * (72 + 2 * 3 * 20),) and state[0].dtype == "float32"
    names = model.declared_tensors()
    for n, shape in (("embed", (211, 88)), ("final.norm", (88,)), ("final.norm.b", (88,)), ("final.norm.alpha", ()),
                     ("l0.norm1.alpha", ()), ("l0.mix.q", (144, 88)), ("l0.mix.k", (48, 88)), ("l0.mix.v", (80, 88)),
                     ("l0.mix.g", (240, 88)), ("l0.mix.o", (88, 240)), ("l0.mix.sink", (6,)), ("l0.mix.rel", (None, 6)),
                     ("l0.mlp.up", (50, 88)), ("l1.mix.dq", (19, 88)), ("l1.mix.dq.norm", (19,)),
                     ("l1.mix.uq", (78, 19)), ("l1.mix.dkv", (43, 88)), ("l1.mix.dkv.norm", (37,)),
                     ("l1.mix.uk", (60, 37)), ("l1.mix.uv", (36, 37)), ("l1.mix.sink", (3,)), ("l1.mix.o", (88, 36)),
                     ("l1.mlp.router", (5, 88)), ("l1.mlp.e4.up", (20, 88)), ("l1.mlp.shared.down", (88, 12)),
                     ("l2.mix.left.q", (80, 88)), ("l2.mix.left.k", (20, 88)), ("l2.mix.left.v", (28, 88)),
                     ("l2.mix.left.sink", (4,)), ("l2.mix.left.o", (88, 112)), ("l2.mix.right.in", (2 * 72 + 120 + 6, 88)),
                     ("l2.mix.right.conv", (192, 3)), ("l2.mix.right.conv.b", (192,)), ("l2.mix.right.dt_bias", (6,)),
                     ("l2.mix.right.A_log", (6,)), ("l2.mix.right.D", (6,)), ("l2.mix.right.norm", (72,)),
                     ("l2.mix.right.o", (88, 72)), ("l3.mlp.e2.down", (88, 44))):
        assert tuple(names[n].shape) == shape, n
    assert names["head"].optional                                     # the head is the embedding table
    for n in ("l2.norm2", "l2.mlp.up", "l3.mlp.shared.up", "l1.mix.q", "l2.mix.left.g", "l2.mix.left.rel",
              "l2.mix.left.out", "l2.mix.right.out", "l1.mix.rel", "l3.mix.q.b"):
        assert n not in names, n
    # a window longer than anything still releases by the rule; no mask: the group keeps every page
    r = CausalLM(config_from_dict(CASES["R"]["config"]).model_spec())
    assert sorted(g.releases for g in r.cache_groups if g.kind == "paged") == [False, False, False, False, True]


def test_pages_go_back_behind_a_window_but_the_first_tokens_pages_stay():
    from lite_lang_b200.cache.manager import CacheManager, PagedGroupSpec
    ps = 4
    groups = [PagedGroupSpec(1, 8, 6, 1, 8, None, 5), PagedGroupSpec(1, 8, 6, 1, 8, None, 0),
              PagedGroupSpec(1, 8, 6, 1, 8, None, 8)]
    assert [g.kept_pages(ps) for g in groups] == [2, 0, 2]
    mgr = CacheManager(groups, [6, 4, 6], ps, 2, 64)
    s = mgr.open()
    for n in range(1, 41):
        assert mgr.reserve(s, n), n
        mgr.advance(s, n)
        mgr.check_invariants()
        for g in (0, 1, 2):
            held = [lp for lp, p in enumerate(mgr.pages_of(g, s)) if p >= 0]
            first = groups[g].first_needed(n) // ps
            kept = groups[g].kept_pages(ps)
            # every page of a kept position is held (once it was asked for); between them and the window's
            # first page nothing is; the window's first page is (unless it is the one not yet asked for)
            assert all(lp in held for lp in range(min(kept, (n + ps - 1) // ps))), (n, g)
            assert all(lp >= first or lp < kept for lp in held), (n, g)
            assert first in held or first * ps >= n, (n, g)
    assert [p >= 0 for p in mgr.pages_of(0, s)] == [True, True] + [False] * 6 + [True, True]
    assert [p >= 0 for p in mgr.pages_of(1, s)] == [False] * 8 + [True, True]
    assert groups[0].pages_a_request_needs(1000, ps, 8) == (6 + 8 + 3) // 4 + 1 + 2
    # a pool of the bound serves a request of any length; pages are used again, the kept ones never
    first_two = mgr.pages_of(0, s)[:2]
    for n in range(41, 64):
        assert mgr.reserve(s, n), n
        mgr.advance(s, n)
    assert mgr.pages_of(0, s)[:2] == first_two and mgr.pages_reused > 0
    mgr.close(s)
    mgr.check_invariants()
    assert all(mgr.num_free_pages(g) == n for g, n in ((0, 6), (1, 4), (2, 6)))


def test_distance_buckets_and_frequencies_of_the_parts_are_the_plain_ones():
    from lite_lang_b200.config.spec import PartSpec
    from lite_lang_b200.parts import build_part
    from lite_lang_b200.parts.modulated_attention import distance_bucket
    for B, D in ((32, 100), (12, 50), (7, 30), (2, 1000), (9, 64), (16, 40.5)):
        assert [distance_bucket(n, B, D) for n in range(300)] == [P.distance_bucket(n, B, D) for n in range(300)]
    # the closed form: exact below B // 2, then logarithmic steps (17 is still in bucket 16, since
    # 16 ln(17/16) / ln(6.25) < 1; 64 = 16 x 4 lies 16 ln 4 / ln 6.25 = 12.1 steps on), capped at the last row,
    # which D has reached; never decreasing
    b = [P.distance_bucket(n, 32, 100) for n in range(200)]
    assert b[:16] == list(range(16)) and b[16] == 16 and b[17] == 16 and b[64] == 28 and b[100] == 31 and b[199] == 31
    assert all(x <= y for x, y in zip(b, b[1:])) and set(b) == set(range(32))
    for dims, base, sc in ((4, 10000.0, (4.0, 64, 32.0, 1.0)), (16, 30000.0, None), (4, 77.0, (2.0, 16, 2.0, 1.0))):
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        part = build_part("position", PartSpec("rope_computed", {"rotary_dim": dims, "theta": base,
                                                                "layout": "interleaved", "scaling": rot.get("scaling")}))
        f, amp = P.scaled_frequencies(rot)
        assert torch.allclose(part.frequencies(), f, rtol=1e-14, atol=0) and abs(part.amplitude - amp) < 1e-15


def test_plain_pieces_against_closed_forms():
    g = torch.Generator().manual_seed(0)
    # a sink of minus infinity is the ordinary softmax; a huge one takes all the weight
    s = torch.randn(5, 5, generator=g, dtype=P.F)
    vis = P.visible_window_keep(5, None, 0)
    w = P.softmax_with_sink(s, vis, torch.tensor(-1e30, dtype=P.F))
    assert torch.allclose(w.sum(-1), torch.ones(5, dtype=P.F)) and float(w[0, 0]) == 1.0 and float(w[1, 2]) == 0.0
    assert float(P.softmax_with_sink(s, vis, torch.tensor(50.0, dtype=P.F)).sum(-1).max()) < 1e-15
    w = P.softmax_with_sink(s, vis, torch.tensor(0.3, dtype=P.F))
    assert abs(float(w[2].sum()) - float(torch.exp(s[2, :3]).sum() / (math.exp(0.3) + torch.exp(s[2, :3]).sum()))) < 1e-15
    # window with kept first tokens
    v = P.visible_window_keep(12, 4, 2)
    assert v[10].tolist() == [True, True] + [False] * 5 + [True] * 4 + [False]
    assert v[3].tolist() == [True] * 4 + [False] * 8 and P.visible_window_keep(6, None, 0)[5].all()
    # the convolution: the last tap weighs the token itself; zeros before the start
    x = torch.randn(6, 3, generator=g, dtype=P.F)
    cw = torch.randn(3, 4, generator=g, dtype=P.F)
    cb = torch.randn(3, generator=g, dtype=P.F)
    y = P.causal_convolution(x, cw, cb)
    assert torch.allclose(y[0], cb + cw[:, 3] * x[0])
    assert torch.allclose(y[4], cb + cw[:, 0] * x[1] + cw[:, 1] * x[2] + cw[:, 2] * x[3] + cw[:, 3] * x[4])
    # the scan as a sum: y_t = sum_s<=t (prod_(s<r<=t) a_r) dt_s (C_t . B_s) x_s + D x_t  (one head, one group)
    m = {"heads": 1, "vdim": 3, "state": 4, "groups": 1, "conv": 1, "norm_groups": 1}
    width = 5
    wts = {"in": torch.randn(2 * 3 + 8 + 1, width, generator=g, dtype=P.F), "conv": torch.ones(11, 1, dtype=P.F),
           "conv.b": torch.zeros(11, dtype=P.F), "dt_bias": torch.tensor([0.2], dtype=P.F),
           "A_log": torch.tensor([-0.5], dtype=P.F), "D": torch.tensor([0.7], dtype=P.F),
           "norm": torch.ones(3, dtype=P.F), "o": torch.eye(3, dtype=P.F)[:, :3].repeat(2, 1)[:width]}
    u = torch.randn(7, width, generator=g, dtype=P.F)
    got = P.state_space(u, m, wts, "", 1e-6)
    proj = u @ wts["in"].T
    z, xx, Bm, Cm, dt = proj[:, :3], P.silu(proj[:, 3:6]), P.silu(proj[:, 6:10]), P.silu(proj[:, 10:14]), proj[:, 14]
    dt = torch.log1p(torch.exp(dt + 0.2))
    a = torch.exp(-math.exp(-0.5) * dt)
    y = torch.zeros(7, 3, dtype=P.F)
    for t in range(7):
        for s_ in range(t + 1):
            y[t] += a[s_ + 1:t + 1].prod() * dt[s_] * (Cm[t] @ Bm[s_]) * xx[s_]
        y[t] += 0.7 * xx[t]
    y = P.unit_rms(y * P.silu(z), 1e-6)
    assert torch.allclose(got, y @ wts["o"].T, atol=1e-12)
    # routed experts: with every expert chosen and scores s the output is sum_e D_e gelu(s_e U_e u)
    assert abs(float(P.gelu_erf(torch.tensor(1.0, dtype=P.F))) - 0.8413447460685429) < 1e-12
    assert float(P.softplus(torch.tensor(100.0, dtype=P.F))) == 100.0


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
    s.cu_q = torch.tensor(np.concatenate([[0], np.cumsum(entries)]), dtype=torch.int32, device=dev())
    s.ctx_len = torch.tensor(ctx, dtype=torch.int32, device=dev())
    s.num_entries = len(entries)
    s.status = torch.zeros(1, dtype=torch.int32, device=dev())
    return s


def _paged(dtype, seqs_k, seqs_v, ps, nkv, hd, vd, rng, live):
    """Keys/values of several requests scattered over a pool whose other slots hold NaN.  ``live(r, page)`` says
    whether a logical page of request r is there; the others are -1 in the table, as when a window has given
    them back."""
    n_pages = sum((len(k) + ps - 1) // ps for k in seqs_k) + 3
    order = rng.permutation(n_pages)
    kc = torch.full((n_pages, nkv, ps, hd), float("nan"), dtype=dtype)
    vc = torch.full((n_pages, nkv, ps, vd), float("nan"), dtype=dtype)
    max_blocks = max((len(k) + ps - 1) // ps for k in seqs_k)
    bt = torch.full((len(seqs_k), max_blocks), -1, dtype=torch.int32)
    at = 0
    for r, (k, v) in enumerate(zip(seqs_k, seqs_v)):
        for j in range(len(k)):
            if not live(r, j // ps):
                continue
            if bt[r, j // ps] < 0:
                bt[r, j // ps] = int(order[at])
                at += 1
            kc[bt[r, j // ps], :, j % ps] = k[j].to(dtype)
            vc[bt[r, j // ps], :, j % ps] = v[j].to(dtype)
    return kc.to(dev()), vc.to(dev()), bt.to(dev())


def _attention_case(dtype, nh, nkv, hd, vd, ps, size, keep, buckets, far, cap, q_temp, gate, lens, new, seed=0,
                    kernel="blocks", out_scale=1.0):
    """Prompt portions and single tokens of several requests in one launch; pages that neither the window nor the
    kept first tokens need are not there.  The last queries of every request are aimed (a large dot product with
    one key) at the keys on both sides of the window's edge, at the last kept token and the first one not kept,
    and at a key far back (which only a request without a window, or a kept token, may read).  ``kernel``:
    "blocks" (a block a token, any sizes) or "shaped" (tensor cores; single tokens first, as the batch builder
    orders a step, their keys cut into parts)."""
    from lite_lang_b200 import ops
    from lite_lang_b200.parts.modulated_attention import distance_bucket
    if kernel == "shaped":
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
        targets = []
        p_last = lens[r] - 1
        if size is not None:
            targets += [("window_out", lambda p: p - size), ("window_in", lambda p: p - size + 1)]
            if keep:
                targets += [("first_in", lambda p: keep - 1), ("first_out", lambda p: keep)]
        else:
            targets += [("far", lambda p: 1)]
        for back, (which, where) in enumerate(targets):
            row = new[r] - 1 - back
            if row < 0:
                continue
            p = p_last - back
            j = where(p)
            if j < 0 or j > p:
                continue
            for h in range(nh):
                qs[r][row, h] = 6.0 * ks[r][j, h // group]
            visible = size is None or p - j < size or j < keep
            aimed.append((r, row, j, which, visible))
    ks, vs, qs = ([t.to(dtype).float() for t in ts] for ts in (ks, vs, qs))

    def live(r, page):
        first = lens[r] - new[r]                         # the first query's position
        lo = 0 if size is None else max(0, first - size + 1)
        return page >= lo // ps or page * ps < keep

    kc, vc, bt = _paged(dtype, ks, vs, ps, nkv, hd, vd, rng, live)
    step = _step(new, [n - c for n, c in zip(lens, new)], list(range(R)))
    n_tok = sum(new)
    gate_in = (torch.randn(n_tok, nh * vd, generator=g) * 2).to(dtype).float() if gate else None
    width = nh * hd + 3 + (nh * vd if gate else 0)
    proj = torch.zeros(n_tok, (width + 7) // 8 * 8, dtype=dtype)                  # q, three other columns, the gate
    proj[:, :nh * hd] = torch.cat([x.reshape(x.shape[0], -1) for x in qs]).to(dtype)
    if gate:
        proj[:, nh * hd + 3:nh * hd + 3 + nh * vd] = gate_in.to(dtype)
    proj = proj.to(dev())
    sink = torch.randn(nh, generator=g) + 2.0
    table = torch.randn(buckets, nh, generator=g) if buckets else None
    by_distance = None
    if table is not None:
        by_distance = table[[distance_bucket(n, buckets, far) for n in range(int(math.ceil(far)) + 1)]].to(dev())
    out = torch.full((n_tok, nh * vd), float("nan"), dtype=dtype, device=dev())
    scale = 0.9 / math.sqrt(hd)
    gate_view = proj[:, nh * hd + 3:nh * hd + 3 + nh * vd] if gate else None
    mask = "causal" if size is None else "window"
    if kernel == "blocks":
        ops.attention_modulated(out, proj, proj.stride(0), gate_view, kc, vc, bt, step.token_req, step.req_slot,
                                step.positions, n_tok, nh, nkv, hd, vd, ps, mask, size, True, scale, None, None,
                                step.status, sink_values=sink.to(dev()), distance_bias=by_distance,
                                keep_first=keep or 0, softcap=cap, query_temperature=q_temp, gate_channels=gate,
                                out_scale=out_scale)
    else:
        n_single = sum(1 for c in new if c == 1)
        more = dict(sink_values=sink.to(dev()), distance_bias=by_distance, keep_first=keep or 0, softcap=cap,
                    query_temperature=q_temp, gate_channels=gate, out_scale=out_scale)
        tail = (nh, nkv, hd, vd, ps, mask, size, True, scale, step.status)
        head = (out, proj, proj.stride(0), False, gate_view, None, kc, vc, bt)
        if n_single:
            stages = (max(lens) + 63) // 64 + 1 if mask == "causal" else (size + 62) // 64 + 1
            for want_parts in ((32, 2) if seed == 0 else (32,)):       # many parts of few stages, and few of many
                span = (stages + want_parts - 1) // want_parts
                ops.attn_shaped(*head, step.cu_q, step.ctx_len, step.req_slot, n_single,
                                n_single * ((group + 127) // 128), *tail, nsplit=(stages + span - 1) // span, span=span,
                                **more)
        if R > n_single:
            ops.attn_shaped(*head, step.cu_q[n_single:], step.ctx_len[n_single:], step.req_slot[n_single:], R - n_single,
                            ops.attn_shaped_blocks(new[n_single:], group), *tail, **more)
    assert int(step.status.item()) == 0
    want, at = [], 0
    for r in range(R):
        T, c = lens[r], new[r]
        qfull = torch.cat([torch.zeros(T - c, nh, hd, dtype=P.F), qs[r].double()])
        if q_temp:
            pos = torch.arange(T, dtype=P.F)
            qfull = qfull * (1.0 + q_temp[0] * torch.log(torch.floor((pos + 1.0) / q_temp[1]) + 1.0))[:, None, None]
        o = P.sink_attention(qfull, ks[r].double(), vs[r].double(), scale, P.visible_window_keep(T, size, keep or 0),
                             sink.double(), bias=None if table is None else P.distance_bias(table.double(), T, far),
                             cap=cap)
        o = o[-c:].reshape(c, nh * vd) * out_scale
        if gate:
            o = o * P.sigmoid(gate_in[at:at + c].double())
        want.append(o)
        at += c
    want = torch.cat(want)
    assert not bool(torch.isnan(out).any())
    got = out.float().cpu()
    assert rel_err(got.numpy(), want.numpy()) <= kernel_tol(dtype), (size, keep)
    return got, want, aimed, vs, new


ATTN_SHAPES = [  # nh, nkv, hd, vd, page size
    (6, 2, 24, 40, 4), (9, 1, 20, 28, 8), (1, 1, 36, 20, 4), (8, 2, 64, 64, 16), (4, 4, 128, 128, 16),
    (2, 1, 128, 128, 64), (5, 5, 12, 20, 8), (4, 2, 96, 80, 16)]


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,ps", ATTN_SHAPES)
def test_window_with_kept_tokens_distance_bias_sink_and_channel_gate(dtype, nh, nkv, hd, vd, ps):
    lens, new = [150, 61, 97, 300, 34], [40, 1, 97, 1, 5]
    for size, keep, buckets, far in ((23, 5, 12, 50), (44, 16, 16, 40), (9, 0, 7, 30), (120, 24, 32, 200),
                                     (1000, 7, 2, 1000), (None, None, 9, 64)):
        _attention_case(dtype, nh, nkv, hd, vd, ps, size, keep, buckets, far, None, None, True, lens, new)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,ps", ATTN_SHAPES)
def test_query_temperature_cap_and_sink(dtype, nh, nkv, hd, vd, ps):
    lens, new = [150, 61, 97, 300, 34], [40, 1, 97, 1, 5]
    for cap, q_temp, out_scale in ((5.0, (0.4, 7), 0.7), (30.0, (0.25, 16), 1.0), (None, None, 1.3), (2.0, (1.0, 1), 2.0),
                                   (15.0, (0.35, 48), 1.1)):
        _attention_case(dtype, nh, nkv, hd, vd, ps, None, None, None, None, cap, q_temp, False, lens, new,
                        out_scale=out_scale)


SHAPED_SHAPES = [(8, 2, 64, 64, 16), (4, 4, 128, 128, 16), (2, 1, 128, 128, 64), (16, 8, 64, 128, 32), (7, 1, 128, 64, 16)]


@gpu
@pytest.mark.parametrize("nh,nkv,hd,vd,ps", SHAPED_SHAPES)
def test_the_same_shapes_of_the_scores_on_tensor_cores(nh, nkv, hd, vd, ps):
    lens, new = [150, 61, 97, 300, 34, 700], [40, 1, 97, 1, 5, 1]
    dt = torch.bfloat16
    for size, keep, buckets, far in ((23, 5, 12, 50), (44, 16, 16, 40), (120, 24, 32, 200), (100, 70, 32, 300),
                                     (1000, 7, 2, 1000), (None, None, 9, 64), (64, 64, 8, 64), (200, 130, 8, 64)):
        _attention_case(dt, nh, nkv, hd, vd, ps, size, keep, buckets, far, None, None, True, lens, new, kernel="shaped")
    for cap, q_temp, out_scale in ((5.0, (0.4, 7), 0.7), (30.0, (0.25, 16), 1.0), (None, None, 1.3), (2.0, (1.0, 1), 2.0)):
        _attention_case(dt, nh, nkv, hd, vd, ps, None, None, None, None, cap, q_temp, False, lens, new, kernel="shaped",
                        out_scale=out_scale)
    # aimed queries on this kernel too: inside and outside every edge, and far back
    seen = set()
    for size, keep in ((24, 5), (100, 70), (None, None)):
        got, want, aimed, vs, new_ = _attention_case(dt, nh, nkv, hd, vd, ps, size, keep, None, None, None, None, False,
                                                     [400, 131], [40, 1], seed=1, kernel="shaped")
        offs = np.concatenate([[0], np.cumsum(new_)])
        for r, row, j, which, visible in aimed:
            o = got[offs[r] + row].view(nh, vd)[0]
            hit = float((o - vs[r][j, 0]).abs().max()) < 0.15 * float(vs[r][j, 0].abs().max())
            assert hit == visible, (size, keep, r, row, j, which)
            seen.add(which)
    assert seen == {"window_in", "window_out", "first_in", "first_out", "far"}


@gpu
def test_an_aimed_query_reads_its_key_inside_an_edge_and_not_the_one_outside():
    """The plain formulas agree with the kernel above; here the statement itself: a query aimed at the first key of
    its window, at the last kept token or at a key hundreds of positions back (without a window) returns that
    key's value; one aimed at the key just outside the window, or at the first token that is not kept, does not;
    and a query that no key answers, before a high sink, returns almost nothing."""
    nh, nkv, hd, vd, ps = 2, 1, 32, 16, 8
    seen = set()
    for size, keep in ((24, 5), (64, 16), (24, 0), (None, None)):
        got, want, aimed, vs, new = _attention_case(torch.float32, nh, nkv, hd, vd, ps, size, keep, None, None, None,
                                                    None, False, [400, 131], [40, 1], seed=1)
        offs = np.concatenate([[0], np.cumsum(new)])
        for r, row, j, which, visible in aimed:
            o = got[offs[r] + row].view(nh, vd)[0]
            hit = float((o - vs[r][j, 0]).abs().max()) < 0.1 * float(vs[r][j, 0].abs().max())
            assert hit == visible, (size, keep, r, row, j, which)
            assert visible == (which in ("window_in", "first_in", "far")), which
            seen.add(which)
    assert seen == {"window_in", "window_out", "first_in", "first_out", "far"}
    from lite_lang_b200 import ops
    T = 50
    kc = torch.zeros(8, 1, ps, hd)
    vc = torch.zeros(8, 1, ps, vd)
    kc.view(-1, hd)[:T], vc.view(-1, vd)[:T] = torch.ones(T, hd), torch.randn(T, vd)
    bt = torch.arange(8, dtype=torch.int32).view(1, 8)
    q = -torch.ones(1, 2 * hd)
    step = _step([1], [T - 1], [0])
    out = torch.empty(1, 2 * vd, device=dev())
    for sink, small in ((torch.tensor([9.0, 9.0]), True), (torch.tensor([-30.0, -30.0]), False)):
        ops.attention_modulated(out, q.to(dev()), 2 * hd, None, kc.to(dev()), vc.to(dev()), bt.to(dev()), step.token_req,
                                step.req_slot, step.positions, 1, 2, 1, hd, vd, ps, "causal", None, True, 0.5, None, None,
                                step.status, sink_values=sink.to(dev()))
        assert (float(out.abs().max()) < 1e-4) == small


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,r,ps", [(12, 512, 32, 16), (4, 64, 16, 16), (28, 160, 16, 8), (17, 96, 32, 4), (3, 37, 6, 4),
                                      (1, 32, 0, 16), (16, 256, 64, 64)])
def test_latent_space_attention_with_a_sink_whole_and_in_parts(dtype, H, R, r, ps):
    """Single tokens and a short portion of several requests against cached rows in scattered pages (the others
    NaN), without and with a window, the keys whole or cut into parts that a second kernel merges, with a sink a
    head: against the formula itself.  The sizes with R + r a multiple of 16 and R of 32 run on tensor cores in
    bfloat16; one query is aimed at a key hundreds of positions back."""
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(H * 1000 + R)
    rng = np.random.default_rng(R)
    KD = R + r
    lens, new = [300, 41, 97, 520], [1, 5, 1, 1]
    rows = [(torch.randn(n, KD, generator=g) * 0.5).to(dtype).float() for n in lens]
    qs = [(torch.randn(c, H, KD, generator=g) * 0.3).to(dtype).float() for c in new]
    qs[3][0, :, :] = 40.0 * rows[3][7] / rows[3][7].norm()               # aimed far back: a score of 20 there
    qs = [x.to(dtype).float() for x in qs]
    n_pages = sum((n + ps - 1) // ps for n in lens) + 3
    order = rng.permutation(n_pages)
    pool = torch.full((n_pages, 1, ps, KD), float("nan"), dtype=dtype)
    bt = torch.full((4, max((n + ps - 1) // ps for n in lens)), -1, dtype=torch.int32)
    at = 0
    for i, k in enumerate(rows):
        for j in range(len(k)):
            if bt[i, j // ps] < 0:
                bt[i, j // ps] = int(order[at])
                at += 1
            pool[bt[i, j // ps], 0, j % ps] = k[j].to(dtype)
    step = _step(new, [n - c for n, c in zip(lens, new)], [0, 1, 2, 3])
    q = torch.cat(qs).to(dtype).to(dev()).contiguous()
    sink = torch.randn(H, generator=g) + 1.0
    scale = 1.0 / math.sqrt(KD)
    n_tok = sum(new)
    for window in (None, 64):
        want = []
        for i in range(4):
            T, c = lens[i], new[i]
            K = rows[i].double()
            for a in range(c):
                p = T - c + a
                lo = 0 if window is None else max(0, p - window + 1)
                s = (qs[i][a].double() @ K[lo:p + 1].T) * scale                                   # [H, keys]
                m = torch.maximum(s.max(-1, keepdim=True).values, sink.double()[:, None])
                e = torch.exp(s - m)
                w = e / (torch.exp(sink.double()[:, None] - m) + e.sum(-1, keepdim=True))
                want.append(w @ K[lo:p + 1, :R])
        want = torch.stack(want)
        longest = max(lens) if window is None else window
        tiles = (longest + 31) // 32 + 1
        for nsplit in (1, 4, 16):
            out = torch.full((n_tok, H, R), float("nan"), dtype=dtype, device=dev())
            ops.latent_attention(out, q, pool.to(dev()), bt.to(dev()), step, 0, n_tok, H, R, r, ps, window, scale,
                                 nsplit, (tiles + nsplit - 1) // nsplit, sink=sink.to(dev()))
            assert int(step.status.item()) == 0
            assert rel_err(out.float().cpu().numpy().reshape(n_tok, -1), want.numpy().reshape(n_tok, -1)) <= kernel_tol(dtype), \
                (window, nsplit)
        if window is None:       # the aimed query returns the latent it was aimed at
            hit = out.float().cpu()[-1, 0]
            assert float((hit - rows[3][7, :R]).abs().max()) < 0.1 * float(rows[3][7, :R].abs().max())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Pd,N,G,taps,parts", [(6, 12, 20, 3, 3, 2), (4, 64, 64, 1, 4, 1), (4, 8, 16, 4, 1, 4),
                                                  (1, 24, 12, 1, 2, 1), (6, 40, 56, 2, 4, 3), (8, 64, 128, 2, 4, 1)])
def test_state_space_pieces_in_portions_with_records_used_again(dtype, H, Pd, N, G, taps, parts):
    """Convolution with the record's tail, step sizes and decays, the scan and the gated norm, for three requests
    fed in portions of unequal sizes (down to one token, shorter than the taps) through records that held
    another request's state before, against the plain formulas on the whole sequences."""
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + N)
    inner, C = H * Pd, H * Pd + 2 * G * N
    lens = [37, 9, 64]
    conv_w = (torch.randn(C, taps, generator=g) * 0.4)
    conv_b = torch.randn(C, generator=g) * 0.1
    dt_bias, A_log, D = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g) * 0.5 - 1.0, torch.randn(H, generator=g)
    norm_w = 1 + 0.1 * torch.randn(inner, generator=g)
    off_x, off_dt = (inner + 7) // 8 * 8, (inner + 7) // 8 * 8 + (C + 7) // 8 * 8
    width = off_dt + (H + 7) // 8 * 8
    rows = [torch.randn(n, width, generator=g).to(dtype).float() for n in lens]
    state_floats = H * Pd * N
    state = torch.full((4, state_floats + (taps - 1) * C), 7.0, device=dev())         # what another request left
    eps = 1e-5
    got = [[] for _ in lens]
    cuts = [[5, 1, 2, 20, 9], [1, 1, 7], [64]]
    slots = [2, 0, 3]
    for r in range(3):
        state[slots[r]].zero_()                                                       # a slot is zeroed when opened
    at = [0, 0, 0]
    for k in range(5):
        who = [r for r in range(3) if k < len(cuts[r])]
        n_new = [cuts[r][k] for r in who]
        proj = torch.cat([rows[r][at[r]:at[r] + cuts[r][k]] for r in who]).to(dtype).to(dev())
        step = _step(n_new, [at[r] for r in who], [slots[r] for r in who])
        n = proj.shape[0]
        xbc = torch.empty(n, C, device=dev())
        dt, decay, y = torch.empty(n, H, device=dev()), torch.empty(n, H, device=dev()), torch.empty(n, inner, device=dev())
        ops.ssd_prepare(proj, off_x, off_dt, conv_w.to(dev()), conv_b.to(dev()), A_log.to(dev()), dt_bias.to(dev()), state,
                        state_floats, step, xbc, dt, decay)
        ops.decay_scan(xbc, inner + G * N, inner, 0, None, state, step, y, H, N, Pd, True, heads_per_group=H // G,
                       token_decay=decay, token_scale=dt, skip=D.to(dev()))
        out = torch.empty(n, inner, dtype=dtype, device=dev())
        ops.ssd_gated_norm(out, y, proj[:, :inner], norm_w.to(dev()), eps, parts)
        assert int(step.status.item()) == 0
        o = out.float().cpu()
        for r, c in zip(who, n_new):
            got[r].append(o[:c])
            o = o[c:]
            at[r] += c
    m = {"heads": H, "vdim": Pd, "state": N, "groups": G, "conv": taps, "norm_groups": parts}
    for r in range(3):
        # the plain layer on an input that makes its first product the rows themselves
        row = rows[r].double()
        cols = torch.cat([row[:, :inner], row[:, off_x:off_x + C], row[:, off_dt:off_dt + H]], dim=1)
        w = {"in": torch.eye(cols.shape[1], dtype=P.F), "conv": conv_w.double(), "conv.b": conv_b.double(),
             "dt_bias": dt_bias.double(), "A_log": A_log.double(), "D": D.double(), "norm": norm_w.double(),
             "o": torch.eye(inner, dtype=P.F)}
        want = P.state_space(cols, m, w, "", eps)
        assert rel_err(torch.cat(got[r]).numpy(), want.numpy()) <= (1e-4 if dtype == torch.float32 else 2e-2), r
    assert float(state[1].min()) == 7.0                                               # nobody's record is untouched


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_expert_weights_on_the_activations_input_and_the_new_activations(dtype):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, E, ff, sff = 9, 5, 24, 16
    h = (torch.randn(T, sff + E * ff, generator=g) * 2).to(dtype)
    gates = torch.rand(T, E, generator=g) * (torch.rand(T, E, generator=g) < 0.5)
    hd = h.clone().to(dev())
    ops.moe_act(hd, gates.to(dev()), sff, ff, E, "gelu", weight_in=True)
    w = torch.cat([torch.ones(T, sff), gates.repeat_interleave(ff, dim=1)], dim=1).double()
    want = P.gelu_erf(h.double() * w) * (w != 0)
    assert rel_err(hd.float().cpu().numpy(), want.numpy()) <= kernel_tol(dtype)
    rows = (torch.randn(T, ff, generator=g) * 2).to(dtype)
    rw = torch.rand(T, generator=g)
    rd = rows.clone().to(dev())
    ops.moe_row_act(rd, rw.to(dev()), "gelu", weight_in=True)
    assert rel_err(rd.float().cpu().numpy(), P.gelu_erf(rows.double() * rw.double()[:, None]).numpy()) <= kernel_tol(dtype)
    x = (torch.randn(T, 40, generator=g) * 2).to(dtype)
    xd = x.clone().to(dev())
    ops.act_rows(xd, "relu2")
    assert rel_err(xd.float().cpu().numpy(), (torch.relu(x.double()) ** 2).numpy()) <= kernel_tol(dtype)


@gpu
@pytest.mark.parametrize("M,K,N", [(5, 128, 200), (32, 384, 72), (200, 96, 136), (300, 256, 512)])
def test_squared_relu_in_the_epilogue_of_the_product(M, K, N):
    from lite_lang_b200 import ops
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    got = ops.linear_act(x.to(dev()), w.to(dev()), "relu2").float().cpu()
    want = torch.relu((x.double() @ w.double().T)) ** 2
    assert rel_err(got.numpy(), want.numpy()) <= 2e-2


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
        refs, decided = [], []
        for s in seqs:
            margins = []
            refs.append(P.forward(cfg, w, s, margins=margins).numpy())
            decided.append(decided_rows(margins))
        _FOLDERS[name] = (folder, seqs, refs, decided)
    return _FOLDERS[name][:3]


def _strict(name, i, n=None):
    """The rows of sequence i (its first n) that bfloat16 is held to."""
    _case(name)
    n = len(_FOLDERS[name][1][i]) if n is None else n
    return np.arange(n) < _FOLDERS[name][3][i]


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
def test_residual_after_every_layer():
    """The float32 residual stream after each layer of a short prompt against the plain implementation's."""
    from lite_lang_b200.engine.batch import StepEntry
    from lite_lang_b200.parts.base import whole_output
    for name in ("P", "R"):
        folder, seqs, _ = _case(name)
        cfg, w = P.read_model_folder(folder)
        layers = []
        P.forward(cfg, w, seqs[4], layers)
        mgr, runner = _runner(folder, torch.float32, CASES[name]["page_size"], 64, graphs=False)
        seen = []
        for block in runner.model.blocks:
            def wrapped(h, delta, step, caches, _f=block.forward):
                h, delta = _f(h, delta, step, caches)
                pending = 0 if delta is None else whole_output(delta, torch.float32).float()
                seen.append((h.float() + pending).cpu())
                return h, delta
            block.forward = wrapped
        s = mgr.open()
        assert runner.reserve(s, len(seqs[4]))
        runner.step([StepEntry(s, seqs[4], (0,))])
        assert len(seen) == len(layers)
        for i, (a, b) in enumerate(zip(seen, layers)):
            assert float((a.double() - b).abs().max()) <= 2e-5 * float(b.abs().max()), (name, i)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_whole_decode_and_portions(name, dtype):
    folder, seqs, refs = _case(name)
    mgr, runner = _runner(folder, dtype, CASES[name]["page_size"], 256 // CASES[name]["page_size"])
    for i in (0, 3, 4):                                     # whole prompts (one of them a single token)
        s = mgr.open()
        assert close(_feed(runner, mgr, s, seqs[i]), refs[i], dtype, _strict(name, i)), f"{name} whole {i}"
        mgr.close(s)
    for i, tail in ((0, 120), (2, 40)):                     # a prompt, then many tokens one by one (captured steps):
        s, n = mgr.open(), len(seqs[i])                     # every window passes over decoded tokens
        head = n - tail
        got = [_feed(runner, mgr, s, seqs[i][:head])] + [_feed(runner, mgr, s, seqs[i][t:t + 1]) for t in range(head, n)]
        assert close(np.concatenate(got), refs[i], dtype, _strict(name, i)), f"{name} decode {i}"
        mgr.close(s)
    s, n = mgr.open(), len(seqs[1])                         # from the very first token on, one by one
    got = [_feed(runner, mgr, s, seqs[1][t:t + 1]) for t in range(n)]
    assert close(np.concatenate(got), refs[1], dtype, _strict(name, 1)), f"{name} token by token"
    mgr.close(s)
    sizes = [7, 2, 13, 2, 5, 31, 2, 3, 17, 2, 64, 2, 9]
    for i in (0, 5):                                        # portions of changing size, down to two tokens
        s, n, t, k, got = mgr.open(), len(seqs[i]), 0, 0, []
        while t < n:
            c = min(sizes[k % len(sizes)], n - t)
            got.append(_feed(runner, mgr, s, seqs[i][t:t + c]))
            t, k = t + c, k + 1
        assert close(np.concatenate(got), refs[i], dtype, _strict(name, i)), f"{name} portions {i}"
        mgr.close(s)
    runner.check_status()
    assert runner.graph_replays > 0


@gpu
def test_a_pool_smaller_than_the_prompt_serves_it_through_the_pages_given_back():
    """Every layer of this case has a window, so a request holds a bounded number of pages however long it
    grows (those of its kept first tokens among them): a prompt of several times the pool, fed in portions, and
    the logits are the whole prompt's."""
    folder = write_folder("W")
    ps = CASES["W"]["page_size"]
    cfg, w = P.read_model_folder(folder)
    toks = [int(t) for t in np.random.default_rng(21).integers(0, cfg["vocab"], 400)]
    ref = P.forward(cfg, w, toks).numpy()
    portion = 24
    pages = (20 + portion + ps - 1) // ps + 1 + 2
    assert pages * ps < len(toks) // 4
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
    waiting, live, all_got, all_ref, all_strict = list(enumerate(order)), {}, [], [], []
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
            all_strict.append(_strict(name, i)[[t + w for w in want]])
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
    assert close(np.concatenate(all_got), np.concatenate(all_ref), dtype, np.concatenate(all_strict)), name
    assert mgr.pages_reused > 0


@gpu
def test_a_batch_gives_each_request_what_it_gets_alone():
    """In the attentions, the scan and the norms the order of every sum depends on the token's position only;
    what is left between a request alone and the same request beside others, in other pages and slots and cut
    otherwise, is the rounding of the matrix products, whose shapes differ (float32, where nothing else rounds)."""
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
    assert float(np.abs(got - alone).max()) <= 5e-5 * float(np.abs(alone).max())


@gpu
def test_replay_tool_and_a_prompt_of_many_tokens_in_one_step():
    """The command-line replay on a folder: a prompt long enough for the prompt attention kernels, cut into three
    steps beside a short request that ends early."""
    folder = write_folder("Q")
    cfg, w = P.read_model_folder(folder)
    toks = [int(t) for t in np.random.default_rng(9).integers(0, cfg["vocab"], 260)]
    margins = []
    ref = P.forward(cfg, w, toks, margins=margins).numpy()
    ok = np.arange(260) < decided_rows(margins)
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
        assert close(np.concatenate([a, b[:59], c, b[59:]]), want, dtype,
                     np.concatenate([ok[0:200:7], ok[200:259], ok[259:], ok[4:5]]))


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
