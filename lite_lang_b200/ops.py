"""Typed Python entry points of the hand-written CUDA kernels.

Every function takes torch CUDA tensors, checks what the kernel assumes
(device, dtype, contiguity, sizes) and launches on torch's current stream.
There is no CPU or library fallback: a tensor that is not on a CUDA device, or
a missing kernel library, raises.

Matrix products are the exception: like the reference, which calls cuBLAS
through ``torch.mm`` / ``torch.addmm`` (``litelang/models/qwen2/layer/
transformer_layer.py:79-109,193``), ``linear`` is a library product.  On the
float32 path TF32 is switched off so that it is a true 32-bit product.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional, Tuple

import torch

from .csrc.build import load_library

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle.  (``torch.cuda.current_stream()`` builds a Python object through
    several layers, 15 us a call, with well over a hundred launches in a step that is not captured.)"""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lite_lang_b200 kernels run on CUDA tensors only; there is no CPU path")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


def _f32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.float32 and t.is_contiguous(), f"{name} must be a contiguous float32 tensor")


def core():
    return load_library("core")


def configure_matmul_precision() -> None:
    """True float32 products (no TF32) and float32 accumulation for bfloat16 ones."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:  # pragma: no cover
        pass


# --------------------------------------------------------------------------
def embed_gather(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: Optional[torch.Tensor]) -> None:
    _need_cuda(out, table, ids)
    _i32(ids, "ids")
    _need(out.dtype == table.dtype and out.is_contiguous() and table.is_contiguous(), "embed: dtype/contiguity")
    n, hidden = ids.numel(), table.shape[1]
    _need(out.shape[0] >= n and out.shape[1] == hidden, "embed: out has the wrong shape")
    core().call("ll_embed_gather", c_int(_dtype_code(out)), _ptr(out), _ptr(table), _ptr(ids), c_int(n),
                c_int(hidden), c_int(table.shape[0]), _ptr(status), _stream())


def feed_tokens(ids: torch.Tensor, feed: torch.Tensor, results: torch.Tensor) -> None:
    """ids[i] = results[feed[i]] where feed[i] >= 0: token ids sampled by the step before, taken on the device."""
    _need_cuda(ids, feed, results)
    for t, nm in ((ids, "ids"), (feed, "feed"), (results, "results")):
        _i32(t, nm)
    _need(feed.numel() >= ids.numel(), "feed_tokens: one feed index per token id")
    core().call("ll_feed_tokens", _ptr(ids), _ptr(feed), _ptr(results), c_int(ids.numel()), c_int(results.numel()),
                _stream())


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    _need_cuda(out, x, weight)
    _f32(weight, "norm weight")
    _need(x.dim() == 2 and out.shape == x.shape and out.dtype == x.dtype, "rmsnorm: shapes")
    _need(x.stride(1) == 1 and out.stride(1) == 1, "rmsnorm: rows must be contiguous")
    _need(weight.numel() == x.shape[1], "rmsnorm: weight size")
    core().call("ll_rmsnorm", c_int(_dtype_code(x)), _ptr(out), _ptr(x), _ptr(weight), c_float(eps),
                c_int(x.shape[0]), c_int(x.shape[1]), c_long(x.stride(0)), c_long(out.stride(0)), _stream())


def add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None, write_residual: bool = True) -> None:
    """out[i] = norm(residual[r] + delta[r]); r = rows[i] if rows is given, else i.

    Without ``rows`` the rounded sum is written back into ``residual``.
    """
    _need_cuda(out, residual, delta, weight, rows)
    _f32(weight, "norm weight")
    _i32(rows, "rows")
    hidden = residual.shape[1]
    _need(residual.is_contiguous() and out.is_contiguous() and out.dtype == residual.dtype, "add_rmsnorm: layout")
    if delta is not None and delta.dim() == 2:
        _need(delta.is_contiguous() and delta.dtype == residual.dtype and delta.shape[1] == hidden,
              "add_rmsnorm: delta layout")
    n_out = rows.numel() if rows is not None else residual.shape[0]
    _need(out.shape[0] >= n_out and out.shape[1] == hidden, "add_rmsnorm: out shape")
    wr = 1 if (write_residual and rows is None and delta is not None) else 0
    partial, parts, part_stride = None, 0, 0
    if delta is not None and delta.dim() == 3:      # float32 partial sums [parts, tokens, hidden]
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and delta.shape[2] == hidden,
              "add_rmsnorm: partial sums must be contiguous float32 [parts, tokens, hidden]")
        partial, parts, part_stride, delta = delta, delta.shape[0], delta.shape[1] * hidden, None
    core().call("ll_add_rmsnorm", c_int(_dtype_code(residual)), _ptr(out), _ptr(residual), _ptr(delta),
                _ptr(partial), c_int(parts), c_long(part_stride), _ptr(weight), c_float(eps), c_int(n_out),
                c_int(hidden), _ptr(rows), c_int(wr), _stream())


def bias_rope_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: Optional[torch.Tensor],
                    cos_sin: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int,
                    slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                    v_cache: Optional[torch.Tensor], page_size: int, status: Optional[torch.Tensor],
                    num_tokens: Optional[int] = None) -> None:
    """Bias, half-split rotation of q and k, and the store of k and v into a cache plane.

    Each of the three is skipped when its argument is None.  ``cos_sin`` is the
    float32 table [max_positions, rot_dim] (cos half, then sin half).
    """
    _need_cuda(qkv, bias, positions, cos_sin, slot_map, k_cache, v_cache)
    _f32(bias, "bias")
    _f32(cos_sin, "cos_sin")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv.dim() == 2 and qkv.shape[1] == width and qkv.stride(1) == 1, "qkv must be [tokens, (nh+2nkv)*hd]")
    n = qkv.shape[0] if num_tokens is None else num_tokens
    if bias is not None:
        _need(bias.numel() == width, "bias size")
    rot_dim, max_pos = 0, 0
    if cos_sin is not None:
        _need(positions is not None, "rotation needs positions")
        max_pos, rot_dim = cos_sin.shape
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None, "store needs the cache plane")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache dtype differs from activations")
        _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
        _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
        num_slots = k_cache.shape[0] * page_size
    core().call("ll_bias_rope_store", c_int(_dtype_code(qkv)), _ptr(qkv), c_long(qkv.stride(0)), _ptr(bias),
                _ptr(positions), _ptr(cos_sin), c_int(max_pos), c_int(rot_dim), c_int(num_heads),
                c_int(num_kv_heads), c_int(head_dim), _ptr(slot_map), _ptr(k_cache), _ptr(v_cache),
                c_int(page_size), c_long(num_slots), c_int(n), _ptr(status), _stream())


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    _need_cuda(out, gate_up)
    _need(gate_up.is_contiguous() and out.is_contiguous() and out.dtype == gate_up.dtype, "silu_mul: layout")
    n, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape[0] == n and out.shape[1] == two_i // 2, "silu_mul: shapes")
    core().call("ll_silu_mul", c_int(_dtype_code(out)), _ptr(out), _ptr(gate_up), c_int(n), c_int(two_i // 2),
                _stream())


def paged_attention_generic(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, block_table: torch.Tensor, token_req: torch.Tensor,
                            req_slot: torch.Tensor, positions: torch.Tensor, num_tokens: int, num_heads: int,
                            num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int], scale: float,
                            status: Optional[torch.Tensor], value_head_dim: Optional[int] = None) -> None:
    """Attention of every new token over its request's cached keys (any sizes, both dtypes).

    ``q`` points at the first query head of the first token; head h of token t
    is at ``q + t*q_stride + h*head_dim`` (elements).  ``value_head_dim``: width of a value head
    (and of an output head) where it differs from the keys'.
    """
    vd = head_dim if value_head_dim is None else int(value_head_dim)
    _need_cuda(out, q, k_cache, v_cache, block_table, token_req, req_slot, positions)
    for t, nm in ((block_table, "block_table"), (token_req, "token_req"), (req_slot, "req_slot"),
                  (positions, "positions")):
        _i32(t, nm)
    _need(head_dim <= 256 and vd <= 512, f"heads of {head_dim} keys / {vd} values are larger than the generic "
          "attention kernel takes (256 / 512)")
    _need(num_heads % num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads")
    _need(out.dtype == q.dtype == k_cache.dtype == v_cache.dtype, "attention: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * vd, "attention: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
          and tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, vd), "cache plane shape")
    core().call("ll_paged_attention_generic", c_int(_dtype_code(out)), _ptr(out), c_long(out.stride(0)), _ptr(q),
                c_long(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.stride(0)),
                _ptr(token_req), _ptr(req_slot), _ptr(positions), c_int(num_tokens), c_int(num_heads),
                c_int(num_kv_heads), c_int(head_dim), c_int(vd), c_int(page_size), c_int(k_cache.shape[0]),
                c_int(window or 0), c_float(scale), _ptr(status), _stream())


def bias_rotate_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: Optional[torch.Tensor],
                      freq: Optional[torch.Tensor], interleaved: bool, num_heads: int, num_kv_heads: int,
                      head_dim: int, value_head_dim: int, slot_map: Optional[torch.Tensor],
                      k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], page_size: int,
                      status: Optional[torch.Tensor]) -> None:
    """Bias, rotation of q and k by angles made in the kernel (float32 position x ``freq`` [rot_dim / 2]; pairs
    (2i, 2i+1) if ``interleaved`` else (i, i + rot_dim/2); the heads' other channels pass), and the store of k and
    v into a cache plane whose values may be wider or narrower than its keys.  In place on ``qkv``
    [tokens, (nh + nkv) * head_dim + nkv * value_head_dim]."""
    _need_cuda(qkv, bias, positions, freq, slot_map, k_cache, v_cache)
    _f32(bias, "bias")
    _f32(freq, "freq")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    width = (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_head_dim
    _need(qkv.dim() == 2 and qkv.shape[1] == width and qkv.stride(1) == 1, "qkv must be [tokens, (nh+nkv)*hd + nkv*vd]")
    _need(bias is None or bias.numel() == width, "bias size")
    rot_dim = 0 if freq is None else 2 * freq.numel()
    _need(rot_dim <= head_dim and (rot_dim == 0 or positions is not None), "rotation: rot_dim <= head_dim, positions")
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None, "store needs the cache plane")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache dtype differs from activations")
        _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
        _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
              and tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, value_head_dim), "cache plane shape")
        num_slots = k_cache.shape[0] * page_size
    core().call("ll_bias_rotate_store", c_int(_dtype_code(qkv)), _ptr(qkv), c_long(qkv.stride(0)), _ptr(bias),
                _ptr(positions), _ptr(freq), c_int(rot_dim), c_int(1 if interleaved else 0), c_int(num_heads),
                c_int(num_kv_heads), c_int(head_dim), c_int(value_head_dim), _ptr(slot_map), _ptr(k_cache),
                _ptr(v_cache), c_int(page_size), c_long(num_slots), c_int(qkv.shape[0]), _ptr(status), _stream())


GATE_ACT = {"silu": 0, "relu": 1}


def act_mul(out: torch.Tensor, gate_up: torch.Tensor, act: str) -> None:
    """out = act(gate) * up for the fused projection [tokens, 2 * I] (gate columns first); act silu or relu."""
    _need_cuda(out, gate_up)
    _need(gate_up.is_contiguous() and out.is_contiguous() and out.dtype == gate_up.dtype, "act_mul: layout")
    n, two_i = gate_up.shape
    _need(two_i % 2 == 0 and out.shape[0] == n and out.shape[1] == two_i // 2, "act_mul: shapes")
    core().call("ll_act_mul", c_int(_dtype_code(out)), _ptr(out), _ptr(gate_up), c_int(n), c_int(two_i // 2),
                c_int(GATE_ACT[act]), _stream())


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[t] += bias in place (float32 sum, one rounding)."""
    _need_cuda(x, bias)
    _f32(bias, "bias")
    _need(x.dim() == 2 and x.stride(1) == 1 and bias.numel() == x.shape[1], "add_bias: shapes")
    core().call("ll_add_bias", c_int(_dtype_code(x)), _ptr(x), c_long(x.stride(0)), _ptr(bias), c_int(x.shape[0]),
                c_int(x.shape[1]), _stream())


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap) in place (float32)."""
    _need_cuda(logits)
    _f32(logits, "logits")
    core().call("ll_softcap", _ptr(logits), c_long(logits.numel()), c_float(cap), _stream())


def rms_pair_mean(out: torch.Tensor, a: torch.Tensor, bias_a: Optional[torch.Tensor], wa: torch.Tensor,
                  b: torch.Tensor, wb: torch.Tensor, eps: float) -> None:
    """out = (rms(a + bias_a) * wa + rms(b) * wb) / 2 row by row: two mixers' outputs joined."""
    _need_cuda(out, a, bias_a, wa, b, wb)
    for t, nm in ((bias_a, "bias"), (wa, "weight"), (wb, "weight")):
        _f32(t, nm)
    n, width = a.shape
    _need(tuple(b.shape) == (n, width) and tuple(out.shape) == (n, width) and out.is_contiguous()
          and a.stride(1) == 1 and b.stride(1) == 1 and a.dtype == b.dtype == out.dtype
          and wa.numel() == width and wb.numel() == width, "rms_pair_mean: shapes")
    core().call("ll_rms_pair_mean", c_int(_dtype_code(out)), _ptr(out), _ptr(a), c_long(a.stride(0)), _ptr(bias_a),
                _ptr(wa), _ptr(b), c_long(b.stride(0)), _ptr(wb), c_float(eps), c_int(n), c_int(width), _stream())


def attn_mma_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int) -> bool:
    """Shapes the tensor-core attention kernel takes; everything else goes to the generic kernel."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0 and q_stride % 8 == 0


def attn_mma_scratch_floats(row_blocks: int, num_kv_heads: int, nsplit: int, head_dim: int) -> int:
    return row_blocks * num_kv_heads * nsplit * 16 * (head_dim + 2)


def attn_mma(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
             block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor,
             num_entries: int, row_blocks: int, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
             window: Optional[int], scale: float, nsplit: int, scratch: Optional[torch.Tensor],
             counters: Optional[torch.Tensor], status: Optional[torch.Tensor], all_single: bool = False,
             cluster: bool = False, warps: int = 4) -> None:
    """Tensor-core paged attention (bfloat16) of the step's entries: decode and prompt portions.

    ``row_blocks`` is the sum over entries of ceil(q_len * group / 16).  With ``nsplit`` > 1 the
    keys of every row block are split over that many CTAs, which park partial results in
    ``scratch`` (float32, ``attn_mma_scratch_floats`` elements); ``counters`` (int32
    [row_blocks * num_kv_heads]) must be zero and are left zero.  ``all_single`` promises that
    every entry brings exactly one token (a decode step).  ``cluster`` (nsplit 2, 4 or 8) makes the
    splits of a row block one thread-block cluster that merges through distributed shared memory;
    scratch and counters are then not needed.  ``warps``: 4 or 8 warps a CTA (8 pays when the step
    has few row blocks).
    """
    _need_cuda(out, q, k_cache, v_cache, block_table, cu_q, ctx_len, req_slot, scratch, counters)
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_len, "ctx_len"), (req_slot, "req_slot"),
                  (counters, "counters")):
        _i32(t, nm)
    _f32(scratch, "scratch")
    _need(attn_mma_supported(q.dtype, head_dim, page_size, q_stride),
          f"attn_mma takes bfloat16, head_dim 64 or 128 and pages of a multiple of 16 tokens, "
          f"not {q.dtype}, {head_dim}, {page_size}")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_mma: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 2 == 0, "attn_mma: out")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(cu_q.numel() >= num_entries + 1 and ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries,
          "attn_mma: entry arrays too short")
    if cluster:
        _need(nsplit in (2, 4, 8, 16), "attn_mma: a cluster has 2, 4, 8 or 16 splits")
    if nsplit > 1 and not cluster:
        _need(scratch is not None and counters is not None, "attn_mma: splits need scratch and counters")
        _need(scratch.numel() >= attn_mma_scratch_floats(row_blocks, num_kv_heads, nsplit, head_dim),
              "attn_mma: scratch too small")
        _need(counters.numel() >= row_blocks * num_kv_heads, "attn_mma: counters too small")
    load_library("attn_mma").call(
        "ll_attn_mma_ex", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(cu_q), _ptr(ctx_len), _ptr(req_slot),
        c_int(num_entries), c_int(row_blocks), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(k_cache.shape[0]), c_int(window or 0), c_float(scale), c_int(nsplit),
        c_int(1 if all_single else 0), c_int(1 if cluster else 0), c_int(warps), _ptr(scratch), _ptr(counters),
        _ptr(status), _stream())


_attn_decode_scratch = {}   # per device: (partial results, counters) of attn_decode's clusters that meet through memory
_DECODE_SCRATCH_FLOATS = 1 << 19    # 2 MB; a plan's need is (CTAs / 4) * 8 * (head size + 2 splits) floats: far less
_DECODE_SCRATCH_COUNTERS = 4096


def _decode_scratch(device, floats: int, counters: int):
    """One buffer a device, of a fixed size and never replaced: captured steps keep its address."""
    _need(floats <= _DECODE_SCRATCH_FLOATS and counters <= _DECODE_SCRATCH_COUNTERS,
          "attn_decode: too many clusters for the scratch memory of their partial results")
    have = _attn_decode_scratch.get(device)
    if have is None:
        have = (torch.empty(_DECODE_SCRATCH_FLOATS, dtype=torch.float32, device=device),
                torch.zeros(_DECODE_SCRATCH_COUNTERS, dtype=torch.int32, device=device))
        _attn_decode_scratch[device] = have
    return have


def attn_decode(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                block_table: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor, num_entries: int,
                num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: Optional[int],
                scale: float, nsplit: int, status: Optional[torch.Tensor], warps: int = 4, depth: int = 0,
                nouter: int = 1) -> None:
    """Tensor-core decode attention (bfloat16), transposed product: one new token per entry, groups of at
    most 8 query heads.  ``nsplit`` in (1, 2, 4, 8) CTAs per (entry, kv head) form a cluster; ``warps`` (4 or 8)
    a CTA take the split's tiles in turn through rings of ``depth`` tiles a warp (0: the kernel's choice; 2 to 4
    for 4 warps, 2 or 3 for 8).  ``nouter`` > 1 (few requests, very long contexts; needs nsplit >= 2): that many
    clusters a (entry, kv head), each with a range of the keys, which meet through scratch memory kept by this
    module."""
    _need_cuda(out, q, k_cache, v_cache, block_table, ctx_len, req_slot)
    for t, nm in ((block_table, "block_table"), (ctx_len, "ctx_len"), (req_slot, "req_slot")):
        _i32(t, nm)
    _need(attn_mma_supported(q.dtype, head_dim, page_size, q_stride) and num_heads // num_kv_heads <= 8,
          "attn_decode takes bfloat16, head_dim 64 or 128, pages of a multiple of 16 tokens, groups of at most 8")
    _need(nsplit in (1, 2, 4, 8), "attn_decode: 1, 2, 4 or 8 splits")
    _need(warps in (4, 8), "attn_decode: 4 or 8 warps")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_decode: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 2 == 0, "attn_decode: out")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries, "attn_decode: entry arrays too short")
    scratch = counters = None
    if nouter > 1:
        _need(nsplit >= 2 and 1 < nouter <= 64 and warps == 8 and depth in (0, 2),
              "attn_decode: several clusters a (entry, kv head) need nsplit >= 2, 8 warps and rings of two tiles")
        depth = 2
        scratch, counters = _decode_scratch(q.device, num_entries * num_kv_heads * nouter * 8 * (head_dim + 2 * nsplit),
                                            num_entries * num_kv_heads * nsplit)
    load_library("attn_mma").call(
        "ll_attn_decode", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(ctx_len), _ptr(req_slot), c_int(num_entries),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(page_size), c_int(k_cache.shape[0]),
        c_int(window or 0), c_float(scale), c_int(nsplit), c_int(warps), c_int(depth), c_int(nouter), _ptr(scratch),
        _ptr(counters), _ptr(status), _stream())


def attn_prefill(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor,
                 num_entries: int, row_blocks: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 page_size: int, window: Optional[int], scale: float, status: Optional[torch.Tensor]) -> None:
    """Tensor-core paged attention (bfloat16) for portions of prompts: 128 query rows a CTA share the
    keys and values through shared memory.  ``row_blocks`` is the sum over the entries of
    ceil(q_len * group / 128).  Same shapes as ``attn_mma``."""
    _need_cuda(out, q, k_cache, v_cache, block_table, cu_q, ctx_len, req_slot)
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_len, "ctx_len"), (req_slot, "req_slot")):
        _i32(t, nm)
    _need(attn_mma_supported(q.dtype, head_dim, page_size, q_stride),
          f"attn_prefill takes bfloat16, head_dim 64 or 128 and pages of a multiple of 16 tokens, "
          f"not {q.dtype}, {head_dim}, {page_size}")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_prefill: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 8 == 0,
          "attn_prefill: out")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(cu_q.numel() >= num_entries + 1 and ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries,
          "attn_prefill: entry arrays too short")
    load_library("attn_mma").call(
        "ll_attn_prefill", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(cu_q), _ptr(ctx_len), _ptr(req_slot),
        c_int(num_entries), c_int(row_blocks), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(page_size), c_int(k_cache.shape[0]), c_int(window or 0), c_float(scale), _ptr(status), _stream())


def attn_prefill_tc_supported(dtype: torch.dtype, head_dim: int, page_size: int, q_stride: int, group: int) -> bool:
    """Whether the tcgen05 prefill attention takes this shape."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and q_stride % 8 == 0 and 1 <= group <= 128
            and (page_size in (8, 16, 32) or (page_size > 0 and page_size % 64 == 0)))


def attn_prefill_tc_blocks(q_lens, group: int) -> int:
    """Row blocks of a step for ``attn_prefill_tc``: a CTA takes floor(128 / group) tokens of one entry."""
    tpb = 128 // group
    return sum((int(n) + tpb - 1) // tpb for n in q_lens)


_attn_tc_scratch = {}


def attn_prefill_tc_plan(entries, group: int, window: Optional[int], num_kv_heads: int = 1, slots: int = 0):
    """(row blocks, nsplit, split_len) of a step for ``attn_prefill_tc``.  ``entries``: (cached tokens, new tokens)
    per entry; a row block takes floor(128 / group) tokens and walks n key blocks of 64.

    A CTA's blocks are a chain (scores, softmax, P V: about 1.4 us a block), so a step lasts as long as its
    longest CTA, and a CTA that finds no room on the SMs at once waits for a whole one to end (the hardware hands
    CTAs out in order).  So row blocks are cut into splits of at most ``split_len`` blocks, with the smallest
    ``split_len`` for which all CTAs of the step fit the ``slots`` (two an SM) at once: a whole causal prompt of
    2,048 tokens (row blocks of 1..32 blocks, 2 kv heads) gets 16, i.e. its longer half is cut in two.  Not below
    4 blocks a split or over 8 splits (every split's partial result goes through scratch memory); when the
    unsplit row blocks already exceed the slots, nothing is cut."""
    tpb = 128 // group
    lengths = []
    for ctx, q in entries:
        for first in range(0, q, tpb):
            hi = ctx + min(first + tpb, q) - 1
            lo = max(0, ctx + first - window + 1) if window else 0
            lengths.append(hi // 64 - lo // 64 + 1)
    blocks = len(lengths)
    if not lengths or slots <= 0 or blocks * num_kv_heads > slots:
        return blocks, 1, 1 << 20
    longest = max(lengths)
    best = longest
    for t in range(max(4, (longest + 7) // 8), longest + 1):
        if sum((n + t - 1) // t for n in lengths) * num_kv_heads <= slots:
            best = t
            break
    if best * 5 > longest * 4:      # cutting off less than a fifth of the longest chain does not pay for the merges
        return blocks, 1, 1 << 20   # (four portions of 512 behind 1,536 tokens: 49 us uncut, 52.5 us cut at 29 of 32)
    most = (longest + best - 1) // best
    nsplit = 1 if most <= 1 else 2 if most <= 2 else 4 if most <= 4 else 8
    return blocks, nsplit, best


def attn_prefill_tc_splits(row_blocks: int, num_kv_heads: int, device) -> int:
    """CTAs a row block's keys may be split over when nothing is known about the entries' lengths: as many as
    still fit the SMs (two CTAs each) at once."""
    ctas = row_blocks * num_kv_heads
    slots = 2 * sm_count(device)
    for n in (8, 4, 2):
        if ctas * n <= slots:
            return n
    return 1


def attn_prefill_tc(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor,
                    num_entries: int, row_blocks: int, num_heads: int, num_kv_heads: int, head_dim: int,
                    page_size: int, window: Optional[int], scale: float, status: Optional[torch.Tensor],
                    nsplit: Optional[int] = None, split_len: int = 8, gate: Optional[torch.Tensor] = None) -> None:
    """Paged attention for portions of prompts on the tcgen05 tensor cores (TMA loads, S and O in tensor
    memory).  ``row_blocks`` from ``attn_prefill_tc_blocks``.  Otherwise as ``attn_prefill``.
    ``nsplit`` (1, 2, 4, 8; default: by the size of the step): the keys of a row block are split over up to that
    many CTAs of about ``split_len`` blocks of 64 keys each (``attn_prefill_tc_plan`` chooses both), which merge
    through scratch memory kept by this module (grown when needed, never shrunk).
    ``gate`` (bfloat16 [tokens, num_heads], any row stride): every head's output times the sigmoid of its gate."""
    _need_cuda(out, q, k_cache, v_cache, block_table, cu_q, ctx_len, req_slot, gate)
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_len, "ctx_len"), (req_slot, "req_slot")):
        _i32(t, nm)
    _need(attn_prefill_tc_supported(q.dtype, head_dim, page_size, q_stride, num_heads // num_kv_heads),
          f"attn_prefill_tc takes bfloat16, head_dim 64 or 128 and pages of 8, 16, 32 or a multiple of 64 tokens, "
          f"not {q.dtype}, {head_dim}, {page_size}")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_prefill_tc: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * head_dim and out.stride(0) % 8 == 0,
          "attn_prefill_tc: out")
    _need(q.stride(1) == 1 and q.shape[1] >= num_heads * head_dim and q.stride(0) == q_stride, "attn_prefill_tc: q")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane shape")
    _need(cu_q.numel() >= num_entries + 1 and ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries,
          "attn_prefill_tc: entry arrays too short")
    if nsplit is None:
        nsplit = attn_prefill_tc_splits(row_blocks, num_kv_heads, q.device)
    _need(nsplit in (1, 2, 4, 8), "attn_prefill_tc: nsplit is 1, 2, 4 or 8")
    scratch = counters = None
    if nsplit > 1:
        floats = row_blocks * num_kv_heads * nsplit * 128 * (head_dim + 2)
        have = _attn_tc_scratch.get(q.device)
        if have is None or have[0].numel() < floats or have[1].numel() < row_blocks * num_kv_heads:
            have = (torch.empty(max(floats, have[0].numel() if have else 0), dtype=torch.float32, device=q.device),
                    torch.zeros(max(row_blocks * num_kv_heads, 1024), dtype=torch.int32, device=q.device))
            _attn_tc_scratch[q.device] = have
        scratch, counters = have
    args = (_ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), c_int(q.shape[0]),
            _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.stride(0)), _ptr(cu_q), _ptr(ctx_len),
            _ptr(req_slot), c_int(num_entries), c_int(row_blocks), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
            c_int(page_size), c_int(k_cache.shape[0]), c_int(window or 0), c_float(scale), c_int(nsplit),
            c_int(max(1, int(split_len))), _ptr(scratch), _ptr(counters))
    if gate is not None:
        _need(gate.dtype == torch.bfloat16 and gate.dim() == 2 and gate.shape[0] == q.shape[0]
              and gate.shape[1] == num_heads and gate.stride(1) == 1, "attn_prefill_tc: gate is bfloat16 [tokens, heads]")
        load_library("attn_tc").call("ll_attn_prefill_tc_gated", *args, _ptr(gate), c_long(gate.stride(0)), _ptr(status),
                                     _stream())
        return
    load_library("attn_tc").call("ll_attn_prefill_tc", *args, _ptr(status), _stream())


_sample_scratch = {}


def sample_scratch_floats(rows: int, vocab: int) -> int:
    return rows * ((vocab + 2047) // 2048) * 3


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, rows: Optional[int] = None,
           scratch: Optional[torch.Tensor] = None) -> None:
    """Greedy (temperature None or <= 0) or temperature sampling of each row of float32 logits.

    Two kernels (per-chunk partial results, then one block per row); ``scratch`` holds the partial
    results (float32, ``sample_scratch_floats`` elements) and is taken from a per-device cache if
    not given."""
    _need_cuda(logits, out, temperature, uniform)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 2-D")
    _i32(out, "out")
    _f32(temperature, "temperature")
    _f32(uniform, "uniform")
    n = logits.shape[0] if rows is None else rows
    _need(out.numel() >= n, "sample: out too small")
    need = sample_scratch_floats(n, logits.shape[1])
    if scratch is None:
        scratch = _sample_scratch.get(logits.device)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(max(need, 1024), dtype=torch.float32, device=logits.device)
            _sample_scratch[logits.device] = scratch
    _f32(scratch, "scratch")
    _need(scratch.numel() >= need, "sample: scratch too small")
    core().call("ll_sample", _ptr(logits), c_long(logits.stride(0)), _ptr(temperature), _ptr(uniform), _ptr(out),
                c_int(n), c_int(logits.shape[1]), _ptr(scratch), _stream())


# --------------------------------------------------------------------------
SMALL_M = 64          # the most tokens the weight-streaming kernel takes


def smallm_preferred(x: torch.Tensor, weight: torch.Tensor, gated: bool = False) -> bool:
    """Where the hand-written kernel is used instead of the library product: few tokens and a
    weight matrix small enough that the library's tile shapes leave most SMs idle (measured on
    B200: the q|k|v and output projections; the library wins on the wide feed-forward and
    lm_head products)."""
    if not smallm_supported(x, weight):
        return False
    n, k = weight.shape
    return x.shape[0] <= 16 and n <= 4096 and k <= 2048 and not gated


def smallm_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= SMALL_M and x.shape[1] % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_smallm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
                act: str = "silu") -> torch.Tensor:
    """out = x @ weight.T for up to 64 tokens with the weight-streaming kernel.

    ``gated``: weight holds gate rows then up rows ([2 I, K]); out [M, I] = silu(gate) * up.
    out may be bfloat16 or (not gated) float32.
    """
    _need_cuda(x, weight, out)
    _need(smallm_supported(x, weight), "gemm_smallm: bfloat16, at most 64 tokens, K a multiple of 32")
    m, k = x.shape
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    _need(weight.shape[1] == k and (not gated or weight.shape[0] % 2 == 0), "gemm_smallm: weight shape")
    _need(out.shape[0] == m and out.shape[1] == n and out.stride(1) == 1, "gemm_smallm: out shape")
    _need(out.dtype in (torch.bfloat16, torch.float32) and not (gated and out.dtype != torch.bfloat16),
          "gemm_smallm: out dtype")
    load_library("gemm_smallm").call(
        "ll_gemm_smallm", _ptr(out), c_long(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0), _ptr(x),
        c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k), c_int(1 + GATE_ACT[act] if gated else 0),
        _stream())
    return out


STREAM_M = 32         # the most tokens the bulk-copy streaming kernel takes
STREAM_M_NARROW = 64  # ... for its units of 16 features (q|k|v, o): the tokens then go in two blocks of 32
_sm_count = {}


def sm_count(device) -> int:
    n = _sm_count.get(device)
    if n is None:
        n = torch.cuda.get_device_properties(device).multi_processor_count
        _sm_count[device] = n
    return n


def stream_mode(x: torch.Tensor, weight: torch.Tensor, gated: bool = False) -> Optional[int]:
    """Work-unit shape of ``gemm_stream`` for this product (0 wide, 1 gated, 2 narrow), or None."""
    if not (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= STREAM_M_NARROW and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0):
        return None
    k = x.shape[1]
    if x.shape[0] > STREAM_M:
        # 33 to 64 tokens: only small products with units of 16 features (bfloat16 out, k whole), a unit a CTA in
        # both blocks of tokens at once and k up to 1,536: a CTA re-reads its 32 token rows (twice its weights' bytes)
        # with every unit, which a larger product pays for (Qwen2-7B sizes at batch 64: 4.33 -> 4.85 ms a step;
        # 2.5-3B sizes 3.27 -> 3.43, and 3.32 with the o projection, k = 2,048, alone) and the 1.5B sizes gain from
        # (2.06 -> 2.00)
        units = (weight.shape[0] + 15) // 16
        return 2 if (not gated and k % 256 == 0 and k <= 1536 and 2 * units <= 2 * sm_count(x.device)) else None
    if gated:
        return 1 if k % 128 == 0 else None
    n = weight.shape[0]
    if n >= 8192 and k % 128 == 0:
        return 0
    if k % 256 == 0:
        return 2
    return 0 if k % 128 == 0 else None


def stream_ksplit(n: int, k: int, mode: int, device) -> int:
    """Parts to cut k into so that a product with few output features still has work units for every
    SM (only worth it for a long k).  The kernel needs every part non-empty: the count is normalised."""
    if mode == 1 or k < 4096:
        return 1
    feats, chunk = (64, 128) if mode == 0 else (16, 256)
    units = (n + feats - 1) // feats
    chunks = k // chunk
    want = max(1, min((2 * sm_count(device)) // units, chunks // 4))
    cpp = (chunks + want - 1) // want
    return (chunks + cpp - 1) // cpp


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, mode: int,
                status: Optional[torch.Tensor] = None, act: str = "silu", row_act: Optional[str] = None) -> torch.Tensor:
    """out = x @ weight.T for up to 32 bfloat16 tokens (64 for mode 2 to bfloat16 with k whole) with the TMA
    weight-streaming kernel.

    mode 0: units of 64 output features; 1: SiLU-gated (weight [2 I, K], out [M, I]);
    2: units of 16 features with k split over the warps.  A float32 ``out`` of shape
    [parts, M, N] receives partial sums of a k range cut into ``parts`` (see ``stream_ksplit``).
    ``row_act`` (mode 0 to bfloat16, k whole): an activation of ``ROW_ACT`` on the result.
    """
    _need_cuda(x, weight, out, status)
    m, k = x.shape
    gated = mode == 1
    row_code = 0
    if row_act is not None:
        _need(mode == 0 and out.dim() == 2 and out.dtype == torch.bfloat16, "gemm_stream: an activation goes with mode 0 "
                                                                          "to bfloat16 and an unsplit k")
        row_code = ROW_ACT[row_act] + 1
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    _need(stream_mode(x, weight, gated) is not None, "gemm_stream: bfloat16, at most 32 tokens (64 for mode 2), K % 128 == 0")
    _need(mode in (0, 1, 2) and k % (256 if mode == 2 else 128) == 0, "gemm_stream: K does not fit the mode")
    _need(weight.shape[1] == k, "gemm_stream: weight shape")
    ksplit = 1
    if out.dim() == 3:
        ksplit = out.shape[0]
        _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (m, n) and not gated,
              "gemm_stream: partial sums go to a contiguous float32 [parts, M, N]")
        out_stride = n
    else:
        _need(out.shape[0] == m and out.shape[1] == n and out.stride(1) == 1, "gemm_stream: out shape")
        out_stride = out.stride(0)
    _need(out.dtype == torch.bfloat16 or (out.dtype == torch.float32 and not gated), "gemm_stream: out dtype")
    load_library("gemm_stream").call(
        "ll_gemm_stream", _ptr(out), c_long(out_stride), c_int(1 if out.dtype == torch.float32 else 0), _ptr(x),
        c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k), c_int(mode | (GATE_ACT[act] << 8) | (row_code << 16)),
        c_int(ksplit), c_int(sm_count(x.device)), _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return out


SUMSQ_ROWS = 64     # rows of a sums-of-squares record (the most tokens ``gemm_stream`` takes)
NORM_SPLIT = os.environ.get("LITE_LANG_B200_NORM_SPLIT", "1") != "0"   # 0: the norm between two streaming products
                                                                        # stays a kernel of its own (for comparisons)


def into_norm_supported(x: torch.Tensor, w_before: torch.Tensor, residual: torch.Tensor) -> bool:
    """Whether ``gemm_stream_into_norm`` takes the product ``x @ w_before.T`` added to ``residual``: a streaming
    product of a decode step with units of 16 features and an unsplit k, bfloat16 residual rows of its shape."""
    n = w_before.shape[0]
    return (NORM_SPLIT and stream_mode(x, w_before) == 2 and n % 16 == 0 and residual.dtype == torch.bfloat16
            and residual.dim() == 2 and tuple(residual.shape) == (x.shape[0], n) and residual.stride(1) == 1)


def gated_scaled_supported(rows: torch.Tensor, w_gate_up: torch.Tensor) -> bool:
    """Whether ``gemm_stream_gated_scaled`` takes rows of this shape: where the streaming gated product runs."""
    if not (NORM_SPLIT and w_gate_up.shape[1] == rows.shape[1] and rows.shape[0] <= SUMSQ_ROWS):
        return False
    if tc_preferred(rows, w_gate_up, gated=True):      # 17 tokens and more: the tcgen05 kernel has the same epilogue
        return True
    return stream_mode(rows, w_gate_up, gated=True) == 1


def gemm_stream_into_norm(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                          status: Optional[torch.Tensor] = None):
    """residual += x @ weight.T (rounded as the separate product and sum would be); returns (u, sumsq): u = the new
    residual rows times ``norm_weight`` (bfloat16), sumsq float32 [out / 16, 64] = the sums of squares of each
    row's 16 values of a unit.  With ``gemm_stream_gated_scaled`` after it, this is the residual sum, the RMS norm
    and the two products around them in two kernels instead of three."""
    _need_cuda(x, weight, residual, norm_weight, status)
    m, k = x.shape
    n = weight.shape[0]
    _need(into_norm_supported(x, weight, residual), "gemm_stream_into_norm: bfloat16, at most 64 tokens, K % 256 == 0, "
                                                    "N % 16 == 0, residual bfloat16 [tokens, N]")
    _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == n and norm_weight.is_contiguous(),
          "gemm_stream_into_norm: the norm's weight is float32 [out]")
    u = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty((n // 16, SUMSQ_ROWS), dtype=torch.float32, device=x.device)
    load_library("gemm_stream").call(
        "ll_gemm_stream_into_norm", _ptr(u), c_long(u.stride(0)), _ptr(residual), c_long(residual.stride(0)),
        _ptr(norm_weight), _ptr(sumsq), _ptr(x), c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k),
        c_int(sm_count(x.device)), _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return u, sumsq


def gemm_stream_gated_scaled(u: torch.Tensor, w_gate_up: torch.Tensor, sumsq: torch.Tensor, eps: float,
                             status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(g) * up of the rows x = u / sqrt(mean of squares + eps), where u is already multiplied by the norm's
    weight and ``sumsq`` [units, 64] holds the rows' sums of squares in parts (``gemm_stream_into_norm``)."""
    _need_cuda(u, w_gate_up, sumsq, status)
    m, k = u.shape
    inter = w_gate_up.shape[0] // 2
    _need(gated_scaled_supported(u, w_gate_up), "gemm_stream_gated_scaled: bfloat16, K % 128 == 0, at most 32 tokens (64 where the tcgen05 kernel takes the product)")
    _need(sumsq.dtype == torch.float32 and sumsq.dim() == 2 and sumsq.shape[1] == SUMSQ_ROWS and sumsq.is_contiguous(),
          "gemm_stream_gated_scaled: sums of squares are float32 [units, 64]")
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=u.device)
    if tc_preferred(u, w_gate_up, gated=True):
        return gemm_tc(u, w_gate_up, act, gated=True, status=status, sumsq=sumsq, eps=eps)
    load_library("gemm_stream").call(
        "ll_gemm_stream_gated_scaled", _ptr(act), c_long(act.stride(0)), _ptr(u), c_long(u.stride(0)), _ptr(w_gate_up),
        c_int(m), c_int(inter), c_int(k), _ptr(sumsq), c_int(sumsq.shape[0]), c_float(eps),
        c_int(sm_count(u.device)), _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return act


def qkv_rope_supported(x: torch.Tensor, w_qkv: torch.Tensor, head_dim: int, rot_dim: int) -> bool:
    """Whether the fused projection + bias + rotation + cache write kernel takes this step."""
    return (stream_mode(x, w_qkv) is not None and x.shape[1] % 256 == 0 and head_dim % 16 == 0
            and rot_dim == head_dim)


def gemm_stream_qkv_rope(q_out: torch.Tensor, x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                         positions: torch.Tensor, cos_sin: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                         v_cache: Optional[torch.Tensor], page_size: int, status: Optional[torch.Tensor]) -> None:
    """q|k|v projection of up to 32 tokens with what follows it, in one kernel: bias, half-split rotation
    of q and k, q into ``q_out`` [tokens, num_heads * head_dim], k and v into the cache plane."""
    _need_cuda(q_out, x, w_qkv, bias, positions, cos_sin, slot_map, k_cache, v_cache, status)
    _f32(bias, "bias")
    _f32(cos_sin, "cos_sin")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    m, k = x.shape
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv_rope_supported(x, w_qkv, head_dim, cos_sin.shape[1]), "gemm_stream_qkv_rope: shapes")
    _need(tuple(w_qkv.shape) == (width, k), "gemm_stream_qkv_rope: weight shape")
    _need(q_out.dtype == torch.bfloat16 and q_out.shape[0] == m and q_out.shape[1] >= num_heads * head_dim
          and q_out.stride(1) == 1, "gemm_stream_qkv_rope: q_out")
    if bias is not None:
        _need(bias.numel() == width, "bias size")
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None and k_cache.dtype == torch.bfloat16
              and k_cache.is_contiguous() and v_cache.is_contiguous()
              and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane")
        num_slots = k_cache.shape[0] * page_size
    load_library("gemm_stream").call(
        "ll_gemm_stream_qkv_rope", _ptr(q_out), c_long(q_out.stride(0)), _ptr(x), c_long(x.stride(0)), _ptr(w_qkv),
        c_int(m), c_int(k), _ptr(bias), _ptr(positions), _ptr(cos_sin), c_int(cos_sin.shape[0]), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), _ptr(slot_map), _ptr(k_cache), _ptr(v_cache), c_int(page_size),
        c_long(num_slots), c_int(sm_count(x.device)), _ptr(status), _stream())


# A timeline build (LITE_LANG_B200_TIMELINE=1, see csrc/common.cuh): the kernels stamp the clock behind the status
# word that the runner hands out; those that a caller gives no status word get the runner's.
TIMELINE_KERNELS = ("qkv", "attention", "o", "gated", "down", "logits")
TIMELINE_SLOTS = len(TIMELINE_KERNELS) * 512 * 4
TIMELINE_STATUS = None


def timeline_build() -> bool:
    from .csrc.build import timeline_build as on
    return on()


TC_M = 128          # most tokens the tcgen05 weight-streaming kernel takes
TC_ENABLED = os.environ.get("LITE_LANG_B200_TC", "1") != "0"   # 0: library products instead (for comparisons)


def tc_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``gemm_tc`` takes this product: bfloat16, at most 128 tokens, K % 64 == 0, aligned rows."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and 0 < x.shape[0] <= TC_M and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 64 == 0
            and weight.is_contiguous() and weight.shape[1] == x.shape[1]
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


TC_MIN_M = 17       # from this many tokens on the tcgen05 kernel was measured ahead of gemm_stream's mma.sync tiles


def tc_preferred(x: torch.Tensor, weight: torch.Tensor, gated: bool = False, wide: bool = False) -> bool:
    """Where the tcgen05 kernel was measured ahead on a B200: more tokens than ``gemm_stream`` takes well
    (its mma.sync tiles get slower from 16 tokens up) and few enough that the step is still bound by reading
    the weights.  The gated feed-forward and a wide product (the logits) up to 64 tokens; a product with a
    long k (split over k, partial sums to the norm) up to 128.  Other products of such steps go to
    ``gemm_stream`` (up to 32 tokens) or the library."""
    if not (TC_ENABLED and tc_supported(x, weight) and x.shape[0] >= TC_MIN_M):
        return False
    if gated or wide:
        return x.shape[0] <= 64
    return x.shape[1] >= 4096 and tc_ksplit(weight.shape[0], x.shape[1], x.device) > 1


def tc_ksplit(n: int, k: int, device) -> int:
    """Parts to cut k into so that a product with few output features (units of 128) has a unit for
    every SM; every part keeps at least four 64-wide boxes.  Normalised so that no part is empty."""
    units = (n + 127) // 128
    boxes = k // 64
    want = max(1, min(sm_count(device) // units, boxes // 4))
    per = (boxes + want - 1) // want
    return (boxes + per - 1) // per


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False, act: str = "silu",
            status: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None, eps: float = 0.0) -> torch.Tensor:
    """out = x @ weight.T for up to 128 bfloat16 tokens on the tcgen05 tensor cores (weights streamed
    by TMA, accumulator in tensor memory).  ``gated``: weight is [2 I, K] and out = silu(gate) * up.
    A float32 ``out`` of shape [parts, M, N] receives the partial sums of a k range cut into parts."""
    _need_cuda(x, weight, out, status)
    _need(tc_supported(x, weight), "gemm_tc: bfloat16, at most 128 tokens, K % 64 == 0, 16-byte aligned rows")
    m, k = x.shape
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    ksplit = 1
    if out.dim() == 3:
        ksplit = out.shape[0]
        _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape[1:]) == (m, n) and not gated,
              "gemm_tc: partial sums go to a contiguous float32 [parts, M, N]")
        per = (k // 64 + ksplit - 1) // ksplit
        _need((k // 64 + per - 1) // per == ksplit, "gemm_tc: a part of k would be empty")
        out_stride = n
    else:
        _need(out.shape[0] == m and out.shape[1] == n and out.stride(1) == 1, "gemm_tc: out shape")
        out_stride = out.stride(0)
    _need(out.dtype == torch.bfloat16 or (out.dtype == torch.float32 and not gated), "gemm_tc: out dtype")
    load_library("gemm_tc").call(
        "ll_gemm_tc", _ptr(out), c_long(out_stride), c_int(1 if out.dtype == torch.float32 else 0), _ptr(x),
        c_long(x.stride(0)), _ptr(weight), c_int(m), c_int(n), c_int(k), c_int(1 + GATE_ACT[act] if gated else 0),
        c_int(ksplit),
        c_int(sm_count(x.device)), _ptr(sumsq), c_int(0 if sumsq is None else sumsq.shape[0]), c_float(eps),
        _ptr(status if status is not None else TIMELINE_STATUS), _stream())
    return out


PAIR_MIN_M = 65     # from this many tokens on (measured from 129 to 4,096) the two-SM tcgen05 kernel with the
                    # activation in its epilogue is ahead of a library product followed by ``silu_mul``


def pair_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``gemm_pair`` takes this product: bfloat16, K % 8 == 0, 16-byte aligned rows."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] > 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0
            and weight.is_contiguous() and weight.shape[1] == x.shape[1]
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
              status: Optional[torch.Tensor] = None, act: str = "silu", row_act: Optional[str] = None) -> torch.Tensor:
    """out = x @ weight.T for many bfloat16 tokens on the tcgen05 tensor cores, a pair of SMs a tile of
    256 tokens x 256 columns.  ``gated``: weight is [2 I, K] and out = silu(gate) * up, the activation done
    on the accumulator, so gate and up never go to memory."""
    _need_cuda(x, weight, out, status)
    _need(pair_supported(x, weight), "gemm_pair: bfloat16, K % 8 == 0, 16-byte aligned rows")
    m, k = x.shape
    n = weight.shape[0] // 2 if gated else weight.shape[0]
    _need(out.dtype == torch.bfloat16 and out.dim() == 2 and out.shape[0] == m and out.shape[1] == n
          and out.stride(1) == 1, "gemm_pair: out is bfloat16 [M, N] with unit column stride")
    if row_act is not None:      # a feed-forward without a gate: out = act(x @ weight.T), act of ``ROW_ACT``
        _need(not gated, "gemm_pair: row_act goes with the plain product")
        load_library("gemm_pair").call(
            "ll_gemm_pair_act", _ptr(out), c_long(out.stride(0)), _ptr(x), c_long(x.stride(0)), _ptr(weight), c_int(m),
            c_int(n), c_int(k), c_int(ROW_ACT[row_act] + 1), c_int(sm_count(x.device)), _ptr(status), _stream())
        return out
    load_library("gemm_pair").call(
        "ll_gemm_pair", _ptr(out), c_long(out.stride(0)), _ptr(x), c_long(x.stride(0)), _ptr(weight), c_int(m),
        c_int(n), c_int(k), c_int(1 + GATE_ACT[act] if gated else 0), c_int(sm_count(x.device)), _ptr(status),
        _stream())
    return out


def pair_qkv_supported(x: torch.Tensor, w_qkv: torch.Tensor, head_dim: int, rot_dim: int) -> bool:
    """Whether the two-SM tcgen05 projection with bias, rotation and cache write in its epilogue takes
    this step: whole heads in a tile of 256 columns, rotation of the whole head."""
    return TC_ENABLED and pair_supported(x, w_qkv) and head_dim in (64, 128, 256) and rot_dim == head_dim


def pair_qkv_preferred(x: torch.Tensor, w_qkv: torch.Tensor) -> bool:
    """Where it was measured ahead of a library product followed by ``bias_rope_store``: when the
    tiles of 256 tokens x 256 columns are enough for a good part of the SM pairs."""
    tiles = ((x.shape[0] + 255) // 256) * ((w_qkv.shape[0] + 255) // 256)
    return tiles * 4 >= sm_count(x.device)


def gemm_pair_qkv_rope(q_out: torch.Tensor, x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor],
                       positions: torch.Tensor, cos_sin: torch.Tensor, num_heads: int, num_kv_heads: int,
                       head_dim: int, slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], page_size: int, status: Optional[torch.Tensor]) -> None:
    """q|k|v projection of many tokens with what follows it, in one kernel: bias, half-split rotation of q
    and k, q into ``q_out`` [tokens, num_heads * head_dim], k and v into the cache plane."""
    _need_cuda(q_out, x, w_qkv, bias, positions, cos_sin, slot_map, k_cache, v_cache, status)
    _f32(bias, "bias")
    _f32(cos_sin, "cos_sin")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    m, k = x.shape
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(pair_qkv_supported(x, w_qkv, head_dim, cos_sin.shape[1]), "gemm_pair_qkv_rope: shapes")
    _need(tuple(w_qkv.shape) == (width, k), "gemm_pair_qkv_rope: weight shape")
    _need(q_out.dtype == torch.bfloat16 and q_out.shape[0] == m and q_out.shape[1] >= num_heads * head_dim
          and q_out.stride(1) == 1 and q_out.stride(0) % 8 == 0, "gemm_pair_qkv_rope: q_out")
    _need(cos_sin.is_contiguous() and positions.numel() >= m, "gemm_pair_qkv_rope: table and positions")
    if bias is not None:
        _need(bias.numel() == width and bias.is_contiguous(), "bias size")
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None and k_cache.dtype == torch.bfloat16
              and k_cache.is_contiguous() and v_cache.is_contiguous() and slot_map.numel() >= m
              and tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim), "cache plane")
        num_slots = k_cache.shape[0] * page_size
    load_library("gemm_pair").call(
        "ll_gemm_pair_qkv_rope", _ptr(q_out), c_long(q_out.stride(0)), _ptr(x), c_long(x.stride(0)), _ptr(w_qkv),
        c_int(m), c_int(k), _ptr(bias), _ptr(positions), _ptr(cos_sin), c_int(cos_sin.shape[0]), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), _ptr(slot_map), _ptr(k_cache), _ptr(v_cache), c_int(page_size),
        c_long(num_slots), c_int(sm_count(x.device)), _ptr(status), _stream())


ACCUMULATE_MIN_M = 129   # more tokens than any of the hand-written plain products takes: library territory


def accumulate_preferred(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``linear_accumulate`` should stand for ``linear`` + a later residual sum: when the product
    is a library one anyway (portions of prompts), its epilogue adds the residual for the price of reading it."""
    return x.shape[0] >= ACCUMULATE_MIN_M and x.dtype == weight.dtype


def linear_accumulate(x: torch.Tensor, weight: torch.Tensor, acc: torch.Tensor) -> None:
    """acc += x @ weight.T in place (library product with beta = 1: float32 accumulation, the sum with ``acc``
    in float32, one rounding), so that the norm after it reads the residual stream only."""
    _need_cuda(x, weight, acc)
    _need(acc.dtype == x.dtype and acc.shape[0] == x.shape[0] and acc.shape[1] == weight.shape[0]
          and acc.stride(1) == 1, "linear_accumulate: acc is [tokens, out] of the operands' dtype")
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("TF32 is on; call ops.configure_matmul_precision() before a float32 product")
    torch.addmm(acc, x, weight.t(), out=acc)


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """act(x @ Wg.T) * (x @ Wu.T) with W = [Wg; Wu], act SiLU or ReLU: fused for few tokens, else product + kernel."""
    inter = w_gate_up.shape[0] // 2
    act = torch.empty((x.shape[0], inter), dtype=x.dtype, device=x.device)
    if tc_preferred(x, w_gate_up, gated=True):
        return gemm_tc(x, w_gate_up, act, gated=True, act=activation)
    if stream_mode(x, w_gate_up, gated=True) is not None:
        return gemm_stream(x, w_gate_up, act, 1, act=activation)
    if smallm_preferred(x, w_gate_up, gated=True):
        return gemm_smallm(x, w_gate_up, act, gated=True, act=activation)
    if TC_ENABLED and x.shape[0] >= PAIR_MIN_M and pair_supported(x, w_gate_up):
        return gemm_pair(x, w_gate_up, act, gated=True, act=activation)
    gu = linear(x, w_gate_up)
    if activation == "silu":
        silu_mul(act, gu)
    else:
        act_mul(act, gu, activation)
    return act


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, partial_ok: bool = False) -> torch.Tensor:
    """x [n, in] times weight [out, in] transposed.

    Up to 32 bfloat16 tokens (decode) go to the hand-written TMA weight-streaming kernel
    (``gemm_stream``), or to ``gemm_smallm`` for shapes that one does not take.  Everything
    else is a library (cuBLAS) product, as in the reference: float32 operands give a true
    float32 product (TF32 is off); bfloat16 operands accumulate in float32.
    ``out_dtype=torch.float32`` with bfloat16 operands keeps the float32 accumulator as the
    result (the logits).  ``partial_ok``: the caller's consumer (the fused residual-and-norm
    kernel) accepts float32 partial sums [parts, n, out] of a product split over k.
    """
    _need_cuda(x, weight)
    if out is None and partial_ok and out_dtype in (None, x.dtype) and tc_preferred(x, weight):
        parts = tc_ksplit(weight.shape[0], x.shape[1], x.device)
        out = torch.empty((parts, x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        return gemm_tc(x, weight, out)
    if out is None and weight.shape[0] >= 8192 and tc_preferred(x, weight, wide=True):
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
        return gemm_tc(x, weight, out)
    mode = stream_mode(x, weight) if (out is None or out.stride(1) == 1) else None
    many = x.shape[0] > STREAM_M       # 33 to 64 tokens: bfloat16 out, k whole
    if mode is not None and many and ((out_dtype or x.dtype) != torch.bfloat16 or (out is not None and out.dtype != torch.bfloat16)):
        mode = None
    if mode is not None:
        dt = out_dtype or x.dtype
        if out is None:
            parts = (stream_ksplit(weight.shape[0], x.shape[1], mode, x.device)
                     if (partial_ok and dt == x.dtype and not many) else 1)
            if parts > 1:
                out = torch.empty((parts, x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
                return gemm_stream(x, weight, out, mode)
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=dt, device=x.device)
        if out.dtype == dt:
            return gemm_stream(x, weight, out, mode)
    if smallm_preferred(x, weight) and (out is None or out.stride(1) == 1):
        dt = out_dtype or x.dtype
        if out is None:
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=dt, device=x.device)
        if out.dtype == dt:
            return gemm_smallm(x, weight, out)
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("TF32 is on; call ops.configure_matmul_precision() before a float32 product")
    if out_dtype is not None and out_dtype != x.dtype:
        res = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is not None:
        return torch.mm(x, weight.t(), out=out)
    return torch.mm(x, weight.t())


# --------------------------------------------------------------------------
# float32 residual stream: scaled embedding and layer norm
# --------------------------------------------------------------------------
def embed_scaled_f32(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float,
                     status: Optional[torch.Tensor]) -> None:
    """out[t] = scale * table[ids[t]] as float32 rows (the residual stream of a model that keeps it in 32-bit)."""
    _need_cuda(out, table, ids)
    _i32(ids, "ids")
    _f32(out, "out")
    _need(table.is_contiguous() and out.shape[1] == table.shape[1] and out.shape[0] >= ids.numel(),
          "embed_scaled_f32: shapes")
    core().call("ll_embed_scaled_f32", c_int(_dtype_code(table)), _ptr(out), _ptr(table), _ptr(ids),
                c_int(ids.numel()), c_int(table.shape[1]), c_int(table.shape[0]), c_float(scale), _ptr(status),
                _stream())


def add_layernorm(out: torch.Tensor, residual: torch.Tensor, d1: Optional[torch.Tensor], d2: Optional[torch.Tensor],
                  weight: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                  partial: Optional[torch.Tensor] = None) -> None:
    """residual (float32) += d1 + d2 (written back unless ``rows`` selects rows); out = layer norm of it
    times ``weight``, in ``out``'s dtype.  ``partial``: a further addend as float32 partial sums
    [parts, tokens, hidden] of a product that was split over its inner dimension."""
    _need_cuda(out, residual, d1, d2, weight, rows)
    _f32(weight, "norm weight")
    _f32(residual, "residual")
    _i32(rows, "rows")
    hidden = residual.shape[1]
    for d in (d1, d2):
        if d is not None:
            _need(d.dtype == out.dtype and d.is_contiguous() and tuple(d.shape) == tuple(residual.shape),
                  "add_layernorm: a delta is [tokens, hidden] of the output's dtype")
    n_out = rows.numel() if rows is not None else residual.shape[0]
    _need(out.is_contiguous() and out.shape[0] >= n_out and out.shape[1] == hidden and weight.numel() == hidden,
          "add_layernorm: out shape")
    parts, part_stride = 0, 0
    if partial is not None:
        _need(partial.dtype == torch.float32 and partial.is_contiguous() and partial.dim() == 3
              and tuple(partial.shape[1:]) == tuple(residual.shape), "add_layernorm: partial sums are float32 "
              "[parts, tokens, hidden]")
        parts, part_stride = partial.shape[0], partial.shape[1] * hidden
    core().call("ll_add_layernorm", c_int(_dtype_code(out)), _ptr(out), _ptr(residual), _ptr(d1), _ptr(d2),
                _ptr(partial), c_int(parts), c_long(part_stride), _ptr(weight), c_float(eps), c_int(n_out),
                c_int(hidden), _ptr(rows), c_int(1 if rows is None else 0), _stream())


# --------------------------------------------------------------------------
# gated delta rule
# --------------------------------------------------------------------------
def delta_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, b_off: int, a_in: torch.Tensor,
                  conv_q: torch.Tensor, conv_k: torch.Tensor, conv_v: torch.Tensor, A_log: torch.Tensor,
                  dt_bias: torch.Tensor, state: torch.Tensor, tail_off: int, step, qn: torch.Tensor, kn: torch.Tensor,
                  vc: torch.Tensor, beta: torch.Tensor, g: torch.Tensor, H: int, Hk: int, dk: int, dv: int, taps: int,
                  per_channel: bool) -> None:
    """Convolution + SiLU of q, k, v (continuing from the records' last inputs), unit vectors, beta and decay of
    the step's tokens into float32 buffers; then the records' last ``taps - 1`` inputs are brought up to date."""
    _need_cuda(proj, a_in, conv_q, conv_k, conv_v, A_log, dt_bias, state, qn, kn, vc, beta, g)
    for t, nm in ((conv_q, "conv_q"), (conv_k, "conv_k"), (conv_v, "conv_v"), (A_log, "A_log"), (dt_bias, "dt_bias"),
                  (state, "state"), (qn, "qn"), (kn, "kn"), (vc, "vc"), (beta, "beta"), (g, "g")):
        _f32(t, nm)
    _need(proj.dim() == 2 and proj.stride(1) == 1 and a_in.stride(1) == 1 and a_in.dtype == proj.dtype,
          "delta_prepare: projections are rows of one dtype")
    _need(state.dim() == 2 and state.shape[1] == tail_off + (taps - 1) * (2 * Hk * dk + H * dv),
          "delta_prepare: the state record is S followed by the convolutions' last inputs")
    n = proj.shape[0]
    load_library("delta_rule").call(
        "ll_delta_prepare", c_int(_dtype_code(proj)), _ptr(proj), c_long(proj.stride(0)), c_int(q_off), c_int(k_off),
        c_int(v_off), c_int(b_off), _ptr(a_in), c_long(a_in.stride(0)), _ptr(conv_q), _ptr(conv_k), _ptr(conv_v),
        _ptr(A_log), _ptr(dt_bias), _ptr(state), c_long(state.stride(0)), c_long(tail_off), _ptr(step.token_req),
        _ptr(step.cu_q), _ptr(step.ctx_len), _ptr(step.req_slot), _ptr(step.positions), _ptr(qn), _ptr(kn), _ptr(vc),
        _ptr(beta), _ptr(g), c_int(n), c_int(step.num_entries), c_int(H), c_int(Hk), c_int(dk), c_int(dv),
        c_int(taps), c_int(1 if per_channel else 0), _stream())


def delta_recurrence(qn: torch.Tensor, kn: torch.Tensor, vc: torch.Tensor, beta: torch.Tensor, g: torch.Tensor,
                     state: torch.Tensor, step, o: torch.Tensor, H: int, Hk: int, dk: int, dv: int,
                     per_channel: bool) -> None:
    """The scan of every entry's tokens through its request's state; o float32 [tokens, H, dv]."""
    _need_cuda(qn, kn, vc, beta, g, state, o)
    _need(dk <= 256, f"delta rule: key heads of {dk} channels are wider than the scan kernel takes (256)")
    load_library("delta_rule").call(
        "ll_delta_recurrence", _ptr(qn), _ptr(kn), _ptr(vc), _ptr(beta), _ptr(g), _ptr(state), c_long(state.stride(0)),
        _ptr(step.cu_q), _ptr(step.req_slot), _ptr(o), c_int(step.num_entries), c_int(H), c_int(Hk), c_int(dk),
        c_int(dv), c_int(1 if per_channel else 0), _stream())


def delta_out(out: torch.Tensor, o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, eps: float, H: int,
              dv: int, gate_act: int) -> None:
    """out = o / rms(o over dv) * weight * act(gate); act 0 SiLU, 1 sigmoid."""
    _need_cuda(out, o, weight, gate)
    _f32(o, "o")
    _f32(weight, "weight")
    _need(out.is_contiguous() and gate.stride(1) == 1 and gate.dtype == out.dtype, "delta_out: layout")
    load_library("delta_rule").call(
        "ll_delta_out", c_int(_dtype_code(out)), _ptr(out), _ptr(o), _ptr(weight), _ptr(gate), c_long(gate.stride(0)),
        c_float(eps), c_int(out.shape[0]), c_int(H), c_int(dv), c_int(gate_act), _stream())


# --------------------------------------------------------------------------
# latent attention
# --------------------------------------------------------------------------
def latent_prepare(proj: torch.Tensor, q_off: int, kv_off: int, norm_w: torch.Tensor, eps: float, freq: torch.Tensor,
                   rot_dims: int, positions: torch.Tensor, slot_map: Optional[torch.Tensor], cache: torch.Tensor,
                   q_full: torch.Tensor, H: int, d: int, r: int, R: int, status: Optional[torch.Tensor],
                   amplitude: float = 1.0, q: Optional[torch.Tensor] = None) -> None:
    """Per token: the latent's RMS norm and the rotated key part into the cache row, and every head's rotated
    query part into ``q_full`` [tokens, H, R + r] behind the R latent-space numbers (which a product fills).
    ``q``: the rows that hold the query heads at ``q_off`` when they are not rows of ``proj`` (queries made by a
    second product); ``amplitude``: a factor on cos and sin."""
    _need_cuda(proj, norm_w, freq, positions, slot_map, cache, q_full, q)
    q = proj if q is None else q
    _need(q.dtype == proj.dtype and q.stride(1) == 1 and q.shape[0] == proj.shape[0], "latent_prepare: q rows")
    _f32(norm_w, "norm_w")
    _f32(freq, "freq")
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    _need(proj.stride(1) == 1 and cache.is_contiguous() and cache.dtype == proj.dtype and cache.shape[-1] == R + r
          and cache.shape[1] == 1, "latent_prepare: the cache plane is [pages, 1, page, latent + rotated]")
    _need(q_full.is_contiguous() and q_full.dtype == proj.dtype and tuple(q_full.shape[1:]) == (H, R + r),
          "latent_prepare: q_full is [tokens, H, latent + rotated] of the projections' dtype")
    load_library("latent_attn").call(
        "ll_latent_prepare", c_int(_dtype_code(proj)), _ptr(proj), c_long(proj.stride(0)), c_int(q_off), c_int(kv_off),
        _ptr(norm_w), c_float(eps), _ptr(freq), c_int(rot_dims), _ptr(positions), _ptr(slot_map), _ptr(cache),
        c_long(cache.shape[0] * cache.shape[2]), _ptr(q_full), c_int(proj.shape[0]), c_int(H), c_int(d), c_int(r),
        c_int(R), _ptr(status), c_float(amplitude), _ptr(q), c_long(q.stride(0)), _stream())


def latent_attention(out: torch.Tensor, q_full: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, step,
                     first: int, count: int, H: int, R: int, r: int, page_size: int, window: Optional[int],
                     scale: float, nsplit: int = 1, tiles_per_split: int = 0,
                     sink: Optional[torch.Tensor] = None) -> None:
    """Attention in the latent space for tokens ``first .. first + count - 1`` of the step.  ``q_full``
    [tokens, H, R + r] and ``out`` [tokens, H, R] (sum_j p_j c_j per head) have the cache's dtype.
    ``nsplit`` > 1: every query's keys are shared out over that many CTAs, ``tiles_per_split`` tiles of 32
    positions each (counted from the query's first visible tile; together they must cover the longest run of
    keys a query of the step sees), and merged by a second kernel.  ``sink`` float32 [H]: every head's softmax
    has one more key of that score, which carries no value."""
    _need_cuda(out, q_full, cache, block_table, sink)
    _f32(sink, "sink")
    _need(sink is None or sink.numel() == H, "latent_attention: sink is a number a head")
    _need(q_full.is_contiguous() and out.is_contiguous() and q_full.dtype == cache.dtype == out.dtype
          and tuple(q_full.shape[1:]) == (H, R + r) and tuple(out.shape[1:]) == (H, R), "latent_attention: layouts")
    _need(R <= 512, f"latent_attention: a latent of {R} numbers is wider than the kernel takes (512)")
    _need(0 <= first and first + count <= q_full.shape[0], "latent_attention: token range")
    part_acc = part_ml = None
    if nsplit > 1:
        _need(tiles_per_split >= 1, "latent_attention: splits need tiles_per_split")
        part_acc = torch.empty((count, H, nsplit, R), dtype=torch.float32, device=out.device)
        part_ml = torch.empty((count, H, nsplit, 2), dtype=torch.float32, device=out.device)
    load_library("latent_attn").call(
        "ll_latent_attention", c_int(_dtype_code(out)), _ptr(out), _ptr(q_full), _ptr(cache), _ptr(block_table),
        c_int(block_table.stride(0)), _ptr(step.token_req), _ptr(step.req_slot), _ptr(step.positions), c_int(first),
        c_int(count), c_int(H), c_int(R), c_int(r), c_int(page_size), c_int(cache.shape[0]), c_int(window or 0),
        c_float(scale), _ptr(step.status), c_int(nsplit), c_int(tiles_per_split), _ptr(part_acc), _ptr(part_ml),
        _ptr(sink), _stream())


def latent_attention_heads(dtype: torch.dtype, R: int, r: int) -> int:
    """Heads a CTA of ``latent_attention`` takes for these sizes (16 on tensor cores: bfloat16, R + r a multiple of
    16, R a multiple of 32; else 8): what a plan of the parts counts its CTAs with."""
    if dtype not in _DT:
        return 8
    return int(load_library("latent_attn").fn("ll_latent_attention_heads")(c_int(_DT[dtype]), c_int(R), c_int(r)))


def latent_gather(dst: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, slot: int, lo: int, page_size: int,
                  status: Optional[torch.Tensor], first: Optional[int] = None, last: Optional[int] = None) -> None:
    """dst [n, width]: row j = the cached row of position lo + j of the request in ``slot``, for positions
    ``first .. last`` (default: all n); zeros for the others (padding of the run)."""
    _need_cuda(dst, cache, block_table)
    _need(dst.is_contiguous() and dst.dtype == cache.dtype and dst.shape[1] == cache.shape[-1], "latent_gather: dst")
    row = block_table[slot]
    first = lo if first is None else first
    last = lo + dst.shape[0] - 1 if last is None else last
    load_library("latent_attn").call(
        "ll_latent_gather", c_int(_dtype_code(dst)), _ptr(dst), _ptr(cache), _ptr(row), c_int(lo), c_int(first),
        c_int(last), c_int(dst.shape[0]), c_int(dst.shape[1]), c_int(page_size), c_int(cache.shape[0]), _ptr(status),
        _stream())


def latent_masked_softmax(P: torch.Tensor, S: torch.Tensor, H: int, p0: int, lo: int, window: Optional[int],
                          scale: float, sink: Optional[torch.Tensor] = None) -> None:
    """P = softmax(scale * S) over the keys each row may see, zero elsewhere.  Row i is query position
    p0 + i // H; column j is key position lo + j; a query at p sees max(lo, p - window + 1) .. p."""
    _need_cuda(P, S)
    _f32(S, "S")
    _need(P.is_contiguous() and tuple(P.shape) == tuple(S.shape), "latent_masked_softmax: shapes")
    load_library("latent_attn").call(
        "ll_latent_masked_softmax", c_int(_dtype_code(P)), _ptr(P), _ptr(S), c_int(S.shape[0]), c_int(S.shape[1]),
        c_int(H), c_int(p0), c_int(lo), c_int(window or 0), c_float(scale), _ptr(sink), _stream())


def batched_heads(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
                  out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Library batched product over heads: a [H, n, k] times b [H, k, m] (any strides a BLAS takes); float32
    operands give a true float32 product, bfloat16 operands accumulate in float32."""
    if a.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("TF32 is on; call ops.configure_matmul_precision() before a float32 product")
    if out is not None:
        return torch.bmm(a, b, out=out)
    if out_dtype is not None and out_dtype != a.dtype:
        return torch.bmm(a, b, out_dtype=out_dtype)
    return torch.bmm(a, b)


def product(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Library product a [n, k] times b [k, m] (b not transposed, any row stride): true float32 for float32
    operands, float32 accumulation for bfloat16 ones."""
    _need_cuda(a, b, out)
    if a.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("TF32 is on; call ops.configure_matmul_precision() before a float32 product")
    return torch.mm(a, b, out=out) if out is not None else torch.mm(a, b)


# --------------------------------------------------------------------------
# routed feed-forward
# --------------------------------------------------------------------------
MOE_SCORE = {"softmax": 0, "sigmoid": 1, "softmax_top": 2}
MOE_ACT = {"relu2": 0, "silu": 1, "gelu_tanh": 2, "gelu": 3}
MOE_ACT_WEIGHT_IN = 16     # added to an activation's code: the expert's weight multiplies the activation's input


def moe_router(x: torch.Tensor, w_router: torch.Tensor, gates: torch.Tensor, top_idx: torch.Tensor,
               top_w: torch.Tensor, top: int, score: str = "softmax", renormalize: bool = False,
               bias: Optional[torch.Tensor] = None, shared_w: Optional[torch.Tensor] = None) -> None:
    """Scores over the experts in float32 and the ``top`` largest: ``gates`` float32 [tokens, E] (zero where an
    expert was not chosen), ``top_idx`` int32 and ``top_w`` float32 [tokens, top].  ``score`` "softmax_top": the
    largest logits are chosen and weighted by the softmax over the chosen ones.  ``bias`` float32 [E] is added to
    the logits.  With ``shared_w`` float32 [tokens], ``w_router`` has one more row and shared_w = sigmoid of it."""
    _need_cuda(x, w_router, gates, top_idx, top_w, bias, shared_w)
    _f32(bias, "router bias")
    _f32(shared_w, "shared_w")
    _f32(w_router, "router weight")
    _f32(gates, "gates")
    _f32(top_w, "top_w")
    _i32(top_idx, "top_idx")
    E, hidden = w_router.shape
    if shared_w is not None:
        E -= 1
    _need(E == gates.shape[1] and (bias is None or bias.numel() == E), "moe_router: experts")
    _need(E <= 256, f"moe_router: {E} experts are more than the kernel takes (256)")
    _need(x.stride(1) == 1 and x.shape[1] == hidden, "moe_router: x rows")
    load_library("moe").call(
        "ll_moe_router", c_int(_dtype_code(x)), _ptr(x), c_long(x.stride(0)), _ptr(w_router), _ptr(bias), _ptr(gates),
        _ptr(top_idx), _ptr(top_w), _ptr(shared_w), c_int(x.shape[0]), c_int(hidden), c_int(E), c_int(top),
        c_int(MOE_SCORE[score]), c_int(1 if renormalize else 0), _stream())


def moe_gated_act(h: torch.Tensor, gates: torch.Tensor, shared_w: Optional[torch.Tensor], shared_ff: int, ff: int,
                  E: int, limit: float, shared_limit: float, alpha: float) -> torch.Tensor:
    """[tokens, shared_ff + E * ff] from the first product over all experts' gate and up rows
    [tokens, 2 * (shared_ff + E * ff)]: a * sigmoid(alpha a) * (c + 1) with a = min(gate, limit),
    c = clamp(up, -limit, limit), times the expert's weight for the token (``shared_w`` for the always-on one)."""
    _need_cuda(h, gates, shared_w)
    _f32(gates, "gates")
    _f32(shared_w, "shared_w")
    width = shared_ff + E * ff
    _need(h.is_contiguous() and h.shape[1] == 2 * width, "moe_gated_act: h is [tokens, 2 * (shared + experts * ff)]")
    out = torch.empty((h.shape[0], width), dtype=h.dtype, device=h.device)
    load_library("moe").call("ll_moe_gated_act", c_int(_dtype_code(h)), _ptr(out), _ptr(h), _ptr(gates), _ptr(shared_w),
                             c_int(h.shape[0]), c_int(shared_ff), c_int(ff), c_int(E), c_float(limit),
                             c_float(shared_limit), c_float(alpha), c_int(sm_count(h.device)), _stream())
    return out


def moe_row_gated_act(h: torch.Tensor, row_w: Optional[torch.Tensor], limit: float, alpha: float) -> torch.Tensor:
    """[rows, ff] from [rows, 2 * ff] (gate columns, then up columns): the gated activation times the row's weight."""
    _need_cuda(h, row_w)
    _f32(row_w, "row_w")
    _need(h.is_contiguous() and h.shape[1] % 2 == 0 and (row_w is None or row_w.numel() == h.shape[0]),
          "moe_row_gated_act: layout")
    ff = h.shape[1] // 2
    out = torch.empty((h.shape[0], ff), dtype=h.dtype, device=h.device)
    load_library("moe").call("ll_moe_row_gated_act", c_int(_dtype_code(h)), _ptr(out), _ptr(h), _ptr(row_w),
                             c_int(h.shape[0]), c_int(ff), c_float(limit), c_float(alpha), c_int(sm_count(h.device)),
                             _stream())
    return out


def moe_act(h: torch.Tensor, gates: torch.Tensor, shared_ff: int, ff: int, E: int, act: str,
            weight_in: bool = False) -> None:
    """In place on the first product over all experts' rows: activation times the expert's weight for the token
    (``weight_in``: the activation of the weight times the unit, i.e. the expert works on the weighted row)."""
    _need_cuda(h, gates)
    _f32(gates, "gates")
    _need(h.stride(1) == 1 and h.stride(0) == h.shape[1] and h.shape[1] == shared_ff + E * ff,
          "moe_act: h is [tokens, shared + experts * ff]")
    load_library("moe").call("ll_moe_act", c_int(_dtype_code(h)), _ptr(h), _ptr(gates), c_int(h.shape[0]),
                             c_int(shared_ff), c_int(ff), c_int(E),
                             c_int(MOE_ACT[act] + (MOE_ACT_WEIGHT_IN if weight_in else 0)), c_int(sm_count(h.device)),
                             _stream())


def moe_sort(top_idx: torch.Tensor, top_w: torch.Tensor, E: int):
    """The (token, chosen expert) pairs in the order of the experts, decided on the device: ``ends`` int32 [E]
    (end of every expert's run of rows), ``row_token`` int32 and ``row_w`` float32 [pairs + E] (every run starts
    with a row of weight 0 that no pair points at, so no run is empty), ``pair_row`` int32 [tokens, top] (the row
    of every pair)."""
    _need_cuda(top_idx, top_w)
    _i32(top_idx, "top_idx")
    _f32(top_w, "top_w")
    n, top = top_idx.shape
    dev = top_idx.device
    ends = torch.empty(E, dtype=torch.int32, device=dev)
    row_token = torch.empty(n * top + E, dtype=torch.int32, device=dev)
    row_w = torch.empty(n * top + E, dtype=torch.float32, device=dev)
    pair_row = torch.empty((n, top), dtype=torch.int32, device=dev)
    load_library("moe").call("ll_moe_sort", _ptr(top_idx), _ptr(top_w), c_int(n), c_int(top), c_int(E), _ptr(ends),
                             _ptr(row_token), _ptr(row_w), _ptr(pair_row), _stream())
    return ends, row_token, row_w, pair_row


def moe_gather_rows(x: torch.Tensor, row_token: torch.Tensor) -> torch.Tensor:
    """[rows, hidden]: x[row_token[row]]."""
    _need_cuda(x, row_token)
    _i32(row_token, "row_token")
    _need(x.stride(1) == 1, "moe_gather_rows: x rows")
    out = torch.empty((row_token.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    load_library("moe").call("ll_moe_gather_rows", c_int(_dtype_code(x)), _ptr(out), _ptr(x), c_long(x.stride(0)),
                             _ptr(row_token), c_int(row_token.numel()), c_int(x.shape[1]), _stream())
    return out


def moe_row_act(h: torch.Tensor, row_w: torch.Tensor, act: str, weight_in: bool = False) -> None:
    """In place: activation of every row times the row's routing weight (``weight_in``: of the row times it)."""
    _need_cuda(h, row_w)
    _f32(row_w, "row_w")
    _need(h.is_contiguous() and row_w.numel() == h.shape[0], "moe_row_act: layout")
    load_library("moe").call("ll_moe_row_act", c_int(_dtype_code(h)), _ptr(h), _ptr(row_w), c_int(h.shape[0]),
                             c_int(h.shape[1]), c_int(MOE_ACT[act] + (MOE_ACT_WEIGHT_IN if weight_in else 0)),
                             c_int(sm_count(h.device)), _stream())


def moe_combine(base: Optional[torch.Tensor], y: torch.Tensor, pair_row: torch.Tensor) -> torch.Tensor:
    """[tokens, hidden]: base + the rows of a token's pairs, added in the order of the pairs (float32 sums)."""
    _need_cuda(base, y, pair_row)
    _i32(pair_row, "pair_row")
    n, top = pair_row.shape
    _need(y.is_contiguous() and (base is None or (base.is_contiguous() and base.dtype == y.dtype
                                                  and tuple(base.shape) == (n, y.shape[1]))), "moe_combine: layout")
    out = torch.empty((n, y.shape[1]), dtype=y.dtype, device=y.device)
    load_library("moe").call("ll_moe_combine", c_int(_dtype_code(y)), _ptr(out), _ptr(base), _ptr(y), _ptr(pair_row),
                             c_int(n), c_int(top), c_int(y.shape[1]), _stream())
    return out


def grouped_product(rows: torch.Tensor, weights: torch.Tensor, ends: torch.Tensor) -> torch.Tensor:
    """Library grouped product: rows [total, k] cut into runs that end at ``ends`` [groups] (int32, on the
    device), run g times weights[g] [n, k] transposed; bfloat16 with float32 accumulation."""
    _need_cuda(rows, weights, ends)
    _i32(ends, "ends")
    _need(rows.dtype == torch.bfloat16 and weights.dtype == torch.bfloat16 and weights.dim() == 3,
          "grouped_product: bfloat16 rows and weights [groups, n, k]")
    return torch.nn.functional.grouped_mm(rows, weights.transpose(1, 2), offs=ends)


def grouped_product_available() -> bool:
    return hasattr(torch.nn.functional, "grouped_mm")


# --------------------------------------------------------------------------
# a residual of several streams, and the norm that reads it
# --------------------------------------------------------------------------
def embed_streams(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, streams: int,
                  status: Optional[torch.Tensor]) -> None:
    """out [tokens, streams * hidden] float32: every stream starts as the token's table row."""
    _need_cuda(out, table, ids)
    _i32(ids, "ids")
    _f32(out, "out")
    hidden = table.shape[1]
    _need(table.is_contiguous() and out.shape[1] == streams * hidden and out.shape[0] >= ids.numel(),
          "embed_streams: shapes")
    load_library("streams").call("ll_embed_streams", c_int(_dtype_code(table)), _ptr(out), _ptr(table), _ptr(ids),
                                 c_int(ids.numel()), c_int(hidden), c_int(table.shape[0]), c_int(streams),
                                 _ptr(status), _stream())


def stream_tanh_norm(out: torch.Tensor, X: torch.Tensor, streams: int, alpha: torch.Tensor, weight: torch.Tensor,
                     bias: Optional[torch.Tensor], read: Optional[torch.Tensor] = None,
                     y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                     write: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """One pass over a residual of ``streams`` rows a token (X float32 [tokens, streams * hidden]): a pending
    sublayer output ``y`` is written back first, X[t] <- sum_s mix[s, t] X[s] + write[t] y (stored unless ``rows``
    selects rows), then out = tanh(alpha * sum_s read[s] X[s]) * weight + bias in ``out``'s dtype (``read`` None:
    all ones).  ``y`` may be [tokens, hidden] of out's dtype or float32 partial sums [parts, tokens, hidden]."""
    _need_cuda(out, X, alpha, weight, bias, read, y, mix, write, rows)
    for t, nm in ((X, "X"), (alpha, "alpha"), (weight, "weight"), (bias, "bias"), (read, "read"), (mix, "mix"),
                  (write, "write")):
        _f32(t, nm)
    _i32(rows, "rows")
    hidden = weight.numel()
    _need(X.dim() == 2 and X.shape[1] == streams * hidden, "stream_tanh_norm: X is [tokens, streams * hidden]")
    n_out = rows.numel() if rows is not None else X.shape[0]
    _need(out.is_contiguous() and out.shape[0] >= n_out and out.shape[1] == hidden, "stream_tanh_norm: out shape")
    _need((mix is None) == (write is None) and (y is None or mix is not None), "stream_tanh_norm: y comes with mix, write")
    _need(mix is None or (mix.numel() == streams * streams and write.numel() == streams), "stream_tanh_norm: mix, write")
    _need(read is None or read.numel() == streams, "stream_tanh_norm: read")
    parts, part_stride, y2, yp = 0, 0, None, None
    if y is not None and y.dim() == 3:
        _need(y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape[1:]) == (X.shape[0], hidden),
              "stream_tanh_norm: partial sums are float32 [parts, tokens, hidden]")
        parts, part_stride, yp = y.shape[0], y.shape[1] * hidden, y
    elif y is not None:
        _need(y.dtype == out.dtype and y.is_contiguous() and tuple(y.shape) == (X.shape[0], hidden),
              "stream_tanh_norm: y is [tokens, hidden] of the output's dtype")
        y2 = y
    load_library("streams").call(
        "ll_stream_tanh_norm", c_int(_dtype_code(out)), _ptr(out), _ptr(X), _ptr(y2), _ptr(yp), c_int(parts),
        c_long(part_stride), _ptr(mix), _ptr(write), _ptr(read), _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(rows),
        c_int(1 if rows is None else 0), c_int(streams), c_int(hidden), c_int(n_out), _stream())


def stream_sum(X: torch.Tensor, streams: int) -> torch.Tensor:
    """float32 [tokens, hidden]: the sum of a token's streams."""
    _need_cuda(X)
    _f32(X, "X")
    hidden = X.shape[1] // streams
    out = torch.empty((X.shape[0], hidden), dtype=torch.float32, device=X.device)
    load_library("streams").call("ll_stream_sum", _ptr(out), _ptr(X), c_int(X.shape[0]), c_int(streams), c_int(hidden),
                                 _stream())
    return out


# --------------------------------------------------------------------------
# linear attention with a decay per head
# --------------------------------------------------------------------------
def silu_rows(x: torch.Tensor) -> None:
    """x <- silu(x) in place (x may be a slice of columns of a wider matrix); float32 arithmetic, one rounding."""
    _need_cuda(x)
    _need(x.dim() == 2 and x.stride(1) == 1, "silu_rows: rows with unit column stride")
    load_library("linear_attn").call("ll_silu_rows", c_int(_dtype_code(x)), _ptr(x), c_long(x.stride(0)),
                                     c_int(x.shape[0]), c_int(x.shape[1]), c_int(sm_count(x.device)), _stream())


def decay_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: Optional[torch.Tensor],
               state: torch.Tensor, step, o: torch.Tensor, H: int, dk: int, dv: int, write_state: bool = True,
               heads_per_group: int = 1, token_decay: Optional[torch.Tensor] = None,
               token_scale: Optional[torch.Tensor] = None, skip: Optional[torch.Tensor] = None) -> None:
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t for every entry's tokens in order; q, k, v are the
    columns of ``proj`` at the three offsets (already activated); ``state`` float32 [slots, >= H * dv * dk] goes on
    from where the request stopped; ``o`` float32 [tokens, H * dv].
    A state-space layer uses the same scan: ``token_decay`` and ``token_scale`` float32 [tokens, H] give every
    token's decay and the factor on what it writes (S_t = a_t S_(t-1) + dt_t k_t v_t^T), ``skip`` float32 [H] adds
    skip_h v_t to the read-out, and the ``heads_per_group`` heads of a group read the same q and k."""
    _need_cuda(proj, decay, state, o, token_decay, token_scale, skip)
    _f32(decay, "decay")
    _f32(state, "state")
    _f32(o, "o")
    for t_, nm in ((token_decay, "token_decay"), (token_scale, "token_scale"), (skip, "skip")):
        _f32(t_, nm)
    _need(decay is not None or token_decay is not None, "decay_scan: a decay a head or a token is needed")
    _need(all(t_ is None or (t_.is_contiguous() and tuple(t_.shape) == (proj.shape[0], H))
              for t_ in (token_decay, token_scale)), "decay_scan: token_decay and token_scale are [tokens, H]")
    _need(proj.stride(1) == 1 and dk <= 256 and (decay is None or decay.numel() == H)
          and (skip is None or skip.numel() == H) and state.shape[1] >= H * dk * dv
          and o.shape[1] == H * dv and o.is_contiguous() and H % heads_per_group == 0,
          "decay_scan: shapes (key heads of at most 256 channels)")
    load_library("linear_attn").call(
        "ll_decay_scan", c_int(_dtype_code(proj)), _ptr(proj), c_long(proj.stride(0)), c_int(q_off), c_int(k_off),
        c_int(v_off), _ptr(decay), _ptr(state), c_long(state.stride(0)), c_int(state.shape[0]), _ptr(step.cu_q),
        _ptr(step.req_slot), _ptr(o), c_int(step.num_entries), c_int(H), c_int(dk), c_int(dv),
        c_int(1 if write_state else 0), _ptr(step.status), c_int(heads_per_group), _ptr(token_decay),
        _ptr(token_scale), _ptr(skip), _stream())


def ssd_prepare(proj: torch.Tensor, x_off: int, dt_off: int, conv_w: torch.Tensor, conv_b: Optional[torch.Tensor],
                A_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, tail_off: int, step,
                xbc: torch.Tensor, dt: torch.Tensor, decay: torch.Tensor, write_state: bool = True) -> None:
    """The pieces of a state-space layer before its scan, a token: the causal convolution (+ bias) and SiLU of the
    ``C`` channels of ``proj`` at ``x_off`` into ``xbc`` float32 [tokens, C], continuing from the last taps - 1
    inputs that the request's record holds at ``tail_off``; dt = softplus(proj[dt_off + h] + dt_bias[h]) and
    decay = exp(-exp(A_log[h]) dt) into float32 [tokens, H].  Then (a second launch) the records' tails are
    brought up to date.  ``conv_w`` float32 [C, taps]."""
    _need_cuda(proj, conv_w, conv_b, A_log, dt_bias, state, xbc, dt, decay)
    for t_, nm in ((conv_w, "conv_w"), (conv_b, "conv_b"), (A_log, "A_log"), (dt_bias, "dt_bias"), (state, "state"),
                   (xbc, "xbc"), (dt, "dt"), (decay, "decay")):
        _f32(t_, nm)
    C, taps = conv_w.shape
    H = A_log.numel()
    n = proj.shape[0]
    _need(proj.stride(1) == 1 and conv_w.is_contiguous() and (conv_b is None or conv_b.numel() == C)
          and dt_bias.numel() == H and xbc.is_contiguous() and tuple(xbc.shape) == (n, C)
          and dt.is_contiguous() and decay.is_contiguous() and tuple(dt.shape) == tuple(decay.shape) == (n, H)
          and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= tail_off + (taps - 1) * C,
          "ssd_prepare: shapes")
    load_library("ssd").call(
        "ll_ssd_prepare", c_int(_dtype_code(proj)), _ptr(proj), c_long(proj.stride(0)), c_int(x_off), c_int(dt_off),
        _ptr(conv_w), _ptr(conv_b), _ptr(A_log), _ptr(dt_bias), _ptr(state), c_long(state.stride(0)), c_long(tail_off),
        c_int(state.shape[0]), _ptr(step.token_req), _ptr(step.cu_q), _ptr(step.req_slot), _ptr(xbc), _ptr(dt),
        _ptr(decay), c_int(n), c_int(step.num_entries), c_int(C), c_int(H), c_int(taps),
        c_int(1 if write_state else 0), _ptr(step.status), _stream())


def ssd_gated_norm(out: torch.Tensor, y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float,
                   parts: int) -> None:
    """out = u / rms(u) * weight over each of ``parts`` equal parts of the row, u = y * silu(z); ``y`` float32
    [tokens, width], ``z`` (a view of the projection's rows) and ``out`` in the engine's dtype."""
    _need_cuda(out, y, z, weight)
    _f32(y, "y")
    _f32(weight, "weight")
    width = y.shape[1]
    _need(y.is_contiguous() and z.stride(1) == 1 and out.stride(1) == 1 and z.dtype == out.dtype
          and tuple(z.shape) == tuple(out.shape) == tuple(y.shape) and weight.numel() == width and width % parts == 0,
          "ssd_gated_norm: shapes")
    load_library("ssd").call("ll_ssd_gated_norm", c_int(_dtype_code(out)), _ptr(out), c_long(out.stride(0)), _ptr(y),
                             _ptr(z), c_long(z.stride(0)), _ptr(weight), c_float(eps), c_int(y.shape[0]), c_int(width),
                             c_int(parts), _stream())


def linear_attn_out(y: torch.Tensor, o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, eps: float) -> None:
    """y = o / rms(o over the whole row) * weight * sigmoid(gate), in y's dtype."""
    _need_cuda(y, o, weight, gate)
    _f32(o, "o")
    _f32(weight, "weight")
    n, width = o.shape
    _need(y.is_contiguous() and tuple(y.shape) == (n, width) and gate.stride(1) == 1 and gate.shape[1] == width
          and gate.dtype == y.dtype and weight.numel() == width, "linear_attn_out: shapes")
    load_library("linear_attn").call("ll_linear_attn_out", c_int(_dtype_code(y)), _ptr(y), _ptr(o), _ptr(weight),
                                     _ptr(gate), c_long(gate.stride(0)), c_float(eps), c_int(n), c_int(width),
                                     _stream())


# --------------------------------------------------------------------------
# a norm on the sublayer's output, a plain feed-forward's activation, scaled logits
# --------------------------------------------------------------------------
def layernorm_into_residual(residual: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                            copy: Optional[torch.Tensor]) -> None:
    """residual (float32) += layer norm of y times ``weight``; ``copy`` (optional) receives the new residual rows
    rounded to its dtype.  ``y`` is [tokens, hidden] of the engine's dtype or float32 partial sums
    [parts, tokens, hidden] of a product split over its inner dimension (added up unrounded)."""
    _need_cuda(residual, y, weight, copy)
    _f32(residual, "residual")
    _f32(weight, "norm weight")
    n, hidden = residual.shape
    _need(weight.numel() == hidden, "layernorm_into_residual: weight size")
    _need(copy is None or (copy.is_contiguous() and tuple(copy.shape) == (n, hidden)),
          "layernorm_into_residual: copy shape")
    if y.dim() == 3:
        _need(y.dtype == torch.float32 and y.is_contiguous() and tuple(y.shape[1:]) == (n, hidden),
              "layernorm_into_residual: partial sums are float32 [parts, tokens, hidden]")
        dt = _dtype_code(copy) if copy is not None else 0
        core().call("ll_layernorm_into_residual", c_int(dt), _ptr(copy), _ptr(residual), c_void_p(0), _ptr(y),
                    c_int(y.shape[0]), c_long(n * hidden), _ptr(weight), c_float(eps), c_int(n), c_int(hidden),
                    _stream())
        return
    _need(y.is_contiguous() and tuple(y.shape) == (n, hidden) and (copy is None or copy.dtype == y.dtype),
          "layernorm_into_residual: y is [tokens, hidden] of the copy's dtype")
    core().call("ll_layernorm_into_residual", c_int(_dtype_code(y)), _ptr(copy), _ptr(residual), _ptr(y), c_void_p(0),
                c_int(0), c_long(0), _ptr(weight), c_float(eps), c_int(n), c_int(hidden), _stream())


def round_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A float32 residual stream rounded to ``dtype``, as a product's operand (float32: the rows themselves)."""
    _need_cuda(x)
    _f32(x, "x")
    if dtype == torch.float32:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    core().call("ll_round_rows", c_int(_dtype_code(out)), _ptr(out), _ptr(x), c_long(x.numel()), _stream())
    return out


ROW_ACT = {"gelu_tanh": 0, "relu": 1, "silu": 2, "relu2": 3}


def linear_act(x: torch.Tensor, weight: torch.Tensor, act: str) -> torch.Tensor:
    """act(x @ weight.T) for a feed-forward without a gate (``act`` of ``ROW_ACT``).  In bfloat16 the activation is
    the epilogue of the product where a kernel of this package makes it: the weight-streaming one for a few tokens
    (units of 64 features, k whole), the two-SM tcgen05 one for many.  Else a product and ``act_rows``."""
    _need_cuda(x, weight)
    if (x.dtype == torch.bfloat16 and x.shape[0] <= STREAM_M and stream_mode(x, weight) == 0
            and not (weight.shape[0] >= 8192 and tc_preferred(x, weight, wide=True))):
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        return gemm_stream(x, weight, out, 0, row_act=act)
    if TC_ENABLED and x.shape[0] >= PAIR_MIN_M and pair_supported(x, weight):
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        return gemm_pair(x, weight, out, row_act=act)
    out = linear(x, weight)
    act_rows(out, act)
    return out


def act_rows(x: torch.Tensor, act: str) -> None:
    """x <- act(x) in place (float32 arithmetic, one rounding): the activation of a feed-forward without a gate."""
    _need_cuda(x)
    _need(x.is_contiguous(), "act_rows: x must be contiguous")
    core().call("ll_act_rows", c_int(_dtype_code(x)), _ptr(x), c_long(x.numel()), c_int(ROW_ACT[act]), _stream())


def scale_logits(logits: torch.Tensor, factor: float) -> None:
    """logits <- logits * factor in place (float32)."""
    _need_cuda(logits)
    _f32(logits, "logits")
    core().call("ll_scale_f32", _ptr(logits), c_long(logits.numel()), c_float(factor), _stream())


# --------------------------------------------------------------------------
# attention with normalised q, k, v and shaped scores
# --------------------------------------------------------------------------
QK_NORM = {None: 0, "none": 0, "head_unit": 1, "projection": 2}
ATTN_MASK = {"causal": 0, "window": 1, "chunk": 2}


def qkv_norm_rotate_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
                          freq: Optional[torch.Tensor], amplitude: float, interleaved: bool, num_heads: int,
                          num_kv_heads: int, head_dim: int, value_head_dim: int, qk_norm: Optional[str],
                          q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], value_norm: bool,
                          eps: float, slot_map: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], page_size: int, status: Optional[torch.Tensor],
                          head_mix: Optional[torch.Tensor] = None, mix_temperature: Optional[torch.Tensor] = None,
                          mixed_q: Optional[torch.Tensor] = None) -> None:
    """Bias, the norms of q, k and v (``qk_norm``: "projection": an RMS norm with weights over all of q and all of
    k before the rotation; "head_unit": every head divided by its root mean square after it; ``value_norm``: the
    same for every value head), the rotation by angles made in the kernel (cos and sin times ``amplitude``), and
    the store of k and v.  In place on the first (nh + nkv) * head_dim + nkv * value_head_dim columns of ``qkv``.
    With ``head_mix`` [nh, nh] and ``mixed_q`` [tokens, nh * nkv * head_dim] also the queries of an attention that
    mixes its heads' scores, as one wider query a head over all kv heads' keys side by side (``attn_shaped``)."""
    _need_cuda(qkv, bias, positions, freq, q_weight, k_weight, slot_map, k_cache, v_cache, head_mix, mix_temperature,
               mixed_q)
    _f32(head_mix, "head_mix")
    _f32(mix_temperature, "mix_temperature")
    if mixed_q is not None:
        _need(head_mix is not None and tuple(head_mix.shape) == (num_heads, num_heads) and head_mix.is_contiguous(),
              "mixed queries need head_mix [heads, heads]")
        _need(mixed_q.dtype == qkv.dtype and mixed_q.is_contiguous()
              and tuple(mixed_q.shape) == (qkv.shape[0], num_heads * num_kv_heads * head_dim), "mixed_q shape")
    for t, nm in ((bias, "bias"), (freq, "freq"), (q_weight, "q norm weight"), (k_weight, "k norm weight")):
        _f32(t, nm)
    _i32(positions, "positions")
    _i32(slot_map, "slot_map")
    width = (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_head_dim
    _need(qkv.dim() == 2 and qkv.shape[1] >= width and qkv.stride(1) == 1, "qkv must be [tokens, >= (nh+nkv)*hd + nkv*vd]")
    _need(bias is None or bias.numel() == width, "bias size")
    mode = QK_NORM[qk_norm]
    if mode == 2:
        _need(q_weight is not None and q_weight.numel() == num_heads * head_dim and k_weight is not None
              and k_weight.numel() == num_kv_heads * head_dim, "projection norm: weights over all of q and all of k")
    rot_dim = 0 if freq is None else 2 * freq.numel()
    _need(rot_dim <= head_dim, "rotation: rot_dim <= head_dim")
    num_slots = 0
    if slot_map is not None:
        _need(k_cache is not None and v_cache is not None, "store needs the cache plane")
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype, "cache dtype differs from activations")
        _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
        _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
              and tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, value_head_dim), "cache plane shape")
        num_slots = k_cache.shape[0] * page_size
    load_library("attn_mod").call(
        "ll_qkv_norm_rotate_store", c_int(_dtype_code(qkv)), _ptr(qkv), c_long(qkv.stride(0)), _ptr(bias),
        _ptr(positions), _ptr(freq), c_int(rot_dim), c_float(amplitude), c_int(1 if interleaved else 0),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(value_head_dim), c_int(mode), _ptr(q_weight),
        _ptr(k_weight), c_int(1 if value_norm else 0), c_float(eps), _ptr(slot_map), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), c_long(num_slots), c_int(qkv.shape[0]), _ptr(head_mix if mixed_q is not None else None),
        _ptr(mix_temperature), _ptr(mixed_q), _ptr(status), _stream())


def attn_shaped_supported(dtype: torch.dtype, num_kv_heads: int, head_dim: int, value_head_dim: int, page_size: int,
                          q_stride: int, mixed: bool) -> bool:
    """Whether the tensor-core attention with shaped scores takes this shape (else ``attention_modulated``)."""
    if not (dtype == torch.bfloat16 and head_dim in (64, 128) and value_head_dim in (64, 128)
            and page_size % 16 == 0 and q_stride % 8 == 0):
        return False
    stage = 2 * 64 * (num_kv_heads if mixed else 1) * head_dim * 2 + 2 * 64 * value_head_dim * 2
    return stage <= 200 * 1024


def attn_shaped_blocks(q_lens, group: int) -> int:
    """Row blocks of these entries for ``attn_shaped``: a CTA takes 128 (token, head of the group) rows of one entry."""
    return sum((int(n) * group + 127) // 128 for n in q_lens)


def attn_shaped(out: torch.Tensor, q: torch.Tensor, q_stride: int, mixed: bool, gate: Optional[torch.Tensor],
                temperature: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor,
                block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor, req_slot: torch.Tensor,
                num_entries: int, row_blocks: int, num_heads: int, num_kv_heads: int, head_dim: int,
                value_head_dim: int, page_size: int, mask: str, mask_size: Optional[int], sink: bool, scale: float,
                status: Optional[torch.Tensor], nsplit: int = 1, span: int = 1,
                sink_values: Optional[torch.Tensor] = None, distance_bias: Optional[torch.Tensor] = None,
                keep_first: int = 0, softcap: Optional[float] = None,
                query_temperature: Optional[Tuple[float, int]] = None, gate_channels: bool = False,
                out_scale: float = 1.0) -> None:
    """Tensor-core paged attention (bfloat16) with shaped scores: the mechanisms of ``attention_modulated`` for
    head sizes 64 and 128.  ``q``: the projection's rows (head h at h * head_dim), or with ``mixed`` the wider
    queries that ``qkv_norm_rotate_store`` leaves for mixed heads (then ``temperature`` is inside them).
    ``nsplit`` > 1 (every entry brings one token): the keys of a row are cut into parts of ``span`` stages of 64
    keys, each a CTA, joined by a second kernel; nsplit * span must cover the stages any token sees (kept first
    tokens' stages before the window's are walked by the first part besides).  ``sink_values``, ``distance_bias``,
    ``keep_first``, ``softcap``, ``query_temperature``, ``gate_channels`` and ``out_scale`` are those of
    ``attention_modulated``.  Launches one kernel, two with ``nsplit`` > 1."""
    _need_cuda(out, q, gate, temperature, k_cache, v_cache, block_table, cu_q, ctx_len, req_slot, sink_values,
               distance_bias)
    _f32(sink_values, "sink_values")
    _f32(distance_bias, "distance_bias")
    _need(sink_values is None or (sink and sink_values.numel() == num_heads), "sink_values: a number a head")
    _need(distance_bias is None or (distance_bias.dim() == 2 and distance_bias.shape[1] == num_heads
                                    and distance_bias.is_contiguous()), "distance_bias is [distances, heads]")
    qt_coef, qt_every = (0.0, 0) if query_temperature is None else (float(query_temperature[0]), int(query_temperature[1]))
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_len, "ctx_len"), (req_slot, "req_slot")):
        _i32(t, nm)
    _f32(temperature, "temperature")
    _need(attn_shaped_supported(q.dtype, num_kv_heads, head_dim, value_head_dim, page_size, q_stride, mixed),
          "attn_shaped takes bfloat16, head sizes 64 and 128 and pages of a multiple of 16 tokens")
    _need(out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16,
          "attn_shaped: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * value_head_dim and out.stride(0) % 8 == 0,
          "attn_shaped: out")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
          and tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, value_head_dim), "cache plane shape")
    _need(cu_q.numel() >= num_entries + 1 and ctx_len.numel() >= num_entries and req_slot.numel() >= num_entries,
          "attn_shaped: entry arrays too short")
    _need(temperature is None or temperature.numel() == num_heads, "temperature: a number a head")
    _need(gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1
                           and gate.shape[1] == (num_heads * value_head_dim if gate_channels else num_heads)),
          "gate: [tokens, heads] rows (or a number a channel)")
    _need(mask == "causal" or (mask_size or 0) > 0, "a window or chunks need a size")
    part = None
    if nsplit > 1:
        part = torch.empty((out.shape[0], num_heads, nsplit, value_head_dim + 2), dtype=torch.float32,
                           device=out.device)
    load_library("attn_shaped").call(
        "ll_attn_shaped", _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride), c_int(1 if mixed else 0),
        _ptr(gate), c_long(0 if gate is None else gate.stride(0)), _ptr(temperature), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(cu_q), _ptr(ctx_len), _ptr(req_slot),
        c_int(num_entries), c_int(row_blocks), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(value_head_dim), c_int(page_size), c_int(k_cache.shape[0]), c_int(ATTN_MASK[mask]),
        c_int(int(mask_size or 0)), c_int(1 if sink else 0), c_float(scale), c_int(nsplit), c_int(span), _ptr(part),
        _ptr(status), _ptr(sink_values), _ptr(distance_bias),
        c_int(0 if distance_bias is None else distance_bias.shape[0]), c_int(int(keep_first or 0)),
        c_float(float(softcap or 0.0)), c_float(qt_coef), c_int(qt_every), c_int(1 if gate_channels else 0),
        c_float(out_scale), _stream())


def attention_modulated(out: torch.Tensor, q: torch.Tensor, q_stride: int, gate: Optional[torch.Tensor],
                        k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                        token_req: torch.Tensor, req_slot: torch.Tensor, positions: torch.Tensor, num_tokens: int,
                        num_heads: int, num_kv_heads: int, head_dim: int, value_head_dim: int, page_size: int,
                        mask: str, mask_size: Optional[int], sink: bool, scale: float,
                        temperature: Optional[torch.Tensor], head_mix: Optional[torch.Tensor],
                        status: Optional[torch.Tensor], sink_values: Optional[torch.Tensor] = None,
                        distance_bias: Optional[torch.Tensor] = None, keep_first: int = 0,
                        softcap: Optional[float] = None, query_temperature: Optional[Tuple[float, int]] = None,
                        gate_channels: bool = False, out_scale: float = 1.0) -> None:
    """Attention of every new token over its request's cached keys with shaped scores (any sizes, both dtypes):
    a number a head on the scores (``temperature``), the heads' scores mixed by ``head_mix`` [nh, nh], a window
    or chunks (``mask``, ``mask_size``), one more key of score 0 without a value (``sink``), a sigmoid gate a
    head on the output (``gate``: a view whose element [t, h] is token t's gate input of head h).
    ``sink_values`` float32 [nh]: the score of the key without a value, a head.  ``distance_bias`` float32
    [distances, nh]: added to the score of a key ``min(n, distances - 1)`` positions back.  ``keep_first``: with a
    window, the request's first positions stay visible.  ``softcap``: s <- cap tanh(s / cap) before the bias.
    ``query_temperature`` (coef, every): the scores of the query at position p times
    1 + coef ln(floor((p + 1) / every) + 1).  ``gate_channels``: ``gate`` is [tokens, nh * vd], a gate a channel.
    ``out_scale``: a constant on the output, applied before its one rounding."""
    _need_cuda(out, q, gate, k_cache, v_cache, block_table, token_req, req_slot, positions, temperature, head_mix,
               sink_values, distance_bias)
    _f32(sink_values, "sink_values")
    _f32(distance_bias, "distance_bias")
    _need(sink_values is None or (sink and sink_values.numel() == num_heads), "sink_values: a number a head")
    _need(distance_bias is None or (distance_bias.dim() == 2 and distance_bias.shape[1] == num_heads
                                    and distance_bias.is_contiguous()), "distance_bias is [distances, heads]")
    for t, nm in ((block_table, "block_table"), (token_req, "token_req"), (req_slot, "req_slot"),
                  (positions, "positions")):
        _i32(t, nm)
    _f32(temperature, "temperature")
    _f32(head_mix, "head_mix")
    _need(num_heads % num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads")
    _need(out.dtype == q.dtype == k_cache.dtype == v_cache.dtype, "attention: dtypes differ")
    _need(out.stride(1) == 1 and out.shape[1] == num_heads * value_head_dim, "attention: out shape")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache plane must be contiguous")
    _need(tuple(k_cache.shape[1:]) == (num_kv_heads, page_size, head_dim)
          and tuple(v_cache.shape[1:]) == (num_kv_heads, page_size, value_head_dim), "cache plane shape")
    _need(temperature is None or temperature.numel() == num_heads, "temperature: a number a head")
    _need(head_mix is None or tuple(head_mix.shape) == (num_heads, num_heads), "head_mix is [heads, heads]")
    _need(gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1
                           and gate.shape[1] == (num_heads * value_head_dim if gate_channels else num_heads)),
          "gate: a number a head (or a channel) and token, rows of the projection's dtype")
    qt_coef, qt_every = (0.0, 0) if query_temperature is None else (float(query_temperature[0]), int(query_temperature[1]))
    load_library("attn_mod").call(
        "ll_attention_modulated", c_int(_dtype_code(out)), _ptr(out), c_long(out.stride(0)), _ptr(q), c_long(q_stride),
        _ptr(gate), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), c_int(block_table.stride(0)), _ptr(token_req),
        _ptr(req_slot), _ptr(positions), c_int(num_tokens), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(value_head_dim), c_int(page_size), c_int(k_cache.shape[0]), c_int(ATTN_MASK[mask]),
        c_int(int(mask_size or 0)), c_int(1 if sink else 0), c_float(scale), _ptr(temperature), _ptr(head_mix),
        _ptr(status), _ptr(sink_values), _ptr(distance_bias),
        c_int(0 if distance_bias is None else distance_bias.shape[0]), c_int(int(keep_first or 0)),
        c_float(float(softcap or 0.0)), c_float(qt_coef), c_int(qt_every),
        c_long(0 if gate is None else gate.stride(0)), c_int(1 if gate_channels else 0), c_float(out_scale),
        _stream())
