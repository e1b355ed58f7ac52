"""The reference project's operator names and signatures, backed by the CUDA kernels.

The reference wires its Llama decode path in by assignment: the attention hook
replaces ``transformers.models.llama.modeling_llama.eager_attention_forward``
(``condition_block_triton_impl/core.py:1372-1379``) and its own experiments
replace the functional operators the same way
(``condition_block_ball/run_latency.py:34``).  This module offers drop-ins for
those seams:

    _build_prompt_blocks(k_all, v_all, block_size)                    core.py:449-500
    _select_prompt_blocks(q_grouped, prefix, eps)                     core.py:503-555
    _run_condition_block_selection_stats(q_grouped, prefix, ...)      core.py:573-698
    _condition_block_decode_output_fused_triton(*, q_grouped, ...)    core.py:1035-1155
    ConditionBlockDecodeRunner / condition_block_decode_context       core.py:1203-1379

Conventions follow the reference: ``q_grouped`` is ``[Hkv, G, 1, D]``, the
prefix dict carries the same keys, errors are ``ValueError``.  Differences are
additive: every function also accepts ``top_k=`` (k best blocks instead of the
epsilon rule) and ``rep_mode=`` ("hybrid" is the reference behaviour), and the
runner accepts batches.  The K/V cache is never copied: a ``[Hkv, T, D]`` cache
view is addressed as 16-token pages with an identity block table.  All tensors
must live on a CUDA device; there is no CPU path.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib, ops
from ._lib import Geom, IA_REP_HYBRID, IA_REP_SPARSE_ONLY, IA_SELECT_EPS, IA_SELECT_TOPK, check

PAGE = 16
_REP = {"sparse_only": IA_REP_SPARSE_ONLY, "hybrid": IA_REP_HYBRID}


# --------------------------------------------------------------------------
# cache views as paged pools
# --------------------------------------------------------------------------

def _check_cache_view(x: torch.Tensor, name: str) -> None:
    if not x.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if x.dim() != 3 or x.stride(2) != 1 or x.stride(1) != x.shape[2]:
        raise ValueError(f"{name} must be a [Hkv, T, D] view whose [T, D] rows are contiguous")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"{name}: dtype {x.dtype} not supported (float32, bfloat16)")
    if (x.stride(0) * x.element_size()) % 16 != 0 or x.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: head stride and base address must be 16-byte aligned")


class _CacheGeometry:
    """A ``[Hkv, T, D]`` cache addressed as 16-token pages: page p of head h starts at
    ``base + h * head_stride + p * 16 * D`` - the pool layout of the C ABI with an
    identity block table.  Holds the small device tensors that description needs."""

    def __init__(self, device, max_tokens: int):
        self.device = device
        self.capacity_pages = 0
        self.table = None
        self.prefix_lens = torch.zeros((1,), dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros((1,), dtype=torch.int32, device=device)
        self.ensure(max_tokens)

    def ensure(self, max_tokens: int) -> None:
        need = (int(max_tokens) + PAGE - 1) // PAGE
        if need > self.capacity_pages:
            self.capacity_pages = max(need, 2 * self.capacity_pages, 64)
            self.table = torch.arange(self.capacity_pages, dtype=torch.int32, device=self.device).view(1, -1)

    def geom(self, k: torch.Tensor, group: int, block_size: int, max_blocks: int, summ=None,
             n_tokens: Optional[int] = None) -> Geom:
        """``k`` gives the base pointer and strides of the cache; ``n_tokens`` how many of its token rows
        exist behind that pointer (prefix + suffix) - pages past them are outside the pool."""
        n_tokens = int(k.shape[1]) if n_tokens is None else int(n_tokens)
        return Geom(batch=1, n_kv_heads=int(k.shape[0]), group_size=int(group), head_dim=int(k.shape[2]),
                    page_size=PAGE, block_size=int(block_size), max_pages=self.capacity_pages,
                    max_blocks=int(max_blocks), dtype=ops._DTYPES[k.dtype], reserved=ops._geom_flags(summ),
                    n_pool_pages=(n_tokens + PAGE - 1) // PAGE, reserved2=0,
                    pool_page_stride=PAGE * int(k.shape[2]), pool_head_stride=int(k.stride(0)))


class _PrefixHandle:
    """What the kernels need about one summarised prefix (kept in the prefix dict)."""

    def __init__(self, k_all, v_all, block_size, summ, geometry):
        self.k_all, self.v_all = k_all, v_all
        self.block_size = int(block_size)
        self.prompt_len = int(k_all.shape[1])
        self.summ = summ
        self.geometry = geometry


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# --------------------------------------------------------------------------
# _build_prompt_blocks
# --------------------------------------------------------------------------

def _build_prompt_blocks(k_all: torch.Tensor, v_all: torch.Tensor, block_size: int) -> Dict[str, object]:
    """Block summaries of a prompt.  Same keys as the reference's dict; k_bar is
    fp32, v_bar and the coordinate bounds are kept in the cache dtype (the
    reference's "mixed" storage) unless ``CONDITION_BLOCK_MIXED_SUMMARIES`` is
    unset, in which case fp32 copies are returned like the reference default.
    ``k_block_attn`` / ``v_block_attn`` are views of the cache when the prompt
    length is a multiple of the block size and zero-padded copies otherwise
    (as in the reference)."""
    _check_cache_view(k_all, "k_all")
    _check_cache_view(v_all, "v_all")
    if k_all.shape != v_all.shape or k_all.dtype != v_all.dtype or k_all.stride() != v_all.stride():
        raise ValueError("k_all and v_all must have the same shape, dtype and strides")
    block_size = int(block_size)
    if block_size % PAGE != 0 or not 0 < block_size <= 128:
        raise ValueError(f"block_size {block_size} must be a multiple of {PAGE}, at most 128")
    lib = _lib.load()
    hkv, length, d = (int(x) for x in k_all.shape)
    nb = max(1, (length + block_size - 1) // block_size)
    dev = k_all.device
    geometry = _CacheGeometry(dev, length)
    geometry.prefix_lens.fill_(length)
    geometry.seq_lens.fill_(length)
    # the reference's switch for the storage of k_bar (core.py:428-446): bf16 only next to bf16 K/V
    k_bar_name = os.environ.get("CONDITION_BLOCK_K_BAR_DTYPE", "float32")
    if k_bar_name not in ("float32", "bfloat16"):
        raise ValueError(f"CONDITION_BLOCK_K_BAR_DTYPE must be float32 or bfloat16, got {k_bar_name!r}.")
    if k_bar_name != "float32" and k_all.dtype != torch.bfloat16:
        raise ValueError("CONDITION_BLOCK_K_BAR_DTYPE=bfloat16 needs bfloat16 keys and values.")
    # the reference's switch for the packed coordinate range (core.py:490-499)
    packed = os.environ.get("CONDITION_BLOCK_TMA_BOUNDS") == "1"
    summ = ops.BlockSummaries.empty(1, hkv, nb, d, k_all.dtype, dev, block_size, getattr(torch, k_bar_name),
                                    packed_bounds=packed)
    g = geometry.geom(k_all, 1, block_size, nb, summ)
    s = summ.c_struct()
    check(lib.ia_build_summaries(ctypes.c_void_p(k_all.data_ptr()), ctypes.c_void_p(v_all.data_ptr()),
                                 ctypes.c_void_p(geometry.table.data_ptr()),
                                 ctypes.c_void_p(geometry.prefix_lens.data_ptr()),
                                 ctypes.byref(g), ctypes.byref(s), _stream()))
    n_real = (length + block_size - 1) // block_size
    token_idx = torch.arange(n_real * block_size, device=dev).reshape(n_real, block_size)
    valid_token = token_idx < length
    counts = valid_token.sum(dim=1).long()
    mixed = os.environ.get("CONDITION_BLOCK_MIXED_SUMMARIES") == "1"

    def stored(t):
        t = t[0, :, :n_real]
        return t if mixed else t.float()

    def blocked(x):
        pad = n_real * block_size - length
        if pad:
            x = torch.cat([x, x.new_zeros((hkv, pad, d))], dim=1)
        return x.reshape(hkv, n_real, block_size, d)

    v_norm_max = summ.v_norm_max[0, :, :n_real]
    prefix = {
        "k_block_attn": blocked(k_all), "v_block_attn": blocked(v_all),
        "token_idx": token_idx, "valid_token": valid_token,
        "k_bar": summ.k_bar[0, :, :n_real], "v_bar": stored(summ.v_bar),
        "k_max": stored(summ.k_max), "k_min": stored(summ.k_min),
        "v_norm_max": v_norm_max,
        "v_norm_all": v_norm_max.amax(dim=-1) if n_real else v_norm_max.new_zeros((hkv,)),
        "block_valid_counts": counts,
        "_b200": _PrefixHandle(k_all, v_all, block_size, summ, geometry),
    }
    if packed:  # as the reference: the packed array, and k_max / k_min as views into it (no duplicate storage)
        prefix["k_bounds"] = summ.k_bounds[0, :, :n_real]
        pairs = prefix["k_bounds"].view(hkv, n_real, d, 2)
        prefix["k_max"], prefix["k_min"] = pairs[..., 0], pairs[..., 1]
    return prefix


def _handle(prefix) -> _PrefixHandle:
    h = prefix.get("_b200")
    if h is None:
        raise ValueError("this prefix was not built by interattn_b200._build_prompt_blocks")
    return h


def _check_q(q_grouped: torch.Tensor, hkv: int, d: int) -> Tuple[int, torch.Tensor]:
    if q_grouped.dim() != 4 or q_grouped.shape[0] != hkv or q_grouped.shape[3] != d:
        raise ValueError("q_grouped must be [Hkv, G, 1, D]")
    if q_grouped.shape[2] != 1:
        raise ValueError("Triton selection stats expects q_len=1.")
    g = int(q_grouped.shape[1])
    return g, q_grouped.reshape(1, hkv * g, d).contiguous()


def _mask_from_indices(idx: torch.Tensor, nb: int, group: int) -> torch.Tensor:
    """idx int32 [1, Hkv, max_sel] (-1 padded) -> bool [Hkv, G, 1, nb]."""
    hkv = idx.shape[1]
    mask = torch.zeros((hkv, nb + 1), dtype=torch.bool, device=idx.device)
    mask.scatter_(1, torch.where(idx[0] >= 0, idx[0], torch.full_like(idx[0], nb)).long(), True)
    return mask[:, None, None, :nb].expand(hkv, group, 1, nb)


# --------------------------------------------------------------------------
# selection
# --------------------------------------------------------------------------

def _select_prompt_blocks(q_grouped, prefix, eps, *, top_k: Optional[int] = None):
    """-> (selected bool [Hkv,G,1,nb], z_logits f32 [Hkv,G,1,nb], v_bar expanded,
    size [1,nb], cluster_exists [1,nb]) - the reference's 5-tuple."""
    h = _handle(prefix)
    hkv, d = int(h.k_all.shape[0]), int(h.k_all.shape[2])
    group, q = _check_q(q_grouped.to(h.k_all.dtype), hkv, d)
    nb = int(prefix["block_valid_counts"].numel())
    kw = dict(top_k=int(top_k)) if top_k is not None else dict(eps=float(eps))
    idx, cnt, aux = ops.select_blocks(q, h.summ, h.geometry.prefix_lens, want=("z",), max_sel=max(nb, 1), **kw)
    selected = _mask_from_indices(idx, nb, group)
    z_logits = aux["z"][0, :, :nb].reshape(hkv, group, 1, nb)
    v_bar = prefix["v_bar"][:, None, None].expand(hkv, group, 1, nb, d)
    size = prefix["block_valid_counts"].view(1, -1)
    return selected, z_logits, v_bar, size, size > 0


def _run_condition_block_selection_stats(q_grouped, prefix, workspace=None, reduce_globals=True,
                                         term1_mass_exp=False):
    """-> (q [rows,D], s_cache [rows,nb], delta_cache [rows,nb], partial [4,rows,1],
    global_stats [4,rows] | None, n_blocks, n_chunks).  The kernel normalises in
    one piece, so there is a single chunk and ``partial`` equals the globals:
    (z_m, z_l) and a pair (c_m, c_l) with c_l e^{c_m} = sum_b e^{z_b} cosh(delta_b)
    (e^{delta_b} in place of the cosh with ``term1_mass_exp``)."""
    h = _handle(prefix)
    hkv, d = int(h.k_all.shape[0]), int(h.k_all.shape[2])
    group, q = _check_q(q_grouped.to(h.k_all.dtype), hkv, d)
    nb = int(prefix["block_valid_counts"].numel())
    rows = hkv * group
    ws = workspace if workspace is not None else {}
    bufs = {}
    for name, shape in (("s", (1, rows, nb)), ("delta", (1, rows, nb)), ("globals", (1, 4, rows))):
        t = ws.get("b200_" + name)
        if t is None or tuple(t.shape) != shape or t.device != q.device:
            t = torch.zeros(shape, device=q.device, dtype=torch.float32)
            ws["b200_" + name] = t
        bufs[name] = t
    ops.select_blocks(q, h.summ, h.geometry.prefix_lens, eps=float("inf"), max_sel=max(nb, 1),
                      want=("s", "delta", "globals"), aux_buffers=bufs, term1_mass_exp=bool(term1_mass_exp))
    globals_ = bufs["globals"][0]
    partial = globals_.reshape(4, rows, 1)
    return (q[0], bufs["s"][0], bufs["delta"][0], partial, globals_ if reduce_globals else None, nb, 1)


# --------------------------------------------------------------------------
# fused decode attention
# --------------------------------------------------------------------------

class _StepWorkspace:
    """Device scratch of one layer, reused across steps (the reference keeps a
    dict of tensors per layer; this object lives in that dict)."""

    def __init__(self, lib, geom: Geom, max_sel: int, n_splits: int, rep_mode: int, device, dtype, rows, d):
        self.key = (geom.n_kv_heads, geom.group_size, geom.max_blocks, max_sel, n_splits, rep_mode, dtype)
        need = lib.ia_workspace_bytes(ctypes.byref(geom), max_sel, n_splits, rep_mode)
        if need < 0:
            check(_lib.IA_ERR_BAD_ARG)
        self.bytes = int(need)
        self.buf = torch.empty((self.bytes + 256,), device=device, dtype=torch.uint8)
        self.off = (-self.buf.data_ptr()) % 256
        self.sel_idx = torch.empty((1, geom.n_kv_heads, max_sel), device=device, dtype=torch.int32)
        self.sel_count = torch.empty((1, geom.n_kv_heads), device=device, dtype=torch.int32)
        self.out = torch.empty((1, rows, d), device=device, dtype=dtype)

    def ptr(self):
        return ctypes.c_void_p(self.buf.data_ptr() + self.off)


def _suffix_continues_prefix(h: _PrefixHandle, k_suffix, v_suffix) -> bool:
    esz = h.k_all.element_size()
    d = int(h.k_all.shape[2])
    for cache, suf in ((h.k_all, k_suffix), (h.v_all, v_suffix)):
        if suf.dim() != 3 or suf.dtype != cache.dtype or suf.shape[0] != cache.shape[0] or suf.shape[2] != d:
            return False
        if suf.shape[1] and (suf.stride(2) != 1 or suf.stride(1) != d or suf.stride(0) != cache.stride(0)):
            return False
        if suf.shape[1] and suf.data_ptr() != cache.data_ptr() + h.prompt_len * d * esz:
            return False
    return True


def _condition_block_decode_output_fused_triton(
    *, q_grouped, prompt_prefix, k_suffix, v_suffix, suffix_len_dev, eps, page_size, store_selected,
    output_dtype, workspace=None, term1_mass_exp=False, top_k: Optional[int] = None,
    rep_mode: str = "hybrid", kv_cache: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
):
    """One decode-attention layer-step for one sequence -> (out [Hkv,G,1,D], selected | None).

    ``k_suffix`` / ``v_suffix`` are normally the tail of the very cache tensor the
    prefix was built from (that is what the attention hook passes); the kernels
    then read prefix and suffix in place.  ``kv_cache=(k_all, v_all)`` names the
    current full cache explicitly (a dynamic cache is re-allocated every step).
    Any other suffix tensor is supported through a slow path that copies prefix
    and suffix into one contiguous cache first."""
    if rep_mode not in _REP:
        raise ValueError(f"rep_mode must be one of {sorted(_REP)}")
    lib = _lib.load()
    h = _handle(prompt_prefix)
    if int(page_size) != h.block_size:
        raise ValueError(f"page_size {page_size} differs from the block size {h.block_size} of the prefix")
    hkv, d = int(h.k_all.shape[0]), int(h.k_all.shape[2])
    group, q = _check_q(q_grouped.to(h.k_all.dtype), hkv, d)
    nb = h.summ.max_blocks
    n_real = int(prompt_prefix["block_valid_counts"].numel())
    if kv_cache is not None:
        k_all, v_all = kv_cache
        _check_cache_view(k_all, "kv_cache[0]")
        _check_cache_view(v_all, "kv_cache[1]")
    elif _suffix_continues_prefix(h, k_suffix, v_suffix):
        k_all, v_all = h.k_all, h.v_all      # base pointers; the suffix follows in the same storage
    else:                                    # slow path: materialise one cache
        k_all = torch.cat([h.k_all, k_suffix.to(h.k_all.dtype)], dim=1).contiguous()
        v_all = torch.cat([h.v_all, v_suffix.to(h.v_all.dtype)], dim=1).contiguous()
    geo = h.geometry
    geo.ensure(h.prompt_len + int(k_suffix.shape[1]) + 1)
    if not (torch.is_tensor(suffix_len_dev) and suffix_len_dev.is_cuda):
        raise ValueError("suffix_len_dev must be a CUDA int32 scalar tensor")
    torch.add(geo.prefix_lens, suffix_len_dev.reshape(1).to(torch.int32), out=geo.seq_lens)

    mode = IA_SELECT_TOPK if top_k is not None else IA_SELECT_EPS
    if term1_mass_exp:
        mode |= _lib.IA_SELECT_TERM1_MASS_EXP
    max_sel = max(nb, 1)
    g = geo.geom(k_all, group, h.block_size, nb, h.summ,
                 n_tokens=max(int(k_all.shape[1]), h.prompt_len + int(k_suffix.shape[1])))
    ws_dict = workspace if workspace is not None else {}
    n_splits = ws_dict.get("b200_n_splits")
    if n_splits is None:
        expect = min(int(top_k), nb) if top_k is not None else max(1, nb // 16)
        n_splits = int(lib.ia_suggest_splits(ctypes.byref(g), expect))
        ws_dict["b200_n_splits"] = n_splits
    ws = ws_dict.get("b200_step")
    key = (hkv, group, nb, max_sel, n_splits, _REP[rep_mode], k_all.dtype)
    if ws is None or ws.key != key or ws.buf.device != q.device:
        ws = _StepWorkspace(lib, g, max_sel, n_splits, _REP[rep_mode], q.device, k_all.dtype, hkv * group, d)
        ws_dict["b200_step"] = ws
    s = h.summ.c_struct()
    check(lib.ia_decode_attention(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k_all.data_ptr()), ctypes.c_void_p(v_all.data_ptr()),
        ctypes.c_void_p(geo.table.data_ptr()), ctypes.c_void_p(geo.prefix_lens.data_ptr()),
        ctypes.c_void_p(geo.seq_lens.data_ptr()), ctypes.byref(s), ctypes.byref(g), mode, int(top_k or 0),
        float(eps or 0.0), max_sel, _REP[rep_mode], n_splits, ws.ptr(), ws.bytes,
        ctypes.c_void_p(ws.sel_idx.data_ptr()), ctypes.c_void_p(ws.sel_count.data_ptr()),
        ctypes.c_void_p(ws.out.data_ptr()), _stream()))
    out = ws.out.reshape(hkv, group, 1, d)
    if output_dtype is not None and out.dtype != output_dtype:
        out = out.to(output_dtype)
    selected = _mask_from_indices(ws.sel_idx, n_real, group) if store_selected else None
    return out, selected


# --------------------------------------------------------------------------
# the Hugging Face attention hook
# --------------------------------------------------------------------------

def _sdpa_prefill(query, key, value, scaling):
    out = F.scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=True,
                                         scale=scaling, enable_gqa=query.shape[1] != key.shape[1])
    return out.transpose(1, 2).contiguous(), None


def _sdpa_full(query, key, value, scaling):
    out = F.scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False,
                                         scale=scaling, enable_gqa=query.shape[1] != key.shape[1])
    return out.transpose(1, 2).contiguous(), None


class ConditionBlockDecodeRunner:
    """Decode-time attention hook with the reference runner's interface
    (``core.py:1203-1353``): prefill (q_len > 1) and the first
    ``full_attention_layers`` layers run dense SDPA, every other layer runs the
    block-sparse path on the prompt summaries it builds on first use.

    ``eps`` selects by the reference rule; ``top_k`` (if given) keeps the k best
    blocks instead.  ``rep_mode="hybrid"`` is the reference behaviour.  Batch 1,
    as in the reference; ``reset_step(pos)`` before every decode step (or advance
    ``suffix_len_dev`` on the device inside a captured graph)."""

    def __init__(self, *, model=None, model_config=None, layer_idx_list=None, full_attention_layers=0,
                 block_size=64, eps=0.0, prompt_len, pos=None, prompt_prefix_cache=None, term1_mass_exp=False,
                 top_k: Optional[int] = None, rep_mode: str = "hybrid", device=None):
        self.term1_mass_exp = bool(term1_mass_exp)
        self.model_config = model_config
        self.module_to_layer_idx = {}
        if model is not None:
            self.module_to_layer_idx = {id(layer.self_attn): i for i, layer in enumerate(model.model.layers)}
            device = device or next(model.parameters()).device
        self.layer_idx_set = None if layer_idx_list is None else {int(i) for i in layer_idx_list}
        self.full_attention_layers = int(full_attention_layers)
        self.block_size, self.eps, self.top_k, self.rep_mode = int(block_size), float(eps), top_k, rep_mode
        self.prompt_len = int(prompt_len)
        self.pos = int(pos if pos is not None else prompt_len)
        self.prompt_prefix_cache = {} if prompt_prefix_cache is None else prompt_prefix_cache
        self.workspace_by_layer: Dict[int, dict] = {}
        # Per-step statistics, as the reference keeps them (core.py:1229-1231): one dict per layer and
        # their sum, values left as GPU scalars so that a step never waits for the device; they are
        # turned into numbers after generation (summarize_condition_block_step_metadata).
        self.stats_by_layer: Dict[int, dict] = {}
        self.aggregate_stats: Dict[str, object] = {}
        self.skip_stats = os.environ.get("CONDITION_BLOCK_SKIP_STATS") == "1"
        self.static_suffix = False
        self.suffix_len_dev = torch.zeros((), dtype=torch.int32, device=device or "cuda")

    def should_compress(self, layer_idx) -> bool:
        inside = self.layer_idx_set is None or int(layer_idx) in self.layer_idx_set
        return inside and int(layer_idx) >= self.full_attention_layers

    def summarize(self) -> dict:
        """The step's statistics, still lazy (core.py:1250-1251, 1429-1438)."""
        return _summarize_stats_lazy(self.aggregate_stats, self.stats_by_layer)

    def reset_step(self, pos) -> None:
        self.pos = int(pos)
        self.suffix_len_dev.fill_(max(self.pos + 1 - self.prompt_len, 0))
        self.stats_by_layer.clear()
        self.aggregate_stats.clear()

    def _record(self, layer_idx, stats) -> None:
        if stats is None:
            return
        self.stats_by_layer[int(layer_idx)] = stats
        _merge_stats_lazy(self.aggregate_stats, stats)

    def hybrid_attention_forward(self, module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
        layer_idx = getattr(module, "layer_idx", None)
        if layer_idx is None:
            layer_idx = self.module_to_layer_idx.get(id(module))
        if query.shape[2] != 1:
            return _sdpa_prefill(query, key, value, scaling)
        if layer_idx is None or not self.should_compress(layer_idx):
            visible = self.pos + 1
            if not self.skip_stats and layer_idx is not None:
                self._record(layer_idx, full_attention_stats_for_heads(query.shape[1], [self.pos]))
            return _sdpa_full(query, key[:, :, :visible], value[:, :, :visible], scaling)
        if query.shape[0] != 1:
            raise ValueError("condition_block fast path expects batch_size=1 and q_len=1.")
        if self.pos < self.prompt_len:
            raise ValueError("condition_block fast path expects generated-token decode positions.")
        n_heads, n_kv_heads, d = int(query.shape[1]), int(key.shape[1]), int(query.shape[3])
        if n_heads % n_kv_heads != 0:
            raise ValueError("condition_block fast path expects grouped query attention.")
        q_grouped = query[0].reshape(n_kv_heads, n_heads // n_kv_heads, 1, d)
        k_all, v_all = key[0], value[0]
        if not self.static_suffix:
            k_all, v_all = k_all[:, : self.pos + 1], v_all[:, : self.pos + 1]
        cache_key = (int(layer_idx), self.prompt_len, self.block_size)
        prefix = self.prompt_prefix_cache.get(cache_key)
        if prefix is None:
            prefix = _build_prompt_blocks(k_all[:, : self.prompt_len], v_all[:, : self.prompt_len], self.block_size)
            self.prompt_prefix_cache[cache_key] = prefix
        out, _ = _condition_block_decode_output_fused_triton(
            q_grouped=q_grouped, prompt_prefix=prefix, k_suffix=k_all[:, self.prompt_len:],
            v_suffix=v_all[:, self.prompt_len:], suffix_len_dev=self.suffix_len_dev, eps=self.eps,
            page_size=self.block_size, store_selected=False, output_dtype=query.dtype,
            workspace=self.workspace_by_layer.setdefault(int(layer_idx), {}), top_k=self.top_k,
            rep_mode=self.rep_mode, kv_cache=(k_all, v_all), term1_mass_exp=self.term1_mass_exp)
        if not self.skip_stats:
            ws = self.workspace_by_layer[int(layer_idx)]["b200_step"]
            self._record(layer_idx, _condition_stats_from_selection(
                ws.sel_idx, ws.sel_count, group_size=n_heads // n_kv_heads,
                block_size=self.block_size, prompt_len=self.prompt_len,
                suffix_len=max(self.pos + 1 - self.prompt_len, 0), rep_mode=self.rep_mode))
        out = out.reshape(n_heads, 1, d).permute(1, 0, 2).unsqueeze(0)
        return out.to(query.dtype), None


# --------------------------------------------------------------------------
# statistics (core.py:1382-1523)
# --------------------------------------------------------------------------

def _condition_stats_from_selection(sel_idx, sel_count, *, group_size, block_size, prompt_len, suffix_len,
                                    rep_mode="hybrid"):
    """The reference's ``_condition_stats`` (core.py:1441-1456) from an index list instead of a boolean
    mask: ``sel_idx [1, Hkv, max_sel]`` / ``sel_count [1, Hkv]`` on the device.  The reference's mask is
    the per-kv-head selection broadcast over the G query rows, so every sum over it is G times the sum
    over kv heads.  Tensor-valued entries stay on the device (no synchronisation here).  With
    ``rep_mode="sparse_only"`` no representative is attended, so ``hybrid_tokens`` leaves them out."""
    n_kv_heads = int(sel_count.shape[-1])
    # blocks of the prompt: all full but possibly the last (host arithmetic: nothing is read back)
    n_real = (int(prompt_len) + block_size - 1) // block_size
    n_exist = n_real
    tail = int(prompt_len) - (n_real - 1) * block_size if n_real else 0
    cnt = sel_count.reshape(n_kv_heads).to(torch.int64)
    has_last = (sel_idx.reshape(n_kv_heads, -1) == n_real - 1).any(dim=-1).to(torch.int64)
    selected_clusters = cnt.sum() * group_size
    selected_tokens = (cnt * block_size - has_last * (block_size - tail)).sum() * group_size
    n_rows = n_kv_heads * group_size
    suffix_tokens = max(int(suffix_len), 0) * n_rows
    hybrid = selected_tokens + suffix_tokens
    if rep_mode == "hybrid":
        hybrid = hybrid + (n_exist * n_kv_heads - cnt.sum()) * group_size
    return {
        "rows": n_rows,
        "clusters": n_exist * n_rows,
        "selected_clusters": selected_clusters,
        "selected_tokens": selected_tokens,
        "hybrid_tokens": hybrid,
        "total_available": (int(prompt_len) + max(int(suffix_len), 0)) * n_rows,
    }


def full_attention_stats_for_heads(n_heads, pos_list):
    """Statistics of a dense layer-step (core.py:1463-1473): every visible token is attended."""
    total_available = sum(int(pos) + 1 for pos in pos_list) * int(n_heads)
    return {"rows": int(n_heads) * len(pos_list), "clusters": 0, "selected_clusters": 0,
            "selected_tokens": total_available, "hybrid_tokens": total_available,
            "total_available": total_available}


def _merge_stats_lazy(total, add):
    for key, value in add.items():
        total[key] = total[key] + value if key in total else value


def _summarize_stats_lazy(aggregate_stats, stats_by_layer):
    return {"aggregate": dict(aggregate_stats),
            "by_layer": {int(i): dict(st) for i, st in stats_by_layer.items()}}


def _to_python_number(value):
    if torch.is_tensor(value):
        if value.numel() != 1:
            raise ValueError("Expected scalar tensor in condition-block stats.")
        return int(value.detach().cpu().item())
    return int(value)


def _full_generation_step_metadata(model, pos_list):
    """Statistics of a step in which every layer attends densely (the prefill step, core.py:1476-1483)."""
    aggregate, by_layer = {}, {}
    n_heads = int(model.config.num_attention_heads)
    for layer_idx in range(int(model.config.num_hidden_layers)):
        st = full_attention_stats_for_heads(n_heads, pos_list)
        by_layer[layer_idx] = st
        _merge_stats_lazy(aggregate, st)
    return _summarize_stats_lazy(aggregate, by_layer)


def summarize_condition_block_step_metadata(step_metadata):
    """Per-generation summary of the per-step statistics (core.py:1486-1523): the only place where the
    lazy GPU scalars are read back.  ``condition_block_equiv_budget`` = attended entries / visible tokens."""
    if os.environ.get("CONDITION_BLOCK_SKIP_STATS") == "1":
        return {"condition_block_stats_disabled": True}
    aggregate, by_step = {}, []
    for step_idx, metadata in enumerate(step_metadata):
        if not metadata:
            continue
        step_aggregate = metadata.get("aggregate", {})
        num = _to_python_number(step_aggregate.get("hybrid_tokens", 0))
        den = max(_to_python_number(step_aggregate.get("total_available", 0)), 1)
        by_step.append({"step": step_idx, "equiv_budget": float(num / den)})
        for key, value in step_aggregate.items():
            if not key.startswith("mean_"):
                _merge_stats_lazy(aggregate, {key: value})
    materialized = {key: _to_python_number(value) for key, value in aggregate.items()}
    total_available = max(int(materialized.get("total_available", 0)), 1)
    rows = max(int(materialized.get("rows", 0)), 1)
    hybrid_tokens = int(materialized.get("hybrid_tokens", 0))
    equiv_budget = float(hybrid_tokens / total_available)
    return {
        "condition_block_equiv_budget": equiv_budget,
        "condition_block_budget": {**materialized, "mean_hybrid_tokens": float(hybrid_tokens / rows),
                                   "mean_budget_causal": equiv_budget, "mean_budget_visible": equiv_budget,
                                   "by_step": by_step},
    }


def generate_condition_block_cached(*, model, tokenizer, input_ids, attention_mask, method, device=None,
                                    dataset=None, term1_mass_exp=False):
    """Greedy generation with block-sparse decode attention; the interface of the
    reference's ``generate_condition_block_cached`` (``core.py:60-187``).

    The prompt is prefilled with dense causal attention, every later token runs
    through ``ConditionBlockDecodeRunner``.  ``method`` supplies
    ``max_new_tokens``, ``full_attention_layers``, ``condition_block_size``,
    ``condition_eps`` (and optionally ``condition_top_k`` / ``condition_rep_mode``).
    Returns ``(output_ids [1, n], metadata)``; generation stops early at the
    tokenizer's EOS id.  Batch size 1, as in the reference.  ``metadata`` is what the
    reference returns (``condition_block_equiv_budget`` and ``condition_block_budget``
    summed over the prefill and every decode step, or ``condition_block_stats_disabled``
    under ``CONDITION_BLOCK_SKIP_STATS=1``) plus ``method`` / ``prompt_len`` / ``decode_steps``."""
    if getattr(method, "condition_delta_mode", "range_bound") != "range_bound":
        raise ValueError("condition_block only supports delta_mode='range_bound'.")
    if int(input_ids.shape[0]) != 1:
        raise ValueError("condition_block generate currently expects batch_size=1.")
    prompt_len = int(input_ids.shape[1])
    budget = int(method.max_new_tokens)
    meta = {"method": "condition_block_b200", "prompt_len": prompt_len, "decode_steps": 0}
    if budget <= 0:
        meta.update(summarize_condition_block_step_metadata([]))
        return torch.empty((1, 0), device=input_ids.device, dtype=input_ids.dtype), meta
    collect_stats = os.environ.get("CONDITION_BLOCK_SKIP_STATS") != "1"
    step_metadata = []
    stop = set()
    eos = getattr(tokenizer, "eos_token_id", None) if tokenizer is not None else None
    if eos is not None:
        stop.update(eos if isinstance(eos, (list, tuple)) else [eos])
    with torch.no_grad():
        out = model(input_ids=input_ids, attention_mask=attention_mask, use_cache=True)
    cache = out.past_key_values
    if collect_stats:
        step_metadata.append(_full_generation_step_metadata(model, [prompt_len - 1]))
    token = torch.argmax(out.logits[:, -1, :].float(), dim=-1, keepdim=True)
    tokens = [token]
    mask = attention_mask
    runner = ConditionBlockDecodeRunner(
        model=model, model_config=model.config, full_attention_layers=method.full_attention_layers,
        block_size=method.condition_block_size, eps=method.condition_eps, prompt_len=prompt_len,
        top_k=getattr(method, "condition_top_k", None), rep_mode=getattr(method, "condition_rep_mode", "hybrid"),
        term1_mass_exp=term1_mass_exp)
    total = prompt_len + 1
    with condition_block_decode_context(runner):
        while len(tokens) < budget and int(token) not in stop:
            runner.reset_step(total - 1)
            if mask is not None:
                mask = torch.cat([mask, torch.ones_like(token)], dim=1)
            with torch.no_grad():
                out = model(input_ids=token, attention_mask=mask, past_key_values=cache, use_cache=True)
            cache = out.past_key_values
            if collect_stats:
                step_metadata.append(runner.summarize())
            token = torch.argmax(out.logits[:, -1, :].float(), dim=-1, keepdim=True)
            tokens.append(token)
            total += 1
            meta["decode_steps"] += 1
    meta.update(summarize_condition_block_step_metadata(step_metadata))
    return torch.cat(tokens, dim=1), meta


@contextlib.contextmanager
def condition_block_decode_context(runner: ConditionBlockDecodeRunner):
    """Install the runner as ``modeling_llama.eager_attention_forward`` for the
    duration of the block (the model must use ``attn_implementation="eager"``)."""
    from transformers.models.llama import modeling_llama
    original = modeling_llama.eager_attention_forward
    modeling_llama.eager_attention_forward = runner.hybrid_attention_forward
    try:
        yield runner
    finally:
        modeling_llama.eager_attention_forward = original
