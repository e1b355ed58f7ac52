"""Batched, paged operators of the condition-block decode path (CUDA only).

Thin host code over the C ABI (``include/interattn_b200.h``): tensors become
raw device pointers, the current torch stream becomes the CUDA stream, status
codes become exceptions.  PyTorch is used for device memory and streams only;
none of these functions computes anything in PyTorch and none has a CPU path.

Shapes (B sequences, Hkv kv heads, G query heads per kv head, D head_dim,
P = 16 tokens per physical page, block = selection block, nb = blocks):

    q            [B, Hkv * G, D]              query head = kv * G + g
    k_pool       [n_pages, Hkv, P, D]         any page / head strides, inner [P, D] contiguous
    block_table  int32 [B, max_pages]
    prefix_lens  int32 [B]   tokens covered by summaries (the prompt)
    seq_lens     int32 [B]   prefix + generated suffix
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import (Geom, IA_BF16, IA_F32, IA_REP_HYBRID, IA_REP_SPARSE_ONLY, IA_SELECT_EPS,
                   IA_SELECT_TOPK, SelectAux, Summaries, check)

_DTYPES = {torch.float32: IA_F32, torch.bfloat16: IA_BF16}
_REP = {"sparse_only": IA_REP_SPARSE_ONLY, "hybrid": IA_REP_HYBRID}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("interattn_b200 operators take CUDA tensors only (there is no CPU path)")


def _geom_flags(summ, bound: str = "range") -> int:
    """Geometry flags: how the summaries are stored (bf16 k_bar: IA_GEOM_KBAR_BF16) and which bound
    the selection uses (``bound="diag_ell"``: IA_GEOM_DIAG_ELL, needs summaries built with w and rho)."""
    if bound not in ("range", "diag_ell"):
        raise ValueError("bound must be 'range' or 'diag_ell'")
    flags = _lib.IA_GEOM_KBAR_BF16 if summ is not None and summ.k_bar.dtype == torch.bfloat16 else 0
    if summ is not None and summ.k_bounds is not None:
        if bound == "diag_ell":
            raise ValueError("summaries with the packed range layout do not carry the diag_ell pair")
        flags |= _lib.IA_GEOM_PACKED_BOUNDS
    if bound == "diag_ell":
        if summ is None or summ.w is None or summ.rho is None:
            raise ValueError("the diag_ell bound needs summaries built with diag_ell=True (w and rho)")
        flags |= _lib.IA_GEOM_DIAG_ELL
    return flags


@dataclass
class PagedKV:
    """A paged KV cache: physical pools + per-sequence page lists + lengths."""

    k_pool: torch.Tensor
    v_pool: torch.Tensor
    block_table: torch.Tensor
    prefix_lens: torch.Tensor
    seq_lens: torch.Tensor
    # Pages the kernels may address (block-table entries are checked against it before use; an
    # entry outside is skipped and reported in the device status word).  Default: the whole pool.
    n_pool_pages: Optional[int] = None

    def __post_init__(self):
        _need_cuda(self.k_pool, self.v_pool, self.block_table, self.prefix_lens, self.seq_lens)
        k, v = self.k_pool, self.v_pool
        if k.dim() != 4 or k.shape != v.shape or k.dtype != v.dtype or k.stride() != v.stride():
            raise ValueError("k_pool / v_pool must be [n_pages, Hkv, P, D] tensors of equal shape, dtype and strides")
        if k.dtype not in _DTYPES:
            raise ValueError(f"KV dtype {k.dtype} not supported (float32, bfloat16)")
        if k.stride(3) != 1 or k.stride(2) != k.shape[3]:
            raise ValueError("the [P, D] run of one (page, kv head) must be contiguous")
        for name in ("block_table", "prefix_lens", "seq_lens"):
            t = getattr(self, name)
            if t.dtype != torch.int32 or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous int32 tensor")
        if self.block_table.dim() != 2:
            raise ValueError("block_table must be [B, max_pages]")

    @property
    def batch(self) -> int:
        return int(self.block_table.shape[0])

    @property
    def n_kv_heads(self) -> int:
        return int(self.k_pool.shape[1])

    @property
    def page_size(self) -> int:
        return int(self.k_pool.shape[2])

    @property
    def head_dim(self) -> int:
        return int(self.k_pool.shape[3])

    def geom(self, group_size: int, block_size: int, max_blocks: int, summ: Optional["BlockSummaries"] = None,
             bound: str = "range") -> Geom:
        return Geom(
            batch=self.batch, n_kv_heads=self.n_kv_heads, group_size=int(group_size), head_dim=self.head_dim,
            page_size=self.page_size, block_size=int(block_size), max_pages=int(self.block_table.shape[1]),
            max_blocks=int(max_blocks), dtype=_DTYPES[self.k_pool.dtype], reserved=_geom_flags(summ, bound),
            n_pool_pages=int(self.k_pool.shape[0] if self.n_pool_pages is None else self.n_pool_pages), reserved2=0,
            pool_page_stride=int(self.k_pool.stride(0)), pool_head_stride=int(self.k_pool.stride(1)))


@dataclass
class BlockSummaries:
    """Per (sequence, kv head, block) statistics: k_bar f32 (or bf16: the reference's
    CONDITION_BLOCK_K_BAR_DTYPE=bfloat16 option, approximate), the rest in the KV dtype."""

    k_bar: torch.Tensor       # [B, Hkv, nb, D] f32 | bf16
    k_max: torch.Tensor       # [B, Hkv, nb, D]
    k_min: torch.Tensor
    v_bar: torch.Tensor
    v_norm_max: torch.Tensor  # [B, Hkv, nb] f32
    block_size: int
    # optional diagonal-ellipsoid pair (the reference's condition_block_ball "diag_ell" bound):
    w: Optional[torch.Tensor] = None     # [B, Hkv, nb, D] KV dtype, max_t |k_t - k_bar| (rounded up in bf16)
    rho: Optional[torch.Tensor] = None   # [B, Hkv, nb] f32, max_t |(k_t - k_bar) / w|
    # optional packed range (the reference's CONDITION_BLOCK_TMA_BOUNDS layout, IMPL/core.py:490-499):
    # [B, Hkv, nb, 2 D] with (k_max[d], k_min[d]) pairs; k_max / k_min are then strided views into it
    k_bounds: Optional[torch.Tensor] = None

    @property
    def max_blocks(self) -> int:
        return int(self.k_bar.shape[2])

    def c_struct(self) -> Summaries:
        if self.k_bounds is not None:  # the kernels read the packed array through the k_max member; k_min is unused
            return Summaries(self.k_bar.data_ptr(), self.k_bounds.data_ptr(), None, self.v_bar.data_ptr(),
                             self.v_norm_max.data_ptr(), None, None)
        return Summaries(self.k_bar.data_ptr(), self.k_max.data_ptr(), self.k_min.data_ptr(),
                         self.v_bar.data_ptr(), self.v_norm_max.data_ptr(),
                         None if self.w is None else self.w.data_ptr(),
                         None if self.rho is None else self.rho.data_ptr())

    @staticmethod
    def empty(batch: int, n_kv_heads: int, max_blocks: int, head_dim: int, dtype: torch.dtype, device,
              block_size: int, k_bar_dtype: torch.dtype = torch.float32, diag_ell: bool = False,
              packed_bounds: bool = False) -> "BlockSummaries":
        shape = (batch, n_kv_heads, max_blocks, head_dim)
        if k_bar_dtype not in (torch.float32, torch.bfloat16) or (k_bar_dtype != torch.float32 and dtype != torch.bfloat16):
            raise ValueError("k_bar is float32, or bfloat16 next to bfloat16 pools")
        if packed_bounds and diag_ell:
            raise ValueError("the packed range layout and the diag_ell pair exclude one another")
        k_bounds = torch.zeros(shape[:3] + (2 * head_dim,), device=device, dtype=dtype) if packed_bounds else None
        pairs = k_bounds.view(*shape, 2) if packed_bounds else None
        return BlockSummaries(
            k_bar=torch.zeros(shape, device=device, dtype=k_bar_dtype),
            k_max=pairs[..., 0] if packed_bounds else torch.zeros(shape, device=device, dtype=dtype),
            k_min=pairs[..., 1] if packed_bounds else torch.zeros(shape, device=device, dtype=dtype),
            k_bounds=k_bounds,
            v_bar=torch.zeros(shape, device=device, dtype=dtype),
            v_norm_max=torch.zeros(shape[:3], device=device, dtype=torch.float32),
            block_size=int(block_size),
            w=torch.zeros(shape, device=device, dtype=dtype) if diag_ell else None,
            rho=torch.zeros(shape[:3], device=device, dtype=torch.float32) if diag_ell else None)


def build_summaries(kv: PagedKV, block_size: int, max_blocks: Optional[int] = None,
                    out: Optional[BlockSummaries] = None,
                    first_blocks: Optional[torch.Tensor] = None,
                    k_bar_dtype: torch.dtype = torch.float32, diag_ell: bool = False,
                    packed_bounds: bool = False) -> BlockSummaries:
    """Block summaries of every sequence's prefix (reference: ``_build_prompt_blocks``).
    ``packed_bounds=True`` stores the coordinate range as the reference does with
    ``CONDITION_BLOCK_TMA_BOUNDS=1`` (``IMPL/core.py:490-499``): one array ``k_bounds`` of ``(k_max[d], k_min[d])``
    pairs, ``k_max`` / ``k_min`` being strided views into it; the selection reads that layout directly.
    ``diag_ell=True`` also keeps the diagonal-ellipsoid pair ``w, rho`` (the reference's
    ``condition_block_ball`` bound; ``select_blocks(..., bound="diag_ell")`` then reads two vectors and a
    scalar per block instead of three vectors).

    ``first_blocks`` (int32 [B], device; needs ``out``) makes it an incremental
    update: only blocks ``b >= first_blocks[seq]`` are recomputed - used when
    the generated suffix has grown by whole blocks and ``kv.prefix_lens`` was
    raised to take them into the summarised prefix."""
    lib = _lib.load()
    if first_blocks is not None:
        if out is None:
            raise ValueError("an incremental update needs the summaries to update (out=)")
        _need_cuda(first_blocks)
        if first_blocks.dtype != torch.int32 or not first_blocks.is_contiguous() or first_blocks.numel() != kv.batch:
            raise ValueError("first_blocks must be a contiguous int32 tensor with one entry per sequence")
        g = kv.geom(1, block_size, out.max_blocks, out)
        s = out.c_struct()
        check(lib.ia_update_summaries(_ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.block_table), _ptr(kv.prefix_lens),
                                      _ptr(first_blocks), ctypes.byref(g), ctypes.byref(s), _stream()))
        return out
    if max_blocks is None:
        max_blocks = out.max_blocks if out is not None else max(
            1, (int(kv.block_table.shape[1]) * kv.page_size + block_size - 1) // block_size)
    if out is None:
        out = BlockSummaries.empty(kv.batch, kv.n_kv_heads, max_blocks, kv.head_dim, kv.k_pool.dtype,
                                   kv.k_pool.device, block_size, k_bar_dtype, diag_ell, packed_bounds)
    g = kv.geom(1, block_size, max_blocks, out)
    s = out.c_struct()
    check(lib.ia_build_summaries(_ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.block_table), _ptr(kv.prefix_lens),
                                 ctypes.byref(g), ctypes.byref(s), _stream()))
    return out


def _q_geom(q: torch.Tensor, n_kv_heads: int) -> int:
    if q.dim() != 3 or not q.is_contiguous():
        raise ValueError("q must be a contiguous [B, Hq, D] tensor")
    if q.shape[1] % n_kv_heads != 0:
        raise ValueError("query heads must be a multiple of kv heads (grouped-query attention)")
    return int(q.shape[1]) // n_kv_heads


def select_blocks(
    q: torch.Tensor, summ: BlockSummaries, prefix_lens: torch.Tensor, *,
    top_k: Optional[int] = None, eps: Optional[float] = None, max_sel: Optional[int] = None,
    want: Sequence[str] = (), out_idx: Optional[torch.Tensor] = None, out_count: Optional[torch.Tensor] = None,
    aux_buffers: Optional[Dict[str, torch.Tensor]] = None, term1_mass_exp: bool = False, bound: str = "range",
) -> Tuple[torch.Tensor, torch.Tensor, Dict[str, torch.Tensor]]:
    """Score every block and route.

    ``bound="diag_ell"`` bounds the in-block spread of the logits with the diagonal-ellipsoid pair
    ``(w, rho)`` of the summaries instead of the coordinate range ``(k_max, k_min)`` (the reference's
    ``condition_block_ball`` variant, ``gen_selection.py:82-87``).

    ``term1_mass_exp`` switches the first term of the score to ``2 b_all softmax(z + delta)``
    (the reference's variant of the same name, ``core.py:798-803``).

    Exactly one of ``top_k`` (k best blocks per (sequence, kv head); ties go to
    the lower block index) and ``eps`` (the reference rule ``score > eps``) is
    given.  Returns ``(idx int32 [B, Hkv, max_sel] ascending, -1 padded,
    count int32 [B, Hkv], aux)`` where ``aux`` holds the tensors named in
    ``want`` out of: score [B,Hkv,nb], z / s / delta [B,rows,nb], globals [B,4,rows].
    """
    lib = _lib.load()
    _need_cuda(q, prefix_lens, summ.k_bar)
    if (top_k is None) == (eps is None):
        raise ValueError("give exactly one of top_k and eps")
    b, hkv, nb, d = summ.k_bar.shape
    group = _q_geom(q, hkv)
    if q.dtype != summ.k_max.dtype:
        raise ValueError("q and the summaries must share the KV dtype")
    mode = IA_SELECT_TOPK if top_k is not None else IA_SELECT_EPS
    if max_sel is None:
        max_sel = int(top_k) if mode == IA_SELECT_TOPK else nb
        max_sel = max(max_sel, 1)
    if term1_mass_exp:
        mode |= _lib.IA_SELECT_TERM1_MASS_EXP
    rows = hkv * group
    dev = q.device
    idx = out_idx if out_idx is not None else torch.empty((b, hkv, max_sel), device=dev, dtype=torch.int32)
    cnt = out_count if out_count is not None else torch.empty((b, hkv), device=dev, dtype=torch.int32)
    shapes = {"score": (b, hkv, nb), "z": (b, rows, nb), "s": (b, rows, nb), "delta": (b, rows, nb),
              "globals": (b, 4, rows)}
    aux: Dict[str, torch.Tensor] = {}
    for name in want:
        if name not in shapes:
            raise ValueError(f"unknown diagnostic {name!r}")
        buf = None if aux_buffers is None else aux_buffers.get(name)
        if buf is None:  # blocks past a sequence's prefix are never written: give them neutral values
            buf = torch.full(shapes[name], float("-inf") if name == "z" else 0.0, device=dev, dtype=torch.float32)
        aux[name] = buf
    c_aux = SelectAux(*[aux[n].data_ptr() if n in aux else None for n in ("score", "z", "s", "delta", "globals")])
    g = Geom(batch=b, n_kv_heads=hkv, group_size=group, head_dim=d, page_size=16, block_size=summ.block_size,
             max_pages=1, max_blocks=nb, dtype=_DTYPES[q.dtype], reserved=_geom_flags(summ, bound),
             pool_page_stride=16 * d, pool_head_stride=16 * d)
    s = summ.c_struct()
    check(lib.ia_select(_ptr(q), ctypes.byref(s), _ptr(prefix_lens), ctypes.byref(g), mode,
                        int(top_k or 0), float(eps or 0.0), int(max_sel), _ptr(idx), _ptr(cnt),
                        ctypes.byref(c_aux), _stream()))
    return idx, cnt, aux


def sparse_decode(
    q: torch.Tensor, kv: PagedKV, idx: torch.Tensor, count: torch.Tensor, *, block_size: int,
    max_blocks: int, rep_mode: str = "sparse_only", summ: Optional[BlockSummaries] = None,
    z: Optional[torch.Tensor] = None, n_splits: int = 1, block_range: Optional[Tuple[int, int]] = None,
    with_suffix: bool = True, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention over the selected blocks (+ representatives, + suffix).

    Returns normalised partials ``(o f32 [B, rows, n_splits, D], lse f32 [B, rows, n_splits])``."""
    lib = _lib.load()
    _need_cuda(q, idx, count)
    group = _q_geom(q, kv.n_kv_heads)
    if q.dtype != kv.k_pool.dtype:
        raise ValueError("q and the KV pools must share a dtype")
    if rep_mode not in _REP:
        raise ValueError(f"rep_mode must be one of {sorted(_REP)}")
    if rep_mode == "hybrid" and (summ is None or z is None):
        raise ValueError("hybrid mode needs the block summaries (v_bar) and z from select_blocks(want=('z',))")
    rows = kv.n_kv_heads * group
    b = kv.batch
    if out is None:
        o = torch.empty((b, rows, n_splits, kv.head_dim), device=q.device, dtype=torch.float32)
        lse = torch.empty((b, rows, n_splits), device=q.device, dtype=torch.float32)
    else:
        o, lse = out
    lo, hi = (0, max_blocks) if block_range is None else block_range
    g = kv.geom(group, block_size, max_blocks, summ)
    s = summ.c_struct() if summ is not None else None
    check(lib.ia_sparse_decode(
        _ptr(q), _ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.block_table), _ptr(kv.prefix_lens), _ptr(kv.seq_lens),
        _ptr(idx), _ptr(count), int(idx.shape[-1]), ctypes.byref(s) if s is not None else None, _ptr(z),
        ctypes.byref(g), _REP[rep_mode], int(n_splits), int(lo), int(hi), int(bool(with_suffix)),
        _ptr(o), _ptr(lse), _stream()))
    return o, lse


def finalize(o_partial: torch.Tensor, lse_partial: torch.Tensor, out_dtype: torch.dtype,
             return_lse: bool = False, out: Optional[torch.Tensor] = None):
    """Log-sum-exp merge of partials along their second-to-last axis.

    o_partial [..., n_parts, D], lse_partial [..., n_parts] -> out [..., D]."""
    lib = _lib.load()
    _need_cuda(o_partial, lse_partial)
    if o_partial.dtype != torch.float32 or lse_partial.dtype != torch.float32:
        raise ValueError("partials are float32")
    if not (o_partial.is_contiguous() and lse_partial.is_contiguous()):
        raise ValueError("partials must be contiguous")
    *lead, parts, d = o_partial.shape
    if tuple(lse_partial.shape) != (*lead, parts):
        raise ValueError("lse_partial must be o_partial without its last axis")
    n_rows = 1
    for x in lead:
        n_rows *= int(x)
    if out is None:
        out = torch.empty((*lead, d), device=o_partial.device, dtype=out_dtype)
    lse = torch.empty(lead, device=o_partial.device, dtype=torch.float32) if return_lse else None
    check(lib.ia_finalize(_ptr(o_partial), _ptr(lse_partial), n_rows, int(parts), int(d), _ptr(out),
                          _DTYPES[out_dtype], _ptr(lse), _stream()))
    return (out, lse) if return_lse else out


def finalize_gathered(gathered: torch.Tensor, n_ranks: int, rank_stride: int, n_rows: int, n_parts: int,
                      head_dim: int, out: torch.Tensor) -> torch.Tensor:
    """Merge the split-KV partials of ``n_ranks`` GPUs read in place from an all-gather buffer:
    chunk ``w`` starts ``w * rank_stride`` floats in and holds ``o [n_rows, n_parts, head_dim]``
    followed by ``lse [n_rows, n_parts]``.  ``out`` (``n_rows * head_dim`` elements) is written."""
    _need_cuda(gathered, out)
    if gathered.dtype != torch.float32 or not gathered.is_contiguous() or not out.is_contiguous():
        raise ValueError("gathered is a contiguous float32 buffer, out a contiguous tensor")
    if gathered.numel() < (n_ranks - 1) * rank_stride + n_rows * n_parts * (head_dim + 1):
        raise ValueError("the gathered buffer is too small")
    if out.numel() != n_rows * head_dim or out.dtype not in _DTYPES:
        raise ValueError("out holds n_rows * head_dim float32 or bfloat16 elements")
    check(_lib.load().ia_finalize_gathered(_ptr(gathered), int(n_ranks), int(rank_stride), int(n_rows), int(n_parts),
                                           int(head_dim), _ptr(out), _DTYPES[out.dtype], _stream()))
    return out


class DecodeAttention:
    """One decode-attention layer-step behind a single call, with all scratch
    preallocated: selection -> sparse attention -> finalize.

    ``step(q)`` enqueues the three kernels on the current stream and returns
    the output tensor it owns (overwritten by the next call); it allocates
    nothing and does not synchronise, so it can be captured in a CUDA graph.
    ``step_host(q_host, out_host)`` is the same step for callers holding the
    query on the host: pinned q -> device, the step, output -> pinned host,
    then a stream synchronise.
    """

    def __init__(self, kv: PagedKV, summ: BlockSummaries, n_q_heads: int, *, top_k: Optional[int] = None,
                 eps: Optional[float] = None, rep_mode: str = "sparse_only", n_splits: Optional[int] = None,
                 max_sel: Optional[int] = None, expected_blocks: Optional[int] = None,
                 term1_mass_exp: bool = False, bound: str = "range"):
        self.lib = _lib.load()
        if (top_k is None) == (eps is None):
            raise ValueError("give exactly one of top_k and eps")
        if n_q_heads % kv.n_kv_heads != 0:
            raise ValueError("query heads must be a multiple of kv heads")
        if rep_mode not in _REP:
            raise ValueError(f"rep_mode must be one of {sorted(_REP)}")
        self.kv, self.summ = kv, summ
        self.group = n_q_heads // kv.n_kv_heads
        self.mode = IA_SELECT_TOPK if top_k is not None else IA_SELECT_EPS
        if term1_mass_exp:
            self.mode |= _lib.IA_SELECT_TERM1_MASS_EXP
        self.top_k, self.eps = int(top_k or 0), float(eps or 0.0)
        nb = summ.max_blocks
        self.max_sel = int(max_sel) if max_sel is not None else (max(self.top_k, 1) if top_k is not None else nb)
        self.geom = kv.geom(self.group, summ.block_size, nb, summ, bound)
        if n_splits is None:   # wave-aware choice for this device
            expect = expected_blocks or (min(self.top_k, nb) if top_k is not None else max(1, nb // 16))
            n_splits = self.lib.ia_suggest_splits(ctypes.byref(self.geom), int(max(1, expect)))
        self.rep_mode, self.n_splits = rep_mode, int(n_splits)
        self.c_summ = summ.c_struct()
        need = self.lib.ia_workspace_bytes(ctypes.byref(self.geom), self.max_sel, self.n_splits, _REP[rep_mode])
        if need < 0:
            check(_lib.IA_ERR_BAD_ARG)
        dev = kv.k_pool.device
        self.workspace = torch.empty((int(need) + 256,), device=dev, dtype=torch.uint8)
        self._ws_off = (-self.workspace.data_ptr()) % 256
        self.ws_bytes = int(need)
        b, rows = kv.batch, kv.n_kv_heads * self.group
        self.sel_idx = torch.empty((b, kv.n_kv_heads, self.max_sel), device=dev, dtype=torch.int32)
        self.sel_count = torch.empty((b, kv.n_kv_heads), device=dev, dtype=torch.int32)
        self.out = torch.empty((b, rows, kv.head_dim), device=dev, dtype=kv.k_pool.dtype)
        self.q_dev = torch.empty((b, rows, kv.head_dim), device=dev, dtype=kv.k_pool.dtype)
        # The step is called once per layer per token: everything that does not change from call to call is
        # turned into ctypes objects here, once.  The tensors of ``kv`` and ``summ`` are therefore bound at
        # construction - update them in place (lengths, table entries), do not replace them.
        self._dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
        self._shape, self._dtype = tuple(self.out.shape), self.out.dtype
        self._kv_args = (_ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.block_table), _ptr(kv.prefix_lens),
                         _ptr(kv.seq_lens), ctypes.byref(self.c_summ), ctypes.byref(self.geom), self.mode,
                         self.top_k, self.eps, self.max_sel, _REP[self.rep_mode], self.n_splits, self._ws_ptr(),
                         self.ws_bytes)
        self._out_args = (_ptr(self.sel_idx), _ptr(self.sel_count), _ptr(self.out))
        self._q_dev_ptr, self._out_ptr = _ptr(self.q_dev), _ptr(self.out)

    def _ws_ptr(self):
        return ctypes.c_void_p(self.workspace.data_ptr() + self._ws_off)

    def _stream(self):
        return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(self._dev_index))

    def step(self, q: torch.Tensor) -> torch.Tensor:
        if not q.is_cuda or q.shape != self._shape or q.dtype != self._dtype or not q.is_contiguous():
            raise ValueError(f"q must be a contiguous CUDA {self._shape} {self._dtype} tensor")
        check(self.lib.ia_decode_attention(ctypes.c_void_p(q.data_ptr()), *self._kv_args, *self._out_args,
                                           self._stream()))
        return self.out

    def step_timed(self, q: torch.Tensor, events: Sequence[torch.cuda.Event]) -> torch.Tensor:
        """``step`` that also records four timing events (before selection, after
        selection, after attention, after finalize) on the current stream.  The
        events must have been recorded once before (torch creates the CUDA event
        lazily on first use)."""
        _need_cuda(q)
        if len(events) != 4:
            raise ValueError("four events are needed")
        handles = (ctypes.c_void_p * 4)(*[ctypes.c_void_p(e.cuda_event) for e in events])
        kv = self.kv
        check(self.lib.ia_decode_attention_timed(
            _ptr(q), _ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.block_table), _ptr(kv.prefix_lens),
            _ptr(kv.seq_lens), ctypes.byref(self.c_summ), ctypes.byref(self.geom), self.mode, self.top_k,
            self.eps, self.max_sel, _REP[self.rep_mode], self.n_splits, self._ws_ptr(), self.ws_bytes,
            _ptr(self.sel_idx), _ptr(self.sel_count), _ptr(self.out), handles, _stream()))
        return self.out

    def step_host(self, q_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        if q_host.is_cuda or out_host.is_cuda:
            raise ValueError("step_host takes host tensors (pinned for full speed)")
        if q_host.shape != self._shape or q_host.dtype != self._dtype or not q_host.is_contiguous():
            raise ValueError(f"q_host must be a contiguous {self._shape} {self._dtype} tensor")
        if out_host.shape != self._shape or out_host.dtype != self._dtype or not out_host.is_contiguous():
            raise ValueError("out_host must match q_host")
        check(self.lib.ia_decode_attention_host(
            ctypes.c_void_p(q_host.data_ptr()), self._q_dev_ptr, *self._kv_args, self._out_ptr,
            ctypes.c_void_p(out_host.data_ptr()), self._stream()))
        return out_host


def decode_attention_noalloc(
    q: torch.Tensor, kv: PagedKV, summ: BlockSummaries, out: torch.Tensor, *, top_k: Optional[int] = None,
    eps: Optional[float] = None, rep_mode: str = "sparse_only", n_splits: int = 1,
    max_sel: Optional[int] = None,
) -> torch.Tensor:
    """One decode-attention layer-step with no device allocation anywhere.

    For hosts that cannot allocate device memory once they are running (an
    inference server that reserved all of HBM for its KV pool; a loop that must
    stay allocation-free).  The caller passes ``q`` and ``out`` (same shape and
    dtype); the step's scratch is a fixed array inside the shared library
    instead of a workspace tensor, so neither this function nor the library
    calls an allocator.  Limits and caveats: the step must fit in
    ``ia_noalloc_scratch_bytes()`` (else ValueError); the first call on a
    device should come before any stream capture; calls share the array, so
    calls that overlap on the GPU race - keep them on one stream.
    """
    lib = _lib.load()
    _need_cuda(q, out)
    if (top_k is None) == (eps is None):
        raise ValueError("give exactly one of top_k and eps")
    if rep_mode not in _REP:
        raise ValueError(f"rep_mode must be one of {sorted(_REP)}")
    group = _q_geom(q, kv.n_kv_heads)
    if out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous() or q.dtype != kv.k_pool.dtype:
        raise ValueError("out must be a contiguous tensor of q's shape and dtype (the KV dtype)")
    mode = IA_SELECT_TOPK if top_k is not None else IA_SELECT_EPS
    if max_sel is None:
        max_sel = max(int(top_k), 1) if top_k is not None else summ.max_blocks
    g = kv.geom(group, summ.block_size, summ.max_blocks, summ)
    s = summ.c_struct()
    check(lib.ia_decode_attention_noalloc(
        _ptr(q), _ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.block_table), _ptr(kv.prefix_lens), _ptr(kv.seq_lens),
        ctypes.byref(s), ctypes.byref(g), mode, int(top_k or 0), float(eps or 0.0), int(max_sel), _REP[rep_mode],
        int(n_splits), _ptr(out), _stream()))
    return out


def last_decode_fused() -> bool:
    """True when this thread's last layer step (``DecodeAttention.step`` and its variants) ran as the single
    fused launch ``condition_block_select_attend_kernel`` rather than as selection + attention."""
    return bool(_lib.load().ia_last_decode_fused())


def last_step_phases() -> Tuple[float, float]:
    """(selection_us, attention_us) of the last completed one-kernel step on the current device, as seen by
    the kernel's first CTA.  Synchronises (a device-to-host copy)."""
    sel, att = ctypes.c_double(0.0), ctypes.c_double(0.0)
    check(_lib.load().ia_last_step_phases(ctypes.byref(sel), ctypes.byref(att)))
    return float(sel.value), float(att.value)


def set_fused_step(enabled: bool) -> bool:
    """Allow (default) or forbid the one-kernel form of the layer step, process-wide; returns the previous
    setting.  For A/B measurements: the two-kernel form is what runs anyway where the fused one does not apply."""
    return bool(_lib.load().ia_set_fused_step(1 if enabled else 0))


def device_status() -> int:
    """Read and clear the device status word, an OR of the ``_lib.IA_DEV_STATUS_*`` masks: a bounded
    wait inside a kernel ran out (SELECT_WAIT, GEMM_WAIT, PEER_WAIT: that result is invalid), or a
    caller-supplied block index / block-table entry was out of range and skipped (BAD_INDEX).
    Synchronises the device."""
    lib = _lib.load()
    v = ctypes.c_int(0)
    check(lib.ia_read_device_status(ctypes.byref(v)))
    return int(v.value)
