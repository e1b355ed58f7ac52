"""1/2/4/8-GPU partitioning of the decode-attention layer-step.

Two ways the step shards (one process per GPU, ``torch.distributed``):

* **batch x kv-head sharding** - the units (sequence, kv head) share nothing:
  summaries, selection, pages and output rows are all per unit.  Each rank
  owns a subset of units and runs the ordinary single-GPU step on them; there
  is no collective on the data path.  ``plan_unit_shards`` balances the
  subsets by attended tokens (longest-processing-time greedy), which matters
  for ragged batches.

* **split-KV** for long single sequences - each rank owns a contiguous range
  of logical blocks of every sequence (their K/V pages).  Block summaries are
  small (about 1 KB per 64 tokens) and are replicated, so every rank computes
  the same global selection with no exchange; it then attends over the
  selected blocks inside its own range (the suffix lives on the last rank)
  and the ranks all-gather their normalised partials ``(o, lse)`` -
  ``rows x (D + 1)`` floats per rank, tens of KB - over NCCL / NVLink and
  merge them with the same log-sum-exp finalize kernel that merges split-KV
  parts inside one GPU.

The reference has no multi-GPU form of this path; its single-GPU building
block is the ``(acc, m, l)`` merge of
``condition_block_triton_impl/legacy.py:765-794``.
"""

from __future__ import annotations

import os
import threading
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

# The peer buffers of the in-kernel exchange are written with plain NVLink stores only.  By default
# torch's symmetric memory also binds every buffer to an NVSwitch multicast object; a rank that
# exits while its memory is bound to one can fault the other ranks' GPUs, and nothing here uses
# multimem, so the binding is switched off before the first symmetric allocation.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


def ordered_shutdown(graphs: Sequence = (), steps: Sequence = (), group=None, watchdog_s: float = 30.0) -> bool:
    """Leave a multi-GPU run in the order the libraries need.

    A communicator cannot be destroyed while a captured CUDA graph still holds its kernels: NCCL
    counts every graph that captured one of its collectives as a reference on the communicator and
    its teardown waits until those references are gone, i.e. until the graphs are destroyed - a
    teardown issued while the Python objects holding the graphs are alive therefore never returns.
    So: (1) destroy the graphs, (2) release the split-KV step objects (their symmetric-memory
    handles), (3) drain the device, (4) meet the other ranks, (5) destroy the process group.  The
    last call runs under a watchdog thread: if it has not returned after ``watchdog_s`` seconds the
    process leaves with ``os._exit(0)`` - the device is idle at that point, so nothing is cut off.
    Returns True when the process group was destroyed normally."""
    for g in graphs:
        try:
            g.reset()
        except Exception:
            pass
    for s in steps:
        close = getattr(s, "close", None)
        if close is not None:
            close()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if not dist.is_initialized():
        return True
    dist.barrier(group)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    done = threading.Event()

    def guard():
        if not done.wait(watchdog_s):
            os._exit(0)

    threading.Thread(target=guard, daemon=True).start()
    dist.destroy_process_group()
    done.set()
    return True


# --------------------------------------------------------------------------
# plans (pure host arithmetic)
# --------------------------------------------------------------------------

def plan_block_ranges(n_blocks: int, world: int, align: int = 1) -> List[Tuple[int, int]]:
    """Contiguous, near-equal block ranges [lo, hi) for ranks 0..world-1 (some may be empty).
    ``align``: every boundary but the last is a multiple of it (the split-KV selection kernel
    streams summaries in tiles of 32 blocks, so its ranges are cut with ``align=32``)."""
    if world <= 0 or n_blocks < 0 or align <= 0:
        raise ValueError("world and align must be positive and n_blocks non-negative")
    units = (n_blocks + align - 1) // align
    cuts = [min(units * r // world * align, n_blocks) for r in range(world + 1)]
    cuts[-1] = n_blocks
    return [(cuts[r], cuts[r + 1]) for r in range(world)]


# --------------------------------------------------------------------------
# split-KV selection: what the ranks exchange, as host arithmetic
# --------------------------------------------------------------------------
# The selection kernel of a split-KV group (ia_select_split) exchanges two small things between the
# GPUs: per query row the softmax normalisers of its own blocks, and its own top-k candidates.  The
# two merges below are the same arithmetic on the host - for tests on any backend, and as the
# definition of what the kernel must compute.

def merge_row_normalisers(m: torch.Tensor, l: torch.Tensor, d: torch.Tensor, b_all: torch.Tensor):
    """Per-rank running-softmax states of every query row -> the global ones.

    ``m, l, d, b_all``: [world, rows]; on each rank ``m`` = max of z over its blocks, ``l`` = sum of
    e^(z - m), ``d`` = sum of e^(z - m) cosh(delta), ``b_all`` = its largest value norm (a rank
    without blocks has m = -inf, l = d = 0).  Returns ``(M, L, D, B)`` [rows] with the same meaning
    over all blocks; ranks are summed in rank order."""
    top = m.amax(dim=0)
    safe = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    w = torch.where(torch.isfinite(m), torch.exp(m - safe), torch.zeros_like(m))
    return top, (l * w).sum(dim=0), (d * w).sum(dim=0), b_all.amax(dim=0)


def merge_topk_candidates(scores: Sequence[torch.Tensor], blocks: Sequence[torch.Tensor], k: int) -> torch.Tensor:
    """Per-rank candidate lists (scores and ascending global block indices, ranks in ascending block
    order) -> the global top-k block indices, ascending.  Higher score first; among equal scores
    the lower block index, which is the earlier position of the concatenated list."""
    sc = torch.cat([x.flatten() for x in scores])
    bl = torch.cat([x.flatten() for x in blocks])
    k_eff = min(int(k), int(sc.numel()))
    order = torch.sort(sc, descending=True, stable=True).indices[:k_eff]
    return torch.sort(bl[order]).values


def unit_costs(prefix_lens: Sequence[int], n_kv_heads: int, block_size: int, top_k: int,
               suffix_lens: Optional[Sequence[int]] = None) -> List[int]:
    """Attended tokens of every unit (sequence-major, then kv head): min(k, blocks) * block + suffix."""
    costs = []
    for i, n in enumerate(prefix_lens):
        blocks = (int(n) + block_size - 1) // block_size
        tokens = min(int(top_k), blocks) * block_size + (int(suffix_lens[i]) if suffix_lens is not None else 0)
        costs.extend([tokens] * n_kv_heads)
    return costs


def plan_unit_shards(costs: Sequence[int], world: int) -> List[List[int]]:
    """Assign units to ranks, heaviest first onto the lightest rank; ties go to the lower rank.
    Returns, per rank, the sorted unit ids it owns."""
    if world <= 0:
        raise ValueError("world must be positive")
    loads = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for unit in sorted(range(len(costs)), key=lambda u: (-costs[u], u)):
        r = min(range(world), key=lambda i: (loads[i], i))
        owned[r].append(unit)
        loads[r] += costs[unit]
    return [sorted(x) for x in owned]


def plan_head_shards(n_kv_heads: int, world: int) -> List[Tuple[int, int]]:
    """kv heads [lo, hi) per rank when the head count divides over the ranks
    (8 kv heads: one per GPU on 8, two on 4, four on 2)."""
    if n_kv_heads % world != 0:
        raise ValueError(f"{n_kv_heads} kv heads do not divide over {world} ranks")
    per = n_kv_heads // world
    return [(r * per, (r + 1) * per) for r in range(world)]


# --------------------------------------------------------------------------
# the one exchange step of split-KV
# --------------------------------------------------------------------------

def allgather_partials(o: torch.Tensor, lse: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """o [rows, D] f32 and lse [rows] f32 of this rank -> (o [rows, world, D], lse [rows, world]).

    One all-gather of the packed ``[rows, D + 1]`` buffer; works on any backend
    (NCCL on GPUs, gloo on the CPU for tests)."""
    if o.dtype != torch.float32 or lse.dtype != torch.float32:
        raise ValueError("partials are float32")
    world = dist.get_world_size(group)
    rows, d = o.shape
    packed = torch.cat([o, lse.unsqueeze(1)], dim=1).contiguous()
    gathered = torch.empty((world * rows, d + 1), dtype=torch.float32, device=o.device)  # rank-major concatenation
    dist.all_gather_into_tensor(gathered, packed, group=group)
    gathered = gathered.view(world, rows, d + 1).permute(1, 0, 2)
    return gathered[..., :d].contiguous(), gathered[..., d].contiguous()


@dataclass
class SplitKVStep:
    """One rank's half of a split-KV decode-attention layer-step.

    ``select`` returns the global selection (identical on every rank),
    ``attend(block_range, with_suffix)`` this rank's normalised partial
    ``(o [rows, D], lse [rows])`` over its share, ``merge(o [rows, W, D],
    lse [rows, W])`` the final output.  On GPUs these are the CUDA operators
    (see ``cuda_split_kv_step``); the CPU tests plug in the oracle."""

    select: Callable[[], object]
    attend: Callable[[object, Tuple[int, int], bool], Tuple[torch.Tensor, torch.Tensor]]
    merge: Callable[[torch.Tensor, torch.Tensor], torch.Tensor]

    def run(self, n_blocks: int, group=None) -> torch.Tensor:
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        lo, hi = plan_block_ranges(n_blocks, world)[rank]
        selection = self.select()
        o, lse = self.attend(selection, (lo, hi), rank == world - 1)
        all_o, all_lse = allgather_partials(o, lse, group)
        return self.merge(all_o, all_lse)


def cuda_split_kv_step(q, kv, summ, *, top_k=None, eps=None, rep_mode="sparse_only", n_splits=2,
                       out_dtype=None) -> SplitKVStep:
    """The CUDA operators wired into a ``SplitKVStep``.

    ``kv`` is this rank's paged cache: its block table needs valid entries only
    for the pages of its own block range (and, on the last rank, the suffix);
    ``summ`` holds the summaries of all blocks (replicated)."""
    from . import ops
    nb = summ.max_blocks
    rows, d = q.shape[0] * q.shape[1], q.shape[2]
    out_dtype = out_dtype or q.dtype

    def select():
        idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=top_k, eps=eps,
                                          want=("z",) if rep_mode == "hybrid" else ())
        return idx, cnt, aux.get("z")

    def attend(selection, block_range, with_suffix):
        idx, cnt, z = selection
        o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=summ.block_size, max_blocks=nb, rep_mode=rep_mode,
                                   summ=summ, z=z, n_splits=n_splits, block_range=block_range,
                                   with_suffix=with_suffix)
        part, part_lse = ops.finalize(o, lse, torch.float32, return_lse=True)
        return part.reshape(rows, d), part_lse.reshape(rows)

    def merge(all_o, all_lse):
        return ops.finalize(all_o, all_lse, out_dtype).reshape(q.shape)

    return SplitKVStep(select, attend, merge)


class SplitKVDecodeAttention:
    """One rank's split-KV layer-step with every buffer preallocated: four launches
    (selection, attention over this rank's block range, one NCCL all-gather of the
    partials, merge), nothing allocated per step, so the step can be captured into a
    CUDA graph together with its collective.

    ``kv`` needs valid pages only for this rank's block range (and the suffix on the
    last rank); ``summ`` holds the summaries of all blocks (replicated), so every rank
    computes the same global selection without an exchange.  The all-gather moves each
    rank's split partials as they are (``[rows, n_splits, D]`` values and ``[rows,
    n_splits]`` log-sum-exps, adjacent in one buffer) and the merge reads the gathered
    chunks in place (``ia_finalize_gathered``)."""

    def __init__(self, kv, summ, n_q_heads: int, *, top_k=None, eps=None, rep_mode: str = "sparse_only",
                 n_splits: int = 4, group=None):
        from . import ops
        self.ops, self.kv, self.summ, self.group = ops, kv, summ, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.top_k, self.eps, self.rep_mode, self.n_splits = top_k, eps, rep_mode, int(n_splits)
        nb = summ.max_blocks
        self.block_range = plan_block_ranges(nb, self.world)[self.rank]
        self.with_suffix = self.rank == self.world - 1
        b, d = kv.batch, kv.head_dim
        self.rows = b * int(n_q_heads)
        dev = kv.k_pool.device
        max_sel = max(int(top_k), 1) if top_k is not None else nb
        self.sel_idx = torch.empty((b, kv.n_kv_heads, max_sel), device=dev, dtype=torch.int32)
        self.sel_count = torch.empty((b, kv.n_kv_heads), device=dev, dtype=torch.int32)
        self.aux = {}
        if rep_mode == "hybrid":
            self.aux["z"] = torch.full((b, int(n_q_heads), nb), float("-inf"), device=dev, dtype=torch.float32)
        n_o = self.rows * self.n_splits * d
        self.chunk = (n_o + self.rows * self.n_splits + 3) // 4 * 4          # floats per rank, 16-byte multiple
        self.mine = torch.zeros((self.chunk,), device=dev, dtype=torch.float32)
        self.o_part = self.mine[:n_o].view(b, int(n_q_heads), self.n_splits, d)
        self.lse_part = self.mine[n_o:n_o + self.rows * self.n_splits].view(b, int(n_q_heads), self.n_splits)
        self.gathered = torch.empty((self.world * self.chunk,), device=dev, dtype=torch.float32)
        self.out = torch.empty((b, int(n_q_heads), d), device=dev, dtype=kv.k_pool.dtype)
        self.n_q_heads = int(n_q_heads)

    def step(self, q: torch.Tensor) -> torch.Tensor:
        ops = self.ops
        kw = dict(top_k=self.top_k) if self.top_k is not None else dict(eps=self.eps)
        ops.select_blocks(q, self.summ, self.kv.prefix_lens, out_idx=self.sel_idx, out_count=self.sel_count,
                          max_sel=int(self.sel_idx.shape[-1]), want=tuple(self.aux), aux_buffers=self.aux, **kw)
        ops.sparse_decode(q, self.kv, self.sel_idx, self.sel_count, block_size=self.summ.block_size,
                          max_blocks=self.summ.max_blocks, rep_mode=self.rep_mode, summ=self.summ,
                          z=self.aux.get("z"), n_splits=self.n_splits, block_range=self.block_range,
                          with_suffix=self.with_suffix, out=(self.o_part, self.lse_part))
        dist.all_gather_into_tensor(self.gathered, self.mine, group=self.group)
        ops.finalize_gathered(self.gathered, self.world, self.chunk, self.rows, self.n_splits, self.kv.head_dim,
                              self.out)
        return self.out


class SplitKVDecodeAttentionP2P:
    """The split-KV layer-step with every exchange inside the kernels: three launches (selection,
    attention, merge) and no collective call.

    ``selection="distributed"`` (default): every rank streams only the block summaries of its own
    range; the selection kernel exchanges the row normalisers and each rank's top-k candidates with
    the other ranks and every rank ends up with the same global selection (``ia_select_split``) -
    the selection's HBM traffic and time shrink with the number of GPUs.  ``"replicated"``: every
    rank holds all summaries and selects on its own (no exchange, no shrinking).

    The attention kernel stores every partial into the gather buffer of every rank through peer
    pointers (NVLink stores) and its last CTA publishes the step number in a flag on every rank;
    the merge kernel waits - bounded, about a second - for the flags of all ranks and merges the
    chunks in place.  All buffers are one block of symmetric memory
    (``torch.distributed._symmetric_memory``), mapped once at construction; a step allocates
    nothing and keeps its step counters on the device, so it can be captured into a CUDA graph.
    Plain peer stores only: the buffers are not bound to an NVSwitch multicast object
    (``TORCH_SYMM_MEM_DISABLE_MULTICAST``).  Every rank must construct the object (a collective),
    run the same number of steps and ``close()`` it (or leave through ``ordered_shutdown``) before
    the process group goes away.  ``check()`` reads the device status word at a point where the
    host waits anyway: a peer wait that ran out means ``out`` of that step is invalid."""

    launches_per_step = 3

    def __init__(self, kv, summ, n_q_heads: int, *, top_k=None, eps=None, rep_mode: str = "sparse_only",
                 n_splits: int = 4, group=None, selection: str = "distributed"):
        import ctypes
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"   # plain peer pointers only (see the module top)
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib, ops
        self.ops, self.lib, self.kv, self.summ = ops, _lib.load(), kv, summ
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        if selection not in ("distributed", "replicated"):
            raise ValueError("selection must be 'distributed' or 'replicated'")
        if selection == "distributed" and top_k is None:
            raise ValueError("the distributed selection is built for top-k routing; use selection='replicated' "
                             "with the epsilon rule")
        self.selection = selection
        self.top_k, self.eps, self.rep_mode, self.n_splits = top_k, eps, rep_mode, int(n_splits)
        nb = summ.max_blocks
        lo, hi = plan_block_ranges(nb, self.world, align=32)[self.rank]
        self.block_range = (lo, nb if hi >= nb else hi)
        self.with_suffix = self.rank == self.world - 1
        b, d = kv.batch, kv.head_dim
        self.n_q_heads, self.rows = int(n_q_heads), b * int(n_q_heads)
        pairs = b * kv.n_kv_heads
        dev = kv.k_pool.device
        max_sel = max(int(top_k), 1) if top_k is not None else nb
        self.sel_idx = torch.empty((b, kv.n_kv_heads, max_sel), device=dev, dtype=torch.int32)
        self.sel_count = torch.empty((b, kv.n_kv_heads), device=dev, dtype=torch.int32)
        self.aux = {}
        if rep_mode == "hybrid":
            self.aux["z"] = torch.full((b, self.n_q_heads, nb), float("-inf"), device=dev, dtype=torch.float32)
        # one symmetric buffer (floats): attention partials | attention flags | normalisers | candidates | flags
        W = self.world
        n_o = self.rows * self.n_splits * d
        chunk = (n_o + self.rows * self.n_splits + 3) // 4 * 4

        def take(n_floats, at=[0]):
            start = at[0]
            at[0] = (start + n_floats + 63) // 64 * 64          # 256-byte slots
            return start
        off_gather = take(2 * W * chunk)
        off_aflags = take(2 * W)
        off_norm = take(2 * pairs * W * 64)
        off_cand = take(2 * pairs * W * (max_sel + 1) * 2)
        off_sflags = take(2 * 2 * pairs * W)
        total = take(0)
        self.buf = symm_mem.empty(total, dtype=torch.float32, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize(dev)
        self.handle = symm_mem.rendezvous(self.buf, group=group.group_name)
        self.counters = torch.zeros(4, device=dev, dtype=torch.int32)   # attention step / grid, selection step / grid
        px, sx = _lib.PeerExchange(), _lib.SelectExchange()
        px.n_ranks, px.my_rank = W, self.rank
        sx.n_ranks, sx.my_rank = W, self.rank
        for w in range(W):
            base = int(self.handle.buffer_ptrs[w])
            px.gather[w] = base + 4 * off_gather
            px.flags[w] = base + 4 * off_aflags
            sx.norm[w] = base + 4 * off_norm
            sx.cand[w] = base + 4 * off_cand
            sx.flags[w] = base + 4 * off_sflags
        px.chunk_floats, px.lse_offset = chunk, n_o
        px.step_counter = self.counters.data_ptr()
        px.grid_counter = self.counters.data_ptr() + 4
        sx.step_counter = self.counters.data_ptr() + 8
        sx.grid_counter = self.counters.data_ptr() + 12
        self.px, self.sx, self._byref = px, sx, ctypes.byref
        self.out = torch.empty((b, self.n_q_heads, d), device=dev, dtype=kv.k_pool.dtype)
        self.geom = kv.geom(self.n_q_heads // kv.n_kv_heads, summ.block_size, nb, summ)
        self.c_summ = summ.c_struct()
        self.c_aux = _lib.SelectAux(None, self.aux["z"].data_ptr() if "z" in self.aux else None, None, None, None)
        self._group = group
        dist.barrier(group)                                # every rank's buffer is zeroed and mapped

    def check(self) -> None:
        """Synchronise and raise if a bounded wait for a peer ran out during the steps so far."""
        from ._lib import IA_DEV_STATUS_PEER_WAIT
        status = self.ops.device_status()
        if status & IA_DEV_STATUS_PEER_WAIT:
            raise RuntimeError("split-KV exchange: a wait for a peer ran out; the output of that step is invalid "
                               "(a rank is missing or far behind)")

    def close(self) -> None:
        """Release the peer mappings.  Collective: every rank drains its device and meets the others
        first, so that no peer is still storing into or polling this rank's buffers."""
        if getattr(self, "buf", None) is None:
            return
        torch.cuda.synchronize()
        dist.barrier(self._group)
        self.handle = None
        self.buf = None
        self.px = self.sx = None

    def step(self, q: torch.Tensor) -> torch.Tensor:
        from ._lib import check
        ops, kv = self.ops, self.kv
        p, s = ops._ptr, ops._stream()
        lo, hi = self.block_range
        max_sel = int(self.sel_idx.shape[-1])
        if self.selection == "distributed":
            check(self.lib.ia_select_split(
                p(q), self._byref(self.c_summ), p(kv.prefix_lens), self._byref(self.geom), int(self.top_k), max_sel,
                int(lo), int(hi), p(self.sel_idx), p(self.sel_count), self._byref(self.c_aux), self._byref(self.sx), s))
        else:
            kw = dict(top_k=self.top_k) if self.top_k is not None else dict(eps=self.eps)
            ops.select_blocks(q, self.summ, kv.prefix_lens, out_idx=self.sel_idx, out_count=self.sel_count,
                              max_sel=max_sel, want=tuple(self.aux), aux_buffers=self.aux, **kw)
        check(self.lib.ia_sparse_decode_exchange(
            p(q), p(kv.k_pool), p(kv.v_pool), p(kv.block_table), p(kv.prefix_lens), p(kv.seq_lens),
            p(self.sel_idx), p(self.sel_count), max_sel, self._byref(self.c_summ),
            p(self.aux.get("z")), self._byref(self.geom), ops._REP[self.rep_mode], self.n_splits, int(lo), int(hi),
            int(self.with_suffix), self._byref(self.px), s))
        check(self.lib.ia_finalize_exchange(self._byref(self.px), self.rows, self.n_splits, kv.head_dim,
                                            p(self.out), ops._DTYPES[self.out.dtype], s))
        return self.out
