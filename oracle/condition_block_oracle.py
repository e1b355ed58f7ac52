"""CPU oracle for the condition-block sparse decode-attention path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
only the test-suite, the smoke check and the benchmark's CPU-baseline leg do,
and there only as the checker / the timed CPU arm.

Every function restates, in plain fp32 torch on the CPU, one piece of the
reference algorithm (paths are relative to the reference project root;
``IMPL`` = ``llama/script/analysis/condition_block_gen/methods/
condition_block_triton_impl``, ``GEN`` = ``llama/script/analysis/
condition_block_gen``):

* ``block_summaries``      - IMPL/core.py:449-500 (and the fp32 twin
                             GEN/methods/condition_block.py:150-180)
* ``condition_terms``      - IMPL/core.py:509-546, stopping before the
                             ``> eps`` comparison
* ``score_from_stats``     - condition_block_ppl/runner_cond_block.py:279-294
* ``diag_ell_stats`` / ``condition_terms(bound="diag_ell")`` - the diagonal-
                             ellipsoid bound of condition_block_ball/gen_selection.py:
                             21-87 (w, rho per block; delta = rho |q * w| / sqrt(D))
* ``select_threshold``     - IMPL/core.py:546 (the reference's epsilon rule)
* ``select_topk``          - no reference counterpart for blocks; the ranking
                             precedent is GEN/methods/quest.py:91-103 (GQA-mean
                             score, top-k).  Tie order is defined here: higher
                             score first, lower block index first among equals.
* ``decode_attention``     - IMPL/legacy.py:797-868 (hybrid: unselected blocks
                             contribute one representative each) and
                             condition_block_ppl/runner_quest.py:230-239
                             (sparse-only: selected blocks + suffix)
* ``decode_attention_dense`` - the same result in the dense masked form of
                             IMPL/legacy.py:797-868: every prefix token is
                             scored, unselected ones are masked (the
                             reference's dense CPU leg, timed by the benchmark)
* ``merge_acc_m_l``        - IMPL/legacy.py:781-793
* ``merge_o_lse``          - the same merge written for (o, lse) partials
* ``condition_stats``      - IMPL/core.py:1441-1456 (per-step statistics)

Parity status: pinned.  ``tests/test_oracle_vs_reference.py`` checks these
functions against the reference's own functions when the reference tree is
importable, and ``tests/test_oracle_golden.py`` checks them against vectors
produced by the reference and committed under ``tests/golden/``.  Both modes of
``decode_attention`` are pinned: ``hybrid`` to the reference's dense function
and to its compact-SDPA function, ``sparse_only`` to the dense function called
with ``cluster_exists`` all false (IMPL/legacy.py:828-829 then masks every
representative, leaving selected tokens + suffix).
One exception - parity unpinned: the ``term1_mass_exp`` branch of
``score_from_stats`` restates a variant the reference has only as a Triton
kernel (IMPL/core.py:798-803, 893-896), which cannot run where the pins run.

The reference handles one sequence at a time; so does every function here
(``*_batch`` helpers loop).  Physical paging is not a reference concept: pages
are gathered into logical token order first (``gather_logical``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


# --------------------------------------------------------------------------
# paging
# --------------------------------------------------------------------------

def gather_logical(pool: torch.Tensor, table_row: torch.Tensor, n_tokens: int) -> torch.Tensor:
    """pool [n_pages, Hkv, P, D] + one sequence's page list -> [Hkv, n_tokens, D]."""
    page = int(pool.shape[2])
    n_pages = (int(n_tokens) + page - 1) // page
    idx = table_row[:n_pages].long()
    x = pool[idx]                       # [n_pages, Hkv, P, D]
    x = x.permute(1, 0, 2, 3).reshape(pool.shape[1], n_pages * page, pool.shape[3])
    return x[:, : int(n_tokens)]


# --------------------------------------------------------------------------
# block summaries
# --------------------------------------------------------------------------

@dataclass
class Summaries:
    """Per-(kv head, block) statistics of the summarised prefix."""

    k_bar: torch.Tensor        # [Hkv, nb, D] fp32 (or the storage dtype)
    v_bar: torch.Tensor        # [Hkv, nb, D]
    k_max: torch.Tensor        # [Hkv, nb, D]
    k_min: torch.Tensor        # [Hkv, nb, D]
    v_norm_max: torch.Tensor   # [Hkv, nb] fp32
    counts: torch.Tensor       # [nb] int64, valid tokens per block
    block_size: int

    @property
    def n_blocks(self) -> int:
        return int(self.counts.numel())


def block_counts(prefix_len: int, block_size: int) -> torch.Tensor:
    nb = (int(prefix_len) + block_size - 1) // block_size
    starts = torch.arange(nb, dtype=torch.long) * block_size
    return (int(prefix_len) - starts).clamp(min=0, max=block_size)


def _blocked(x: torch.Tensor, block_size: int) -> Tuple[torch.Tensor, int]:
    heads, length = x.shape[:2]
    nb = (length + block_size - 1) // block_size
    tail = nb * block_size - length
    if tail:
        x = torch.cat([x, x.new_zeros((heads, tail, x.shape[2]))], dim=1)
    return x.reshape(heads, nb, block_size, x.shape[2]), nb


def block_summaries(
    k_all: torch.Tensor,
    v_all: torch.Tensor,
    block_size: int,
    storage: str = "fp32",
) -> Summaries:
    """Summaries of a [Hkv, L, D] prefix.

    ``storage="fp32"`` keeps every statistic in fp32 (the reference default);
    ``storage="mixed"`` keeps k_bar in fp32, v_bar and the coordinate bounds in
    the source dtype (the reference's CONDITION_BLOCK_MIXED_SUMMARIES layout,
    IMPL/core.py:411-446).  Sums are accumulated in fp32 in both cases.
    """
    kb, nb = _blocked(k_all, block_size)
    vb, _ = _blocked(v_all, block_size)
    length = int(k_all.shape[1])
    tok = torch.arange(nb * block_size).reshape(nb, block_size)
    live = tok < length                                   # [nb, B]
    live4 = live.view(1, nb, block_size, 1)
    counts = live.sum(dim=1).long()
    denom = counts.clamp_min(1).float().view(1, nb, 1)

    k_sum = (kb * live4).sum(dim=2, dtype=torch.float32)
    v_sum = (vb * live4).sum(dim=2, dtype=torch.float32)
    k_hi = kb.masked_fill(~live4, float("-inf")).amax(dim=2)
    k_lo = kb.masked_fill(~live4, float("inf")).amin(dim=2)
    v_len = torch.linalg.vector_norm(vb, dim=-1, dtype=torch.float32)
    v_len = v_len.masked_fill(~live.view(1, nb, block_size), float("-inf"))

    k_bar = k_sum / denom
    v_bar = v_sum / denom
    if storage == "fp32":
        k_hi, k_lo = k_hi.float(), k_lo.float()
    elif storage == "mixed":
        v_bar = v_bar.to(v_all.dtype)
    else:
        raise ValueError(f"unknown summary storage {storage!r}")
    return Summaries(
        k_bar=k_bar, v_bar=v_bar, k_max=k_hi, k_min=k_lo,
        v_norm_max=v_len.amax(dim=2), counts=counts, block_size=int(block_size),
    )


# --------------------------------------------------------------------------
# condition score
# --------------------------------------------------------------------------

def score_from_stats(p: torch.Tensor, delta: torch.Tensor, b_c: torch.Tensor, b_all: torch.Tensor,
                     term1_mass_exp: bool = False) -> torch.Tensor:
    """Two-term block condition given softmax mass p, range bound delta and the
    value-norm bounds (per block b_c, global b_all).

    ``term1_mass_exp``: the first term is ``2 b_all softmax(z + delta)`` - the variant the
    reference has only as a Triton kernel (core.py:798-803 forms ``zc = z + delta``,
    core.py:893-896 ``term1 = 2 b_all exp(z + delta - c_m) / c_l``), restated here from those
    lines; no CPU implementation of it exists in the reference, so this variant's parity is
    unpinned."""
    if term1_mass_exp:
        e = torch.exp(delta)
        norm = (p * e).sum(dim=-1).clamp_min(1e-30)
        first = 2.0 * b_all.unsqueeze(-1) * e / norm.unsqueeze(-1)
        return p * (first + 2.0 * b_c * torch.tanh(delta / 2.0))
    ch = torch.cosh(delta)
    norm = (p * ch).sum(dim=-1).clamp_min(1e-30)
    first = 2.0 * b_all.unsqueeze(-1) * (ch - 1.0) / norm.unsqueeze(-1)
    second = 2.0 * b_c * torch.tanh(delta / 2.0)
    return p * (first + second)


def diag_ell_stats(k_all: torch.Tensor, summ: Summaries, w_dtype: Optional[torch.dtype] = None):
    """The diagonal-ellipsoid summaries of condition_block_ball/gen_selection.py:21-73:
    ``w = max(k_max - k_bar, k_bar - k_min)`` clamped at 1e-6 (one vector per block), optionally stored
    in bf16 after a round-up bump of ``1 + 2^-7`` (their CONDITION_BLOCK_BALL_W_DTYPE option), and
    ``rho = max_t |(k_t - k_bar) / w|`` computed with the stored w - in the reference's expanded form
    ``|k|^2_w - 2 k . k_bar_w + |k_bar|^2_w``.  k_all [Hkv, L, D] is the summarised prefix.
    Returns (w [Hkv, nb, D], rho [Hkv, nb] fp32)."""
    k_bar = summ.k_bar.float()
    w = torch.maximum(summ.k_max.float() - k_bar, k_bar - summ.k_min.float()).clamp_min(1e-6)
    if w_dtype == torch.bfloat16:
        w = (w * (1.0 + 2.0 ** -7)).to(torch.bfloat16)
    inv_w2 = w.float().pow(-2)
    kb, nb = _blocked(k_all.float(), summ.block_size)                  # [Hkv, nb, B, D]
    live = torch.arange(summ.block_size).view(1, -1) < summ.counts.view(-1, 1)
    k_norm2 = torch.einsum("hbtd,hbd->hbt", kb.pow(2), inv_w2)
    dot = torch.einsum("hbtd,hbd->hbt", kb, k_bar * inv_w2)
    offset = (k_bar.pow(2) * inv_w2).sum(dim=-1)
    dist2 = (k_norm2 - 2.0 * dot + offset.unsqueeze(-1)).masked_fill(~live.unsqueeze(0), float("-inf"))
    return w, dist2.amax(dim=-1).clamp_min(0.0).sqrt()


def condition_terms(q_grouped: torch.Tensor, summ: Summaries, term1_mass_exp: bool = False,
                    diag_ell=None) -> Dict[str, torch.Tensor]:
    """q_grouped [Hkv, G, D] -> per-row and per-head quantities of the score.

    Returns ``s`` (q.k_bar/sqrt(D)), ``delta`` (range bound), ``z`` (s + log
    count, -inf for empty blocks), ``cond`` [Hkv, G, nb] and ``score`` =
    mean over the G query rows of a kv head, [Hkv, nb].
    ``diag_ell=(w, rho)``: the bound is ``rho |q * w| / sqrt(D)`` (condition_block_ball/
    gen_selection.py:82-87) instead of the coordinate-range bound; everything else is the same.
    """
    q = q_grouped.float()
    hkv, g, d = q.shape
    root = d ** 0.5
    exists = (summ.counts > 0).view(1, 1, -1)
    k_bar = summ.k_bar.to(q.dtype)

    q4 = q.view(hkv, g, 1, d)
    s = (torch.einsum("gsqd,gbd->gsqb", q4, k_bar) / root)[:, :, 0]
    if diag_ell is not None:
        w, rho = diag_ell
        qw = torch.sqrt(torch.einsum("gsqd,gbd->gsqb", q4.pow(2), w.float().pow(2)).clamp_min(0.0))[:, :, 0]
        delta = (rho.float()[:, None, :] * qw / root).masked_fill(~exists, 0.0)
    else:
        k_hi = summ.k_max.to(q.dtype)
        k_lo = summ.k_min.to(q.dtype)
        qb = q4[:, :, :, None, :]
        hi_prod = qb * k_hi[:, None, None]
        lo_prod = qb * k_lo[:, None, None]
        upper = (torch.maximum(hi_prod, lo_prod).sum(dim=-1) / root)[:, :, 0]
        lower = (torch.minimum(hi_prod, lo_prod).sum(dim=-1) / root)[:, :, 0]
        delta = torch.maximum((upper - s).abs(), (lower - s).abs()).masked_fill(~exists, 0.0)

    b_c = summ.v_norm_max.float()[:, None, :].expand(hkv, g, -1).masked_fill(~exists, 0.0)
    b_all = b_c.amax(dim=-1)
    z = torch.log(summ.counts.clamp_min(1).float()).view(1, 1, -1) + s
    z = z.masked_fill(~exists, float("-inf"))
    p = torch.softmax(z, dim=-1)
    cond = score_from_stats(p, delta, b_c, b_all, term1_mass_exp)
    return {"s": s, "delta": delta, "z": z, "p": p, "cond": cond, "score": cond.mean(dim=1)}


def select_threshold(score: torch.Tensor, counts: torch.Tensor, eps: float) -> torch.Tensor:
    """bool [Hkv, nb]: blocks whose score exceeds eps and that hold a token."""
    return (score > eps) & (counts > 0).view(1, -1)


def select_topk(score: torch.Tensor, counts: torch.Tensor, k: int) -> Tuple[List[List[int]], torch.Tensor]:
    """Top-k blocks per kv head among blocks that hold a token.

    Order: score descending, block index ascending among equal scores (a stable
    sort of the negated scores).  Returns (ranked index lists, bool mask)."""
    hkv, nb = score.shape
    alive = (counts > 0).nonzero().flatten()
    k_eff = min(int(k), int(alive.numel()))
    ranked: List[List[int]] = []
    mask = torch.zeros((hkv, nb), dtype=torch.bool)
    for h in range(hkv):
        vals = score[h, alive]
        order = torch.sort(vals, descending=True, stable=True).indices[:k_eff]
        chosen = alive[order]
        ranked.append([int(i) for i in chosen])
        mask[h, chosen] = True
    return ranked, mask


# --------------------------------------------------------------------------
# decode attention given a block mask
# --------------------------------------------------------------------------

def decode_attention(
    q_grouped: torch.Tensor,
    k_all: torch.Tensor,
    v_all: torch.Tensor,
    prefix_len: int,
    block_size: int,
    mask: torch.Tensor,
    *,
    rep_mode: str,
    z: Optional[torch.Tensor] = None,
    v_bar: Optional[torch.Tensor] = None,
    block_range: Optional[Tuple[int, int]] = None,
    with_suffix: bool = True,
    return_lse: bool = False,
):
    """One decode step for one sequence.

    q_grouped [Hkv, G, D]; k_all/v_all [Hkv, L, D] hold the summarised prefix
    (first ``prefix_len`` tokens) followed by the generated suffix.  ``mask``
    [Hkv, nb] marks the selected blocks.  A joint softmax runs over (i) every
    token of a selected block, (ii) in ``rep_mode="hybrid"`` one representative
    per unselected non-empty block with logit ``z`` and value ``v_bar``,
    (iii) every suffix token.  ``rep_mode="sparse_only"`` drops (ii).
    ``block_range=(lo, hi)`` restricts (i) and (ii) to blocks lo <= b < hi (one
    rank's share in split-KV); ``with_suffix=False`` drops (iii).
    Returns out [Hkv, G, D] fp32 (and lse [Hkv, G] when asked; rows with
    nothing to attend to give out = 0, lse = -inf).
    """
    q = q_grouped.float()
    hkv, g, d = q.shape
    root = d ** 0.5
    total = int(k_all.shape[1])
    nb = int(mask.shape[1])
    lo, hi = (0, nb) if block_range is None else block_range
    in_range = torch.zeros(nb, dtype=torch.bool)
    in_range[lo:hi] = True
    counts = block_counts(prefix_len, block_size)

    out = torch.zeros((hkv, g, d), dtype=torch.float32)
    lse = torch.full((hkv, g), float("-inf"), dtype=torch.float32)
    for h in range(hkv):
        logits: List[torch.Tensor] = []
        values: List[torch.Tensor] = []
        picked = (mask[h] & in_range & (counts > 0)).nonzero().flatten().tolist()
        if picked:
            tok = torch.cat([
                torch.arange(b * block_size, b * block_size + int(counts[b])) for b in picked
            ])
            kk = k_all[h, tok].float()
            logits.append(q[h] @ kk.T / root)                      # [G, n_tok]
            values.append(v_all[h, tok].float()[None].expand(g, -1, -1))
        if rep_mode == "hybrid":
            reps = ((~mask[h]) & in_range & (counts > 0)).nonzero().flatten()
            if reps.numel():
                logits.append(z[h][:, reps].float())
                values.append(v_bar[h, reps].float()[None].expand(g, -1, -1))
        elif rep_mode != "sparse_only":
            raise ValueError(f"unknown rep_mode {rep_mode!r}")
        if with_suffix and total > prefix_len:
            ks = k_all[h, prefix_len:total].float()
            logits.append(q[h] @ ks.T / root)
            values.append(v_all[h, prefix_len:total].float()[None].expand(g, -1, -1))
        if not logits:
            continue
        lg = torch.cat(logits, dim=1)
        vv = torch.cat(values, dim=1)
        top = lg.amax(dim=1, keepdim=True)
        w = torch.exp(lg - top)
        norm = w.sum(dim=1, keepdim=True)
        out[h] = torch.einsum("gt,gtd->gd", w, vv) / norm.clamp_min(1e-30)
        lse[h] = (top + torch.log(norm))[:, 0]
    return (out, lse) if return_lse else out


def decode_attention_dense(
    q_grouped: torch.Tensor,
    k_all: torch.Tensor,
    v_all: torch.Tensor,
    prefix_len: int,
    block_size: int,
    mask: torch.Tensor,
    *,
    rep_mode: str,
    z: Optional[torch.Tensor] = None,
    v_bar: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``decode_attention`` in the dense masked form of IMPL/legacy.py:797-868.

    Every token of the blocked prefix gets a logit (one [G, nb * B] product per
    kv head); tokens of unselected or padded positions are masked to -inf, the
    representatives of unselected non-empty blocks enter with logit ``z``
    (``rep_mode="hybrid"``) or are all masked (``"sparse_only"`` - the reference
    function called with ``cluster_exists`` all false), the suffix follows, and
    one softmax runs over the three parts.  Same result as
    ``decode_attention``; the cost grows with the context instead of with the
    selection, which is what makes it the reference's *dense* CPU leg."""
    if rep_mode not in ("hybrid", "sparse_only"):
        raise ValueError(f"unknown rep_mode {rep_mode!r}")
    q = q_grouped.float()
    hkv, g, d = q.shape
    root = d ** 0.5
    total = int(k_all.shape[1])
    kb, nb = _blocked(k_all[:, :prefix_len].float(), block_size)      # [Hkv, nb, B, D]
    vb, _ = _blocked(v_all[:, :prefix_len].float(), block_size)
    counts = block_counts(prefix_len, block_size)
    live = torch.arange(block_size).view(1, -1) < counts.view(-1, 1)   # [nb, B]
    tok_on = mask.view(hkv, 1, nb, 1) & live.view(1, 1, nb, block_size)
    tok_logit = torch.einsum("hgd,hbtd->hgbt", q, kb) / root
    tok_logit = tok_logit.masked_fill(~tok_on, float("-inf"))
    parts = [tok_logit.flatten(2).amax(dim=-1)]
    rep_on = None
    if rep_mode == "hybrid":
        rep_on = ((~mask) & (counts > 0).view(1, -1)).view(hkv, 1, nb).expand(hkv, g, nb)
        rep_logit = z.float().masked_fill(~rep_on, float("-inf"))
        parts.append(rep_logit.amax(dim=-1))
    suf_logit = None
    if total > prefix_len:
        suf_logit = torch.einsum("hgd,htd->hgt", q, k_all[:, prefix_len:total].float()) / root
        parts.append(suf_logit.amax(dim=-1))
    top = torch.stack(parts, dim=0).amax(dim=0)                        # [Hkv, G]
    safe = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    tok_w = torch.exp(tok_logit - safe[:, :, None, None]).masked_fill(~tok_on, 0.0)
    norm = tok_w.flatten(2).sum(dim=-1)
    num = torch.einsum("hgbt,hbtd->hgd", tok_w, vb)
    if rep_on is not None:
        rep_w = torch.exp(rep_logit - safe[:, :, None]).masked_fill(~rep_on, 0.0)
        norm = norm + rep_w.sum(dim=-1)
        num = num + torch.einsum("hgb,hbd->hgd", rep_w, v_bar.float())
    if suf_logit is not None:
        suf_w = torch.exp(suf_logit - safe[:, :, None])
        norm = norm + suf_w.sum(dim=-1)
        num = num + torch.einsum("hgt,htd->hgd", suf_w, v_all[:, prefix_len:total].float())
    return num / norm.clamp_min(1e-30).unsqueeze(-1)


# --------------------------------------------------------------------------
# split-KV merge
# --------------------------------------------------------------------------

def merge_acc_m_l(acc: torch.Tensor, m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    """acc [rows, C, D], m/l [rows, C] (unnormalised partial sums with running
    maxima) -> out [rows, D]."""
    top = m.amax(dim=1, keepdim=True)
    w = torch.exp(m - top)
    w = torch.where(torch.isfinite(m), w, torch.zeros_like(w))
    den = (w * l).sum(dim=1)
    num = (acc * w.unsqueeze(-1)).sum(dim=1)
    return num / den.clamp_min(1e-30).unsqueeze(-1)


def merge_o_lse(o: torch.Tensor, lse: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """o [rows, C, D] normalised partial outputs, lse [rows, C] their
    log-sum-exp -> (out [rows, D], lse [rows]).  A partial with lse = -inf
    carries no mass; if every partial is empty the row is 0 / -inf."""
    top = lse.amax(dim=1, keepdim=True)
    safe_top = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    w = torch.exp(lse - safe_top)
    den = w.sum(dim=1)
    out = (o * w.unsqueeze(-1)).sum(dim=1) / den.clamp_min(1e-30).unsqueeze(-1)
    total = torch.where(den > 0, safe_top[:, 0] + torch.log(den.clamp_min(1e-30)),
                        torch.full_like(den, float("-inf")))
    return out, total


# --------------------------------------------------------------------------
# per-step statistics
# --------------------------------------------------------------------------

def condition_stats(mask: torch.Tensor, counts: torch.Tensor, group_size: int, prompt_len: int,
                    suffix_len: int) -> Dict[str, int]:
    """The reference's per-layer step statistics (IMPL/core.py:1441-1456) for a per-kv-head block mask
    [Hkv, nb] (the reference's ``selected`` is that mask broadcast over the G query rows)."""
    hkv = int(mask.shape[0])
    rows = hkv * int(group_size)
    exists = counts > 0
    selected_tokens = int((mask.long() * counts.view(1, -1)).sum()) * int(group_size)
    reps = int(((~mask) & exists.view(1, -1)).sum()) * int(group_size)
    suffix_tokens = max(int(suffix_len), 0) * rows
    return {
        "rows": rows,
        "clusters": int(exists.sum()) * rows,
        "selected_clusters": int(mask.sum()) * int(group_size),
        "selected_tokens": selected_tokens,
        "hybrid_tokens": selected_tokens + reps + suffix_tokens,
        "total_available": (int(prompt_len) + max(int(suffix_len), 0)) * rows,
    }


# --------------------------------------------------------------------------
# one full decode-attention step over a paged batch
# --------------------------------------------------------------------------

def decode_step_batch(
    case: Dict[str, torch.Tensor],
    *,
    mode: str = "topk",
    top_k: int = 0,
    eps: float = 0.0,
    rep_mode: str = "sparse_only",
    storage: str = "mixed",
    seqs: Optional[List[int]] = None,
) -> Dict[str, list]:
    """Run summaries -> score -> selection -> attention for the sequences of a
    paged case (see ``oracle.configs.make_case``).  Returns per-sequence lists:
    ``summaries``, ``score`` [Hkv, nb], ``ranked`` (top-k) / ``mask``, ``out``
    [Hkv*G, D] fp32."""
    block = int(case["block_size"])
    hkv = int(case["k_pool"].shape[1])
    hq = int(case["q"].shape[1])
    g = hq // hkv
    res: Dict[str, list] = {"summaries": [], "score": [], "ranked": [], "mask": [], "out": [], "z": []}
    which = range(int(case["q"].shape[0])) if seqs is None else seqs
    for b in which:
        plen = int(case["prefix_lens"][b])
        slen = int(case["seq_lens"][b])
        k_all = gather_logical(case["k_pool"], case["block_table"][b], slen)
        v_all = gather_logical(case["v_pool"], case["block_table"][b], slen)
        summ = block_summaries(k_all[:, :plen], v_all[:, :plen], block, storage=storage)
        qg = case["q"][b].reshape(hkv, g, -1)
        terms = condition_terms(qg, summ)
        if mode == "topk":
            ranked, mask = select_topk(terms["score"], summ.counts, top_k)
        elif mode == "eps":
            mask = select_threshold(terms["score"], summ.counts, eps)
            ranked = [m.nonzero().flatten().tolist() for m in mask]
        else:
            raise ValueError(mode)
        out = decode_attention(
            qg, k_all, v_all, plen, block, mask,
            rep_mode=rep_mode, z=terms["z"], v_bar=summ.v_bar,
        )
        res["summaries"].append(summ)
        res["score"].append(terms["score"])
        res["z"].append(terms["z"])
        res["ranked"].append(ranked)
        res["mask"].append(mask)
        res["out"].append(out.reshape(hq, -1))
    return res
