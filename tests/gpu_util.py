"""Helpers shared by the GPU parity tests: move a seeded case to the device,
run the C-ABI operators, and express their results in the oracle's terms."""

import torch

from interattn_b200 import ops
from oracle import condition_block_oracle as orc


def to_device(case, device="cuda:0"):
    kv = ops.PagedKV(
        k_pool=case["k_pool"].to(device), v_pool=case["v_pool"].to(device),
        block_table=case["block_table"].clamp_min(0).to(device).contiguous(),
        prefix_lens=case["prefix_lens"].to(device), seq_lens=case["seq_lens"].to(device))
    q = case["q"].to(device).contiguous()
    return q, kv


def max_blocks_of(case):
    block = int(case["block_size"])
    return max(1, (int(case["prefix_lens"].max()) + block - 1) // block)


def oracle_summaries_from_gpu(summ, b, prefix_len):
    """The GPU-built summaries of sequence b as an oracle ``Summaries`` (fp32 views)."""
    block = summ.block_size
    counts = orc.block_counts(prefix_len, block)
    nb = counts.numel()
    return orc.Summaries(
        k_bar=summ.k_bar[b, :, :nb].float().cpu(), v_bar=summ.v_bar[b, :, :nb].cpu(),
        k_max=summ.k_max[b, :, :nb].cpu(), k_min=summ.k_min[b, :, :nb].cpu(),
        v_norm_max=summ.v_norm_max[b, :, :nb].float().cpu(), counts=counts, block_size=block)


def logical_kv(case, b):
    slen = int(case["seq_lens"][b])
    k = orc.gather_logical(case["k_pool"], case["block_table"][b], slen)
    v = orc.gather_logical(case["v_pool"], case["block_table"][b], slen)
    return k, v


def rank_gap(score_row, k):
    """Relative gap between the k-th and (k+1)-th best score (inf if there is no (k+1)-th)."""
    vals = torch.sort(score_row, descending=True).values
    if k >= vals.numel() or k <= 0:
        return float("inf")
    a, b = float(vals[k - 1]), float(vals[k])
    return abs(a - b) / max(abs(a), 1e-30)
