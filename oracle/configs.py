"""Seeded synthetic inputs for the decode-attention configurations.

TEST INFRASTRUCTURE (shared by the oracle, the tests and the benchmark's CPU
arm).  The workload table itself (``DecodeConfig``, ``CONFIGS``, ``scaled``)
lives in ``interattn_b200.workloads``; this module materialises a configuration
on the CPU from its seed.

Physical layout of a KV pool: ``[n_pages, n_kv_heads, page_size, head_dim]``,
so that one (page, kv head) is one contiguous run.  ``block_table[b, j]`` is
the physical page holding logical tokens ``16 j .. 16 j + 15`` of sequence b.
"""

from __future__ import annotations

from typing import Dict

import torch

from interattn_b200.workloads import CONFIGS, DecodeConfig, scaled  # noqa: F401  (re-exported)


def make_case(cfg: DecodeConfig, *, spare_pages: int = 0) -> Dict[str, object]:
    """Materialise one configuration on the CPU.

    Returns q [B, Hq, D], k_pool / v_pool [n_pages, Hkv, P, D] (cfg dtype),
    block_table int32 [B, max_pages] (a seeded random permutation of the pool,
    cut per sequence; unused entries are -1), prefix_lens / seq_lens int32 [B],
    plus the scalar geometry.  All draws come from one generator seeded with
    ``cfg.seed``, in a fixed order: q, k_pool, v_pool, channel factor, table.
    """
    g = torch.Generator().manual_seed(cfg.seed)
    dt = cfg.torch_dtype
    P = cfg.page_size
    seq_lens = [p + s for p, s in zip(cfg.prefix_lens, cfg.suffix_lens)]
    pages_per_seq = [(n + P - 1) // P for n in seq_lens]
    n_pages = sum(pages_per_seq) + int(spare_pages)
    max_pages = max(pages_per_seq)

    q = torch.randn((cfg.batch, cfg.n_q_heads, cfg.head_dim), generator=g).to(dt)
    k_pool = torch.randn((n_pages, cfg.n_kv_heads, P, cfg.head_dim), generator=g)
    v_pool = torch.randn((n_pages, cfg.n_kv_heads, P, cfg.head_dim), generator=g)
    if cfg.k_channel_sigma > 0:
        factor = torch.exp(cfg.k_channel_sigma * torch.randn((cfg.head_dim,), generator=g))
        k_pool = k_pool * factor
    k_pool, v_pool = k_pool.to(dt), v_pool.to(dt)

    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    table = torch.full((cfg.batch, max_pages), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per_seq):
        table[b, :n] = perm[at: at + n]
        at += n
    return {
        "cfg": cfg,
        "q": q, "k_pool": k_pool, "v_pool": v_pool, "block_table": table,
        "prefix_lens": torch.tensor(cfg.prefix_lens, dtype=torch.int32),
        "seq_lens": torch.tensor(seq_lens, dtype=torch.int32),
        "page_size": P, "block_size": cfg.block_size, "top_k": cfg.top_k,
    }
