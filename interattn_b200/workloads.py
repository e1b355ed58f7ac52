"""The named decode-attention workloads: geometry and lengths only, no data.

Five configurations follow the benchmark description of the project: a
CPU-runnable fp32 case, the Llama-3-8B attention geometry at 32k context, one
attention layer of the full Llama-3-8B decode, a long-context split-KV case and
a variable-length batch at the Llama-3-70B geometry.  They stand in for the
LongBench / WikiText prompts the reference measures on: same head geometry and
context lengths; the tensors are seeded N(0,1) draws made by the benchmark (on
the device) or by the test generators (on the host).
``scaled()`` shrinks a configuration so that a CPU check finishes in seconds
while keeping its geometry (heads, head_dim, page, block, ragged tail).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional

import torch


@dataclass(frozen=True)
class DecodeConfig:
    name: str
    dtype: str                 # "float32" | "bfloat16"
    batch: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    page_size: int
    block_size: int
    top_k: int
    prefix_lens: tuple         # per sequence: tokens covered by summaries
    suffix_lens: tuple         # per sequence: generated tokens after the prefix
    seed: int = 0
    k_channel_sigma: float = 0.0   # log-normal sigma of the per-channel K scale

    @property
    def group_size(self) -> int:
        return self.n_q_heads // self.n_kv_heads

    @property
    def torch_dtype(self) -> torch.dtype:
        return getattr(torch, self.dtype)


def _uniform_lengths(batch: int, lo: int, hi: int, seed: int) -> tuple:
    g = torch.Generator().manual_seed(seed + 7919)
    return tuple(int(x) for x in torch.randint(lo, hi + 1, (batch,), generator=g))


CONFIGS: Dict[str, DecodeConfig] = {
    # fp32, batch 2, 8 q heads / 2 kv heads, D 64, context 1024, top-4 of 16 blocks
    "cfg1_cpu_fp32": DecodeConfig(
        "cfg1_cpu_fp32", "float32", 2, 8, 2, 64, 16, 64, 4, (1024, 1024), (0, 0), seed=0),
    # Llama-3-8B attention geometry, batch 16, context 32768, top-64 of 512 blocks
    "cfg2_llama8b_32k": DecodeConfig(
        "cfg2_llama8b_32k", "bfloat16", 16, 32, 8, 128, 16, 64, 64,
        (32768,) * 16, (0,) * 16, seed=0, k_channel_sigma=0.5),
    # long-context split-KV: batch 4, context 131072, top-32 of 2048 blocks
    "cfg4_longctx_128k": DecodeConfig(
        "cfg4_longctx_128k", "bfloat16", 4, 32, 8, 128, 16, 64, 32,
        (131072,) * 4, (0,) * 4, seed=0),
    # one attention layer of the full Llama-3-8B decode (batch 32, 8192-token prompts, top-64 of
    # 128 blocks), half way through its 256 generated tokens
    "cfg3_layer_llama8b_8k": DecodeConfig(
        "cfg3_layer_llama8b_8k", "bfloat16", 32, 32, 8, 128, 16, 64, 64,
        (8192,) * 32, (128,) * 32, seed=0),
    # Llama-3-70B attention geometry, batch 64, ragged lengths in [1024, 65536], top-48
    "cfg5_llama70b_ragged": DecodeConfig(
        "cfg5_llama70b_ragged", "bfloat16", 64, 64, 8, 128, 16, 64, 48,
        _uniform_lengths(64, 1024, 65536, 0), (0,) * 64, seed=0),
}


def scaled(cfg: DecodeConfig, *, batch: Optional[int] = None, max_len: int = 2048,
           suffix: int = 0, top_k: Optional[int] = None) -> DecodeConfig:
    """A small twin of ``cfg``: fewer sequences, contexts folded into
    [block_size, max_len] keeping their remainders modulo the block size (so
    ragged tails stay ragged), optional generated suffix."""
    b = cfg.batch if batch is None else min(batch, cfg.batch)
    lens = []
    for i in range(b):
        n = cfg.prefix_lens[i]
        if n > max_len:
            n = cfg.block_size + (n - cfg.block_size) % (max_len - cfg.block_size + 1)
        lens.append(n)
    nb_min = min((n + cfg.block_size - 1) // cfg.block_size for n in lens)
    k = cfg.top_k if top_k is None else top_k
    return replace(
        cfg, name=cfg.name + "_small", batch=b, prefix_lens=tuple(lens),
        suffix_lens=(suffix,) * b, top_k=max(1, min(k, max(1, nb_min // 2))),
    )


def make_device_layer(cfg: DecodeConfig, device, seed: int):
    """One layer's paged KV cache for the whole batch of ``cfg``, generated on the device: N(0,1) K/V
    (K channels scaled by a log-normal factor where the configuration asks for it), a random
    permutation as the block table.  Returns an ``ops.PagedKV``."""
    from . import ops
    g = torch.Generator(device=device).manual_seed(seed)
    P, D, hkv = cfg.page_size, cfg.head_dim, cfg.n_kv_heads
    pages_per_seq = [(n + s + P - 1) // P for n, s in zip(cfg.prefix_lens, cfg.suffix_lens)]
    n_pages, max_pages = sum(pages_per_seq), max(pages_per_seq)
    dt = cfg.torch_dtype
    k_pool = torch.randn((n_pages, hkv, P, D), generator=g, device=device, dtype=torch.float32)
    if cfg.k_channel_sigma > 0:
        k_pool *= torch.exp(cfg.k_channel_sigma * torch.randn((D,), generator=g, device=device))
    k_pool = k_pool.to(dt)
    v_pool = torch.randn((n_pages, hkv, P, D), generator=g, device=device, dtype=torch.float32).to(dt)
    perm = torch.randperm(n_pages, generator=g, device=device).to(torch.int32)
    table = torch.zeros((cfg.batch, max_pages), dtype=torch.int32, device=device)
    at = 0
    for b, n in enumerate(pages_per_seq):
        table[b, :n] = perm[at: at + n]
        at += n
    prefix = torch.tensor(cfg.prefix_lens, dtype=torch.int32, device=device)
    seq = torch.tensor([p + s for p, s in zip(cfg.prefix_lens, cfg.suffix_lens)], dtype=torch.int32, device=device)
    return ops.PagedKV(k_pool, v_pool, table, prefix, seq)
