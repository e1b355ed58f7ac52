"""Soundness of the two in-block spread bounds as the CUDA kernels compute them, on the four synthetic key
geometries of the reference's sanity script (llama/script/analysis/condition_block_ball/sanity.py:29-41, 44-125):
independent normal keys; 0.3 x noise plus a ramp from 0 to 4 along one unit direction per head (a RoPE-like
drift); every 37th token scaled by 8 (outliers); keys scaled by 3 and shifted by 1.5.

Bar (the reference's own): for every (query row, block) that holds a token, the kernel's delta - the coordinate
range bound and the diagonal-ellipsoid bound - is at least the exact spread max_t |q.k_t / sqrt(D) - s| minus
1e-4, the exact spread taken in float64 from the keys as stored in the pool and the block mean as stored in
the summaries.  Also, as there: the bounds are not vacuous (median bound / exact below 50).
"""

import math

import pytest
import torch

from oracle.configs import DecodeConfig, make_case
from tests.gpu_util import logical_kv, max_blocks_of, to_device

pytestmark = pytest.mark.gpu

KINDS = ["iid", "drift", "outlier", "real_scale"]
CASES = [
    DecodeConfig("sound_bf16", "bfloat16", 2, 8, 4, 128, 16, 32, 3, (512, 311), (0, 0), seed=41),
    DecodeConfig("sound_f32", "float32", 2, 8, 4, 128, 16, 32, 3, (256, 100), (0, 0), seed=42),
    DecodeConfig("sound_bf16_b64", "bfloat16", 1, 32, 8, 128, 16, 64, 3, (1000,), (0,), seed=43),
]


def _ops():
    from interattn_b200 import ops
    return ops


def _shape_keys(case, kind, seed):
    """Rewrite the case's key pool, in logical token order, with one of the four geometries."""
    cfg = case["cfg"]
    g = torch.Generator().manual_seed(seed)
    page = cfg.page_size
    for b in range(cfg.batch):
        n = int(case["seq_lens"][b])
        k = torch.randn((cfg.n_kv_heads, n, cfg.head_dim), generator=g)
        if kind == "drift":
            direction = torch.randn((cfg.n_kv_heads, 1, cfg.head_dim), generator=g)
            direction = direction / direction.norm(dim=-1, keepdim=True)
            k = 0.3 * k + torch.linspace(0.0, 4.0, n).view(1, n, 1) * direction
        elif kind == "outlier":
            k[:, ::37] *= 8.0
        elif kind == "real_scale":
            k = 3.0 * k + 1.5
        for j in range((n + page - 1) // page):
            rows = k[:, j * page:(j + 1) * page]
            case["k_pool"][int(case["block_table"][b, j]), :, :rows.shape[1]] = rows.to(cfg.torch_dtype)


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("cfg", CASES, ids=lambda c: c.name)
def test_kernel_bounds_contain_the_exact_spread(cfg, kind):
    ops = _ops()
    case = make_case(cfg, spare_pages=2)
    _shape_keys(case, kind, cfg.seed + KINDS.index(kind))
    q, kv = to_device(case)
    nbmax = max_blocks_of(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nbmax, diag_ell=True)
    deltas = {}
    for bound in ("range", "diag_ell"):
        _, _, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("delta",), bound=bound)
        deltas[bound] = aux["delta"].double().cpu()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    G, D, B = cfg.group_size, cfg.head_dim, cfg.block_size
    ratios = {"range": [], "diag_ell": []}
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        nb = (plen + B - 1) // B
        k, _ = logical_kv(case, b)
        k = k[:, :plen].double()                                         # [Hkv, T, D] as stored
        qg = case["q"][b].double().reshape(cfg.n_kv_heads, G, D)        # as stored
        logits = torch.einsum("hgd,htd->hgt", qg, k) / math.sqrt(D)
        s = torch.einsum("hgd,hbd->hgb", qg, summ.k_bar[b, :, :nb].double().cpu()) / math.sqrt(D)
        pad = nb * B - plen
        spread = torch.nn.functional.pad(logits, (0, pad), value=float("nan")).reshape(cfg.n_kv_heads, G, nb, B)
        exact = (spread - s.unsqueeze(-1)).abs()
        exact = torch.where(torch.isnan(exact), torch.zeros_like(exact), exact).amax(-1)   # [Hkv, G, nb]
        for bound, d in deltas.items():
            got = d[b, :, :nb].reshape(cfg.n_kv_heads, G, nb)
            worst = float((exact - got).max())
            assert worst <= 1e-4, f"{kind} / {bound}: the bound falls {worst:.3e} short of the exact spread"
            keep = exact > 0.01
            ratios[bound].append((got[keep] / exact[keep]))
    for bound, r in ratios.items():
        med = float(torch.cat(r).median())
        assert 1.0 <= med < 50.0, f"{kind} / {bound}: median bound / exact = {med:.2f}"
