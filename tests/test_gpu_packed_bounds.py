"""GPU parity of the packed coordinate-range layout (the reference's ``k_bounds``,
IMPL/core.py:490-499: ``torch.stack((k_max, k_min), dim=-1).flatten(2)``): the summary kernel writes the pairs,
the selection reads them - through the tensor cores as one contraction of length 2 D against the query's signed
parts interleaved, or on the CUDA cores after a de-interleave - and picks exactly what it picks from two arrays.

Bars: the packed array de-interleaves to the two arrays bit for bit; selected indices identical to the plain
layout and to the oracle; scores within 2e-4 relative.
"""

import pytest
import torch

from oracle import condition_block_oracle as orc
from oracle.configs import CONFIGS, DecodeConfig, make_case, scaled
from tests.gpu_util import max_blocks_of, oracle_summaries_from_gpu, to_device

pytestmark = pytest.mark.gpu


def _ops():
    from interattn_b200 import ops
    return ops


CASES = [
    CONFIGS["cfg1_cpu_fp32"],                                                   # fp32, CUDA-core scoring
    scaled(CONFIGS["cfg2_llama8b_32k"], batch=3, max_len=2304, suffix=0),       # bf16, tensor-core scoring
    scaled(CONFIGS["cfg5_llama70b_ragged"], batch=5, max_len=1900, suffix=3),   # G = 8, ragged
    DecodeConfig("f32_d128", "float32", 2, 4, 2, 128, 16, 64, 3, (700, 129), (2, 0), seed=5),
    DecodeConfig("bf16_d64", "bfloat16", 2, 8, 2, 64, 16, 64, 3, (777, 65), (0, 18), seed=6),
    DecodeConfig("bf16_g16", "bfloat16", 1, 16, 1, 128, 16, 64, 5, (1111,), (4,), seed=7),  # bf16 on the CUDA cores
]


@pytest.fixture(scope="module", params=CASES, ids=lambda c: c.name)
def bundle(request):
    ops = _ops()
    cfg = request.param
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    plain = ops.build_summaries(kv, cfg.block_size, max_blocks=nb)
    packed = ops.build_summaries(kv, cfg.block_size, max_blocks=nb, packed_bounds=True)
    torch.cuda.synchronize()
    return cfg, case, q, kv, plain, packed


def test_the_packed_array_holds_the_pairs(bundle):
    cfg, case, q, kv, plain, packed = bundle
    assert packed.k_bounds.shape == plain.k_max.shape[:3] + (2 * cfg.head_dim,)
    assert torch.equal(packed.k_bounds[..., 0::2], plain.k_max) and torch.equal(packed.k_bounds[..., 1::2], plain.k_min)
    assert torch.equal(packed.k_max, plain.k_max) and torch.equal(packed.k_min, plain.k_min)  # the strided views
    for name in ("k_bar", "v_bar", "v_norm_max"):
        assert torch.equal(getattr(packed, name), getattr(plain, name)), name


def test_selection_from_the_packed_layout(bundle):
    ops = _ops()
    cfg, case, q, kv, plain, packed = bundle
    idx_p, cnt_p, aux_p = ops.select_blocks(q, packed, kv.prefix_lens, top_k=cfg.top_k, want=("score", "delta"))
    idx, cnt, aux = ops.select_blocks(q, plain, kv.prefix_lens, top_k=cfg.top_k, want=("score", "delta"))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(idx_p, idx) and torch.equal(cnt_p, cnt)
    assert torch.allclose(aux_p["score"], aux["score"], rtol=2e-4, atol=1e-8)
    assert torch.allclose(aux_p["delta"], aux["delta"], rtol=1e-4, atol=1e-5)
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        osum = oracle_summaries_from_gpu(packed, b, plen)
        qg = case["q"][b].reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim).float()
        terms = orc.condition_terms(qg, osum)
        ranked, _ = orc.select_topk(terms["score"], osum.counts, cfg.top_k)
        for h in range(cfg.n_kv_heads):
            assert idx_p[b, h, :int(cnt_p[b, h])].cpu().tolist() == sorted(ranked[h])


@pytest.mark.parametrize("cluster", [None, 1])
def test_layer_step_from_the_packed_layout(bundle, cluster, monkeypatch):
    """The one-call step (two kernels, or - cluster pinned to 1 where the shape allows - the fused kernel)."""
    ops = _ops()
    cfg, case, q, kv, plain, packed = bundle
    if cluster is not None:
        monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", str(cluster))
    want_step = ops.DecodeAttention(kv, plain, cfg.n_q_heads, top_k=cfg.top_k)
    want = want_step.step(q).clone()
    got_step = ops.DecodeAttention(kv, packed, cfg.n_q_heads, top_k=cfg.top_k)
    got = got_step.step(q).clone()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(got_step.sel_idx, want_step.sel_idx) and torch.equal(got_step.sel_count, want_step.sel_count)
    assert torch.equal(got, want)  # the same blocks through the same attention code


def test_packed_layout_excludes_the_ellipsoid_pair():
    ops = _ops()
    cfg = CASES[1]
    case = make_case(cfg, spare_pages=1)
    q, kv = to_device(case)
    with pytest.raises(ValueError):
        ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case), packed_bounds=True, diag_ell=True)
    packed = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case), packed_bounds=True)
    with pytest.raises(ValueError):
        ops.select_blocks(q, packed, kv.prefix_lens, top_k=cfg.top_k, bound="diag_ell")
