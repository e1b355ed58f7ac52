"""GPU parity of the two-pass selection (``condition_block_select_twopass_kernel``): no per-(row, block)
state in shared memory - row normalisers from a first pass over the summaries, the scores from a second pass
over the same tiles.  It does the one-pass kernel's arithmetic in the one-pass kernel's order.  The form is taken
on request only (``INTERATTN_B200_SELECT_TWOPASS=1``): it fits two CTAs per SM where the one-pass narrow shape
does not, but measured slower than the wide shape there.

Bars: scores, selected indices and the layer step bit-identical to the one-pass narrow kernel; indices
identical to the oracle.
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
    scaled(CONFIGS["cfg2_llama8b_32k"], batch=3, max_len=2304, suffix=0),          # G = 4
    scaled(CONFIGS["cfg5_llama70b_ragged"], batch=5, max_len=1900, suffix=3),      # G = 8, ragged
    scaled(CONFIGS["cfg4_longctx_128k"], batch=2, max_len=4096, suffix=1, top_k=8),
    DecodeConfig("bf16_g1", "bfloat16", 2, 2, 2, 128, 16, 64, 2, (300, 64), (0, 0), seed=8),
    DecodeConfig("bf16_g2_ragged", "bfloat16", 4, 4, 2, 128, 16, 64, 3, (1, 129, 1000, 0), (15, 16, 17, 40), seed=11),
    DecodeConfig("bf16_d64", "bfloat16", 2, 8, 2, 64, 16, 64, 3, (777, 65), (0, 18), seed=6),
]


@pytest.mark.parametrize("k_bar", ["f32", "bf16"])
@pytest.mark.parametrize("cfg", CASES, ids=lambda c: c.name)
def test_two_pass_selection_equals_the_one_pass_kernel(cfg, k_bar, monkeypatch):
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_SHAPE", "narrow")
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case),
                               k_bar_dtype=torch.bfloat16 if k_bar == "bf16" else torch.float32)
    got = {}
    for form in ("0", "1"):
        monkeypatch.setenv("INTERATTN_B200_SELECT_TWOPASS", form)
        idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("score", "z", "delta", "globals"))
        eidx, ecnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, eps=1e-3)
        got[form] = (idx, cnt, aux, eidx, ecnt)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    (idx1, cnt1, aux1, eidx1, ecnt1), (idx2, cnt2, aux2, eidx2, ecnt2) = got["0"], got["1"]
    assert torch.equal(idx1, idx2) and torch.equal(cnt1, cnt2)
    assert torch.equal(eidx1, eidx2) and torch.equal(ecnt1, ecnt2)
    for name in ("score", "z", "delta", "globals"):
        assert torch.equal(aux1[name], aux2[name]), name
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        if plen == 0:
            assert int(cnt2[b].sum()) == 0
            continue
        osum = oracle_summaries_from_gpu(summ, b, plen)
        qg = case["q"][b].reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim).float()
        if k_bar == "bf16":
            osum.k_bar = summ.k_bar[b, :, :osum.n_blocks].float().cpu()
        terms = orc.condition_terms(qg, osum)
        ranked, _ = orc.select_topk(terms["score"], osum.counts, cfg.top_k)
        for h in range(cfg.n_kv_heads):
            assert idx2[b, h, :int(cnt2[b, h])].cpu().tolist() == sorted(ranked[h])


@pytest.mark.parametrize("rep_mode", ["sparse_only", "hybrid"])
def test_layer_step_with_the_two_pass_selection(rep_mode, monkeypatch):
    """Two kernels: the two-pass selection (it writes the representatives' logits to the workspace in its first
    pass) and the attention kernel - same output as with the one-pass selection."""
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_SHAPE", "narrow")
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = CASES[1]
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    before = ops.set_fused_step(False)
    try:
        outs = []
        for form in ("0", "1"):
            monkeypatch.setenv("INTERATTN_B200_SELECT_TWOPASS", form)
            step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode)
            outs.append((step.step(q).clone(), step.sel_idx.clone()))
    finally:
        ops.set_fused_step(before)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(outs[0][1], outs[1][1]) and torch.equal(outs[0][0], outs[1][0])
