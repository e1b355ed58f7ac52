"""The oracle against vectors produced by the unmodified reference
(tests/golden/make_golden.py).  Runs without the reference tree."""

import json
import os

import numpy as np
import pytest
import torch

from oracle import condition_block_oracle as orc
from tests import golden_io


def _cases():
    case, vec = golden_io.ragged_case()
    yield "ragged_bf16", case, vec
    case, vec, ok = golden_io.cfg1_case()
    if ok:
        yield "cfg1_fp32", case, vec


def test_cfg1_inputs_regenerate_bit_exactly():
    _, _, ok = golden_io.cfg1_case()
    if not ok:
        pytest.skip("this torch build draws different seeded normals; cfg1 golden outputs not comparable here")


@pytest.mark.parametrize("name,case,vec", list(_cases()), ids=lambda x: x if isinstance(x, str) else "")
def test_oracle_reproduces_reference_vectors(name, case, vec):
    cfg = case["cfg"]
    g = cfg.group_size
    for b in range(cfg.batch):
        pre = f"seq{b}_"
        plen, slen = int(case["prefix_lens"][b]), int(case["seq_lens"][b])
        k = orc.gather_logical(case["k_pool"], case["block_table"][b], slen)
        v = orc.gather_logical(case["v_pool"], case["block_table"][b], slen)
        summ = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size)
        for key, mine in (("k_bar", summ.k_bar), ("v_bar", summ.v_bar), ("k_max", summ.k_max),
                          ("k_min", summ.k_min), ("v_norm_max", summ.v_norm_max)):
            assert np.array_equal(mine.float().numpy(), vec[pre + key]), key
        assert np.array_equal(summ.counts.numpy(), vec[pre + "counts"])
        qg = case["q"][b].reshape(cfg.n_kv_heads, g, cfg.head_dim).float()
        terms = orc.condition_terms(qg, summ)
        assert np.array_equal(terms["z"].numpy(), vec[pre + "z_logits"])
        assert np.array_equal(terms["score"].numpy(), vec[pre + "score"])
        assert np.array_equal(orc.select_threshold(terms["score"], summ.counts, 0.0).numpy(), vec[pre + "mask_eps0"])
        for qi in (0, 1):
            eps = float(vec[pre + f"eps{qi}"])
            assert np.array_equal(orc.select_threshold(terms["score"], summ.counts, eps).numpy(),
                                  vec[pre + f"mask_eps{qi}q"])
        ranked, mask = orc.select_topk(terms["score"], summ.counts, cfg.top_k)
        assert np.array_equal(np.array(ranked, dtype=np.int32), vec[pre + "topk_ranked"])
        got = orc.decode_attention(qg, k, v, plen, cfg.block_size, mask, rep_mode="hybrid",
                                   z=terms["z"], v_bar=summ.v_bar)
        np.testing.assert_allclose(got.numpy(), vec[pre + "hybrid_topk_out"], rtol=1e-5, atol=2e-6)
        # the dense-form port (every prefix token scored, then masked) against the same reference vectors
        got_dense = orc.decode_attention_dense(qg, k, v, plen, cfg.block_size, mask, rep_mode="hybrid",
                                               z=terms["z"], v_bar=summ.v_bar)
        np.testing.assert_allclose(got_dense.numpy(), vec[pre + "hybrid_topk_out"], rtol=1e-5, atol=2e-6)
        # sparse-only (the benchmark's mode): the reference's dense function with every representative masked
        for fn in (orc.decode_attention, orc.decode_attention_dense):
            got = fn(qg, k, v, plen, cfg.block_size, mask, rep_mode="sparse_only")
            np.testing.assert_allclose(got.numpy(), vec[pre + "sparse_topk_out"], rtol=1e-5, atol=2e-6)
        # The reference's compact-SDPA path recomputes the representatives' logits from k_bar cast to the
        # cache dtype (legacy.py:917) and runs one SDPA call; with a bf16 cache that rounding of k_bar is
        # the whole difference from the dense form, hence the looser tolerance there.
        got = orc.decode_attention(qg, k, v, plen, cfg.block_size, mask, rep_mode="hybrid",
                                   z=terms["z"], v_bar=summ.v_bar)
        loose = dict(rtol=1e-5, atol=2e-6) if cfg.dtype == "float32" else dict(rtol=2e-3, atol=2e-3)
        np.testing.assert_allclose(got.numpy(), vec[pre + "compact_hybrid_topk_out"], **loose)
        if pre + "pr1_eps1_out" in vec.files:
            eps = float(vec[pre + "eps1"])
            m2 = orc.select_threshold(terms["score"], summ.counts, eps)
            got = orc.decode_attention(qg, k, v, plen, cfg.block_size, m2, rep_mode="hybrid",
                                       z=terms["z"], v_bar=summ.v_bar)
            np.testing.assert_allclose(got.numpy(), vec[pre + "pr1_eps1_out"], rtol=1e-5, atol=2e-6)


def test_score_known_answer():
    with open(os.path.join(golden_io.GOLDEN_DIR, "score_known_answer.json")) as f:
        want = torch.tensor([float.fromhex(x) for x in json.load(f)["score_hex"]], dtype=torch.float64)
    z = torch.tensor([[[0.0, 1.0, 2.0], [0.5, -0.5, float("-inf")]]], dtype=torch.float64)
    p = torch.softmax(z, dim=-1)
    delta = torch.tensor([[[0.2, 1.0, 2.0], [0.4, 1.5, 0.0]]], dtype=torch.float64)
    b_c = torch.tensor([[[1.0, 2.0, 1.5], [0.8, 1.2, 0.0]]], dtype=torch.float64)
    got = orc.score_from_stats(p, delta, b_c, b_c.amax(dim=-1))
    assert torch.equal(got.flatten(), want)


def test_topk_tie_break_is_lowest_index():
    score = torch.tensor([[1.0, 3.0, 3.0, 0.5, 3.0, 1.0]])
    counts = torch.tensor([64, 64, 64, 64, 64, 0])
    ranked, mask = orc.select_topk(score, counts, 2)
    assert ranked == [[1, 2]]
    ranked, mask = orc.select_topk(score, counts, 4)
    assert ranked == [[1, 2, 4, 0]]
    ranked, mask = orc.select_topk(score, counts, 9)     # k > live blocks: the empty block never enters
    assert sorted(ranked[0]) == [0, 1, 2, 3, 4] and not mask[0, 5]


def test_split_kv_partials_merge_to_the_whole():
    case, _ = golden_io.ragged_case()
    cfg = case["cfg"]
    g = cfg.group_size
    b = 0
    plen, slen = int(case["prefix_lens"][b]), int(case["seq_lens"][b])
    k = orc.gather_logical(case["k_pool"], case["block_table"][b], slen)
    v = orc.gather_logical(case["v_pool"], case["block_table"][b], slen)
    summ = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size)
    qg = case["q"][b].reshape(cfg.n_kv_heads, g, cfg.head_dim).float()
    terms = orc.condition_terms(qg, summ)
    _, mask = orc.select_topk(terms["score"], summ.counts, 3)
    for rep_mode in ("hybrid", "sparse_only"):
        whole = orc.decode_attention(qg, k, v, plen, cfg.block_size, mask, rep_mode=rep_mode,
                                     z=terms["z"], v_bar=summ.v_bar)
        parts = []
        cuts = [(0, 2), (2, 3), (3, summ.n_blocks)]
        for i, rng in enumerate(cuts):
            parts.append(orc.decode_attention(
                qg, k, v, plen, cfg.block_size, mask, rep_mode=rep_mode, z=terms["z"], v_bar=summ.v_bar,
                block_range=rng, with_suffix=(i == len(cuts) - 1), return_lse=True))
        o = torch.stack([p[0].reshape(-1, cfg.head_dim) for p in parts], dim=1)
        lse = torch.stack([p[1].reshape(-1) for p in parts], dim=1)
        merged, _ = orc.merge_o_lse(o, lse)
        assert torch.allclose(merged, whole.reshape(-1, cfg.head_dim), rtol=1e-5, atol=1e-6)
