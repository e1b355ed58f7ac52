"""Pins the oracle to the reference's own functions (needs the reference tree).

Skipped where the reference is not present (e.g. on a GPU box); the committed
vectors under tests/golden/ carry the same pin there."""

import os
import sys

import pytest
import torch

# the reference checkout: INTERATTN_REFERENCE_ROOT, else a directory `reference` next to this repository
REF_ROOT = os.environ.get("INTERATTN_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
pytestmark = pytest.mark.skipif(
    not os.path.isdir(os.path.join(REF_ROOT, "llama")), reason="reference tree not present")

from oracle import condition_block_oracle as orc
from oracle.configs import CONFIGS, make_case, scaled


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, REF_ROOT)
    try:
        from llama.script.analysis.condition_block_gen.methods import condition_block as pr1
        from llama.script.analysis.condition_block_gen.methods.condition_block_triton_impl import core, legacy
    finally:
        sys.path.remove(REF_ROOT)
    return pr1, core, legacy


def _logical(case, b):
    slen = int(case["seq_lens"][b])
    k = orc.gather_logical(case["k_pool"], case["block_table"][b], slen)
    v = orc.gather_logical(case["v_pool"], case["block_table"][b], slen)
    return k, v


CASES = [
    ("cfg1_cpu_fp32", dict(), 0),
    ("cfg2_llama8b_32k", dict(batch=2, max_len=1500), 5),
    ("cfg5_llama70b_ragged", dict(batch=3, max_len=900), 0),
]


@pytest.mark.parametrize("name,shrink,suffix", CASES)
def test_summaries_match_reference(ref, name, shrink, suffix):
    pr1, core, _ = ref
    cfg = CONFIGS[name] if not shrink else scaled(CONFIGS[name], suffix=suffix, **shrink)
    case = make_case(cfg)
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        k, v = _logical(case, b)
        mine = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size)
        theirs = core._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
        assert torch.equal(mine.k_bar, theirs["k_bar"])
        assert torch.equal(mine.v_bar, theirs["v_bar"])
        assert torch.equal(mine.k_max, theirs["k_max"])
        assert torch.equal(mine.k_min, theirs["k_min"])
        assert torch.equal(mine.v_norm_max, theirs["v_norm_max"])
        assert torch.equal(mine.counts, theirs["block_valid_counts"])
        if cfg.dtype == "float32":
            twin = pr1._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
            assert torch.equal(mine.k_bar, twin["k_bar"])
            assert torch.allclose(mine.v_norm_max, twin["v_norm_max"], rtol=1e-6, atol=0)


@pytest.mark.parametrize("name,shrink,suffix", CASES)
def test_score_and_threshold_selection_match_reference(ref, name, shrink, suffix):
    _, core, _ = ref
    cfg = CONFIGS[name] if not shrink else scaled(CONFIGS[name], suffix=suffix, **shrink)
    case = make_case(cfg)
    g = cfg.group_size
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        k, v = _logical(case, b)
        summ = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size)
        theirs = core._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
        qg = case["q"][b].reshape(cfg.n_kv_heads, g, 1, cfg.head_dim).float()
        terms = orc.condition_terms(qg[:, :, 0], summ)
        # thresholds at quantiles of the score: the reference's mask must follow the oracle score
        for quant in (0.0, 0.3, 0.9):
            eps = float(torch.quantile(terms["score"].flatten(), quant)) if quant else 0.0
            sel, z_logits, v_bar, size, exists = core._select_prompt_blocks_eager(qg, theirs, eps)
            mine = orc.select_threshold(terms["score"], summ.counts, eps)
            assert torch.equal(sel[:, 0, 0], mine)
            assert torch.equal(z_logits[:, :, 0], terms["z"])
        # eps extremes used by the reference's sanity scripts
        sel, *_ = core._select_prompt_blocks_eager(qg, theirs, 1e9)
        assert not sel.any()


def test_score_known_answer_from_reference_pytest(ref):
    """The hand-written 2x3 example of the reference's own score test
    (condition_block_ppl/delta_bound/term_ablation/test_ppl.py:8-40)."""
    import types
    stubbed = []
    for name in ("matplotlib", "matplotlib.pyplot"):  # plotting is not needed for the score
        try:
            __import__(name)
        except ImportError:
            sys.modules[name] = types.ModuleType(name)
            stubbed.append(name)
    sys.path.insert(0, REF_ROOT)
    try:
        from llama.script.analysis.condition_block_ppl import runner_cond_block as rcb
    except Exception as exc:  # other optional deps of that module
        pytest.skip(f"runner_cond_block not importable: {exc}")
    finally:
        sys.path.remove(REF_ROOT)
        for name in stubbed:
            sys.modules.pop(name, None)
    z = torch.tensor([[[0.0, 1.0, 2.0], [0.5, -0.5, float("-inf")]]], dtype=torch.float64)
    p = torch.softmax(z, dim=-1)
    delta = torch.tensor([[[0.2, 1.0, 2.0], [0.4, 1.5, 0.0]]], dtype=torch.float64)
    b_c = torch.tensor([[[1.0, 2.0, 1.5], [0.8, 1.2, 0.0]]], dtype=torch.float64)
    b_all = b_c.amax(dim=-1)
    want = rcb._condition_score_for_blocks(
        p_tensor=p, z_logits=z, delta=delta, b_c=b_c, b_all=b_all, cluster_exists=torch.isfinite(z[0]))
    assert torch.equal(orc.score_from_stats(p, delta, b_c, b_all), want)


@pytest.mark.parametrize("name,shrink,suffix", CASES)
@pytest.mark.parametrize("rep_mode", ["hybrid", "sparse_only"])
def test_attention_matches_reference_dense(ref, name, shrink, suffix, rep_mode):
    pr1, core, legacy = ref
    cfg = CONFIGS[name] if not shrink else scaled(CONFIGS[name], suffix=suffix, **shrink)
    case = make_case(cfg)
    g = cfg.group_size
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        slen = int(case["seq_lens"][b])
        k, v = _logical(case, b)
        summ = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size)
        theirs = core._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
        qg = case["q"][b].reshape(cfg.n_kv_heads, g, 1, cfg.head_dim).float()
        terms = orc.condition_terms(qg[:, :, 0], summ)
        ranked, mask = orc.select_topk(terms["score"], summ.counts, cfg.top_k)
        selected = mask[:, None, None, :].expand(-1, g, 1, -1)
        v_bar = theirs["v_bar"][:, None, None].expand(-1, g, 1, -1, -1)
        want = legacy._condition_block_decode_output_dense(
            q_grouped=qg, pos_tensor=torch.tensor([slen - 1]), prompt_prefix=theirs,
            k_suffix=k[:, plen:].float(), v_suffix=v[:, plen:].float(),
            block_size=cfg.block_size, prompt_len=plen, selected=selected,
            z_logits=terms["z"][:, :, None], v_bar=v_bar,
            # sparse-only = the same reference function with every representative masked (legacy.py:828-829)
            cluster_exists=(summ.counts > 0).view(1, -1) if rep_mode == "hybrid"
            else torch.zeros((1, summ.n_blocks), dtype=torch.bool))
        for fn in (orc.decode_attention, orc.decode_attention_dense):
            got = fn(qg[:, :, 0], k, v, plen, cfg.block_size, mask, rep_mode=rep_mode, z=terms["z"],
                     v_bar=summ.v_bar)
            assert torch.allclose(got, want[:, :, 0], rtol=1e-5, atol=2e-6)
        if rep_mode == "hybrid":
            # the reference's sparse CPU path (compact + one SDPA call); fp32 attention dtype.  With a bf16
            # cache it rounds k_bar to bf16 for the representatives' logits (legacy.py:917): looser there.
            compact = legacy._condition_block_decode_output_compact_sdpa(
                q_grouped=qg, pos_tensor=torch.tensor([slen - 1]), prompt_prefix=theirs,
                k_suffix=k[:, plen:].float(), v_suffix=v[:, plen:].float(), block_size=cfg.block_size,
                prompt_len=plen, selected=selected, attention_dtype=torch.float32)
            tol = dict(rtol=1e-5, atol=2e-6) if cfg.dtype == "float32" else dict(rtol=2e-3, atol=2e-3)
            assert torch.allclose(got, compact[:, :, 0], **tol)


def test_threshold_end_to_end_matches_pr1_reference(ref):
    """fp32 twin: the whole step (selection by eps + hybrid attention)."""
    pr1, _, _ = ref
    cfg = CONFIGS["cfg1_cpu_fp32"]
    case = make_case(cfg)
    g = cfg.group_size
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        k, v = _logical(case, b)
        twin = pr1._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
        qg = case["q"][b].reshape(cfg.n_kv_heads, g, 1, cfg.head_dim)
        summ = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size)
        terms = orc.condition_terms(qg[:, :, 0], summ)
        eps = float(torch.quantile(terms["score"].flatten(), 0.75))
        want, _stats = pr1._condition_block_decode_output(
            q_grouped=qg, pos_tensor=torch.tensor([plen - 1]), prompt_prefix=twin,
            k_suffix=k[:, plen:], v_suffix=v[:, plen:], block_size=cfg.block_size,
            eps=eps, prompt_len=plen)
        mask = orc.select_threshold(terms["score"], summ.counts, eps)
        got = orc.decode_attention(qg[:, :, 0], k, v, plen, cfg.block_size, mask,
                                   rep_mode="hybrid", z=terms["z"], v_bar=summ.v_bar)
        assert torch.allclose(got, want[:, :, 0], rtol=1e-5, atol=2e-6)


def test_merge_matches_reference_math():
    torch.manual_seed(3)
    acc = torch.randn(8, 5, 16)
    m = torch.randn(8, 5)
    l = torch.rand(8, 5) + 0.1
    m[0, 2] = float("-inf"); l[0, 2] = 0.0; acc[0, 2] = 0.0
    top = m.amax(dim=1, keepdim=True)
    want = (acc * torch.exp(m - top)[..., None]).sum(1) / (torch.exp(m - top) * l).sum(1).clamp_min(1e-30)[:, None]
    assert torch.allclose(orc.merge_acc_m_l(acc, m, l), want, rtol=1e-6, atol=1e-7)
    o = acc / l.clamp_min(1e-30)[..., None]
    lse = m + torch.log(l)
    got, _ = orc.merge_o_lse(o, lse)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)


def test_step_statistics_match_reference(ref):
    """oracle.condition_stats against core._condition_stats on a ragged prompt (last block partial)."""
    _, core, _ = ref
    torch.manual_seed(9)
    hkv, g, block, prompt_len, suffix_len = 2, 4, 64, 331, 5
    counts = orc.block_counts(prompt_len, block)
    nb = counts.numel()
    mask = torch.rand(hkv, nb) > 0.5
    mask[0, nb - 1] = True
    selected = mask[:, None, None, :].expand(-1, g, 1, -1)
    want = core._condition_stats(selected=selected, size=counts.view(1, -1), cluster_exists=(counts > 0).view(1, -1),
                                 prompt_len=prompt_len, suffix_len=suffix_len)
    got = orc.condition_stats(mask, counts, g, prompt_len, suffix_len)
    assert {k: int(v) for k, v in want.items()} == got


@pytest.mark.parametrize("w_dtype", [None, torch.bfloat16])
def test_diag_ell_bound_matches_reference(ref, monkeypatch, w_dtype):
    """oracle.diag_ell_stats / condition_terms(diag_ell=...) against condition_block_ball/gen_selection.py
    (w, rho, the delta it gives, and the epsilon masks) on a ragged bf16 prefix."""
    _, core, _ = ref
    sys.path.insert(0, REF_ROOT)
    try:
        from llama.script.analysis.condition_block_ball import gen_selection as ball
    finally:
        sys.path.remove(REF_ROOT)
    if w_dtype == torch.bfloat16:
        monkeypatch.setenv("CONDITION_BLOCK_BALL_W_DTYPE", "bfloat16")
    else:
        monkeypatch.delenv("CONDITION_BLOCK_BALL_W_DTYPE", raising=False)
    cfg = scaled(CONFIGS["cfg2_llama8b_32k"], batch=2, max_len=1100, suffix=0)
    case = make_case(cfg)
    g = cfg.group_size
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        k, v = _logical(case, b)
        theirs = core._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
        summ = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size)
        w, rho = orc.diag_ell_stats(k[:, :plen], summ, w_dtype)
        w_ref, rho_ref = ball.diag_ell_stats(theirs)
        assert torch.equal(w.float(), w_ref.float())
        assert torch.allclose(rho, rho_ref, rtol=1e-5, atol=1e-6)
        qg = case["q"][b].reshape(cfg.n_kv_heads, g, 1, cfg.head_dim).float()
        terms = orc.condition_terms(qg[:, :, 0], summ, diag_ell=(w_ref, rho_ref))
        delta_ref = ball._diag_ell_delta(qg, theirs, cfg.head_dim ** 0.5)[:, :, 0]
        assert torch.allclose(terms["delta"], delta_ref, rtol=1e-6, atol=1e-7)
        for quant in (0.25, 0.75):
            eps = float(torch.quantile(terms["score"].flatten(), quant))
            sel, z_logits, *_ = ball.select_prompt_blocks_diag_ell(qg, theirs, eps)
            assert torch.equal(sel[:, 0, 0], orc.select_threshold(terms["score"], summ.counts, eps))
            assert torch.equal(z_logits[:, :, 0], terms["z"])
