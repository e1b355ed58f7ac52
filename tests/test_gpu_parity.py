"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and the
committed reference vectors, on the same seeded inputs.

Bars: selected block indices identical; attention output within 1e-5 for fp32
pools and 2e-2 abs / 1e-2 rel for bf16 pools (the project's stated
tolerances); summaries: bounds bit-exact, fp32 means within a few ulp.
"""

import numpy as np
import pytest
import torch

from oracle import condition_block_oracle as orc
from oracle.configs import CONFIGS, DecodeConfig, make_case, scaled
from tests import golden_io
from tests.gpu_util import logical_kv, max_blocks_of, oracle_summaries_from_gpu, rank_gap, to_device

pytestmark = pytest.mark.gpu

TOL = {"float32": dict(rtol=1e-5, atol=1e-5), "bfloat16": dict(rtol=1e-2, atol=2e-2)}


def _ops():
    from interattn_b200 import ops
    return ops


def small_cases():
    yield CONFIGS["cfg1_cpu_fp32"]
    yield scaled(CONFIGS["cfg1_cpu_fp32"], max_len=1000, suffix=7)
    yield scaled(CONFIGS["cfg2_llama8b_32k"], batch=3, max_len=2304, suffix=0)
    yield scaled(CONFIGS["cfg2_llama8b_32k"], batch=2, max_len=1500, suffix=33)
    yield scaled(CONFIGS["cfg4_longctx_128k"], batch=2, max_len=4096, suffix=1, top_k=8)
    yield scaled(CONFIGS["cfg5_llama70b_ragged"], batch=5, max_len=1900, suffix=3)
    # fp32 with head_dim 128 and bf16 with head_dim 64: the other two kernel instantiations
    yield DecodeConfig("f32_d128", "float32", 2, 4, 2, 128, 16, 64, 3, (700, 129), (2, 0), seed=5)
    yield DecodeConfig("bf16_d64", "bfloat16", 2, 8, 2, 64, 16, 64, 3, (777, 65), (0, 18), seed=6)
    yield DecodeConfig("bf16_g16", "bfloat16", 1, 16, 1, 128, 16, 64, 5, (1111,), (4,), seed=7)
    yield DecodeConfig("bf16_g1", "bfloat16", 2, 2, 2, 128, 16, 64, 2, (300, 64), (0, 0), seed=8)


CASES = list(small_cases())


@pytest.fixture(scope="module", params=CASES, ids=lambda c: c.name)
def bundle(request):
    ops = _ops()
    cfg = request.param
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb)
    torch.cuda.synchronize()
    return cfg, case, q, kv, summ


def test_summaries(bundle):
    cfg, case, q, kv, summ = bundle
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        k, v = logical_kv(case, b)
        want = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size, storage="mixed")
        got = oracle_summaries_from_gpu(summ, b, plen)
        assert torch.equal(got.k_max.float(), want.k_max.float())
        assert torch.equal(got.k_min.float(), want.k_min.float())
        assert torch.allclose(got.k_bar, want.k_bar, rtol=2e-6, atol=2e-6)
        assert torch.allclose(got.v_norm_max, want.v_norm_max, rtol=2e-6, atol=0)
        if cfg.dtype == "float32":
            assert torch.allclose(got.v_bar, want.v_bar, rtol=2e-6, atol=2e-6)
        else:  # bf16 storage: at most one rounding step apart
            assert torch.allclose(got.v_bar.float(), want.v_bar.float(), rtol=8e-3, atol=1e-6)


def _oracle_selection(cfg, case, summ, b, k):
    plen = int(case["prefix_lens"][b])
    osum = oracle_summaries_from_gpu(summ, b, plen)
    qg = case["q"][b].reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim).float()
    terms = orc.condition_terms(qg, osum)
    ranked, mask = orc.select_topk(terms["score"], osum.counts, k)
    return osum, terms, ranked, mask


def test_topk_indices_bit_exact(bundle):
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("score", "z", "delta", "s"))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    idx, cnt = idx.cpu(), cnt.cpu()
    for b in range(cfg.batch):
        osum, terms, ranked, mask = _oracle_selection(cfg, case, summ, b, cfg.top_k)
        nb = osum.n_blocks
        score = aux["score"][b, :, :nb].cpu()
        # a one-token block has delta = 0 exactly, hence score 0; the CPU float noise there is ~1e-9
        assert torch.allclose(score, terms["score"], rtol=2e-4, atol=1e-8), "condition score"
        assert torch.allclose(aux["z"][b, :, :nb].cpu().reshape(cfg.n_kv_heads, cfg.group_size, nb),
                              terms["z"], rtol=1e-5, atol=1e-5)
        assert torch.allclose(aux["delta"][b, :, :nb].cpu().reshape(cfg.n_kv_heads, cfg.group_size, nb),
                              terms["delta"], rtol=1e-4, atol=1e-5)
        for h in range(cfg.n_kv_heads):
            want = sorted(ranked[h])
            n = int(cnt[b, h])
            got = idx[b, h, :n].tolist()
            assert n == len(want)
            assert got == sorted(got) and len(set(got)) == n
            assert (idx[b, h, n:] == -1).all()
            assert got == want, (
                f"seq {b} head {h}: index sets differ; relative score gap at the cut "
                f"{rank_gap(terms['score'][h], len(want)):.3e}")


def test_term1_mass_exp_variant(bundle):
    """Score variant with the first term 2 b_all softmax(z + delta): scores, top-k indices and the
    one-call step against the oracle's restatement of the variant.  The query is scaled down so that
    delta is small - for large delta the two forms of the first term coincide."""
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    q = (q.float() * 0.04).to(q.dtype)
    idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("score",),
                                      term1_mass_exp=True)
    plain = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("score",))[2]["score"]
    idx, cnt = idx.cpu(), cnt.cpu()
    differs = False
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        osum = oracle_summaries_from_gpu(summ, b, plen)
        qg = q[b].cpu().reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim).float()
        terms = orc.condition_terms(qg, osum, term1_mass_exp=True)
        ranked, _ = orc.select_topk(terms["score"], osum.counts, cfg.top_k)
        nb = osum.n_blocks
        score = aux["score"][b, :, :nb].cpu()
        assert torch.allclose(score, terms["score"], rtol=2e-4, atol=1e-8)
        differs |= not torch.allclose(score, plain[b, :, :nb].cpu(), rtol=1e-2, atol=1e-8)
        for h in range(cfg.n_kv_heads):
            n = int(cnt[b, h])
            assert idx[b, h, :n].tolist() == sorted(ranked[h])
    assert differs, "the variant must change the score"
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, term1_mass_exp=True)
    step.step(q)
    assert torch.equal(step.sel_idx.cpu()[:, :, :idx.shape[2]], idx)


def test_bf16_k_bar_option(bundle):
    """The reference's bf16 storage of the block key means (CONDITION_BLOCK_K_BAR_DTYPE=bfloat16): the stored
    mean is the fp32 mean rounded once; selection is identical to the oracle evaluated on those stored
    means; the layer-step runs on them."""
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    if cfg.dtype != "bfloat16":
        with pytest.raises(ValueError):
            ops.build_summaries(kv, cfg.block_size, max_blocks=summ.max_blocks, k_bar_dtype=torch.bfloat16)
        return
    low = ops.build_summaries(kv, cfg.block_size, max_blocks=summ.max_blocks, k_bar_dtype=torch.bfloat16)
    assert low.k_bar.dtype == torch.bfloat16
    for b in range(cfg.batch):
        nbv = (int(case["prefix_lens"][b]) + cfg.block_size - 1) // cfg.block_size
        assert torch.equal(low.k_bar[b, :, :nbv], summ.k_bar[b, :, :nbv].to(torch.bfloat16))
        assert torch.equal(low.k_max[b, :, :nbv], summ.k_max[b, :, :nbv])
    idx, cnt, aux = ops.select_blocks(q, low, kv.prefix_lens, top_k=cfg.top_k, want=("score", "s"))
    assert ops.device_status() == 0
    idx, cnt = idx.cpu(), cnt.cpu()
    for b in range(cfg.batch):
        osum, terms, ranked, _ = _oracle_selection(cfg, case, low, b, cfg.top_k)
        nb = osum.n_blocks
        assert torch.allclose(aux["s"][b, :, :nb].cpu().reshape(cfg.n_kv_heads, cfg.group_size, nb), terms["s"],
                              rtol=1e-5, atol=1e-5)
        assert torch.allclose(aux["score"][b, :, :nb].cpu(), terms["score"], rtol=2e-4, atol=1e-8)
        for h in range(cfg.n_kv_heads):
            assert idx[b, h, :int(cnt[b, h])].tolist() == sorted(ranked[h])
    step = ops.DecodeAttention(kv, low, cfg.n_q_heads, top_k=cfg.top_k)
    step.step(q)
    assert torch.equal(step.sel_idx.cpu()[:, :, :idx.shape[2]], idx)
    assert bool(torch.isfinite(step.out.float()).all())


def test_eps_selection(bundle):
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    # thresholds: the reference's sanity extremes and one mid-range value taken from the data
    _, terms0, _, _ = _oracle_selection(cfg, case, summ, 0, 1)
    mid = float(torch.quantile(terms0["score"].flatten(), 0.6))
    for eps in (0.0, mid, 1e9):
        idx, cnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, eps=eps)
        idx, cnt = idx.cpu(), cnt.cpu()
        for b in range(cfg.batch):
            osum, terms, _, _ = _oracle_selection(cfg, case, summ, b, 1)
            want_mask = orc.select_threshold(terms["score"], osum.counts, eps)
            for h in range(cfg.n_kv_heads):
                want = want_mask[h].nonzero().flatten().tolist()
                got = idx[b, h, : int(cnt[b, h])].tolist()
                if eps == 0.0:
                    # every block that holds a token, except a one-token block (zero width: score 0)
                    everyone = list(range(osum.n_blocks))
                    assert got == everyone or (int(osum.counts[-1]) == 1 and got == everyone[:-1])
                elif eps == 1e9:
                    assert got == []
                else:
                    sc = terms["score"][h]
                    near = ((sc - eps).abs() <= 2e-4 * sc.abs() + 1e-8).nonzero().flatten().tolist()
                    assert set(got) ^ set(want) <= set(near)


def test_eps_threshold_sweep(bundle):
    """Routing near the threshold: the reference probes its kernels with thresholds at quantiles of the reference
    scores so that 0.1 % ... 50 % of the blocks are selected and counts the blocks on which two implementations
    disagree (llama/script/implementation/tensorcore_selection/benchmark.py:70-117).  Here: the selected sets of
    the CUDA kernel and of the oracle differ at most in blocks whose score lies within the score tolerance of
    the threshold, at every such quantile; selected counts fall as the threshold rises."""
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    per_seq = [_oracle_selection(cfg, case, summ, b, 1) for b in range(cfg.batch)]
    live = torch.cat([terms["score"][:, osum.counts > 0].flatten() for osum, terms, _, _ in per_seq])
    if live.numel() < 8:
        pytest.skip("too few blocks for quantiles")
    totals = []
    for frac in (0.5, 0.1, 0.01, 0.001):
        eps = float(torch.quantile(live.double(), 1.0 - frac))
        idx, cnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, eps=eps)
        idx, cnt = idx.cpu(), cnt.cpu()
        disagree = 0
        for b, (osum, terms, _, _) in enumerate(per_seq):
            want_mask = orc.select_threshold(terms["score"], osum.counts, eps)
            for h in range(cfg.n_kv_heads):
                want = set(want_mask[h].nonzero().flatten().tolist())
                got = idx[b, h, : int(cnt[b, h])].tolist()
                assert got == sorted(got) and len(set(got)) == len(got)
                sc = terms["score"][h]
                near = set(((sc - eps).abs() <= 2e-4 * sc.abs() + 1e-8).nonzero().flatten().tolist())
                assert set(got) ^ want <= near, f"quantile {frac}: seq {b} head {h}"
                disagree += len(set(got) ^ want)
        assert disagree <= max(1, live.numel() // 1000)
        totals.append(int(cnt.sum()))
    assert totals == sorted(totals, reverse=True)


@pytest.mark.parametrize("rep_mode", ["sparse_only", "hybrid"])
@pytest.mark.parametrize("n_splits", [1, 3])
def test_attention_output(bundle, rep_mode, n_splits):
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    nb = summ.max_blocks
    idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("z",))
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=cfg.block_size, max_blocks=nb, rep_mode=rep_mode,
                               summ=summ, z=aux["z"], n_splits=n_splits)
    out = ops.finalize(o, lse, q.dtype)
    torch.cuda.synchronize()
    idx, cnt = idx.cpu(), cnt.cpu()
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        osum = oracle_summaries_from_gpu(summ, b, plen)
        k, v = logical_kv(case, b)
        mask = torch.zeros((cfg.n_kv_heads, osum.n_blocks), dtype=torch.bool)
        for h in range(cfg.n_kv_heads):
            mask[h, idx[b, h, : int(cnt[b, h])].long()] = True
        z = aux["z"][b, :, : osum.n_blocks].cpu().reshape(cfg.n_kv_heads, cfg.group_size, -1)
        qg = case["q"][b].reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim).float()
        want = orc.decode_attention(qg, k, v, plen, cfg.block_size, mask, rep_mode=rep_mode, z=z, v_bar=osum.v_bar)
        got = out[b].float().cpu().reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim)
        torch.testing.assert_close(got, want, **TOL[cfg.dtype])


def test_one_call_layer_step_matches_the_three_calls(bundle):
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    for rep_mode in ("sparse_only", "hybrid"):
        step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode, n_splits=2)
        out = step.step(q).clone()
        idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("z",))
        o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=cfg.block_size, max_blocks=summ.max_blocks,
                                   rep_mode=rep_mode, summ=summ, z=aux["z"], n_splits=2)
        want = ops.finalize(o, lse, q.dtype)
        torch.cuda.synchronize()
        assert torch.equal(step.sel_idx, idx) and torch.equal(step.sel_count, cnt)
        # the single fused launch (one CTA per pair, no representatives) partitions the pages differently
        same = torch.equal if not ops.last_decode_fused() else (
            lambda a, b: torch.allclose(a.float(), b.float(), **TOL[cfg.dtype]))
        assert same(out, want)
        # host-buffer entry point: pinned q in, pinned out back
        q_host = case["q"].contiguous().pin_memory()
        out_host = torch.empty_like(q_host).pin_memory()
        step.step_host(q_host, out_host)
        assert same(out_host, want.cpu())


def test_equal_share_grid_matches_the_pair_grid(bundle, monkeypatch):
    """INTERATTN_B200_DECODE_GRID=flat: the attention kernel on a fixed grid of two CTAs per SM, every
    CTA an equal slice of all pairs' pages (slices cross pair boundaries).  Same selection, outputs
    within tolerance of the pair grid and of the oracle (the partition differs, so not the same bits);
    twice in a row, because the per-pair arrival counters must come back to zero."""
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    for rep_mode in ("sparse_only", "hybrid"):
        monkeypatch.delenv("INTERATTN_B200_DECODE_GRID", raising=False)
        pairs = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode, n_splits=2)
        want = pairs.step(q).clone()
        monkeypatch.setenv("INTERATTN_B200_DECODE_GRID", "flat")
        flat = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode, n_splits=2)
        for _ in range(2):
            got = flat.step(q).clone()
            torch.cuda.synchronize()
            assert torch.equal(flat.sel_idx, pairs.sel_idx)
            torch.testing.assert_close(got.float(), want.float(), **TOL[cfg.dtype])
        assert ops.device_status() == 0


def test_layer_step_replays_from_a_cuda_graph():
    """The step allocates nothing and reads its per-step quantities from device
    memory, so it can be captured once and replayed (the reference's graphed
    decode loop, condition_block_triton_impl/core.py:190-316): new q and a longer
    suffix are picked up by the replay."""
    ops = _ops()
    cfg = scaled(CONFIGS["cfg2_llama8b_32k"], batch=2, max_len=2304, suffix=40)
    case = make_case(cfg)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb)
    full_seq = kv.seq_lens.clone()
    kv.seq_lens.copy_(kv.prefix_lens + 3)                 # start with 3 suffix tokens
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode="hybrid", n_splits=3)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step.step(q)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step.step(q)
    for extra in (3, 17, 40):
        kv.seq_lens.copy_(kv.prefix_lens + extra)
        q.copy_(torch.roll(q, extra, dims=2))
        graph.replay()
        got = step.out.clone()
        want = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode="hybrid", n_splits=3).step(q)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    assert torch.equal(kv.seq_lens, full_seq)


def test_incremental_summary_update_equals_full_rebuild():
    """Summary maintenance during decode: when the generated suffix has grown by
    whole blocks, raising prefix_lens and recomputing only the new blocks gives
    the same summaries as rebuilding everything, and the next step then selects
    among the new blocks too."""
    ops = _ops()
    cfg = DecodeConfig("grow", "bfloat16", 2, 8, 2, 128, 16, 64, 3, (640, 200), (150, 70), seed=12)
    case = make_case(cfg)
    q, kv = to_device(case)
    nb = (max(p + s for p, s in zip(cfg.prefix_lens, cfg.suffix_lens)) + 63) // 64
    summ = ops.build_summaries(kv, 64, max_blocks=nb)                  # prompt blocks only
    before = summ.k_bar.clone()
    old_blocks = torch.tensor([(p + 63) // 64 for p in cfg.prefix_lens], dtype=torch.int32, device=q.device)
    # two more whole blocks of the first sequence and one of the second join the summarised prefix
    grown = torch.tensor([cfg.prefix_lens[0] + 128, 256], dtype=torch.int32, device=q.device)
    kv.prefix_lens.copy_(grown)
    first = torch.tensor([cfg.prefix_lens[0] // 64, 200 // 64], dtype=torch.int32, device=q.device)
    ops.build_summaries(kv, 64, out=summ, first_blocks=first)
    full = ops.build_summaries(kv, 64, max_blocks=nb)
    torch.cuda.synchronize()
    for b, n_new in ((0, (640 + 128) // 64), (1, 4)):
        for name in ("k_bar", "k_max", "k_min", "v_bar", "v_norm_max"):
            assert torch.equal(getattr(summ, name)[b, :, :n_new], getattr(full, name)[b, :, :n_new]), name
    assert torch.equal(summ.k_bar[0, :, : int(old_blocks[0])], before[0, :, : int(old_blocks[0])])   # untouched
    # the step over the grown prefix matches the oracle (new blocks selectable, shorter suffix)
    idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("z",))
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=64, max_blocks=nb, n_splits=2)
    out = ops.finalize(o, lse, torch.float32).cpu()
    for b in range(cfg.batch):
        plen = int(grown[b])
        k, v = logical_kv(case, b)
        osum = oracle_summaries_from_gpu(summ, b, plen)
        qg = case["q"][b].reshape(2, 4, 128).float()
        terms = orc.condition_terms(qg, osum)
        ranked, mask = orc.select_topk(terms["score"], osum.counts, cfg.top_k)
        for h in range(2):
            assert idx[b, h, : int(cnt[b, h])].cpu().tolist() == sorted(ranked[h])
        want = orc.decode_attention(qg, k, v, plen, 64, mask, rep_mode="sparse_only")
        torch.testing.assert_close(out[b].reshape(2, 4, 128), want, rtol=1e-2, atol=2e-2)


def test_block_range_shares_merge_to_the_whole(bundle):
    """Split-KV across ranks, emulated on one GPU: each 'rank' attends over its
    own block range (the last one also over the suffix); merging the (o, lse)
    partials reproduces the single-GPU result."""
    ops = _ops()
    cfg, case, q, kv, summ = bundle
    nb = summ.max_blocks
    idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("z",))
    for rep_mode in ("sparse_only", "hybrid"):
        o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=cfg.block_size, max_blocks=nb, rep_mode=rep_mode,
                                   summ=summ, z=aux["z"], n_splits=1)
        whole, whole_lse = ops.finalize(o, lse, torch.float32, return_lse=True)
        ranks = 3
        cuts = [nb * r // ranks for r in range(ranks + 1)]
        parts = []
        for r in range(ranks):
            po, plse = ops.sparse_decode(q, kv, idx, cnt, block_size=cfg.block_size, max_blocks=nb,
                                         rep_mode=rep_mode, summ=summ, z=aux["z"], n_splits=2,
                                         block_range=(cuts[r], cuts[r + 1]), with_suffix=(r == ranks - 1))
            parts.append(ops.finalize(po, plse, torch.float32, return_lse=True))
        go = torch.stack([p[0] for p in parts], dim=2).contiguous()
        glse = torch.stack([p[1] for p in parts], dim=2).contiguous()
        merged, merged_lse = ops.finalize(go, glse, torch.float32, return_lse=True)
        torch.cuda.synchronize()
        # fp32 pools: only the summation order differs.  bf16 pools: the probabilities are
        # rounded to bf16 relative to the running maximum, which depends on the partition.
        tol = dict(rtol=2e-5, atol=2e-5) if cfg.dtype == "float32" else dict(rtol=1e-2, atol=3e-3)
        torch.testing.assert_close(merged, whole, **tol)
        finite = torch.isfinite(whole_lse)
        torch.testing.assert_close(merged_lse[finite], whole_lse[finite], rtol=1e-5, atol=1e-5)


# ---------------------------------------------------------------------------
# committed reference vectors
# ---------------------------------------------------------------------------

def _golden(which):
    if which == "ragged":
        case, vec = golden_io.ragged_case()
    else:
        case, vec, ok = golden_io.cfg1_case()
        if not ok:
            pytest.skip("seeded inputs differ on this torch build")
    return case, vec


@pytest.mark.parametrize("which", ["ragged", "cfg1"])
def test_against_reference_vectors(which):
    """End to end against what the unmodified reference produced: top-k index
    sets from its score, its dense hybrid output for that selection and its
    sparse-only output (the same function with every representative masked)."""
    ops = _ops()
    case, vec = _golden(which)
    cfg = case["cfg"]
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb)
    idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("z", "score"))
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=cfg.block_size, max_blocks=nb, rep_mode="hybrid",
                               summ=summ, z=aux["z"], n_splits=2)
    out = ops.finalize(o, lse, torch.float32).cpu()
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=cfg.block_size, max_blocks=nb, rep_mode="sparse_only",
                               n_splits=3)
    out_sparse = ops.finalize(o, lse, torch.float32).cpu()
    step_sparse = ops.DecodeAttention(kv, summ, q.shape[1], top_k=cfg.top_k, rep_mode="sparse_only").step(q).float().cpu()
    idx, cnt = idx.cpu(), cnt.cpu()
    tol = dict(rtol=1e-5, atol=1e-5) if cfg.dtype == "float32" else dict(rtol=1e-2, atol=2e-2)
    for b in range(cfg.batch):
        want_sparse = torch.from_numpy(vec[f"seq{b}_sparse_topk_out"])
        torch.testing.assert_close(out_sparse[b].reshape(want_sparse.shape), want_sparse, **tol)
        torch.testing.assert_close(step_sparse[b].reshape(want_sparse.shape), want_sparse, **tol)
        pre = f"seq{b}_"
        ranked = vec[pre + "topk_ranked"]
        n_blocks = vec[pre + "score"].shape[1]
        np.testing.assert_allclose(aux["score"][b, :, :n_blocks].cpu().numpy(), vec[pre + "score"], rtol=3e-4, atol=1e-12)
        np.testing.assert_allclose(aux["z"][b, :, :n_blocks].cpu().numpy().reshape(vec[pre + "z_logits"].shape),
                                   vec[pre + "z_logits"], rtol=1e-5, atol=1e-5)
        for h in range(cfg.n_kv_heads):
            assert idx[b, h, : int(cnt[b, h])].tolist() == sorted(ranked[h].tolist())
        want = torch.from_numpy(vec[pre + "hybrid_topk_out"])
        got = out[b].reshape(want.shape)
        torch.testing.assert_close(got, want, **tol)
    # the reference's epsilon rule at the stored thresholds
    for qi in (0, 1):
        for b in range(cfg.batch):
            eps = float(vec[f"seq{b}_eps{qi}"])
            gi, gc, _ = ops.select_blocks(q, summ, kv.prefix_lens, eps=eps)
            for h in range(cfg.n_kv_heads):
                want = np.nonzero(vec[f"seq{b}_mask_eps{qi}q"][h])[0].tolist()
                got = gi[b, h, : int(gc[b, h])].cpu().tolist()
                score = vec[f"seq{b}_score"][h]
                near = np.nonzero(np.abs(score - eps) <= 3e-4 * np.abs(score))[0].tolist()
                assert set(got) ^ set(want) <= set(near)


# ---------------------------------------------------------------------------
# edge cases
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("prefix", [1, 63, 64, 65, 15 * 64, 16 * 64, 17 * 64 + 1, 31 * 64, 32 * 64 + 5, 33 * 64])
def test_block_count_edges(prefix):
    ops = _ops()
    cfg = DecodeConfig("edge", "bfloat16", 1, 8, 2, 128, 16, 64, 4, (prefix,), (2,), seed=prefix)
    case = make_case(cfg)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    summ = ops.build_summaries(kv, 64, max_blocks=nb)
    for top_k in (1, 4, nb, nb + 3):
        idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=top_k, max_sel=nb + 3, want=("z",))
        o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=64, max_blocks=nb, rep_mode="hybrid", summ=summ,
                                   z=aux["z"], n_splits=2)
        out = ops.finalize(o, lse, q.dtype).float().cpu()
        osum, terms, ranked, mask = _oracle_selection(cfg, case, summ, 0, top_k)
        for h in range(cfg.n_kv_heads):
            assert idx[0, h, : int(cnt[0, h])].cpu().tolist() == sorted(ranked[h])
        k, v = logical_kv(case, 0)
        qg = case["q"][0].reshape(2, 4, 128).float()
        want = orc.decode_attention(qg, k, v, prefix, 64, mask, rep_mode="hybrid", z=terms["z"], v_bar=osum.v_bar)
        torch.testing.assert_close(out[0].reshape(2, 4, 128), want, rtol=1e-2, atol=2e-2)


def test_empty_prefix_attends_suffix_only_and_empty_everything_gives_zero():
    ops = _ops()
    cfg = DecodeConfig("nopfx", "bfloat16", 2, 8, 2, 128, 16, 64, 4, (0, 0), (21, 0), seed=3)
    case = make_case(cfg, spare_pages=2)
    case["block_table"] = case["block_table"].clamp_min(0)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, 64, max_blocks=1)
    idx, cnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, top_k=4)
    assert int(cnt.sum()) == 0 and bool((idx == -1).all())
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=64, max_blocks=1, n_splits=2)
    out = ops.finalize(o, lse, torch.float32).cpu()
    k, v = logical_kv(case, 0)
    qg = case["q"][0].reshape(2, 4, 128).float()
    want = orc.decode_attention(qg, k, v, 0, 64, torch.zeros((2, 0), dtype=torch.bool), rep_mode="sparse_only")
    torch.testing.assert_close(out[0].reshape(2, 4, 128), want, rtol=1e-2, atol=2e-2)
    assert bool((out[1] == 0).all())            # nothing to attend to: zeros, not NaN


def test_tied_scores_go_to_the_lowest_index():
    """Identical blocks give bit-identical scores; the k lowest indices must win."""
    ops = _ops()
    cfg = DecodeConfig("ties", "float32", 1, 4, 1, 64, 16, 64, 3, (64 * 9,), (0,), seed=9)
    case = make_case(cfg)
    # make every block a copy of block 0 (same pages repeated in the table)
    case["block_table"][0] = case["block_table"][0, :4].repeat(9)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, 64, max_blocks=9)
    for k in (1, 3, 8):
        idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=k, want=("score",))
        score = aux["score"][0, 0].cpu()
        assert bool((score == score[0]).all())
        assert idx[0, 0, :k].cpu().tolist() == list(range(k))


def test_finalize_matches_oracle_merge():
    ops = _ops()
    torch.manual_seed(0)
    o = torch.randn(37, 5, 128)
    lse = torch.randn(37, 5) * 3
    lse[3] = float("-inf")
    lse[4, 1:] = float("-inf")
    want, want_lse = orc.merge_o_lse(o, lse)
    got, got_lse = ops.finalize(o.cuda(), lse.cuda(), torch.float32, return_lse=True)
    want[3] = 0
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(got_lse.cpu(), want_lse, rtol=1e-5, atol=1e-6)


def test_argument_errors_are_value_errors():
    ops = _ops()
    cfg = DecodeConfig("err", "bfloat16", 1, 8, 2, 128, 16, 64, 2, (128,), (0,), seed=1)
    case = make_case(cfg)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, 64, max_blocks=2)
    with pytest.raises(ValueError):
        ops.select_blocks(q, summ, kv.prefix_lens, top_k=5, max_sel=2)          # k > capacity
    with pytest.raises(ValueError):
        ops.select_blocks(q, summ, kv.prefix_lens)                              # neither rule
    with pytest.raises(ValueError):
        ops.select_blocks(q.float(), summ, kv.prefix_lens, top_k=1)             # dtype mismatch
    with pytest.raises(ValueError):
        ops.select_blocks(case["q"], summ, kv.prefix_lens, top_k=1)             # CPU tensor
    with pytest.raises(ValueError):
        ops.build_summaries(kv, 40)                                             # block not a page multiple
    idx, cnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, top_k=1)
    with pytest.raises(ValueError):
        ops.sparse_decode(q, kv, idx, cnt, block_size=64, max_blocks=2, rep_mode="hybrid")   # no z / summaries
    with pytest.raises(ValueError):
        ops.sparse_decode(q, kv, idx, cnt, block_size=64, max_blocks=2, n_splits=0)


@pytest.mark.parametrize("dtype,head_dim", [("bfloat16", 128), ("bfloat16", 64), ("float32", 128), ("float32", 64)])
def test_streaming_and_direct_summary_kernels_agree(dtype, head_dim, monkeypatch):
    """The two forms of the summary kernel (bulk-copy rings / plain loads) do the same arithmetic in the same
    order per coordinate: means, bounds and mean values are identical bit for bit; the largest value norm only
    differs in how the 32 lanes' partial sums are added (a few ulp).  Ragged lengths, an incremental update
    included."""
    ops = _ops()
    cfg = DecodeConfig("summ_forms", dtype, 5, 8, 2, head_dim, 16, 64, 3, (1, 1000, 64, 2049, 0), (0, 3, 0, 0, 5), seed=17)
    case = make_case(cfg, spare_pages=2)
    case["block_table"] = case["block_table"].clamp_min(0)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    built = {}
    for form in ("stream", "direct"):
        monkeypatch.setenv("INTERATTN_B200_SUMMARIES", form)
        full = ops.build_summaries(kv, cfg.block_size, max_blocks=nb + 2)
        part = ops.build_summaries(kv, cfg.block_size, max_blocks=nb + 2)
        for name in ("k_bar", "k_max", "k_min", "v_bar", "v_norm_max"):
            getattr(part, name).fill_(7.0)  # blocks below first_blocks must keep what they hold
        first = torch.tensor([0, 9, 1, 30, 0], dtype=torch.int32, device=q.device)
        ops.build_summaries(kv, cfg.block_size, max_blocks=nb + 2, out=part, first_blocks=first)
        built[form] = (full, part)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for which in (0, 1):
        a, b = built["stream"][which], built["direct"][which]
        for name in ("k_bar", "k_max", "k_min", "v_bar"):
            assert torch.equal(getattr(a, name), getattr(b, name)), name
        assert torch.allclose(a.v_norm_max, b.v_norm_max, rtol=1e-6, atol=0)
    full, part = built["stream"]
    assert bool((part.k_max[1, :, :9] == 7.0).all()) and torch.equal(part.k_max[1, :, 9:16], full.k_max[1, :, 9:16])
    assert bool((part.k_max[3, :, :30] == 7.0).all()) and torch.equal(part.k_max[3, :, 30:33], full.k_max[3, :, 30:33])
