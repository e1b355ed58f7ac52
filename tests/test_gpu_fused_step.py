"""GPU parity of the one-kernel layer step (``condition_block_select_attend_kernel``): the CTA that
picked the blocks of a (sequence, kv head) attends over their pages and the suffix itself.

The launch shape decides whether a step fuses (the whole grid resident at once); the small cases here pin
the shape through the environment (``INTERATTN_B200_SELECT_CLUSTER``, wide and narrow CTAs) and assert that
the fused kernel ran.  Bars: the selection identical to the stand-alone selection kernel; the output within the
bf16 tolerance (2e-2 abs / 1e-2 rel) of the oracle's attention over exactly those blocks.
"""

import pytest
import torch

from oracle import condition_block_oracle as orc
from oracle.configs import CONFIGS, DecodeConfig, make_case, scaled
from tests.gpu_util import logical_kv, max_blocks_of, oracle_summaries_from_gpu, to_device

pytestmark = pytest.mark.gpu
TOL = dict(rtol=1e-2, atol=2e-2)


def _ops():
    from interattn_b200 import ops
    return ops


CASES = [
    scaled(CONFIGS["cfg2_llama8b_32k"], batch=3, max_len=2304, suffix=0),
    scaled(CONFIGS["cfg2_llama8b_32k"], batch=2, max_len=1500, suffix=33),
    scaled(CONFIGS["cfg4_longctx_128k"], batch=2, max_len=4096, suffix=1, top_k=8),
    scaled(CONFIGS["cfg5_llama70b_ragged"], batch=5, max_len=1900, suffix=3),
    DecodeConfig("bf16_g1", "bfloat16", 2, 2, 2, 128, 16, 64, 2, (300, 64), (0, 0), seed=8),
    DecodeConfig("bf16_g2_ragged", "bfloat16", 4, 4, 2, 128, 16, 64, 3, (1, 129, 1000, 0), (15, 16, 17, 40), seed=11),
    DecodeConfig("bf16_g8_long_suffix", "bfloat16", 2, 8, 1, 128, 16, 64, 2, (520, 7), (300, 5), seed=12),
    # blocks of two and of eight pages
    DecodeConfig("bf16_block32", "bfloat16", 2, 8, 2, 128, 16, 32, 5, (1000, 333), (3, 40), seed=13),
    DecodeConfig("bf16_block128", "bfloat16", 2, 8, 2, 128, 16, 128, 3, (2000, 129), (17, 0), seed=14),
]


def _check_against_oracle(cfg, case, summ, out, idx, cnt, rep_mode="sparse_only", z=None):
    out = out.float().cpu()
    idx, cnt = idx.cpu(), cnt.cpu()
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        osum = oracle_summaries_from_gpu(summ, b, plen)
        k, v = logical_kv(case, b)
        mask = torch.zeros((cfg.n_kv_heads, osum.n_blocks), dtype=torch.bool)
        for h in range(cfg.n_kv_heads):
            mask[h, idx[b, h, :int(cnt[b, h])].long()] = True
        qg = case["q"][b].reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim).float()
        extra = {}
        if rep_mode == "hybrid":
            extra = dict(z=z[b, :, :osum.n_blocks].cpu().reshape(cfg.n_kv_heads, cfg.group_size, -1), v_bar=osum.v_bar)
        want = orc.decode_attention(qg, k, v, plen, cfg.block_size, mask, rep_mode=rep_mode, **extra)
        got = out[b].reshape(cfg.n_kv_heads, cfg.group_size, cfg.head_dim)
        torch.testing.assert_close(got, want, **TOL)


@pytest.mark.parametrize("rep_mode", ["sparse_only", "hybrid"])
@pytest.mark.parametrize("shape,cluster", [("wide", 1), ("narrow", 1), ("wide", 2), ("wide", 4), ("wide", 8), ("narrow", 2)])
@pytest.mark.parametrize("cfg", CASES, ids=lambda c: c.name)
def test_fused_step_matches_selection_and_oracle(cfg, shape, cluster, rep_mode, monkeypatch):
    """cluster > 1: the CTAs that share a (sequence, kv head) also share its pages and rank 0 merges them.
    hybrid: every block that was not picked attends through its representative, straight from the logits the
    selection left in shared memory."""
    ops = _ops()
    resident = torch.cuda.get_device_properties(0).multi_processor_count * (2 if shape == "narrow" else 1)
    if cfg.batch * cfg.n_kv_heads * cluster > resident:
        pytest.skip("more CTAs than resident slots: this batch keeps the two kernels")
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", str(cluster))
    monkeypatch.setenv("INTERATTN_B200_SELECT_SHAPE", shape)
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode)
    for _ in range(2):  # twice: the ring's barriers are initialised per launch
        out = step.step(q).clone()
        assert ops.last_decode_fused(), "the pinned shape must take the one-kernel form"
    idx, cnt, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("z",))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(step.sel_idx[:, :, :idx.shape[2]], idx) and torch.equal(step.sel_count, cnt)
    _check_against_oracle(cfg, case, summ, out, idx, cnt, rep_mode, aux["z"])
    # the two-kernel form on the same inputs, through the three public calls (they never fuse)
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=cfg.block_size, max_blocks=summ.max_blocks, n_splits=2,
                               rep_mode=rep_mode, summ=summ, z=aux["z"])
    two = ops.finalize(o, lse, q.dtype)
    torch.testing.assert_close(out.float(), two.float(), **TOL)


def test_switch_between_the_one_kernel_and_the_two_kernel_form(monkeypatch):
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = CASES[0]
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k)
    one = step.step(q).clone()
    assert ops.last_decode_fused()
    before = ops.set_fused_step(False)
    try:
        two = step.step(q).clone()
        assert not ops.last_decode_fused()
    finally:
        assert ops.set_fused_step(before) is False
    again = step.step(q).clone()
    torch.cuda.synchronize()
    assert ops.last_decode_fused() and ops.device_status() == 0
    assert torch.equal(one, again)
    torch.testing.assert_close(one.float(), two.float(), **TOL)


def test_fused_step_with_epsilon_rule(monkeypatch):
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = CASES[1]
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    _, _, aux = ops.select_blocks(q, summ, kv.prefix_lens, top_k=cfg.top_k, want=("score",))
    eps = float(aux["score"].flatten().sort().values[-40])  # keeps a few dozen blocks in total
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, eps=eps)
    out = step.step(q).clone()
    assert ops.last_decode_fused()
    idx, cnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, eps=eps)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(step.sel_idx[:, :, :idx.shape[2]], idx) and torch.equal(step.sel_count, cnt)
    assert int(cnt.sum()) > 0
    _check_against_oracle(cfg, case, summ, out, idx, cnt)


@pytest.mark.parametrize("cluster", [1, 2])
def test_fused_step_with_more_pages_than_the_page_list_holds(cluster, monkeypatch):
    """One query row per kv head and an epsilon below every score: all blocks are kept, four pages each -
    more items than the shared-memory page list (rows x blocks entries) holds, so the attention phase
    resolves and streams them in several chunks while the ring carries over."""
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", str(cluster))
    cfg = DecodeConfig("g1_keep_all", "bfloat16", 2, 2, 2, 128, 16, 64, 2, (64 * 37 + 5, 64 * 12), (9, 0), seed=31)
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, eps=-1.0)
    out = step.step(q).clone()
    assert ops.last_decode_fused()
    idx, cnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, eps=-1.0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert cnt.cpu().tolist() == [[38, 38], [12, 12]], "every block of every sequence"
    assert torch.equal(step.sel_idx[:, :, :idx.shape[2]], idx) and torch.equal(step.sel_count, cnt)
    _check_against_oracle(cfg, case, summ, out, idx, cnt)


def test_fused_step_empty_prefix_and_empty_sequence(monkeypatch):
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = DecodeConfig("nopfx", "bfloat16", 2, 8, 2, 128, 16, 64, 4, (0, 0), (21, 0), seed=3)
    case = make_case(cfg, spare_pages=2)
    case["block_table"] = case["block_table"].clamp_min(0)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, 64, max_blocks=1)
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=4)
    out = step.step(q).float().cpu()
    assert ops.last_decode_fused() and ops.device_status() == 0
    assert int(step.sel_count.sum()) == 0
    k, v = logical_kv(case, 0)
    qg = case["q"][0].reshape(2, 4, 128).float()
    want = orc.decode_attention(qg, k, v, 0, 64, torch.zeros((2, 0), dtype=torch.bool), rep_mode="sparse_only")
    torch.testing.assert_close(out[0].reshape(2, 4, 128), want, **TOL)
    assert bool((out[1] == 0).all())  # nothing to attend to: zeros, not NaN


def test_fused_step_skips_a_table_entry_outside_the_pool(monkeypatch):
    """A block-table entry past the declared pool size: the page contributes nothing, the device status
    word reports it, nothing outside the pool is read (the TMA unit would zero-fill it anyway)."""
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = CASES[0]
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    good = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k).step(q).clone()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    small = ops.PagedKV(k_pool=kv.k_pool, v_pool=kv.v_pool, block_table=kv.block_table, prefix_lens=kv.prefix_lens,
                        seq_lens=kv.seq_lens, n_pool_pages=int(kv.block_table.max()))  # the last page is "outside"
    out = ops.DecodeAttention(small, summ, cfg.n_q_heads, top_k=cfg.top_k).step(q).clone()
    torch.cuda.synchronize()
    assert ops.last_decode_fused()
    assert ops.device_status() & 8, "IA_DEV_STATUS_BAD_INDEX"  # reading the word clears it
    assert torch.isfinite(out.float()).all() and torch.isfinite(good.float()).all()


@pytest.mark.parametrize("rep_mode", ["sparse_only", "hybrid"])
def test_fused_step_ignores_what_lies_in_dead_rows(rep_mode, monkeypatch):
    """Token slots past a sequence's end (inside its last page) and summary rows past its last block hold
    NaN: the kernel masks their logits and must also keep them out of the P.V product (0 x NaN)."""
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = DecodeConfig("dead_rows", "bfloat16", 2, 8, 2, 128, 16, 64, 3, (1000, 333), (5, 20), seed=21)
    case = make_case(cfg, spare_pages=2)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb + 3)
    clean = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode).step(q).clone()
    assert ops.last_decode_fused()
    for b in range(cfg.batch):
        slen, plen = int(case["seq_lens"][b]), int(case["prefix_lens"][b])
        page = int(case["block_table"][b, (slen - 1) // 16])
        kv.k_pool[page, :, slen % 16:] = float("nan")
        kv.v_pool[page, :, slen % 16:] = float("nan")
        n_blocks = (plen + 63) // 64
        summ.v_bar[b, :, n_blocks:] = float("nan")
    out = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode).step(q).clone()
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, clean)


def test_fused_step_over_a_static_cache_addressed_in_place(monkeypatch):
    """A [batch, kv head, token, head_dim] cache viewed as pages (head stride > page stride): the pools' tensor
    maps put the head outermost; same output as the two-kernel form over the same view."""
    ops = _ops()
    from interattn_b200.llama_decode import cache_as_pool
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    b, hkv, t, d, g = 3, 2, 1024, 128, 4
    gen = torch.Generator(device="cuda").manual_seed(5)
    key = torch.randn((b, hkv, t, d), device="cuda", generator=gen).to(torch.bfloat16)
    value = torch.randn((b, hkv, t, d), device="cuda", generator=gen).to(torch.bfloat16)
    k_pool, v_pool, table = cache_as_pool(key, value)
    prefix = torch.tensor([900, 640, 77], dtype=torch.int32, device="cuda")
    seq = prefix + torch.tensor([5, 100, 16], dtype=torch.int32, device="cuda")
    kv = ops.PagedKV(k_pool, v_pool, table, prefix, seq)
    summ = ops.build_summaries(kv, 64, max_blocks=15)
    q = torch.randn((b, hkv * g, d), device="cuda", generator=gen).to(torch.bfloat16)
    step = ops.DecodeAttention(kv, summ, hkv * g, top_k=4)
    out = step.step(q).clone()
    assert ops.last_decode_fused(), "the strided view must be expressible as a tensor map"
    idx, cnt, _ = ops.select_blocks(q, summ, prefix, top_k=4)
    assert torch.equal(step.sel_idx[:, :, :idx.shape[2]], idx) and torch.equal(step.sel_count, cnt)
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=64, max_blocks=15, n_splits=2)
    two = ops.finalize(o, lse, q.dtype)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    torch.testing.assert_close(out.float(), two.float(), **TOL)


def test_fused_step_replays_from_a_cuda_graph(monkeypatch):
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = CASES[3]
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k)
    want = step.step(q).clone()
    assert ops.last_decode_fused()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step.step(q)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step.step(q)
    torch.cuda.current_stream().wait_stream(side)
    step.out.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(step.out, want)
    assert ops.device_status() == 0


def test_phase_stamps_of_the_last_fused_step(monkeypatch):
    """The first CTA of the one-kernel step leaves three time stamps; the two phases are positive and add up to
    less than the step's duration between events."""
    ops = _ops()
    monkeypatch.setenv("INTERATTN_B200_SELECT_CLUSTER", "1")
    cfg = CASES[0]
    case = make_case(cfg, spare_pages=3)
    q, kv = to_device(case)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=max_blocks_of(case))
    step = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k)
    step.step(q)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    step.step(q)
    b.record()
    torch.cuda.synchronize()
    assert ops.last_decode_fused()
    sel_us, att_us = ops.last_step_phases()
    assert 0.0 < sel_us < 1000.0 and 0.0 < att_us < 1000.0
    # two clocks: the stamps come from the global timer (its tick may be a microsecond), the span from events
    assert sel_us + att_us <= a.elapsed_time(b) * 1e3 + 3.0
