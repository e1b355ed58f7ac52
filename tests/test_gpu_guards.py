"""Index and block-table validation on the public ABI.

``ia_sparse_decode`` takes the caller's index list and block table.  Every entry
is checked on the device before it is used - block index against ``max_blocks``,
logical page against the table row, physical page against ``n_pool_pages`` -
and a bad one is skipped and reported as ``IA_DEV_STATUS_BAD_INDEX`` instead of
being dereferenced.

Every "bad" value below lies outside the range the geometry *declares* but
inside memory this test allocated (fewer blocks / pool pages are declared than
exist), so that even a wrong guard could only read the test's own tensors.
"""

from dataclasses import replace

import pytest
import torch

from oracle import condition_block_oracle as orc
from oracle.configs import DecodeConfig, make_case
from tests.gpu_util import logical_kv, max_blocks_of, to_device

pytestmark = pytest.mark.gpu

CFG = DecodeConfig("guards", "bfloat16", 2, 8, 2, 128, 16, 64, 3, (512, 448), (5, 0), seed=5)


def _setup():
    from interattn_b200 import _lib, ops
    case = make_case(CFG)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    summ = ops.build_summaries(kv, CFG.block_size, max_blocks=nb)
    idx, cnt, _ = ops.select_blocks(q, summ, kv.prefix_lens, top_k=CFG.top_k)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return _lib, ops, case, q, kv, nb, idx, cnt


def _run(ops, q, kv, idx, cnt, nb, **kw):
    o, lse = ops.sparse_decode(q, kv, idx, cnt, block_size=CFG.block_size, max_blocks=nb, n_splits=2, **kw)
    out = ops.finalize(o, lse, torch.float32)
    torch.cuda.synchronize()
    return out


def test_clean_inputs_leave_the_status_word_clear():
    _lib, ops, case, q, kv, nb, idx, cnt = _setup()
    out = _run(ops, q, kv, idx, cnt, nb)
    assert ops.device_status() == 0
    assert bool(torch.isfinite(out).all())


def test_block_index_outside_the_declared_blocks_is_skipped():
    _lib, ops, case, q, kv, nb, idx, cnt = _setup()
    want = _run(ops, q, kv, idx, cnt, nb)
    # declare one block fewer than exist and select the last real block of sequence 0
    declared = nb - 1
    bad = idx.clone()
    bad[0, :, :] = -1
    bad[0, :, 0] = 0
    bad[0, :, 1] = nb - 1                       # >= declared, < the blocks that exist
    n = torch.full_like(cnt, 2)
    n[1] = cnt[1]
    got = _run(ops, q, kv, bad, n, declared)
    assert ops.device_status() & _lib.IA_DEV_STATUS_BAD_INDEX
    assert bool(torch.isfinite(got).all())
    # what is left for sequence 0 is block 0 (+ suffix); the oracle agrees
    k, v = logical_kv(case, 0)
    plen = int(case["prefix_lens"][0])
    # the declared geometry also caps the summarised prefix at `declared` blocks
    mask = torch.zeros((CFG.n_kv_heads, nb), dtype=torch.bool)
    mask[:, 0] = True
    qg = case["q"][0].reshape(CFG.n_kv_heads, CFG.group_size, CFG.head_dim).float()
    ref = orc.decode_attention(qg, k, v, plen, CFG.block_size, mask, rep_mode="sparse_only")
    torch.testing.assert_close(got[0].cpu().reshape(ref.shape), ref, rtol=1e-2, atol=2e-2)
    # the untouched sequence is unaffected
    torch.testing.assert_close(got[1], want[1], rtol=1e-2, atol=2e-2)


def test_negative_block_index_is_skipped():
    _lib, ops, case, q, kv, nb, idx, cnt = _setup()
    bad = idx.clone()
    bad[1, 0, 0] = -2        # sequence 1: even unguarded, a negative logical page would land in table row 0
    got = _run(ops, q, kv, bad, cnt, nb)
    assert ops.device_status() & _lib.IA_DEV_STATUS_BAD_INDEX
    assert bool(torch.isfinite(got).all())


def test_table_entry_outside_the_declared_pool_is_skipped():
    _lib, ops, case, q, kv, nb, idx, cnt = _setup()
    want = _run(ops, q, kv, idx, cnt, nb)
    n_pages = int(kv.k_pool.shape[0])
    declared = n_pages - 8                      # pages [declared, n_pages) exist but are "outside the pool"
    some_outside = bool((kv.block_table[:, : nb * 4] >= declared).any())
    assert some_outside, "the permuted table should use the last pages too"
    small = replace(kv, n_pool_pages=declared)
    got = _run(ops, q, small, idx, cnt, nb)
    status = ops.device_status()
    touched = False
    table = kv.block_table.cpu()
    for b in range(CFG.batch):
        for h in range(CFG.n_kv_heads):
            for blk in idx[b, h, : int(cnt[b, h])].cpu().tolist():
                touched |= bool((table[b, blk * 4: blk * 4 + 4] >= declared).any())
        plen, slen = int(case["prefix_lens"][b]), int(case["seq_lens"][b])
        if slen > plen:
            touched |= bool((table[b, plen // 16: (slen - 1) // 16 + 1] >= declared).any())
    assert bool(status & _lib.IA_DEV_STATUS_BAD_INDEX) == touched
    assert bool(torch.isfinite(got).all())
    if not touched:
        torch.testing.assert_close(got, want, rtol=1e-2, atol=2e-2)
    # the one-call step takes the same guards (equal-share grid)
    step = ops.DecodeAttention(small, ops.build_summaries(kv, CFG.block_size, max_blocks=nb), CFG.n_q_heads,
                               top_k=CFG.top_k)
    out = step.step(q).float()
    torch.cuda.synchronize()
    assert bool(ops.device_status() & _lib.IA_DEV_STATUS_BAD_INDEX) == touched   # same selection, same pages
    assert bool(torch.isfinite(out).all())


def test_index_list_out_of_order_is_reported():
    _lib, ops, case, q, kv, nb, idx, cnt = _setup()
    shuffled = idx.clone()
    shuffled[0, 0, :2] = idx[0, 0, :2].flip(0)  # two valid blocks, wrong order
    got = _run(ops, q, kv, shuffled, cnt, nb, block_range=(0, nb), with_suffix=True)
    assert ops.device_status() & _lib.IA_DEV_STATUS_BAD_INDEX
    assert bool(torch.isfinite(got).all())


def test_summaries_skip_a_table_entry_outside_the_declared_pool():
    """The summary kernel fetches whole (page, kv head) runs with bulk copies: a block-table entry past the
    declared pool is reported and its sixteen tokens are left out of the block's summary - never fetched."""
    from interattn_b200 import _lib, ops
    case = make_case(CFG)
    q, kv = to_device(case)
    nb = max_blocks_of(case)
    clean = ops.build_summaries(kv, CFG.block_size, max_blocks=nb)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    # declare one page less than exist: the highest page id of the table is now "outside"
    top = int(kv.block_table.max())
    small = replace(kv, n_pool_pages=top)
    got = ops.build_summaries(small, CFG.block_size, max_blocks=nb)
    torch.cuda.synchronize()
    assert ops.device_status() & _lib.IA_DEV_STATUS_BAD_INDEX
    where = (kv.block_table == top).nonzero()[0]
    seq, blk = int(where[0]), int(where[1]) // (CFG.block_size // 16)
    same = torch.ones(clean.k_bar.shape[:3], dtype=torch.bool, device=clean.k_bar.device)
    same[seq, :, blk] = False
    assert torch.equal(got.k_bar[same], clean.k_bar[same]) and torch.equal(got.k_max[same], clean.k_max[same])
    assert torch.isfinite(got.k_bar.float()).all()
    if blk * CFG.block_size < int(kv.prefix_lens[seq]):  # the block lies in the summarised prefix: 48 tokens are left
        assert not torch.equal(got.k_bar[seq, :, blk], clean.k_bar[seq, :, blk])
