"""The allocation-free layer-step (ia_decode_attention_noalloc).

Some hosts of the library cannot allocate device memory once they run - a
server that gave all of HBM to its KV pool, a hot loop that must not touch an
allocator - so this entry point keeps its scratch in a fixed array inside the
shared library.  The test drives it through the C ABI and compares it with the
workspace-based entry point (ia_decode_attention) on the same inputs, twice in
a row with different inputs and modes, because the shared array keeps whatever
the previous call left in it - and, so that the test stands on its own, with
the CPU oracle on the same inputs.  It also checks that an over-sized step is
refused instead of overrunning the array.

Collected last (file name) so that a run stopping at the first failure has
already exercised everything else; it needs nothing from the other tests.
"""

import ctypes

import pytest
import torch

from oracle import condition_block_oracle as orc
from oracle.configs import CONFIGS, DecodeConfig, make_case, scaled

pytestmark = pytest.mark.gpu

TOL = {"float32": dict(rtol=1e-5, atol=1e-5), "bfloat16": dict(rtol=1e-2, atol=2e-2)}


def _setup(cfg, device="cuda:0"):
    from interattn_b200 import ops
    case = make_case(cfg, spare_pages=2)
    kv = ops.PagedKV(case["k_pool"].to(device), case["v_pool"].to(device),
                     case["block_table"].clamp_min(0).to(device).contiguous(),
                     case["prefix_lens"].to(device), case["seq_lens"].to(device))
    q = case["q"].to(device).contiguous()
    nb = max(1, (int(case["prefix_lens"].max()) + cfg.block_size - 1) // cfg.block_size)
    summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb)
    return ops, q, kv, summ, case


def _oracle_step(cfg, case, summ, q, rep_mode):
    """The layer-step on the CPU: score -> top-k -> attention from the stored summaries (the
    selection is defined on those), [B, Hq, D] fp32."""
    from tests.gpu_util import logical_kv, oracle_summaries_from_gpu
    g = cfg.group_size
    outs = []
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        osum = oracle_summaries_from_gpu(summ, b, plen)
        qg = q[b].cpu().reshape(cfg.n_kv_heads, g, cfg.head_dim).float()
        terms = orc.condition_terms(qg, osum)
        _, mask = orc.select_topk(terms["score"], osum.counts, cfg.top_k)
        k, v = logical_kv(case, b)
        out = orc.decode_attention(qg, k, v, plen, cfg.block_size, mask, rep_mode=rep_mode, z=terms["z"],
                                   v_bar=osum.v_bar)
        outs.append(out.reshape(cfg.n_q_heads, cfg.head_dim))
    return torch.stack(outs)


def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row():
    calls = [
        (scaled(CONFIGS["cfg2_llama8b_32k"], batch=3, max_len=2304, suffix=9), "hybrid", 3),
        (scaled(CONFIGS["cfg5_llama70b_ragged"], batch=4, max_len=1500, suffix=0), "sparse_only", 2),
        (CONFIGS["cfg1_cpu_fp32"], "hybrid", 1),
    ]
    for cfg, rep_mode, n_splits in calls:          # back to back: the array still holds the previous step
        ops, q, kv, summ, case = _setup(cfg)
        want = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode,
                                   n_splits=n_splits).step(q).clone()
        out = torch.full_like(q, float("nan"))
        before = torch.cuda.memory_allocated()
        got = ops.decode_attention_noalloc(q, kv, summ, out, top_k=cfg.top_k, rep_mode=rep_mode, n_splits=n_splits)
        assert torch.cuda.memory_allocated() == before      # the wrapper did not touch torch's allocator either
        torch.cuda.synchronize()
        assert got.data_ptr() == out.data_ptr()
        torch.testing.assert_close(got.float(), want.float(), **TOL[cfg.dtype])
        # same kernels, same split: in fact the same bits
        assert torch.equal(got, want)
        # and the CPU oracle agrees, so this test does not lean on the other entry point being right
        torch.testing.assert_close(got.float().cpu(), _oracle_step(cfg, case, summ, q, rep_mode), **TOL[cfg.dtype])
        # and once more with a different query on the same cache
        q2 = torch.roll(q, 1, dims=1).contiguous()
        want2 = ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode,
                                    n_splits=n_splits).step(q2).clone()
        got2 = ops.decode_attention_noalloc(q2, kv, summ, out, top_k=cfg.top_k, rep_mode=rep_mode,
                                            n_splits=n_splits)
        torch.cuda.synchronize()
        torch.testing.assert_close(got2.float(), want2.float(), **TOL[cfg.dtype])
        torch.testing.assert_close(got2.float().cpu(), _oracle_step(cfg, case, summ, q2, rep_mode), **TOL[cfg.dtype])
    assert ops.device_status() == 0


def test_noalloc_refuses_a_step_larger_than_its_array():
    from interattn_b200 import _lib
    cfg = DecodeConfig("big", "bfloat16", 2, 8, 2, 128, 16, 64, 2, (256, 256), (0, 0), seed=2)
    ops, q, kv, summ, _ = _setup(cfg)
    lib = _lib.load()
    limit = lib.ia_noalloc_scratch_bytes()
    assert limit == 8 * 1024 * 1024
    g = kv.geom(cfg.group_size, cfg.block_size, summ.max_blocks)
    # pretend the batch is huge: only the size check may look at it
    g.batch = 1 << 16
    need = lib.ia_workspace_bytes(ctypes.byref(g), 2, 4, _lib.IA_REP_SPARSE_ONLY)
    assert need > limit
    s = summ.c_struct()
    out = torch.empty_like(q)
    status = lib.ia_decode_attention_noalloc(
        q.data_ptr(), kv.k_pool.data_ptr(), kv.v_pool.data_ptr(), kv.block_table.data_ptr(),
        kv.prefix_lens.data_ptr(), kv.seq_lens.data_ptr(), ctypes.byref(s), ctypes.byref(g),
        _lib.IA_SELECT_TOPK, 2, 0.0, 2, _lib.IA_REP_SPARSE_ONLY, 4, out.data_ptr(), None)
    assert status == _lib.IA_ERR_UNSUPPORTED
    msg = lib.ia_last_error_string().decode()
    assert "scratch" in msg and str(limit) in msg
    with pytest.raises(ValueError):
        _lib.check(status)
