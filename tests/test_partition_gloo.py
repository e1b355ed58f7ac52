"""The multi-GPU partitioner on the CPU: plans, and the split-KV exchange step
run as two gloo ranks with the oracle standing in for the CUDA operators."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from interattn_b200 import partition
from oracle import condition_block_oracle as orc
from oracle.configs import CONFIGS, make_case, scaled


def test_block_ranges_cover_everything_once():
    for n, w in ((2048, 8), (2048, 4), (7, 4), (3, 8), (0, 2), (513, 2)):
        r = partition.plan_block_ranges(n, w)
        assert len(r) == w and r[0][0] == 0 and r[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        sizes = [hi - lo for lo, hi in r]
        assert max(sizes) - min(sizes) <= 1


def test_head_shards_match_the_variable_length_configuration():
    assert partition.plan_head_shards(8, 8) == [(i, i + 1) for i in range(8)]
    assert partition.plan_head_shards(8, 4) == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert partition.plan_head_shards(8, 2) == [(0, 4), (4, 8)]
    with pytest.raises(ValueError):
        partition.plan_head_shards(8, 3)


def test_unit_shards_balance_ragged_batches():
    cfg = CONFIGS["cfg5_llama70b_ragged"]
    costs = partition.unit_costs(cfg.prefix_lens, cfg.n_kv_heads, cfg.block_size, cfg.top_k)
    assert len(costs) == cfg.batch * cfg.n_kv_heads
    for world in (2, 4, 8):
        owned = partition.plan_unit_shards(costs, world)
        assert sorted(u for part in owned for u in part) == list(range(len(costs)))     # a partition
        loads = [sum(costs[u] for u in part) for part in owned]
        assert max(loads) - min(loads) <= max(costs)                                      # LPT bound
        assert partition.plan_unit_shards(costs, world) == owned                         # deterministic
    # short sequences (fewer blocks than k) cost less than long ones
    assert min(costs) < max(costs) == cfg.top_k * cfg.block_size


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _split_kv_rank(rank, world, port, rep_mode, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = scaled(CONFIGS["cfg4_longctx_128k"], batch=1, max_len=1500, suffix=9, top_k=6)
        case = make_case(cfg)                     # same seed on every rank: replicated inputs
        g = cfg.group_size
        plen, slen = int(case["prefix_lens"][0]), int(case["seq_lens"][0])
        k = orc.gather_logical(case["k_pool"], case["block_table"][0], slen)
        v = orc.gather_logical(case["v_pool"], case["block_table"][0], slen)
        summ = orc.block_summaries(k[:, :plen], v[:, :plen], cfg.block_size, storage="mixed")
        qg = case["q"][0].reshape(cfg.n_kv_heads, g, cfg.head_dim).float()
        rows = cfg.n_q_heads

        def select():
            terms = orc.condition_terms(qg, summ)
            _, mask = orc.select_topk(terms["score"], summ.counts, cfg.top_k)
            return mask, terms["z"]

        def attend(selection, block_range, with_suffix):
            mask, z = selection
            # a rank only ever touches the K/V of its own block range (and the suffix on the last rank)
            lo, hi = block_range
            k_mine, v_mine = torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))
            k_mine[:, lo * cfg.block_size: min(hi * cfg.block_size, plen)] = k[:, lo * cfg.block_size: min(hi * cfg.block_size, plen)]
            v_mine[:, lo * cfg.block_size: min(hi * cfg.block_size, plen)] = v[:, lo * cfg.block_size: min(hi * cfg.block_size, plen)]
            if with_suffix:
                k_mine[:, plen:], v_mine[:, plen:] = k[:, plen:], v[:, plen:]
            o, lse = orc.decode_attention(qg, k_mine, v_mine, plen, cfg.block_size, mask, rep_mode=rep_mode, z=z,
                                          v_bar=summ.v_bar, block_range=block_range, with_suffix=with_suffix,
                                          return_lse=True)
            return o.reshape(rows, -1), lse.reshape(rows)

        def merge(all_o, all_lse):
            return orc.merge_o_lse(all_o, all_lse)[0]

        step = partition.SplitKVStep(select, attend, merge)
        out = step.run(summ.n_blocks)
        mask, z = select()
        whole = orc.decode_attention(qg, k, v, plen, cfg.block_size, mask, rep_mode=rep_mode, z=z, v_bar=summ.v_bar)
        ok = torch.allclose(out, whole.reshape(rows, -1), rtol=1e-5, atol=1e-6) and bool(torch.isfinite(out).all())
        # every rank ends with the same merged output
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        ok = ok and all(torch.equal(gathered[0], x) for x in gathered)
        with open(f"{result_path}.{rank}", "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rep_mode", ["sparse_only", "hybrid"])
@pytest.mark.parametrize("world", [2, 3])
def test_split_kv_exchange_two_gloo_ranks(tmp_path, rep_mode, world):
    port = _free_port()
    result = str(tmp_path / "result")
    mp.spawn(_split_kv_rank, args=(world, port, rep_mode, result), nprocs=world, join=True)
    for r in range(world):
        assert open(f"{result}.{r}").read() == "ok"


def test_allgather_partials_layout_single_rank(tmp_path):
    port = _free_port()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        o, lse = torch.randn(6, 8), torch.randn(6)
        go, gl = partition.allgather_partials(o, lse)
        assert go.shape == (6, 1, 8) and gl.shape == (6, 1)
        assert torch.equal(go[:, 0], o) and torch.equal(gl[:, 0], lse)
        with pytest.raises(ValueError):
            partition.allgather_partials(o.double(), lse)
    finally:
        dist.destroy_process_group()
