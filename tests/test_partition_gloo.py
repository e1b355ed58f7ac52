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


def test_aligned_block_ranges():
    for n, w in ((2048, 8), (2048, 2), (100, 4), (33, 2), (0, 2), (94, 8), (513, 3)):
        r = partition.plan_block_ranges(n, w, align=32)
        assert len(r) == w and r[0][0] == 0 and r[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(lo % 32 == 0 for lo, hi in r if lo < n)           # every start on a 32-block tile
        assert all(hi % 32 == 0 or hi == n for lo, hi in r)


def _distributed_selection_rank(rank, world, port, result_path):
    """What ia_select_split does, with the oracle's per-block terms and the host-side merges of
    interattn_b200.partition, over two all-gathers: every rank scores only its own block range and
    all ranks end up with the oracle's global top-k."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = scaled(CONFIGS["cfg4_longctx_128k"], batch=1, max_len=6000, suffix=0, top_k=12)
        case = make_case(cfg)
        g = cfg.group_size
        plen = int(case["prefix_lens"][0])
        k = orc.gather_logical(case["k_pool"], case["block_table"][0], plen)
        v = orc.gather_logical(case["v_pool"], case["block_table"][0], plen)
        summ = orc.block_summaries(k, v, cfg.block_size, storage="mixed")
        qg = case["q"][0].reshape(cfg.n_kv_heads, g, cfg.head_dim).float()
        nb = summ.n_blocks
        lo, hi = partition.plan_block_ranges(nb, world, align=32)[rank]
        # this rank's summaries only: the other blocks are NaN and must never matter
        mine = orc.Summaries(summ.k_bar[:, lo:hi], summ.v_bar[:, lo:hi], summ.k_max[:, lo:hi], summ.k_min[:, lo:hi],
                             summ.v_norm_max[:, lo:hi], summ.counts[lo:hi], summ.block_size)
        rows = cfg.n_kv_heads * g
        if hi > lo:
            t = orc.condition_terms(qg, mine)                       # z, delta of the own blocks (its p / score are local: unused)
            z, delta = t["z"].reshape(rows, -1), t["delta"].reshape(rows, -1)
            m = z.amax(dim=1)
            w = torch.exp(z - m[:, None])
            l, d = w.sum(dim=1), (w * torch.cosh(delta)).sum(dim=1)
            b_all = mine.v_norm_max.float().amax(dim=1).repeat_interleave(g)
        else:
            z = delta = torch.zeros((rows, 0))
            m, l, d, b_all = torch.full((rows,), float("-inf")), torch.zeros(rows), torch.zeros(rows), torch.zeros(rows)
        # exchange 1: the row normalisers
        packed = torch.stack([m, l, d, b_all])                     # [4, rows]
        gathered = [torch.empty_like(packed) for _ in range(world)]
        dist.all_gather(gathered, packed)
        allp = torch.stack(gathered)                                # [world, 4, rows]
        M, L, D, B = partition.merge_row_normalisers(allp[:, 0], allp[:, 1], allp[:, 2], allp[:, 3])
        # scores of the own blocks with the global normalisers (the reference's condition score)
        p_soft = torch.exp(z - M[:, None]) / L[:, None]
        denom = (D / L).clamp_min(1e-30)
        b_c = mine.v_norm_max.float().repeat_interleave(g, dim=0) if hi > lo else torch.zeros((rows, 0))
        cond = p_soft * (2.0 * B[:, None] * (torch.cosh(delta) - 1.0) / denom[:, None] + 2.0 * b_c * torch.tanh(delta / 2.0))
        score = cond.reshape(cfg.n_kv_heads, g, -1).mean(dim=1)      # [Hkv, own blocks]
        # exchange 2: the own top-k candidates (score, global block), padded to k
        kk = cfg.top_k
        cand_s = torch.full((cfg.n_kv_heads, kk), float("-inf"))
        cand_b = torch.full((cfg.n_kv_heads, kk), -1, dtype=torch.long)
        for h in range(cfg.n_kv_heads):
            ranked, _ = orc.select_topk(score[h:h + 1], mine.counts, kk)
            chosen = sorted(ranked[0])
            cand_s[h, : len(chosen)] = score[h, chosen]
            cand_b[h, : len(chosen)] = torch.tensor(chosen, dtype=torch.long) + lo
        gs = [torch.empty_like(cand_s) for _ in range(world)]
        gb = [torch.empty_like(cand_b) for _ in range(world)]
        dist.all_gather(gs, cand_s)
        dist.all_gather(gb, cand_b)
        # the oracle's selection from all blocks at once
        terms = orc.condition_terms(qg, summ)
        want, _ = orc.select_topk(terms["score"], summ.counts, kk)
        ok = True
        for h in range(cfg.n_kv_heads):
            sc = [x[h][y[h] >= 0] for x, y in zip(gs, gb)]
            bl = [y[h][y[h] >= 0] for y in gb]
            got = partition.merge_topk_candidates(sc, bl, kk).tolist()
            ok = ok and got == sorted(want[h])
        with open(f"{result_path}.{rank}", "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_distributed_selection_protocol_gloo_ranks(tmp_path, world):
    port = _free_port()
    result = str(tmp_path / "result")
    mp.spawn(_distributed_selection_rank, args=(world, port, result), nprocs=world, join=True)
    for r in range(world):
        assert open(f"{result}.{r}").read() == "ok"


def test_candidate_merge_breaks_ties_towards_the_lower_block():
    got = partition.merge_topk_candidates([torch.tensor([3.0, 1.0]), torch.tensor([3.0, 3.0])],
                                          [torch.tensor([2, 5]), torch.tensor([40, 41])], 2)
    assert got.tolist() == [2, 40]
    M, L, D, B = partition.merge_row_normalisers(
        torch.tensor([[0.0], [float("-inf")]]), torch.tensor([[2.0], [0.0]]), torch.tensor([[3.0], [0.0]]),
        torch.tensor([[1.5], [0.0]]))
    assert (float(M), float(L), float(D), float(B)) == (0.0, 2.0, 3.0, 1.5)      # a rank without blocks adds nothing


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
