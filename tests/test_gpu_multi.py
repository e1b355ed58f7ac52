"""Split-KV across real GPUs (one process per GPU, NCCL): every rank holds only
the K/V pages of its own block range, selects globally from replicated
summaries, attends over its share and all-gathers (o, lse); the merged output
must equal the single-GPU layer-step.  The multi-rank tests are skipped on boxes with
one GPU; the same code runs there as a process group of one rank."""

import os
import socket
from datetime import timedelta

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, rep_mode, result_path):
    import torch.distributed as dist
    from interattn_b200 import ops, partition
    from oracle.configs import CONFIGS, make_case, scaled
    # no NVSwitch multicast anywhere in this test: ranks may leave on an error path
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # a short collective timeout: a rank that failed must not leave the others waiting for the job's limit
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(seconds=90))
    try:
        cfg = scaled(CONFIGS["cfg4_longctx_128k"], batch=2, max_len=6000, suffix=11, top_k=12)
        case = make_case(cfg)
        nb = max((n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens)
        q = case["q"].to(dev)
        table = case["block_table"].clamp_min(0).to(dev).contiguous()
        full = ops.PagedKV(case["k_pool"].to(dev), case["v_pool"].to(dev), table,
                           case["prefix_lens"].to(dev), case["seq_lens"].to(dev))
        summ = ops.build_summaries(full, cfg.block_size, max_blocks=nb)        # replicated summaries
        whole = ops.DecodeAttention(full, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode,
                                    n_splits=2).step(q).clone()

        # this rank's pool: NaN everywhere except the pages of its own block range (+ suffix on the last rank)
        lo, hi = partition.plan_block_ranges(nb, world)[rank]
        ppb = cfg.block_size // cfg.page_size
        keep = torch.zeros(case["k_pool"].shape[0], dtype=torch.bool)
        for b in range(cfg.batch):
            n_prefix_pages = (cfg.prefix_lens[b] + cfg.page_size - 1) // cfg.page_size
            mine = [p for p in range(lo * ppb, min(hi * ppb, n_prefix_pages))]
            if rank == world - 1:
                first_suffix = cfg.prefix_lens[b] // cfg.page_size
                last = (cfg.prefix_lens[b] + cfg.suffix_lens[b] - 1) // cfg.page_size
                mine += list(range(first_suffix, last + 1))
            keep[case["block_table"][b, mine].long()] = True
        k_mine = torch.where(keep[:, None, None, None], case["k_pool"].float(), torch.tensor(float("nan"))).to(q.dtype)
        v_mine = torch.where(keep[:, None, None, None], case["v_pool"].float(), torch.tensor(float("nan"))).to(q.dtype)
        local = ops.PagedKV(k_mine.to(dev), v_mine.to(dev), table, full.prefix_lens, full.seq_lens)

        step = partition.cuda_split_kv_step(q, local, summ, top_k=cfg.top_k, rep_mode=rep_mode, n_splits=2)
        out = step.run(nb)
        torch.cuda.synchronize()
        ok = bool(torch.isfinite(out.float()).all())
        ok = ok and torch.allclose(out.float(), whole.float(), rtol=1e-2, atol=3e-3)
        # the preallocated form of the same step: eager, then captured with its all-gather and replayed
        fast = partition.SplitKVDecodeAttention(local, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode,
                                                n_splits=3)
        eager = fast.step(q).clone()
        torch.cuda.synchronize()
        ok = ok and torch.allclose(eager.float(), whole.float(), rtol=1e-2, atol=3e-3)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fast.step(q)                                  # warm-up on the capture stream
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        # thread_local: the process group's watchdog thread polls events while this thread captures
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            fast.step(q)
        fast.out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        ok = ok and torch.equal(fast.out, eager)
        # The same step with every exchange inside the kernels (peer stores + flags, no collective call),
        # selection included: this rank's summaries are NaN outside its own (32-aligned) block range, so
        # the global selection can only come out right through the normaliser and candidate exchange.
        s_lo, s_hi = partition.plan_block_ranges(nb, world, align=32)[rank]

        def own_range_only(t):
            keep_blocks = torch.zeros(nb, dtype=torch.bool, device=dev)
            keep_blocks[s_lo:s_hi] = True
            shape = (1, 1, nb) + (1,) * (t.dim() - 3)
            return torch.where(keep_blocks.view(shape), t.float(), torch.tensor(float("nan"), device=dev)).to(t.dtype)

        summ_mine = ops.BlockSummaries(own_range_only(summ.k_bar), own_range_only(summ.k_max),
                                       own_range_only(summ.k_min), own_range_only(summ.v_bar),
                                       own_range_only(summ.v_norm_max), summ.block_size)
        # this rank's pool for the aligned ranges (they differ from the unaligned ones above)
        keep2 = torch.zeros(case["k_pool"].shape[0], dtype=torch.bool)
        for b in range(cfg.batch):
            n_prefix_pages = (cfg.prefix_lens[b] + cfg.page_size - 1) // cfg.page_size
            mine = [pg for pg in range(s_lo * ppb, min(s_hi * ppb, n_prefix_pages))]
            if rank == world - 1:
                mine += list(range(cfg.prefix_lens[b] // cfg.page_size,
                                   (cfg.prefix_lens[b] + cfg.suffix_lens[b] - 1) // cfg.page_size + 1))
            keep2[case["block_table"][b, mine].long()] = True
        nan = torch.tensor(float("nan"))
        local2 = ops.PagedKV(torch.where(keep2[:, None, None, None], case["k_pool"].float(), nan).to(q.dtype).to(dev),
                             torch.where(keep2[:, None, None, None], case["v_pool"].float(), nan).to(q.dtype).to(dev),
                             table, full.prefix_lens, full.seq_lens)
        p2p = partition.SplitKVDecodeAttentionP2P(local2, summ_mine, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode,
                                                  n_splits=3, selection="distributed")
        direct = p2p.step(q).clone()
        torch.cuda.synchronize()
        want_idx, want_cnt, _ = ops.select_blocks(q, summ, full.prefix_lens, top_k=cfg.top_k)
        ok_p2p = torch.equal(p2p.sel_idx, want_idx) and torch.equal(p2p.sel_count, want_cnt)   # the global selection
        ok_p2p = ok_p2p and torch.allclose(direct.float(), whole.float(), rtol=1e-2, atol=3e-3)
        # and with replicated summaries, every rank selecting on its own
        rep = partition.SplitKVDecodeAttentionP2P(local2, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode,
                                                  n_splits=2, selection="replicated")
        ok_p2p = ok_p2p and torch.allclose(rep.step(q).float(), whole.float(), rtol=1e-2, atol=3e-3)
        torch.cuda.synchronize()
        for _ in range(3):                                # consecutive steps alternate the two buffer parities
            again = p2p.step(q)
        torch.cuda.synchronize()
        ok_p2p = ok_p2p and torch.equal(again, direct)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            p2p.step(q)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2, capture_error_mode="thread_local"):
            p2p.step(q)
        for _ in range(2):
            p2p.out.zero_()
            graph2.replay()
        torch.cuda.synchronize()
        ok_p2p = ok_p2p and torch.equal(p2p.out, direct) and ops.device_status() == 0
        with open(f"{result_path}.{rank}", "w") as f:
            f.write("ok" if ok and ok_p2p else f"mismatch {float((out.float() - whole.float()).abs().max())} "
                                               f"{float((eager.float() - whole.float()).abs().max())} "
                                               f"p2p {ok_p2p} {float((direct.float() - whole.float()).abs().max())}")
        # graphs first, then the peer mappings, a drained device, the other ranks, the communicator
        partition.ordered_shutdown(graphs=[graph, graph2], steps=[p2p, rep])
        with open(f"{result_path}.{rank}.shutdown", "w") as f:
            f.write("clean")
    except Exception as e:   # report and leave at once; the peers' bounded waits let them return too
        with open(f"{result_path}.{rank}", "w") as f:
            f.write(f"error {type(e).__name__}: {e}"[:500])
        torch.cuda.synchronize()
        os._exit(0)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("rep_mode", ["sparse_only", "hybrid"])
def test_split_kv_over_nccl(tmp_path, rep_mode):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    result = str(tmp_path / "result")
    mp.spawn(_rank_main, args=(world, _free_port(), rep_mode, result), nprocs=world, join=True)
    for r in range(world):
        assert open(f"{result}.{r}").read() == "ok"
        assert os.path.exists(f"{result}.{r}.shutdown"), "the ordered teardown did not return"


@pytest.mark.timeout(300)
@pytest.mark.parametrize("rep_mode", ["sparse_only", "hybrid"])
def test_split_kv_step_as_a_group_of_one(tmp_path, rep_mode):
    """One rank owns every block: the preallocated split-KV step (selection, ranged attention,
    all-gather, gathered merge; eager and captured) must reproduce the one-call layer-step."""
    import torch.multiprocessing as mp
    result = str(tmp_path / "result")
    mp.spawn(_rank_main, args=(1, _free_port(), rep_mode, result), nprocs=1, join=True)
    assert open(f"{result}.0").read() == "ok"
    assert os.path.exists(f"{result}.0.shutdown"), "the ordered teardown did not return"
