"""Benchmark of the condition-block sparse decode-attention layer-step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (N = 1): the Llama-3-8B attention geometry - bf16, 32 query / 8 kv
heads, head_dim 128, batch 16, context 32768 per sequence, 16-token pages
behind a randomly permuted block table, selection block 64, top-k 64 - one
decode step of one attention layer: block scoring + top-k routing, paged
sparse attention over the selected pages, split-KV finalize.  Synthetic
N(0,1) tensors (K channels scaled by a log-normal factor) stand in for real
prompts.  A "step" is one such layer-step over the batch.  With N GPUs every
rank owns its own 16 sequences (batch x kv-head sharding: the units share
nothing, so there is no collective on the data path) - weak scaling.

One JSON line on rank 0:
  value      decode tokens advanced through one attention layer per second,
             whole job, inputs resident in HBM (one C-ABI call per step)
  e2e        the same through the host-buffer entry point: pinned q -> device,
             the step, output -> pinned host, every step
  roofline   the paged sparse-attention kernel: K/V bytes of the selected
             tokens / its CUDA-event duration, against the measured HBM peak
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch path) timed
             on this box's host cores on a bounded sample
`--impl reference` times that CPU path alone, with every host thread.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "sparse_decode_attn_layer_tokens_per_s"
UNIT = "tok*layer/s"
WORKLOAD = "cfg2_llama8b_32k"
N_LAYER_POOLS = 4       # default number of KV pools rotated between steps (4 x 320 MiB touched > 126 MB of L2)
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--n-splits", type=int, default=0, help="split-KV parts per (sequence, kv head); 0 = auto")
    ap.add_argument("--rep-mode", default="sparse_only", choices=["sparse_only", "hybrid"])
    ap.add_argument("--workload", default=WORKLOAD)
    ap.add_argument("--cpu-sample-seqs", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="split-KV arm: launch the step eagerly")
    ap.add_argument("--kbar-bf16", action="store_true",
                    help="store the block key means in bf16 (the reference's approximate option) instead of fp32")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="split-KV arm: partials stored into the peers' buffers by the attention kernel (p2p) "
                         "or an NCCL all-gather after it (nccl)")
    ap.add_argument("--llama-steps", type=int, default=48,
                    help="greedy decode steps of the full Llama-3-8B-architecture model (batch 32, 8192-token "
                         "prompts, random weights) timed after the layer-step, 1 GPU only; 0 skips it")
    ap.add_argument("--layer-pools", type=int, default=N_LAYER_POOLS,
                    help="KV pools rotated between steps (1 keeps a profiler capture small)")
    return ap.parse_args()


# ----------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's PyTorch path
# ----------------------------------------------------------------------------

def cpu_prepare(cfg, n_seqs, seed_offset=0):
    """Inputs of ``n_seqs`` sequences of the workload on the host, with their
    block summaries (built once per prompt, hence outside the timed part)."""
    from dataclasses import replace
    from oracle import condition_block_oracle as orc
    from oracle.configs import make_case

    small = replace(cfg, batch=n_seqs, prefix_lens=cfg.prefix_lens[:n_seqs], suffix_lens=cfg.suffix_lens[:n_seqs],
                    seed=cfg.seed + seed_offset)
    case = make_case(small)
    hkv, g = small.n_kv_heads, small.group_size
    prepared = []
    for b in range(n_seqs):
        plen, slen = int(case["prefix_lens"][b]), int(case["seq_lens"][b])
        k = orc.gather_logical(case["k_pool"], case["block_table"][b], slen)
        v = orc.gather_logical(case["v_pool"], case["block_table"][b], slen)
        summ = orc.block_summaries(k[:, :plen], v[:, :plen], small.block_size, storage="mixed")
        prepared.append((plen, k, v, summ, case["q"][b].reshape(hkv, g, -1)))
    return small, prepared


def cpu_layer_step(small, prepared):
    """One layer-step on the host: score + top-k + sparse attention per sequence.  Returns seconds."""
    from oracle import condition_block_oracle as orc
    t0 = time.perf_counter()
    for plen, k, v, summ, qg in prepared:
        terms = orc.condition_terms(qg, summ)
        _, mask = orc.select_topk(terms["score"], summ.counts, small.top_k)
        orc.decode_attention(qg, k, v, plen, small.block_size, mask, rep_mode="sparse_only")
    return time.perf_counter() - t0


def run_reference_arm(args):
    """The reference's CPU implementation of the path (oracle port), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle.configs import CONFIGS
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = CONFIGS[args.workload]
    n = 1 if args.steps > 20 else max(1, min(args.cpu_sample_seqs, 4))
    small, prepared = cpu_prepare(cfg, n)
    for _ in range(args.warmup):
        cpu_layer_step(small, prepared)
    total = 0.0
    for _ in range(args.steps):
        total += cpu_layer_step(small, prepared)
    value = n * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": f"{n} of {cfg.batch} sequences per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{n} sequence(s) x {args.steps} steps: score + top-k + sparse attention, "
                                   "summaries excluded"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

def make_device_layer(cfg, device, seed):
    """One layer's paged KV cache for the whole batch, generated on the device:
    N(0,1) K/V (K channels scaled by a log-normal factor), a random permutation
    as the block table."""
    import torch
    from interattn_b200 import ops
    g = torch.Generator(device=device).manual_seed(seed)
    P, D, hkv = cfg.page_size, cfg.head_dim, cfg.n_kv_heads
    pages_per_seq = [(n + s + P - 1) // P for n, s in zip(cfg.prefix_lens, cfg.suffix_lens)]
    n_pages, max_pages = sum(pages_per_seq), max(pages_per_seq)
    dt = cfg.torch_dtype
    k_pool = torch.randn((n_pages, hkv, P, D), generator=g, device=device, dtype=torch.float32)
    if cfg.k_channel_sigma > 0:
        k_pool *= torch.exp(cfg.k_channel_sigma * torch.randn((D,), generator=g, device=device))
    k_pool = k_pool.to(dt)
    v_pool = torch.randn((n_pages, hkv, P, D), generator=g, device=device, dtype=torch.float32).to(dt)
    perm = torch.randperm(n_pages, generator=g, device=device).to(torch.int32)
    table = torch.zeros((cfg.batch, max_pages), dtype=torch.int32, device=device)
    at = 0
    for b, n in enumerate(pages_per_seq):
        table[b, :n] = perm[at: at + n]
        at += n
    prefix = torch.tensor(cfg.prefix_lens, dtype=torch.int32, device=device)
    seq = torch.tensor([p + s for p, s in zip(cfg.prefix_lens, cfg.suffix_lens)], dtype=torch.int32, device=device)
    return ops.PagedKV(k_pool, v_pool, table, prefix, seq)


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from interattn_b200 import ops
    from oracle.configs import CONFIGS

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    cfg = CONFIGS[args.workload]
    # The variable-length Llama-3-70B configuration shards by kv head (one head per GPU on 8,
    # two on 4, four on 2): every rank holds all sequences but only its heads - strong scaling,
    # still no collective, the output rows of different heads are disjoint.
    head_shard = args.workload == "cfg5_llama70b_ragged" and world > 1
    if head_shard:
        from dataclasses import replace
        from interattn_b200.partition import plan_head_shards
        lo, hi = plan_head_shards(cfg.n_kv_heads, world)[rank]
        cfg = replace(cfg, n_kv_heads=hi - lo, n_q_heads=(hi - lo) * cfg.group_size)
    replicas = 1 if head_shard else world
    props = torch.cuda.get_device_properties(device)
    n_splits = args.n_splits or None      # None: the library picks a wave-aware split count
    nb = max((n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens)
    rows = cfg.n_q_heads

    layers, steppers, qs = [], [], []
    n_pools = max(1, args.layer_pools)
    for l in range(n_pools):
        kv = make_device_layer(cfg, device, seed=1000 * rank + l)
        summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb,
                                   k_bar_dtype=torch.bfloat16 if args.kbar_bf16 else torch.float32)
        layers.append((kv, summ))
        steppers.append(ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=args.rep_mode,
                                            n_splits=n_splits))
        g = torch.Generator(device=device).manual_seed(77 + 1000 * rank + l)
        qs.append(torch.randn((cfg.batch, rows, cfg.head_dim), generator=g, device=device).to(cfg.torch_dtype))
    n_splits = steppers[0].n_splits
    torch.cuda.synchronize()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident arm: K steps, per-kernel events inside the same region -------------
    K, W = args.steps, args.warmup
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K)]
    for row in ev:
        for e in row:
            e.record()
    sampler = ClockSampler(local_rank)   # samples from the warm-up to the end of the second timed region
    sampler.start()
    for i in range(W):
        steppers[i % n_pools].step(qs[i % n_pools])
    sync_all()
    # headline region: K steps through the plain one-call entry point
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(K):
        steppers[i % n_pools].step(qs[i % n_pools])
    t_end.record()
    sync_all()
    elapsed_ms = t_begin.elapsed_time(t_end)
    # the same K steps again with events between the kernels: per-kernel device times for the roofline
    for i in range(K):
        steppers[i % n_pools].step_timed(qs[i % n_pools], ev[i])
    sync_all()
    sel_ms = sum(r[0].elapsed_time(r[1]) for r in ev) / K
    att_ms = sum(r[1].elapsed_time(r[2]) for r in ev) / K
    fin_ms = sum(r[2].elapsed_time(r[3]) for r in ev) / K
    status = ops.device_status()

    # ---- end-to-end arm: host q in, host output back, every step ---------------------------------
    q_host = [q.cpu().pin_memory() for q in qs]
    out_host = [torch.empty_like(q).pin_memory() for q in q_host]
    for i in range(min(W, 5)):
        steppers[i % n_pools].step_host(q_host[i % n_pools], out_host[i % n_pools])
    sync_all()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_begin.record()
    for i in range(K):
        steppers[i % n_pools].step_host(q_host[i % n_pools], out_host[i % n_pools])
    e_end.record()
    sync_all()
    clocks = sampler.stop()
    e2e_ms = e_begin.elapsed_time(e_end)

    times = torch.tensor([elapsed_ms, e2e_ms, att_ms, sel_ms, fin_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, att_ms, sel_ms, fin_ms = [float(x) for x in times.cpu()]

    if rank == 0:
        esz = 2 if cfg.dtype == "bfloat16" else 4
        tokens_sel = sum(min(cfg.top_k * cfg.block_size, n) for n in cfg.prefix_lens) * cfg.n_kv_heads
        suffix_tok = sum(cfg.suffix_lens) * cfg.n_kv_heads
        kv_bytes = (tokens_sel + suffix_tok) * cfg.head_dim * 2 * esz
        sel_bytes = sum((n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens) * cfg.n_kv_heads * (
            cfg.head_dim * (2 if args.kbar_bf16 else 4) + 2 * cfg.head_dim * esz + 4)
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak, peak_src = float(json.load(f)["hbm_gbs"]), "measured"
        except (OSError, KeyError, ValueError):
            pass
        traffic = None   # DRAM bytes per launch of the attention kernel, from the committed ncu summary
        try:
            with open(os.path.join(ROOT, "profiles", "dram_traffic.txt")) as f:
                for ln in f:
                    parts = ln.split()
                    if len(parts) == 3 and parts[0] == args.workload and parts[1] == "sparse_decode":
                        traffic = int(parts[2])
        except (OSError, ValueError):
            pass
        att_gbs = kv_bytes / (att_ms * 1e-3) / 1e9
        sel_gbs = sel_bytes / (sel_ms * 1e-3) / 1e9
        q_bytes = cfg.batch * rows * cfg.head_dim * esz
        line = {
            "metric": METRIC, "value": replicas * cfg.batch * K / (elapsed_ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": elapsed_ms / K,
            "higher_is_better": True, "scaling": "strong" if head_shard else "weak", "vs_baseline": None,
            "dtype": "bf16" if cfg.dtype == "bfloat16" else "f32", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": cfg.batch, "n_q_heads": cfg.n_q_heads,
                       "n_kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim, "context": max(cfg.prefix_lens),
                       "page": cfg.page_size, "block": cfg.block_size, "top_k": cfg.top_k,
                       "rep_mode": args.rep_mode, "n_splits": n_splits, "k_bar": "bf16" if args.kbar_bf16 else "f32", "parallelism": (f"kv-head shard x{world}" if head_shard else f"batch-shard x{world}"),
                       "l2": f"{n_pools} layer pools rotated, {(kv_bytes + sel_bytes) >> 20} MiB read per step "
                             "(> 126 MB L2), no flush"},
            "us_per_layer": 1e3 * elapsed_ms / K,
            "kernel_us": {"select": 1e3 * sel_ms, "sparse_decode": 1e3 * att_ms, "finalize": 1e3 * fin_ms},
            "roofline": {"bound": "hbm", "kernel": "condition_block_finalize_attention_kernel",
                         "achieved": att_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": att_gbs / peak, "traffic": traffic, "bytes_per_launch": kv_bytes},
            "roofline_select": {"bound": "hbm", "kernel": "condition_block_select_kernel", "achieved": sel_gbs,
                                "peak": peak, "unit": "GB/s", "frac": sel_gbs / peak,
                                "bytes_per_launch": sel_bytes},
            "e2e": {"value": replicas * cfg.batch * K / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": q_bytes, "d2h_bytes_per_step": q_bytes,
                    "us_per_layer": 1e3 * e2e_ms / K,
                    "note": "KV pool and block summaries are cache state resident on the device; the step's "
                            "inputs (q) and outputs cross PCIe every step"},
            "gpu_launches": 2 * K,   # selection + attention (finalize fused) per step, headline region
            "clocks": clocks,
            "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            n = max(1, args.cpu_sample_seqs)
            small, prepared = cpu_prepare(cfg, n)
            cpu_layer_step(small, prepared)  # warm-up
            reps = 5
            dt = sum(cpu_layer_step(small, prepared) for _ in range(reps)) / reps
            line["cpu_baseline"] = {
                "value": n / dt, "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"{n} of {cfg.batch} sequences, one layer-step x {reps}: score + top-k + sparse "
                          f"attention ({dt:.2f} s per step), summaries excluded"}
        if args.llama_steps > 1 and world == 1 and args.workload == WORKLOAD:
            line["llama_decode"] = llama_decode_line(args.llama_steps)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def llama_decode_line(steps):
    """Second figure of the metric: decode tokens/s of the whole Llama-3-8B-architecture model
    (32 layers, random bf16 weights, batch 32, 8192 uniform-random prompt ids, block 64, top-64
    in every layer) through the fused decode step captured in a CUDA graph."""
    import torch
    try:
        from interattn_b200 import llama_decode as ld
        torch.cuda.empty_cache()
        model = ld.build_random_llama("llama3-8b")
        g = torch.Generator(device="cuda").manual_seed(0)
        ids = torch.randint(0, model.config.vocab_size, (32, 8192), generator=g, device="cuda")
        _, st = ld.generate_batched(model, ids, int(steps), cuda_graph=True, fused_step=True)
        return {"metric": "llama3_8b_decode_tokens_per_s", "value": st["tokens_per_s"], "unit": "tok/s",
                "ms_per_decode_step": 1e3 * st["decode_s"] / max(st["decode_steps_timed"], 1),
                "decode_steps_timed": st["decode_steps_timed"], "prefill_s": st["prefill_s"],
                "config": {"layers": 32, "batch": 32, "prompt": 8192, "block": 64, "top_k": 64, "dtype": "bf16",
                           "cuda_graph": True, "fused_step": True, "weights": "random init",
                           "data": "uniform random token ids"}}
    except Exception as e:   # the layer-step line above must still be printed
        return {"metric": "llama3_8b_decode_tokens_per_s", "error": f"{type(e).__name__}: {e}"[:300]}


def run_split_kv_arm(args):
    """Long-context split-KV (strong scaling): the blocks of every sequence are cut
    into contiguous ranges, one per rank; every rank selects globally from the
    replicated summaries, attends over its range and the ranks all-gather (o, lse)
    over NCCL before the merge.  A step is the whole exchange: four launches with
    preallocated buffers, captured per layer pool into a CUDA graph (the all-gather
    included) unless --no-graph is given or the capture fails."""
    import torch
    import torch.distributed as dist
    from interattn_b200 import ops, partition
    from oracle.configs import CONFIGS

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    from datetime import timedelta
    dist.init_process_group("nccl", device_id=device, timeout=timedelta(seconds=120))
    cfg = CONFIGS[args.workload]
    nb = max((n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens)
    n_pools = max(1, args.layer_pools)
    steps_obj = []
    for l in range(n_pools):
        kv = make_device_layer(cfg, device, seed=l)      # same seed on every rank: a rank reads only its range
        summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb,
                                   k_bar_dtype=torch.bfloat16 if args.kbar_bf16 else torch.float32)
        g = torch.Generator(device=device).manual_seed(77 + l)
        q = torch.randn((cfg.batch, cfg.n_q_heads, cfg.head_dim), generator=g, device=device).to(cfg.torch_dtype)
        cls = partition.SplitKVDecodeAttentionP2P if args.exchange == "p2p" else partition.SplitKVDecodeAttention
        step = cls(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=args.rep_mode, n_splits=args.n_splits or 4)
        steps_obj.append((step, q))
    K, W = args.steps, args.warmup
    for step, q in steps_obj:          # communicator set-up and first launches outside any capture
        step.step(q)
    torch.cuda.synchronize()
    graphs = None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for step, q in steps_obj:
                    step.step(q)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graphs = []
            for step, q in steps_obj:
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, capture_error_mode="thread_local"):
                    step.step(q)
                graphs.append(g_)
        except Exception as e:   # every rank runs the same code, so every rank falls back together
            print(f"[bench] graph capture of the split-KV step failed ({type(e).__name__}: {e}); running eagerly",
                  file=sys.stderr, flush=True)
            graphs = None
    run_step = (lambda i: graphs[i % n_pools].replay()) if graphs is not None else (
        lambda i: steps_obj[i % n_pools][0].step(steps_obj[i % n_pools][1]))

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(W):
        run_step(i)
    sync_all()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(K):
        run_step(i)
    t1.record()
    sync_all()
    clocks = sampler.stop()
    times = torch.tensor([t0.elapsed_time(t1)], device=device, dtype=torch.float64)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(times[0])
        line = {
            "metric": METRIC, "value": cfg.batch * K / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "batch": cfg.batch, "context": max(cfg.prefix_lens),
                       "top_k": cfg.top_k, "rep_mode": args.rep_mode, "parallelism": f"split-kv x{world}",
                       "exchange": ("peer stores of the (o, lse) partials from the attention kernel + flags"
                                    if args.exchange == "p2p" else "NCCL all_gather of the (o, lse) partials")
                                   + ", selection replicated",
                       "cuda_graph": graphs is not None},
            "us_per_layer": 1e3 * ms / K, "gpu_launches": 3 * K, "clocks": clocks, "device_status": ops.device_status(),
        }
        print(json.dumps(line), flush=True)
    if graphs is not None:
        # the captured graphs hold the communicator's kernels; destroying the communicator under them
        # did not return on two GPUs - drop the graphs, drain the device and leave without the teardown
        del graphs, run_step
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)
    dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "cfg4_longctx_128k" and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_split_kv_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
