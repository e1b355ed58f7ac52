"""Benchmark of the condition-block sparse decode-attention layer-step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--repeats R] [--impl reference]
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

Timing: W warm-up steps, then R regions of exactly K steps each; a region is
bracketed by a device synchronise (and a barrier across ranks) on both sides,
timed with CUDA events, maximum over ranks; the line reports the MEDIAN
region (min and mean beside it) - one 20-step region lasts 1.5 ms, too short
to stand alone.  Four KV pools are rotated between steps (> 126 MB of L2
touched before a pool is seen again); `cold_l2` repeats the steps with a
256 MiB buffer overwritten before each one.

One JSON line on rank 0:
  value      decode tokens advanced through one attention layer per second,
             whole job, inputs resident in HBM (one C-ABI call per step)
  e2e        the same through the host-buffer entry point: pinned q -> device,
             the step, output -> pinned host, every step
  roofline   the one-kernel step (selection, then paged sparse attention, in
             one launch): block summaries read + K/V bytes of the selected
             tokens / its average launch duration over the timed regions
             (which hold nothing but its launches), against the measured HBM
             peak; `isolated_us` = events around single launches; `phases`
             splits a launch at the first CTA's time stamps
  two_kernel the same step as two launches (selection, attention), each with
             its own duration and roofline
  hybrid, kbar_bf16, diag_ell   the same step in the reference's own mode
             (unselected blocks attended through their representatives), with
             the block key means stored in bf16, and with the diagonal-ellipsoid
             bound in place of the coordinate range, each with its own roofline
  cpu_baseline  the CPU port of the reference's PyTorch path timed on this
             box's host cores on a bounded sample: its sparse (gather the
             selected tokens) and dense (score every token, then mask) legs
  llama_decode  tokens/s of the whole Llama-3-8B-architecture decode (N = 1)
  strong_cfg5, split_kv_cfg4   (N > 1) the two strong-scaling arms: kv-head
             shards of the ragged 70B batch, and split-KV of the 128k batch
`--impl reference` times the CPU path alone, with every host thread.
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
FLUSH_BYTES = 256 << 20  # cold-L2 variant: at least twice the 126 MB L2


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20, help="steps per timed region")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeats", type=int, default=25, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--n-splits", type=int, default=0, help="split-KV parts per (sequence, kv head); 0 = auto")
    ap.add_argument("--rep-mode", default="sparse_only", choices=["sparse_only", "hybrid"])
    ap.add_argument("--workload", default=WORKLOAD)
    ap.add_argument("--cpu-sample-seqs", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-variants", action="store_true", help="skip the hybrid / bf16-k_bar / cold-L2 sub-records")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the two strong-scaling sub-records")
    ap.add_argument("--no-graph", action="store_true", help="split-KV arm: launch the step eagerly")
    ap.add_argument("--kbar-bf16", action="store_true",
                    help="store the block key means in bf16 (the reference's approximate option) instead of fp32")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="split-KV arm: partials stored into the peers' buffers by the attention kernel (p2p) "
                         "or an NCCL all-gather after it (nccl)")
    ap.add_argument("--llama-steps", type=int, default=256,
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


def cpu_layer_step(small, prepared, leg="sparse", rep_mode="sparse_only"):
    """One layer-step on the host: score + top-k + attention per sequence.  ``leg`` picks the port of
    the reference's sparse path (gather the selected tokens, IMPL/legacy.py:871-966) or of its dense
    path (score every prefix token, then mask, IMPL/legacy.py:797-868).  Returns seconds."""
    from oracle import condition_block_oracle as orc
    attend = orc.decode_attention if leg == "sparse" else orc.decode_attention_dense
    t0 = time.perf_counter()
    for plen, k, v, summ, qg in prepared:
        terms = orc.condition_terms(qg, summ)
        _, mask = orc.select_topk(terms["score"], summ.counts, small.top_k)
        attend(qg, k, v, plen, small.block_size, mask, rep_mode=rep_mode, z=terms["z"], v_bar=summ.v_bar)
    return time.perf_counter() - t0


def cpu_legs(cfg, n, reps, rep_mode):
    """Both CPU legs on the same ``n`` sampled sequences -> {"sparse": tok*layer/s, "dense": ...}, seconds per step."""
    small, prepared = cpu_prepare(cfg, n)
    out, secs = {}, {}
    for leg in ("sparse", "dense"):
        cpu_layer_step(small, prepared, leg, rep_mode)  # warm-up
        dt = sum(cpu_layer_step(small, prepared, leg, rep_mode) for _ in range(reps)) / reps
        out[leg], secs[leg] = n / dt, dt
    return out, secs


def run_reference_arm(args):
    """The reference's CPU implementation of the path (oracle port), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from interattn_b200.workloads import CONFIGS
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = CONFIGS[args.workload]
    n = 1 if args.steps > 20 else max(1, min(args.cpu_sample_seqs, 4))
    small, prepared = cpu_prepare(cfg, n)
    for _ in range(args.warmup):
        cpu_layer_step(small, prepared, "sparse", args.rep_mode)
    total = 0.0
    for _ in range(args.steps):
        total += cpu_layer_step(small, prepared, "sparse", args.rep_mode)
    value = n * args.steps / total
    dense_dt = sum(cpu_layer_step(small, prepared, "dense", args.rep_mode) for _ in range(3)) / 3
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "rep_mode": args.rep_mode,
                   "sample": f"{n} of {cfg.batch} sequences per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{n} sequence(s) x {args.steps} steps: score + top-k + sparse attention "
                                   "(the port of the reference's sparse CPU leg), summaries excluded",
                         "legs": {"sparse": value, "dense": n / dense_dt}},
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
    from interattn_b200.workloads import make_device_layer as make
    return make(cfg, device, seed)


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return FALLBACK_HBM_GBS, "fallback"


def committed_traffic(workload, kernel):
    """DRAM bytes per launch from the committed ncu summary (profiles/dram_traffic.txt), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.txt")) as f:
            for ln in f:
                parts = ln.split()
                if len(parts) == 3 and parts[0] == workload and parts[1] == kernel:
                    return int(parts[2])
    except (OSError, ValueError):
        pass
    return None


def algorithmic_bytes(cfg, rep_mode, kbar_bf16, bound="range"):
    """(attention kernel, selection kernel) algorithmic bytes per launch.  The selection reads, per block,
    k_bar and either (k_max, k_min) or, with the diagonal-ellipsoid bound, (w, rho)."""
    esz = 2 if cfg.dtype == "bfloat16" else 4
    blocks = [(n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens]
    tokens_sel = sum(min(cfg.top_k * cfg.block_size, n) for n in cfg.prefix_lens) * cfg.n_kv_heads
    suffix_tok = sum(cfg.suffix_lens) * cfg.n_kv_heads
    kv_bytes = (tokens_sel + suffix_tok) * cfg.head_dim * 2 * esz
    if rep_mode == "hybrid":  # one v_bar row per unselected block
        kv_bytes += sum(max(nb - cfg.top_k, 0) for nb in blocks) * cfg.n_kv_heads * cfg.head_dim * esz
    bound_bytes = 2 * cfg.head_dim * esz if bound == "range" else cfg.head_dim * esz + 4
    sel_bytes = sum(blocks) * cfg.n_kv_heads * (cfg.head_dim * (2 if kbar_bf16 else 4) + bound_bytes + 4)
    return kv_bytes, sel_bytes


class Regions:
    """R timed regions of K steps each, bracketed by a synchronise (+ barrier) on both sides."""

    def __init__(self, torch, dist, world, device):
        self.torch, self.dist, self.world, self.device = torch, dist, world, device

    def sync_all(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def run(self, step, K, R, first=0):
        """step(i) enqueues step i.  Returns per-region milliseconds (max over ranks), a list of R."""
        torch = self.torch
        ms = []
        i = first
        for _ in range(R):
            self.sync_all()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(K):
                step(i)
                i += 1
            t1.record()
            self.sync_all()
            ms.append(t0.elapsed_time(t1))
        t = torch.tensor(ms, device=self.device, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.cpu()]


def summarise(ms_regions, K):
    """Median / min / mean microseconds per step over the regions."""
    per = sorted(1e3 * m / K for m in ms_regions)
    return {"median": statistics.median(per), "min": per[0], "mean": sum(per) / len(per), "regions": len(per)}


def kernel_times(torch, steppers, qs, K, repeats):
    """Per-kernel device microseconds (median over K x repeats live steps, events between the launches)."""
    n_pools = len(steppers)
    n = K * repeats
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n)]
    for row in ev:
        for e in row:
            e.record()
    torch.cuda.synchronize()
    for i in range(n):
        steppers[i % n_pools].step_timed(qs[i % n_pools], ev[i])
    torch.cuda.synchronize()
    sel = statistics.median(r[0].elapsed_time(r[1]) for r in ev) * 1e3
    att = statistics.median(r[1].elapsed_time(r[2]) for r in ev) * 1e3
    return sel, att


def kernel_records(fused, sel_us, att_us, kv_bytes, sel_bytes, workload, rep_mode="sparse_only", phases=None,
                   region_us=None):
    """(kernel_us, roofline, roofline_select) of a layer step.  Two kernels: the attention kernel is the
    dominant one and the selection kernel has its own record.  One fused kernel
    (condition_block_select_attend_kernel): it reads the summaries and the picked pages in one launch, so its
    algorithmic bytes are the sum.  Its timed regions hold nothing but its launches, so its average launch
    duration over the timed region is ``region_us`` (region / launches; programmatic launch lets a launch's
    prologue overlap its predecessor's drain); the span between events around single launches, where nothing
    overlaps, is kept beside it as ``isolated_us``."""
    peak, src = hbm_peak()
    if fused:
        isolated = sel_us + att_us  # events 0 -> 2; nothing runs between 1 and 2
        us = region_us if region_us else isolated
        gbs = (kv_bytes + sel_bytes) / (us * 1e-6) / 1e9
        kernel_us = {"select_attend": isolated, "select": 0.0, "sparse_decode": 0.0, "finalize": 0.0}
        roof = {"bound": "hbm", "kernel": "condition_block_select_attend_kernel", "achieved": gbs, "peak": peak,
                "peak_source": src, "unit": "GB/s", "frac": gbs / peak,
                "traffic": committed_traffic(workload, "select_attend"), "bytes_per_launch": kv_bytes + sel_bytes,
                "duration_us": us, "isolated_us": isolated,
                "isolated_frac": (kv_bytes + sel_bytes) / (isolated * 1e-6) / 1e9 / peak,
                "timing": ("duration = timed region / launches (the regions hold this kernel only); "
                           "isolated = CUDA events around single launches" if region_us else
                           "CUDA events around single launches")}
        if phases is not None and phases[0] > 0 and phases[1] > 0:
            # the kernel's own clock (time stamps of its first CTA): the latency-bound selection in front and the
            # streaming attention phase behind it, each with the bytes it moves
            s_us, a_us = phases
            roof["phases"] = {
                "selection": {"us": s_us, "bytes": sel_bytes, "achieved": sel_bytes / (s_us * 1e-6) / 1e9,
                              "frac": sel_bytes / (s_us * 1e-6) / 1e9 / peak},
                "attention": {"us": a_us, "bytes": kv_bytes, "achieved": kv_bytes / (a_us * 1e-6) / 1e9,
                              "frac": kv_bytes / (a_us * 1e-6) / 1e9 / peak},
                "clock": "nanosecond global timer, first CTA of the last launch; the event-timed duration above "
                         "also holds launch and drain"}
        return kernel_us, roof, None
    att_gbs, sel_gbs = kv_bytes / (att_us * 1e-6) / 1e9, sel_bytes / (sel_us * 1e-6) / 1e9
    suffix = "" if rep_mode == "sparse_only" else f"_{rep_mode}"
    kernel_us = {"select": sel_us, "sparse_decode": att_us, "finalize": 0.0}
    roof = {"bound": "hbm", "kernel": "condition_block_finalize_attention_kernel", "achieved": att_gbs, "peak": peak,
            "peak_source": src, "unit": "GB/s", "frac": att_gbs / peak,
            "traffic": committed_traffic(workload, "sparse_decode" + suffix), "bytes_per_launch": kv_bytes}
    roof_sel = {"bound": "hbm", "kernel": "condition_block_select_kernel", "achieved": sel_gbs, "peak": peak,
                "unit": "GB/s", "frac": sel_gbs / peak, "bytes_per_launch": sel_bytes,
                "traffic": committed_traffic(workload, "select")}
    return kernel_us, roof, roof_sel


def variant_record(torch, regions, cfg, layers, qs, rep_mode, kbar_bf16, summaries, n_splits, K, R, workload,
                   bound="range", fused=True):
    """One sub-record: the layer-step in another mode / summary layout / launch form, with its own roofline."""
    from interattn_b200 import ops
    before = ops.set_fused_step(fused)
    try:
        return _variant_record(torch, regions, cfg, layers, qs, rep_mode, kbar_bf16, summaries, n_splits, K, R,
                               workload, bound)
    finally:
        ops.set_fused_step(before)


def _variant_record(torch, regions, cfg, layers, qs, rep_mode, kbar_bf16, summaries, n_splits, K, R, workload, bound):
    from interattn_b200 import ops
    steppers = [ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=rep_mode, n_splits=n_splits,
                                    bound=bound)
                for (kv, _), summ in zip(layers, summaries)]
    n_pools = len(steppers)
    for i in range(8):
        steppers[i % n_pools].step(qs[i % n_pools])
    ms = regions.run(lambda i: steppers[i % n_pools].step(qs[i % n_pools]), K, R)
    sel_us, att_us = kernel_times(torch, steppers, qs, K, max(1, R // 5))
    fused = ops.last_decode_fused()
    phases = ops.last_step_phases() if fused else None
    kv_bytes, sel_bytes = algorithmic_bytes(cfg, rep_mode, kbar_bf16, bound)
    per_step = summarise(ms, K)
    kernel_us, roof, roof_sel = kernel_records(fused, sel_us, att_us, kv_bytes, sel_bytes, workload, rep_mode, phases,
                                               per_step["median"])
    rec = {
        "us_per_layer": per_step, "kernel_us": kernel_us,
        "config": {"rep_mode": rep_mode, "k_bar": "bf16" if kbar_bf16 else "f32", "bound": bound,
                   "launches_per_step": 1 if fused else 2},
        "roofline": roof,
    }
    if roof_sel is not None:
        rec["roofline_select"] = roof_sel
    return rec


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from interattn_b200 import ops
    from interattn_b200.workloads import CONFIGS

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        from datetime import timedelta
        dist.init_process_group("nccl", device_id=device, timeout=timedelta(seconds=180))
    regions = Regions(torch, dist, world, device)
    line = layer_step_record(args, args.workload, torch, dist, regions, world, rank, local_rank, device, main=True)
    if world > 1 and not args.no_strong and args.workload == WORKLOAD:
        # the two strong-scaling arms, every rank takes part; rank 0 attaches them to its line
        for key, fn in (("strong_cfg5", strong_cfg5_record), ("split_kv_cfg4", split_kv_record)):
            try:
                rec = fn(args, torch, dist, regions, world, rank, local_rank, device)
            except Exception as e:  # the same code runs on every rank, so every rank lands here together
                rec = {"error": f"{type(e).__name__}: {e}"[:300]}
            if rank == 0:
                line[key] = rec
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            cfg = CONFIGS[args.workload]
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            n = max(1, args.cpu_sample_seqs)
            legs, secs = cpu_legs(cfg, n, 3, args.rep_mode)
            hyb, _ = cpu_legs(cfg, n, 2, "hybrid") if args.rep_mode != "hybrid" else (legs, secs)
            line["cpu_baseline"] = {
                "value": legs["sparse"], "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"{n} of {cfg.batch} sequences, one layer-step x 3 per leg: score + top-k + attention "
                          f"(sparse leg {secs['sparse']:.2f} s, dense leg {secs['dense']:.2f} s per step), "
                          "summaries excluded",
                "legs": {"sparse": legs["sparse"], "dense": legs["dense"],
                         "hybrid_sparse": hyb["sparse"], "hybrid_dense": hyb["dense"]}}
        if args.llama_steps > 1 and world == 1 and args.workload == WORKLOAD:
            line["llama_decode"] = llama_decode_line(args.llama_steps)
        print(json.dumps(line), flush=True)
    if world > 1:
        from interattn_b200 import partition
        partition.ordered_shutdown()


def layer_step_record(args, workload, torch, dist, regions, world, rank, local_rank, device, main, head_shard=False):
    """The layer-step of one workload on this rank's shard; returns the JSON record (meaningful on rank 0)."""
    from dataclasses import replace
    from interattn_b200 import ops
    from interattn_b200.workloads import CONFIGS
    cfg = CONFIGS[workload]
    if head_shard:
        # kv-head shards: every rank holds all sequences but only its heads - strong scaling, still no
        # collective, the output rows of different heads are disjoint
        from interattn_b200.partition import plan_head_shards
        lo, hi = plan_head_shards(cfg.n_kv_heads, world)[rank]
        cfg = replace(cfg, n_kv_heads=hi - lo, n_q_heads=(hi - lo) * cfg.group_size)
    replicas = 1 if head_shard else world
    n_splits = args.n_splits or None      # None: the library picks a wave-aware split count
    nb = max((n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens)
    rows = cfg.n_q_heads
    kbar_dt = torch.bfloat16 if args.kbar_bf16 else torch.float32

    layers, steppers, qs = [], [], []
    n_pools = max(1, args.layer_pools)
    for l in range(n_pools):
        kv = make_device_layer(cfg, device, seed=1000 * rank + l)
        summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb, k_bar_dtype=kbar_dt)
        layers.append((kv, summ))
        steppers.append(ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode=args.rep_mode,
                                            n_splits=n_splits))
        g = torch.Generator(device=device).manual_seed(77 + 1000 * rank + l)
        qs.append(torch.randn((cfg.batch, rows, cfg.head_dim), generator=g, device=device).to(cfg.torch_dtype))
    n_splits = steppers[0].n_splits
    torch.cuda.synchronize()

    K, W, R = args.steps, args.warmup, max(1, args.repeats)
    sampler = ClockSampler(local_rank)   # samples from the warm-up to the end of the last timed region
    sampler.start()
    for i in range(max(W, 3)):
        steppers[i % n_pools].step(qs[i % n_pools])
    # headline: R regions of K steps through the plain one-call entry point
    ms = regions.run(lambda i: steppers[i % n_pools].step(qs[i % n_pools]), K, R)
    # the same steps again with events between the kernels: per-kernel device times for the roofline
    sel_us, att_us = kernel_times(torch, steppers, qs, K, max(1, R // 5))
    fused = ops.last_decode_fused()  # one launch per step (selection + attention in one kernel) or two
    phases = ops.last_step_phases() if fused else None
    status = ops.device_status()

    # end-to-end: host q in, host output back, every step
    q_host = [q.cpu().pin_memory() for q in qs]
    out_host = [torch.empty_like(q).pin_memory() for q in q_host]
    for i in range(5):
        steppers[i % n_pools].step_host(q_host[i % n_pools], out_host[i % n_pools])
    e2e_ms = regions.run(lambda i: steppers[i % n_pools].step_host(q_host[i % n_pools], out_host[i % n_pools]), K, R)
    clocks = sampler.stop()

    # cold L2: a 256 MiB buffer overwritten before every step, the step timed by its own events
    cold = None
    if main and not args.no_variants:
        flush = torch.empty((FLUSH_BYTES,), device=device, dtype=torch.uint8)
        n = K * max(1, R // 5)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for i in range(n):
            flush.fill_(i & 0xff)
            ev[i][0].record()
            steppers[i % n_pools].step(qs[i % n_pools])
            ev[i][1].record()
        torch.cuda.synchronize()
        per = sorted(a.elapsed_time(b) * 1e3 for a, b in ev)
        cold = {"us_per_layer": {"median": statistics.median(per), "min": per[0], "mean": sum(per) / len(per)},
                "flush_bytes": FLUSH_BYTES, "steps": n,
                "note": "one step at a time between events, so launch latency is not hidden by the next step"}
        del flush

    t = torch.tensor([sel_us, att_us], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sel_us, att_us = [float(x) for x in t.cpu()]
    step_us, e2e_us = summarise(ms, K), summarise(e2e_ms, K)

    esz = 2 if cfg.dtype == "bfloat16" else 4
    kv_bytes, sel_bytes = algorithmic_bytes(cfg, args.rep_mode, args.kbar_bf16)
    kernel_us, roof, roof_sel = kernel_records(fused, sel_us, att_us, kv_bytes, sel_bytes, workload, args.rep_mode,
                                               phases, step_us["median"])
    q_bytes = cfg.batch * rows * cfg.head_dim * esz
    line = {
        "metric": METRIC, "value": replicas * cfg.batch / (step_us["median"] * 1e-6), "unit": UNIT,
        "n_gpus": world, "steps": K, "warmup": W, "repeats": R, "ms_per_step": step_us["median"] * 1e-3,
        "higher_is_better": True, "scaling": "strong" if head_shard else "weak", "vs_baseline": None,
        "dtype": "bf16" if cfg.dtype == "bfloat16" else "f32", "data": "synthetic",
        "config": {"workload": workload, "batch_per_gpu": cfg.batch, "n_q_heads": cfg.n_q_heads,
                   "n_kv_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim, "context": max(cfg.prefix_lens),
                   "page": cfg.page_size, "block": cfg.block_size, "top_k": cfg.top_k,
                   "rep_mode": args.rep_mode, "n_splits": 1 if fused else n_splits,
                   "launches_per_step": 1 if fused else 2, "k_bar": "bf16" if args.kbar_bf16 else "f32",
                   "parallelism": (f"kv-head shard x{world}" if head_shard else f"batch-shard x{world}"),
                   "timing": f"median of {R} regions of {K} steps, each between synchronise + barrier, max over ranks",
                   "l2": f"{n_pools} layer pools rotated, {(kv_bytes + sel_bytes) >> 20} MiB read per step "
                         "(> 126 MB L2), no flush; cold_l2 = flushed before every step"},
        "us_per_layer": step_us["median"], "us_per_layer_stats": step_us,
        "kernel_us": kernel_us,
        "roofline": roof,
        "roofline_select": roof_sel,
        "e2e": {"value": replicas * cfg.batch / (e2e_us["median"] * 1e-6), "unit": UNIT,
                "h2d_bytes_per_step": q_bytes, "d2h_bytes_per_step": q_bytes,
                "us_per_layer": e2e_us["median"], "us_per_layer_stats": e2e_us,
                "note": "KV pool and block summaries are cache state resident on the device; the step's "
                        "inputs (q) and outputs cross PCIe every step"},
        # per timed region: one fused selection-and-attention kernel per step, or selection + attention
        "gpu_launches": (1 if fused else 2) * K,
        "clocks": clocks,
        "device_status": status,
    }
    if cold is not None:
        line["cold_l2"] = cold
    if main and not args.no_variants and world == 1:
        # the reference's own mode (representatives of the unselected blocks) and the bf16 k_bar layout
        Rv = max(5, R // 2)
        summ_f32 = [s for _, s in layers]
        if fused:
            # the same step as selection kernel + attention kernel: what the one-kernel form is measured against,
            # and the per-kernel rooflines of the form that runs where the fused one does not apply
            line["two_kernel"] = variant_record(torch, regions, cfg, layers, qs, args.rep_mode, args.kbar_bf16,
                                                summ_f32, args.n_splits or None, K, Rv, workload, fused=False)
        if args.rep_mode != "hybrid":
            line["hybrid"] = variant_record(torch, regions, cfg, layers, qs, "hybrid", args.kbar_bf16, summ_f32,
                                            n_splits, K, Rv, workload)
        if not args.kbar_bf16:
            summ_bf16 = [ops.build_summaries(kv, cfg.block_size, max_blocks=nb, k_bar_dtype=torch.bfloat16)
                         for kv, _ in layers]
            line["kbar_bf16"] = variant_record(torch, regions, cfg, layers, qs, args.rep_mode, True, summ_bf16,
                                               n_splits, K, Rv, workload)
            del summ_bf16
            # the diagonal-ellipsoid bound: (k_bar, w, rho) per block instead of (k_bar, k_max, k_min)
            summ_ell = [ops.build_summaries(kv, cfg.block_size, max_blocks=nb, diag_ell=True) for kv, _ in layers]
            line["diag_ell"] = variant_record(torch, regions, cfg, layers, qs, args.rep_mode, False, summ_ell,
                                              n_splits, K, Rv, workload, bound="diag_ell")
            del summ_ell
    return line


def strong_cfg5_record(args, torch, dist, regions, world, rank, local_rank, device):
    """kv-head shards of the ragged Llama-3-70B batch (one kv head per GPU on 8, two on 4, four on 2)."""
    import copy
    a = copy.copy(args)
    a.no_variants, a.rep_mode, a.kbar_bf16 = True, "sparse_only", False
    rec = layer_step_record(a, "cfg5_llama70b_ragged", torch, dist, regions, world, rank, local_rank, device,
                            main=False, head_shard=True)
    return {k: rec[k] for k in ("value", "unit", "us_per_layer", "us_per_layer_stats", "kernel_us", "scaling",
                                "config", "roofline", "roofline_select", "device_status")}


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
        from interattn_b200 import ops
        return {"metric": "llama3_8b_decode_tokens_per_s", "value": st["tokens_per_s"], "unit": "tok/s",
                "attention_launches_per_layer": 1 if ops.last_decode_fused() else 2,
                "ms_per_decode_step": 1e3 * st["decode_s"] / max(st["decode_steps_timed"], 1),
                "decode_steps_timed": st["decode_steps_timed"], "prefill_s": st["prefill_s"],
                "config": {"layers": 32, "batch": 32, "prompt": 8192, "new_tokens": int(steps), "block": 64,
                           "top_k": 64, "dtype": "bf16", "cuda_graph": True, "fused_step": True,
                           "weights": "random init", "data": "uniform random token ids"}}
    except Exception as e:   # the layer-step line above must still be printed
        return {"metric": "llama3_8b_decode_tokens_per_s", "error": f"{type(e).__name__}: {e}"[:300]}


def split_kv_record(args, torch, dist, regions, world, rank, local_rank, device):
    """Long-context split-KV (strong scaling): the blocks of every sequence are cut into contiguous
    ranges, one per rank; a step is the whole exchange (selection, attention, merge), captured per
    layer pool into a CUDA graph unless --no-graph is given or the capture fails.  With the in-kernel
    exchange both forms of the selection are timed - distributed (every rank streams its own
    summaries, two small exchanges inside the selection kernel) and replicated (every rank streams
    all summaries, no exchange) - and the faster one is the record's value."""
    from interattn_b200 import ops, partition
    from interattn_b200.workloads import CONFIGS
    workload = "cfg4_longctx_128k"
    cfg = CONFIGS[workload]
    nb = max((n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens)
    n_pools = max(1, args.layer_pools)
    K, R = args.steps, max(1, args.repeats)
    pools = []
    for l in range(n_pools):
        kv = make_device_layer(cfg, device, seed=l)      # same seed on every rank: a rank reads only its range
        summ = ops.build_summaries(kv, cfg.block_size, max_blocks=nb,
                                   k_bar_dtype=torch.bfloat16 if args.kbar_bf16 else torch.float32)
        g = torch.Generator(device=device).manual_seed(77 + l)
        q = torch.randn((cfg.batch, cfg.n_q_heads, cfg.head_dim), generator=g, device=device).to(cfg.torch_dtype)
        pools.append((kv, summ, q))

    def time_form(make_step):
        steps_obj = [(make_step(kv, summ), q) for kv, summ, q in pools]
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
        for i in range(max(args.warmup, 3)):
            run_step(i)
        ms = regions.run(run_step, K, R)
        status = ops.device_status()
        # graphs that captured NCCL kernels keep the communicator referenced: destroy them before anything else
        for g_ in graphs or []:
            g_.reset()
        for step, _ in steps_obj:
            close = getattr(step, "close", None)
            if close is not None:
                close()
        return {"us_per_layer": summarise(ms, K), "cuda_graph": graphs is not None, "device_status": status,
                "gpu_launches_per_step": getattr(steps_obj[0][0], "launches_per_step", 4)}

    n_splits = args.n_splits or 4
    forms = {}
    if args.exchange == "p2p":
        for selection in ("distributed", "replicated"):
            forms[selection] = time_form(lambda kv, summ, sel=selection: partition.SplitKVDecodeAttentionP2P(
                kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode="sparse_only", n_splits=n_splits, selection=sel))
    else:
        forms["replicated"] = time_form(lambda kv, summ: partition.SplitKVDecodeAttention(
            kv, summ, cfg.n_q_heads, top_k=cfg.top_k, rep_mode="sparse_only", n_splits=n_splits))
    best = min(forms, key=lambda k: forms[k]["us_per_layer"]["median"])
    step_us = forms[best]["us_per_layer"]
    return {
        "value": cfg.batch / (step_us["median"] * 1e-6), "unit": UNIT, "us_per_layer": step_us["median"],
        "us_per_layer_stats": step_us, "scaling": "strong",
        "config": {"workload": workload, "batch": cfg.batch, "context": max(cfg.prefix_lens), "top_k": cfg.top_k,
                   "parallelism": f"split-kv x{world}",
                   "exchange": ("peer stores of the (o, lse) partials from the attention kernel + flags"
                                if args.exchange == "p2p" else "NCCL all_gather of the (o, lse) partials"),
                   "selection": best, "cuda_graph": forms[best]["cuda_graph"]},
        "selection_forms_us": {k: v["us_per_layer"]["median"] for k, v in forms.items()},
        "gpu_launches_per_step": forms[best]["gpu_launches_per_step"],
        "device_status": max(v["device_status"] for v in forms.values()),
    }


def run_split_kv_arm(args):
    """`--workload cfg4_longctx_128k` under torchrun: the split-KV arm alone, as the job's headline line."""
    import torch
    import torch.distributed as dist
    from datetime import timedelta
    from interattn_b200 import partition
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device, timeout=timedelta(seconds=180))
    regions = Regions(torch, dist, world, device)
    sampler = ClockSampler(local_rank)
    sampler.start()
    rec = split_kv_record(args, torch, dist, regions, world, rank, local_rank, device)
    clocks = sampler.stop()
    if rank == 0:
        line = {"metric": METRIC, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "repeats": args.repeats, "ms_per_step": rec["us_per_layer"] * 1e-3, "higher_is_better": True,
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "clocks": clocks,
                "gpu_launches": rec["gpu_launches_per_step"] * args.steps}
        line.update(rec)
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    partition.ordered_shutdown()


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
