"""Phase timelines of the selection and attention kernels without a profiler.

    python -m interattn_b200.phase_trace select cfg2_llama8b_32k [more workloads]
    python -m interattn_b200.phase_trace decode cfg3_layer_llama8b_8k
    python -m interattn_b200.phase_trace step cfg2_llama8b_32k      (the one-kernel layer step)

Builds a variant of the library with ``-DIA_SELECT_TRACE -DIA_DECODE_TRACE`` (beside the normal
one, never loaded by anything else).  In that variant thread 0 of every CTA writes time stamps
from the nanosecond global timer at the kernel's phase boundaries: the selection kernel into the
``delta`` diagnostics buffer (16 floats per CTA instead of the deltas), the attention kernel into a
buffer whose address the environment variable ``IA_TRACE_PTR`` gives (``IA_STEP_TRACE_PTR`` for the
selection-and-attention kernel of the one-kernel step).  This module runs the traced
kernel on a named workload - after a launch on another KV pool, so that its inputs come from
HBM - and prints, per stamp, the mean / min / max over the CTAs in microseconds since CTA start.
"""

from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
TRACE_LIB = os.path.join(HERE, "libinterattn_b200_trace.so")

SELECT_STAMPS = ["predecessor complete", "set-up barrier passed", "first tile landed",
                 "thread 0's last tile consumed", "all tiles consumed, lane states reduced",
                 "row normalisers merged", "scores in the routing CTA", "radix select done", "indices written",
                 "radix pass 0", "radix pass 1", "radix pass 2", "radix pass 3"]
STEP_STAMPS = SELECT_STAMPS[:11] + ["attention phase starts", "all pages consumed", "first page consumed",
                                    "output rows written"]
DECODE_STAMPS = ["predecessor complete", "lengths and counts read", "descriptors resolved", "first page landed",
                 "last page consumed", "rings idle", "partial written", "pair finished"]


def _load_trace_library():
    from . import _lib, build
    build.build(defines=("IA_SELECT_TRACE", "IA_DECODE_TRACE"), output=TRACE_LIB)
    _lib.LIB_PATH = TRACE_LIB
    _lib._lib = None
    return _lib.load()


def _report(name, stamps, t):
    t = t[t[:, 15] != 0]
    if t.shape[0] == 0:
        print(f"{name}: no CTA left a stamp")
        return
    start = t[:, 15] - t[:, 15].min()
    print(f"{name}: {t.shape[0]} CTAs, start skew max {float(start.max()) * 1e-3:.2f} us")
    for i, label in enumerate(stamps):
        col = t[:, i]
        col = col[col > 0]
        if col.numel():
            print(f"  {label:42s} mean {float(col.mean()):7.2f}  min {float(col.min()):7.2f}  "
                  f"max {float(col.max()):7.2f}  (n={col.numel()})")
    last = max(i for i in range(len(stamps)) if bool((t[:, i] > 0).any()))
    print(f"  last stamp of the grid {float((start * 1e-3 + t[:, last]).max()):.2f} us after the first CTA started")
    return start * 1e-3


def _report_absolute(stamps, t, picks):
    """The attention kernel's stamps on one clock (us since the first CTA saw its predecessor complete),
    as percentiles over the CTAs, and split by how many CTAs of the grid shared the CTA's SM."""
    t = t[t[:, 15] != 0]
    start = (t[:, 15] - t[:, 15].min()) * 1e-3
    zero = float((start + t[:, 0]).min())
    sm = t[:, 14].long()
    mates = torch.bincount(sm, minlength=int(sm.max()) + 1)[sm]
    print(f"  on one clock (0 = first CTA past its predecessor); SMs used {int(sm.unique().numel())}, "
          f"CTAs by SM occupancy {dict(sorted((int(k), int((mates == k).sum())) for k in mates.unique()))}")
    qs = torch.tensor([0.0, 0.1, 0.5, 0.9, 1.0], dtype=torch.float64)
    for i in picks:
        a = (start + t[:, i] - zero).double()
        row = "  ".join(f"{float(v):6.2f}" for v in torch.quantile(a, qs))
        by = "  ".join(f"[{int(k)} per SM: mean {float(a[mates == k].mean()):.2f}]" for k in mates.unique())
        print(f"  {stamps[i]:28s} min/p10/p50/p90/max  {row}   {by}")


def main(argv):
    if len(argv) < 2 or argv[0] not in ("select", "decode", "step"):
        raise SystemExit(__doc__)
    if not torch.cuda.is_available():
        raise SystemExit("phase_trace needs a CUDA device")
    dev = torch.device("cuda:0")
    trace = torch.zeros(8192 * 16, device=dev, dtype=torch.float32)
    os.environ["IA_STEP_TRACE_PTR" if argv[0] == "step" else "IA_TRACE_PTR"] = hex(trace.data_ptr())
    if argv[0] == "decode":
        os.environ["INTERATTN_B200_FUSED"] = "0"  # the attention kernel of the two-kernel form is the subject
    _load_trace_library()
    from . import ops
    from .workloads import CONFIGS, make_device_layer
    for workload in argv[1:]:
        cfg = CONFIGS[workload]
        nb = max((n + cfg.block_size - 1) // cfg.block_size for n in cfg.prefix_lens)
        pools = []
        for l in range(2):
            kv = make_device_layer(cfg, dev, l)
            pools.append((kv, ops.build_summaries(kv, cfg.block_size, max_blocks=nb)))
        q = torch.randn(cfg.batch, cfg.n_q_heads, cfg.head_dim, device=dev).to(cfg.torch_dtype)
        if argv[0] == "select":
            for _ in range(4):
                ops.select_blocks(q, pools[1][1], pools[1][0].prefix_lens, top_k=cfg.top_k)
                torch.cuda.synchronize()
                _, _, aux = ops.select_blocks(q, pools[0][1], pools[0][0].prefix_lens, top_k=cfg.top_k, want=("delta",))
                torch.cuda.synchronize()
            flat = aux["delta"].reshape(-1)
            _report(f"select {workload}", SELECT_STAMPS, flat[: flat.numel() // 16 * 16].reshape(-1, 16).cpu())
        elif argv[0] == "step":
            steps = [ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k) for kv, summ in pools]
            for _ in range(3):
                steps[1].step(q)
                torch.cuda.synchronize()
                trace.zero_()
                torch.cuda.synchronize()
                steps[0].step(q)
                torch.cuda.synchronize()
            if not ops.last_decode_fused():
                print(f"step {workload}: this workload takes the two-kernel form")
                continue
            _report(f"step {workload}", STEP_STAMPS, trace.reshape(-1, 16).cpu())
        else:
            steps = [ops.DecodeAttention(kv, summ, cfg.n_q_heads, top_k=cfg.top_k) for kv, summ in pools]
            for _ in range(3):
                steps[1].step(q)
                torch.cuda.synchronize()
                trace.zero_()
                torch.cuda.synchronize()
                steps[0].step(q)
                torch.cuda.synchronize()
            t = trace.reshape(-1, 16).cpu()
            _report(f"decode {workload} (n_splits {steps[0].n_splits})", DECODE_STAMPS, t)
            _report_absolute(DECODE_STAMPS, t, (0, 3, 4, 7))


if __name__ == "__main__":
    main(sys.argv[1:])
