"""Generates the committed golden vectors from the UNMODIFIED reference.

Run where the reference tree is present:

    python tests/golden/make_golden.py [--reference /path/to/reference]

For each case the reference's own functions are called on seeded inputs
(``oracle.configs``) and their outputs stored:

* ``_build_prompt_blocks``            -> block summaries
* ``_select_prompt_blocks_eager``     -> z_logits, epsilon masks at several
  thresholds, and the per-(kv head, block) condition score, captured as the
  tensor the reference averages over the query group right before comparing
  with eps (the function does not return it)
* ``_condition_block_decode_output_dense`` -> hybrid attention output for the
  top-k mask (score descending, block index ascending among equals), and the
  sparse-only output for the same mask: the same function with
  ``cluster_exists`` all false, which masks every representative
  (legacy.py:828-829) and leaves selected tokens + suffix
* ``_condition_block_decode_output_compact_sdpa`` -> the reference's sparse CPU
  path (gather the active entries, one SDPA call) for the same mask, fp32
* the fp32 twin ``condition_block._condition_block_decode_output`` end to end

Small cases carry their inputs; for the larger fp32 configuration the inputs
are regenerated from the seed and only their SHA-256 is stored.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import condition_block_oracle as orc  # noqa: E402  (paging helper only)
from oracle.configs import CONFIGS, DecodeConfig, make_case  # noqa: E402


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def _sha(*tensors: torch.Tensor) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(_np(t.contiguous()).tobytes())
    return h.hexdigest()


class _CaptureGroupMean:
    """Records the input of ``Tensor.mean(dim=1, keepdim=True)`` - the call the
    reference makes on the condition tensor just before thresholding."""

    def __enter__(self):
        self.seen = []
        self._orig = torch.Tensor.mean
        outer = self

        def spy(t, *a, **kw):
            if kw.get("keepdim") and (kw.get("dim") == 1 or (a and a[0] == 1)):
                outer.seen.append(t.detach().clone())
            return outer._orig(t, *a, **kw)

        torch.Tensor.mean = spy
        return self

    def __exit__(self, *exc):
        torch.Tensor.mean = self._orig
        return False


def reference_vectors(core, legacy, pr1, cfg: DecodeConfig, eps_quantiles=(0.25, 0.75)):
    case = make_case(cfg)
    g = cfg.group_size
    out = {}
    for b in range(cfg.batch):
        plen = int(case["prefix_lens"][b])
        slen = int(case["seq_lens"][b])
        k = orc.gather_logical(case["k_pool"], case["block_table"][b], slen)
        v = orc.gather_logical(case["v_pool"], case["block_table"][b], slen)
        prefix = core._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
        qg = case["q"][b].reshape(cfg.n_kv_heads, g, 1, cfg.head_dim).float()
        with _CaptureGroupMean() as cap:
            sel0, z_logits, v_bar, size, exists = core._select_prompt_blocks_eager(qg, prefix, 0.0)
        assert len(cap.seen) == 1
        score = cap.seen[0].mean(dim=1)[:, 0]                      # [Hkv, nb]
        pre = f"seq{b}_"
        for key in ("k_bar", "v_bar", "k_max", "k_min", "v_norm_max"):
            out[pre + key] = _np(prefix[key].float())
        out[pre + "counts"] = prefix["block_valid_counts"].numpy()
        out[pre + "z_logits"] = z_logits[:, :, 0].numpy()
        out[pre + "score"] = score.numpy()
        out[pre + "mask_eps0"] = sel0[:, 0, 0].numpy()
        for qi, quant in enumerate(eps_quantiles):
            eps = float(torch.quantile(score.flatten(), quant))
            sel, *_ = core._select_prompt_blocks_eager(qg, prefix, eps)
            out[pre + f"eps{qi}"] = np.float64(eps)
            out[pre + f"mask_eps{qi}q"] = sel[:, 0, 0].numpy()
        # top-k mask from the reference score
        nb = score.shape[1]
        k_eff = min(cfg.top_k, nb)
        order = torch.sort(score, dim=1, descending=True, stable=True).indices[:, :k_eff]
        mask = torch.zeros_like(score, dtype=torch.bool)
        mask.scatter_(1, order, True)
        out[pre + "topk_ranked"] = order.numpy().astype(np.int32)
        dense = legacy._condition_block_decode_output_dense(
            q_grouped=qg, pos_tensor=torch.tensor([slen - 1]), prompt_prefix=prefix,
            k_suffix=k[:, plen:].float(), v_suffix=v[:, plen:].float(),
            block_size=cfg.block_size, prompt_len=plen,
            selected=mask[:, None, None, :].expand(-1, g, 1, -1),
            z_logits=z_logits, v_bar=v_bar, cluster_exists=exists)
        out[pre + "hybrid_topk_out"] = dense[:, :, 0].numpy()
        sparse = legacy._condition_block_decode_output_dense(
            q_grouped=qg, pos_tensor=torch.tensor([slen - 1]), prompt_prefix=prefix,
            k_suffix=k[:, plen:].float(), v_suffix=v[:, plen:].float(),
            block_size=cfg.block_size, prompt_len=plen,
            selected=mask[:, None, None, :].expand(-1, g, 1, -1),
            z_logits=z_logits, v_bar=v_bar, cluster_exists=torch.zeros_like(exists))
        out[pre + "sparse_topk_out"] = sparse[:, :, 0].numpy()
        compact = legacy._condition_block_decode_output_compact_sdpa(
            q_grouped=qg, pos_tensor=torch.tensor([slen - 1]), prompt_prefix=prefix,
            k_suffix=k[:, plen:].float(), v_suffix=v[:, plen:].float(),
            block_size=cfg.block_size, prompt_len=plen,
            selected=mask[:, None, None, :].expand(-1, g, 1, -1),
            attention_dtype=torch.float32)
        out[pre + "compact_hybrid_topk_out"] = compact[:, :, 0].numpy()
        if cfg.dtype == "float32":
            twin = pr1._build_prompt_blocks(k[:, :plen], v[:, :plen], cfg.block_size)
            eps = float(out[pre + "eps1"])
            full, _ = pr1._condition_block_decode_output(
                q_grouped=qg, pos_tensor=torch.tensor([slen - 1]), prompt_prefix=twin,
                k_suffix=k[:, plen:], v_suffix=v[:, plen:], block_size=cfg.block_size,
                eps=eps, prompt_len=plen)
            out[pre + "pr1_eps1_out"] = full[:, :, 0].numpy()
    out["input_sha256"] = np.array(_sha(case["q"], case["k_pool"], case["v_pool"], case["block_table"]))
    return case, out


SMALL_RAGGED = DecodeConfig(
    "golden_ragged_bf16", "bfloat16", 2, 8, 2, 128, 16, 64, 2, (331, 128), (5, 1), seed=11,
    k_channel_sigma=0.5)


def main():
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--reference", default=os.environ.get("INTERATTN_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference"),
        help="the reference checkout (default: a directory `reference` next to this repository)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from llama.script.analysis.condition_block_gen.methods import condition_block as pr1
    from llama.script.analysis.condition_block_gen.methods.condition_block_triton_impl import core, legacy
    sys.path.remove(args.reference)

    # 1. fp32 CPU configuration: outputs + input checksum
    case, vec = reference_vectors(core, legacy, pr1, CONFIGS["cfg1_cpu_fp32"])
    np.savez_compressed(os.path.join(HERE, "cfg1_cpu_fp32_reference.npz"), **vec)

    # 2. small ragged bf16 case with suffix: inputs included
    case, vec = reference_vectors(core, legacy, pr1, SMALL_RAGGED)
    for key in ("q", "k_pool", "v_pool", "block_table", "prefix_lens", "seq_lens"):
        vec["in_" + key] = _np(case[key])
    np.savez_compressed(os.path.join(HERE, "ragged_bf16_reference.npz"), **vec)

    # 3. the hand-written score example of the reference's own pytest
    import types
    for name in ("matplotlib", "matplotlib.pyplot"):
        try:
            __import__(name)
        except ImportError:
            sys.modules[name] = types.ModuleType(name)
    sys.path.insert(0, args.reference)
    from llama.script.analysis.condition_block_ppl import runner_cond_block as rcb
    sys.path.remove(args.reference)
    z = torch.tensor([[[0.0, 1.0, 2.0], [0.5, -0.5, float("-inf")]]], dtype=torch.float64)
    p = torch.softmax(z, dim=-1)
    delta = torch.tensor([[[0.2, 1.0, 2.0], [0.4, 1.5, 0.0]]], dtype=torch.float64)
    b_c = torch.tensor([[[1.0, 2.0, 1.5], [0.8, 1.2, 0.0]]], dtype=torch.float64)
    b_all = b_c.amax(dim=-1)
    want = rcb._condition_score_for_blocks(
        p_tensor=p, z_logits=z, delta=delta, b_c=b_c, b_all=b_all, cluster_exists=torch.isfinite(z[0]))
    with open(os.path.join(HERE, "score_known_answer.json"), "w") as f:
        json.dump({"score_hex": [float(x).hex() for x in want.flatten()]}, f, indent=1)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
