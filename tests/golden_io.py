"""Loader for the committed golden vectors (tests/golden/*.npz)."""

import hashlib
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _to_np(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def input_sha256(case):
    h = hashlib.sha256()
    for key in ("q", "k_pool", "v_pool", "block_table"):
        h.update(_to_np(case[key].contiguous()).tobytes())
    return h.hexdigest()


def load(name):
    return np.load(os.path.join(GOLDEN_DIR, name), allow_pickle=False)


def ragged_case():
    """The small bf16 case whose inputs are stored with its reference outputs."""
    from tests.golden.make_golden import SMALL_RAGGED as cfg
    vec = load("ragged_bf16_reference.npz")

    def bf16(a):
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)

    case = {
        "cfg": cfg,
        "q": bf16(vec["in_q"]), "k_pool": bf16(vec["in_k_pool"]), "v_pool": bf16(vec["in_v_pool"]),
        "block_table": torch.from_numpy(vec["in_block_table"].copy()),
        "prefix_lens": torch.from_numpy(vec["in_prefix_lens"].copy()),
        "seq_lens": torch.from_numpy(vec["in_seq_lens"].copy()),
        "page_size": cfg.page_size, "block_size": cfg.block_size, "top_k": cfg.top_k,
    }
    return case, vec


def cfg1_case():
    """The fp32 configuration: inputs regenerated from the seed, checked by hash."""
    from oracle.configs import CONFIGS, make_case
    vec = load("cfg1_cpu_fp32_reference.npz")
    case = make_case(CONFIGS["cfg1_cpu_fp32"])
    ok = input_sha256(case) == str(vec["input_sha256"])
    return case, vec, ok
