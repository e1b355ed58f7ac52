"""CPU restatement of the element-wise ops of one Llama decode step.

Test infrastructure only: imported by ``tests/`` to check the fused CUDA kernels of
``interattn_b200/csrc/llama_step.cu``; nothing in the product path uses it.

The arithmetic is not the reference's own: the reference runs the unmodified Hugging
Face model around its attention hook (``condition_block_triton_impl/core.py:190-316``),
so the algorithm lives in the third-party package ``transformers`` (5.5.0 in this
image), ``models/llama/modeling_llama.py``:

* ``LlamaRMSNorm.forward``            lines 62-67
* ``rotate_half`` / ``apply_rotary_pos_emb``  lines 138-168
* ``LlamaMLP.forward``                ``down_proj(act_fn(gate_proj(x)) * up_proj(x))``
* ``LlamaDecoderLayer.forward``       ``hidden_states = residual + hidden_states``
* ``cache_utils.StaticLayer.update``  ``index_copy_`` of the new key/value row

Each function restates the published expression with plain torch CPU ops in the
tensor's own dtype, so every bf16 rounding point is where PyTorch puts it.
``tests/test_llama_step_oracle.py`` pins these functions against the modules
themselves.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(new residual, normalised) for rows [n, hidden]."""
    x = residual if delta is None else residual + delta
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    return x, weight * y.to(x.dtype)


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., D] with cos/sin broadcastable to it."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return (x * cos) + (rot * sin)


def rope_append(qkv: torch.Tensor, cos_table: torch.Tensor, sin_table: torch.Tensor, seq_lens: torch.Tensor,
                k_cache: torch.Tensor, v_cache: torch.Tensor, n_q_heads: int) -> torch.Tensor:
    """qkv [B, (Hq + 2 Hkv) * D]; caches [B, Hkv, T, D] updated in place at position
    seq_lens - 1; returns the rotated q [B, Hq, D]."""
    b, hkv, _, d = k_cache.shape
    rows = qkv.view(b, n_q_heads + 2 * hkv, d)
    q, k, v = rows[:, :n_q_heads], rows[:, n_q_heads:n_q_heads + hkv], rows[:, n_q_heads + hkv:]
    pos = (seq_lens.to(torch.int64) - 1)
    cos, sin = cos_table[pos][:, None, :], sin_table[pos][:, None, :]
    q_rot, k_rot = rotate(q, cos, sin), rotate(k, cos, sin)
    for i in range(b):
        k_cache[i, :, int(pos[i])] = k_rot[i]
        v_cache[i, :, int(pos[i])] = v[i]
    return q_rot.contiguous()


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    inter = gate_up.shape[-1] // 2
    return torch.nn.functional.silu(gate_up[..., :inter]) * gate_up[..., inter:]


def argmax_first(logits: torch.Tensor) -> torch.Tensor:
    """Lowest index among the row's maxima, int64 [n]."""
    lf = logits.to(torch.float32)
    top = lf.max(dim=-1, keepdim=True).values
    idx = torch.arange(lf.shape[-1]).expand_as(lf)
    return torch.where(lf == top, idx, torch.full_like(idx, lf.shape[-1])).min(dim=-1).values
