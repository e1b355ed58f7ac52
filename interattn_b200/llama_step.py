"""One batched Llama decode step with every non-GEMM op a single fused launch.

The reference decodes through the unmodified Hugging Face model and replaces
only ``eager_attention_forward`` (``condition_block_triton_impl/core.py:1372-1379``);
its captured step (``core.py:190-316``) therefore replays the model's own
element-wise PyTorch kernels - about forty per layer - around the attention hook.
``FusedLlamaStep`` runs the same arithmetic, on the same weights and the same
static cache, as ten launches per layer:

    add+RMSNorm | QKV GEMM | RoPE+cache append | block selection | sparse attention
    | O GEMM | add+RMSNorm | gate/up GEMM | SiLU*up | down GEMM

The GEMMs run on concatenated weights through ``torch.mm`` (cuBLAS) or, on request,
``csrc/skinny_gemm.cu`` (a tcgen05 weight-streaming kernel for batches of at most
32 rows); everything else is ``csrc/llama_step.cu`` and the attention kernels, keeping the
bf16 rounding points of ``transformers.models.llama.modeling_llama`` so that the
fused and the module-by-module step agree up to fp32 summation order.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .ops import _need_cuda, _ptr, _stream


def _bf16(*tensors):
    for t in tensors:
        if t is not None and (t.dtype != torch.bfloat16 or not t.is_contiguous()):
            raise ValueError("contiguous bfloat16 tensors are needed")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> torch.Tensor:
    """``residual += delta`` (skipped for ``None``), then ``out = weight * rmsnorm(residual)``; rows [n, hidden]."""
    _need_cuda(residual)
    _bf16(residual, delta, weight, out)
    n, hidden = residual.shape
    if out.shape != residual.shape or (delta is not None and delta.shape != residual.shape) or weight.numel() != hidden:
        raise ValueError("add_rmsnorm: shapes differ")
    _lib.check(_lib.load().ia_llama_add_rmsnorm(_ptr(residual), _ptr(delta) if delta is not None else None,
                                                _ptr(weight), _ptr(out), n, hidden, float(eps), _stream()))
    return out


def rope_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_lens: torch.Tensor,
                k_cache: torch.Tensor, v_cache: torch.Tensor, q_out: torch.Tensor) -> torch.Tensor:
    """Rotate the q and k heads of ``qkv [B, (Hq + 2 Hkv) * D]`` at position ``seq_lens - 1``, write k and v
    into the static cache tensors ``[B, Hkv, T, D]`` there and q into ``q_out [B, Hq, D]``."""
    _need_cuda(qkv)
    _bf16(qkv, cos, sin, k_cache, v_cache, q_out)
    b, hkv, t, d = (int(x) for x in k_cache.shape)
    hq = int(q_out.shape[1])
    if qkv.shape != (b, (hq + 2 * hkv) * d) or q_out.shape != (b, hq, d) or v_cache.shape != k_cache.shape:
        raise ValueError("rope_append: shapes differ")
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != d:
        raise ValueError("rope_append: cos/sin are [positions, head_dim]")
    if seq_lens.dtype != torch.int32 or seq_lens.numel() != b:
        raise ValueError("rope_append: seq_lens is int32 [batch]")
    _lib.check(_lib.load().ia_llama_rope_append(
        _ptr(qkv), _ptr(cos), _ptr(sin), int(cos.shape[0]), _ptr(seq_lens), _ptr(k_cache), _ptr(v_cache),
        hkv * t * d, t * d, t, _ptr(q_out), b, hq, hkv, d, _stream()))
    return q_out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]``."""
    _need_cuda(gate_up)
    _bf16(gate_up, out)
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2):
        raise ValueError("silu_mul: shapes differ")
    _lib.check(_lib.load().ia_llama_silu_mul(_ptr(gate_up), _ptr(out), n, two_i // 2, _stream()))
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Row-wise arg-max of bf16 ``logits [n, vocab]`` into int64 ``out`` (n elements); lowest index on ties."""
    _need_cuda(logits)
    if logits.dtype != torch.bfloat16 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("argmax: bfloat16 [rows, vocab] with unit inner stride")
    if out.dtype != torch.int64 or out.numel() != logits.shape[0] or not out.is_contiguous():
        raise ValueError("argmax: out is a contiguous int64 tensor with one element per row")
    _lib.check(_lib.load().ia_llama_argmax(_ptr(logits), int(logits.stride(0)), int(logits.shape[0]),
                                           int(logits.shape[1]), _ptr(out), _stream()))
    return out


def gemm_workspace(n: int, device) -> torch.Tensor:
    """Zeroed scratch for ``gemm`` calls with at most ``n`` output columns (one per stream)."""
    size = int(_lib.load().ia_llama_gemm_workspace_bytes(int(n)))
    return torch.zeros(size, dtype=torch.uint8, device=device)


class PackedWeight:
    """A linear layer's weight ``[n, k]`` in the tile order ``gemm`` streams it (packed once)."""

    def __init__(self, w: torch.Tensor):
        _need_cuda(w)
        _bf16(w)
        if w.dim() != 2:
            raise ValueError("a [n, k] weight is needed")
        self.n, self.k = int(w.shape[0]), int(w.shape[1])
        lib = _lib.load()
        self.data = torch.empty(int(lib.ia_llama_gemm_packed_bytes(self.n, self.k)), dtype=torch.uint8,
                                device=w.device)
        _lib.check(lib.ia_llama_gemm_pack(_ptr(w), self.n, self.k, _ptr(self.data), _stream()))


def gemm(x: torch.Tensor, w: PackedWeight, out: torch.Tensor, workspace: torch.Tensor) -> torch.Tensor:
    """``out [m, n] = x [m, k] @ w [n, k].T`` for m <= 32 (``nn.Linear`` without bias)."""
    _need_cuda(x)
    _bf16(x, out)
    m, k = x.shape
    if k != w.k or out.shape != (m, w.n):
        raise ValueError("gemm: shapes differ")
    _lib.check(_lib.load().ia_llama_gemm(_ptr(x), _ptr(w.data), _ptr(out), m, w.n, k, _ptr(workspace),
                                         int(workspace.numel()), _stream()))
    return out


class FusedLlamaStep:
    """Decode step of a Hugging Face ``LlamaForCausalLM`` over its ``StaticCache``.

    ``attention[i]`` is the ``ops.DecodeAttention`` of layer ``i`` (its ``PagedKV`` views the
    cache tensors in place and shares ``seq_lens``).  ``step(tokens)`` consumes ``tokens
    [B, 1]`` int64, writes the next greedy tokens into it and leaves the logits in
    ``self.logits``.  The position of the incoming token is ``seq_lens - 1`` for every
    sequence; the caller advances ``seq_lens`` between steps.  Nothing is allocated inside
    ``step``: it can be captured into a CUDA graph."""

    PROJECTIONS = ("w_qkv", "w_o", "w_gu", "w_down", "lm_head")

    def __init__(self, model, cache, attention, seq_lens: torch.Tensor, cache_len: int,
                 own_gemm: Optional[str] = None):
        # own_gemm: which projections run on this library's GEMM kernel instead of torch.mm
        # (cuBLAS): "all", "none" or a comma-separated subset of PROJECTIONS.  None reads
        # INTERATTN_B200_LLAMA_GEMM, default "none" (see _linear).  Batches above 32 rows always
        # use torch.mm.
        import os
        if own_gemm is None:
            own_gemm = os.environ.get("INTERATTN_B200_LLAMA_GEMM", "none")
        if own_gemm == "all":
            own = set(self.PROJECTIONS)
        elif own_gemm in ("none", "cublas", ""):
            own = set()
        else:
            own = {name.strip() for name in own_gemm.split(",")}
            if not own <= set(self.PROJECTIONS):
                raise ValueError(f"own_gemm names must come from {self.PROJECTIONS}")
        cfg = model.config
        if getattr(cfg, "attention_bias", False) or getattr(cfg, "mlp_bias", False):
            raise ValueError("projection biases are not supported")
        core = model.model
        p0 = core.embed_tokens.weight
        if p0.dtype != torch.bfloat16:
            raise ValueError("a bfloat16 model is needed")
        self.embed = p0
        self.eps = float(cfg.rms_norm_eps)
        self.seq_lens = seq_lens
        self.attention = list(attention)
        self.hq, self.hkv = int(cfg.num_attention_heads), int(cfg.num_key_value_heads)
        self.d = int(getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads)
        self.layers = []
        for i, layer in enumerate(core.layers):
            a, m = layer.self_attn, layer.mlp
            self.layers.append(dict(
                norm1=layer.input_layernorm.weight, norm2=layer.post_attention_layernorm.weight,
                w_qkv=torch.cat([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight], dim=0).contiguous(),
                w_o=a.o_proj.weight, w_gu=torch.cat([m.gate_proj.weight, m.up_proj.weight], dim=0).contiguous(),
                w_down=m.down_proj.weight, k=cache.layers[i].keys, v=cache.layers[i].values))
        self.final_norm = core.norm.weight
        self.lm_head = model.lm_head.weight
        b = int(seq_lens.numel())
        dev, h, inter = p0.device, int(cfg.hidden_size), int(cfg.intermediate_size)
        with torch.no_grad():
            pos = torch.arange(cache_len, device=dev)[None, :]
            cos, sin = core.rotary_emb(torch.empty((1,), dtype=torch.bfloat16, device=dev), pos)
        self.cos, self.sin = cos[0].contiguous(), sin[0].contiguous()
        new = lambda *shape: torch.empty(shape, dtype=torch.bfloat16, device=dev)  # noqa: E731
        self.x, self.h, self.o, self.down = new(b, h), new(b, h), new(b, h), new(b, h)
        self.qkv, self.q = new(b, (self.hq + 2 * self.hkv) * self.d), new(b, self.hq, self.d)
        self.gu, self.act = new(b, 2 * inter), new(b, inter)
        self.logits = new(b, int(self.lm_head.shape[0]))
        self.own_gemm = set() if b > 32 else own
        self.gemm_ws = None
        if self.own_gemm:   # pack the chosen projections once (their concatenated copies are then dropped)
            self.gemm_ws = gemm_workspace(int(self.lm_head.shape[0]), dev)
            for L in self.layers:
                for name in self.own_gemm - {"lm_head"}:
                    L[name] = PackedWeight(L[name])
            if "lm_head" in self.own_gemm:
                self.lm_head = PackedWeight(self.lm_head)
            torch.cuda.synchronize(dev)

    def _linear(self, x: torch.Tensor, w, out: torch.Tensor) -> torch.Tensor:
        """nn.Linear without bias.  Which kernel: back to back on its own, this library's kernel
        matches cuBLAS at 32 rows and passes it on the widest shape (lm head, 6.6 against 6.5
        TB/s); inside the captured Llama-3-8B step its longer start-up and partial-tile tail
        cost about 7 us per projection (7.6 against 6.7 ms per step with every projection on
        it), so cuBLAS is the default and the kernel is opt-in."""
        if isinstance(w, PackedWeight):
            return gemm(x, w, out, self.gemm_ws)
        return torch.mm(x, w.t(), out=out)

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        b = self.x.shape[0]
        torch.index_select(self.embed, 0, tokens.view(-1), out=self.x)
        delta = None
        for L, attn in zip(self.layers, self.attention):
            add_rmsnorm(self.x, delta, L["norm1"], self.eps, self.h)
            self._linear(self.h, L["w_qkv"], self.qkv)
            rope_append(self.qkv, self.cos, self.sin, self.seq_lens, L["k"], L["v"], self.q)
            ctx = attn.step(self.q)
            self._linear(ctx.view(b, self.hq * self.d), L["w_o"], self.o)
            add_rmsnorm(self.x, self.o, L["norm2"], self.eps, self.h)
            self._linear(self.h, L["w_gu"], self.gu)
            silu_mul(self.gu, self.act)
            self._linear(self.act, L["w_down"], self.down)
            delta = self.down
        add_rmsnorm(self.x, delta, self.final_norm, self.eps, self.h)
        self._linear(self.h, self.lm_head, self.logits)
        argmax(self.logits, tokens)
        return tokens
