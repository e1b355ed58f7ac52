"""The two caller-side seams of the reference, extended by one entry each.

* ``generate_with_method`` dispatches on ``method.kind``
  (``condition_block_gen/methods/generate.py:17-82``); new kinds are added to the
  ``--method`` choices (``methods/config.py:77-92``) and to ``LOCAL_PATCH_METHODS``
  (``condition_block_gen/common.py:18-25``, which forces the eager attention
  implementation the hook needs).  ``METHOD_KIND`` = ``"condition_block_b200"`` is
  that new kind: ``generate_with_method`` here handles it and hands every other kind
  to the dispatcher it wraps; ``register_method_kind`` installs it into the
  reference's modules when they are importable.
* ``attention_factory.create_attention(config, layer_index)`` builds the attention
  module of the nanoGPT stack from ``config.attn.type`` and raises
  ``NotImplementedError`` for unknown types (``attention_factory.py:17-48``); the
  module contract is ``forward(x[B, T, C]) -> y[B, T, C]`` (``model.py:230-231,
  358-366``).  ``create_attention`` here adds the type ``"condition_block_b200"``:
  a causal self-attention module that prefills densely and decodes single tokens
  through the block-sparse operator over its own paged cache.  Nothing on the Llama
  path goes through this seam; it exists so that a nanoGPT config can name the op.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
from torch import nn

from . import ops

METHOD_KIND = "condition_block_b200"
ATTN_TYPE = "condition_block_b200"
PAGE = 16


# --------------------------------------------------------------------------
# generation-method seam
# --------------------------------------------------------------------------

def generate_with_method(model, tokenizer, input_ids, attention_mask, method, device, dataset=None,
                         fallback: Optional[Callable] = None):
    """``generate_with_method`` of the reference with the kind ``condition_block_b200``.

    Batch 1 goes through ``reference_api.generate_condition_block_cached`` (the reference's
    own loop structure); larger batches through ``llama_decode.generate_batched``.  The
    method object is the reference's ``GenerationMethod`` (``methods/config.py:4-31``);
    optional extra attributes ``condition_top_k``, ``condition_rep_mode``,
    ``condition_cuda_graph`` and ``condition_fused_step`` select the top-k rule, the
    value-side mode and the batched loop's options.  Other kinds go to ``fallback`` (the
    dispatcher being wrapped) or raise ``NotImplementedError``."""
    if getattr(method, "kind", None) != METHOD_KIND:
        if fallback is None:
            raise NotImplementedError(f"method kind {getattr(method, 'kind', None)!r} is not handled here")
        return fallback(model, tokenizer, input_ids, attention_mask, method, device, dataset)
    if input_ids.shape[0] == 1:
        from .reference_api import generate_condition_block_cached
        return generate_condition_block_cached(model=model, tokenizer=tokenizer, input_ids=input_ids,
                                               attention_mask=attention_mask, method=method, device=device,
                                               dataset=dataset)
    from .llama_decode import generate_batched
    top_k = getattr(method, "condition_top_k", None)
    tokens, stats = generate_batched(
        model, input_ids.to(device), int(method.max_new_tokens),
        block_size=int(method.condition_block_size or 64), top_k=top_k,
        eps=None if top_k is not None else float(method.condition_eps),
        rep_mode=getattr(method, "condition_rep_mode", "hybrid"),
        full_attention_layers=int(method.full_attention_layers),
        cuda_graph=bool(getattr(method, "condition_cuda_graph", False)),
        fused_step=bool(getattr(method, "condition_fused_step", False)))
    meta = {"method": METHOD_KIND, "batched": True, "decode_tokens_per_s": stats["tokens_per_s"],
            "prefill_s": stats["prefill_s"], "cuda_graph": stats["cuda_graph"], "fused_step": stats["fused_step"]}
    return tokens, meta


def register_method_kind(generate_module=None, common_module=None, parser=None) -> None:
    """Install the kind into the reference's own modules (each argument optional):
    ``generate_module.generate_with_method`` is wrapped, ``common_module.LOCAL_PATCH_METHODS``
    gains the kind, and the ``--method`` argument of ``parser`` accepts it."""
    if generate_module is not None:
        original = generate_module.generate_with_method
        if not getattr(original, "_b200_wrapped", False):
            def dispatch(model, tokenizer, input_ids, attention_mask, method, device, dataset=None):
                return generate_with_method(model, tokenizer, input_ids, attention_mask, method, device, dataset,
                                            fallback=original)
            dispatch._b200_wrapped = True
            generate_module.generate_with_method = dispatch
    if common_module is not None:
        common_module.LOCAL_PATCH_METHODS.add(METHOD_KIND)
    if parser is not None:
        for action in parser._actions:
            if "--method" in action.option_strings and action.choices is not None and METHOD_KIND not in action.choices:
                action.choices = list(action.choices) + [METHOD_KIND]


# --------------------------------------------------------------------------
# attention-factory seam
# --------------------------------------------------------------------------

class ConditionBlockSelfAttention(nn.Module):
    """Causal self-attention with the nanoGPT module contract and a paged KV cache.

    ``forward(x[B, T, C])``: T > 1 is a prefill - dense causal attention over the T
    tokens, which also (re)fills the cache and builds the block summaries; T == 1 decodes
    one token per sequence against the cache through the block-sparse operator (the new
    token is appended first, as the Hugging Face hook sees it).  Config fields: ``n_embd``,
    ``n_head``, optional ``n_kv_head`` (GQA), ``bias``, ``block_size`` (context length, the
    cache capacity), and under ``attn``: ``select_block`` (64), ``top_k`` (64) or ``eps``,
    ``rep_mode`` ("sparse_only").  Inference only: the operator has no backward pass."""

    def __init__(self, config, layer_index=None):
        super().__init__()
        a = config.attn
        self.n_head = int(config.n_head)
        self.n_kv_head = int(getattr(config, "n_kv_head", None) or self.n_head)
        if config.n_embd % self.n_head or self.n_head % self.n_kv_head:
            raise ValueError("n_embd must divide into n_head heads and n_head into n_kv_head groups")
        self.head_dim = config.n_embd // self.n_head
        bias = bool(getattr(config, "bias", False))
        self.c_attn = nn.Linear(config.n_embd, (self.n_head + 2 * self.n_kv_head) * self.head_dim, bias=bias)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=bias)
        self.layer = layer_index
        self.capacity = (int(config.block_size) + PAGE - 1) // PAGE * PAGE
        self.select_block = int(getattr(a, "select_block", 64))
        self.top_k = getattr(a, "top_k", 64)
        self.eps = getattr(a, "eps", None)
        self.rep_mode = getattr(a, "rep_mode", "sparse_only")
        self._state = None

    def _split(self, x):
        b, t, _ = x.shape
        qkv = self.c_attn(x)
        hq, hkv, d = self.n_head, self.n_kv_head, self.head_dim
        q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
        return (q.view(b, t, hq, d).transpose(1, 2), k.view(b, t, hkv, d).transpose(1, 2),
                v.view(b, t, hkv, d).transpose(1, 2))

    def _prefill(self, x):
        b, t, c = x.shape
        if t > self.capacity:
            raise ValueError(f"{t} tokens exceed the context length {self.capacity}")
        q, k, v = self._split(x)
        y = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True,
                                                             enable_gqa=self.n_kv_head != self.n_head)
        hkv, d, dev = self.n_kv_head, self.head_dim, x.device
        k_cache = torch.zeros((b, hkv, self.capacity, d), dtype=x.dtype, device=dev)
        v_cache = torch.zeros_like(k_cache)
        k_cache[:, :, :t], v_cache[:, :, :t] = k.detach(), v.detach()
        from .llama_decode import cache_as_pool
        k_pool, v_pool, table = cache_as_pool(k_cache, v_cache)
        prefix = torch.full((b,), t, dtype=torch.int32, device=dev)
        kv = ops.PagedKV(k_pool, v_pool, table, prefix, prefix.clone())
        nb = max(1, (self.capacity + self.select_block - 1) // self.select_block)
        summ = ops.build_summaries(kv, self.select_block, max_blocks=nb)
        kw = dict(top_k=int(self.top_k)) if self.eps is None else dict(eps=float(self.eps))
        step = ops.DecodeAttention(kv, summ, self.n_head, rep_mode=self.rep_mode, **kw)
        self._state = dict(k=k_cache, v=v_cache, kv=kv, step=step, length=t)
        return self.c_proj(y.transpose(1, 2).reshape(b, t, c))

    def _decode(self, x):
        st = self._state
        if st is None:
            raise ValueError("decode before prefill: call forward with the prompt (T > 1) first")
        b, _, c = x.shape
        pos = st["length"]
        if pos >= self.capacity:
            raise ValueError("the cache is full")
        q, k, v = self._split(x)
        st["k"][:, :, pos], st["v"][:, :, pos] = k[:, :, 0].detach(), v[:, :, 0].detach()
        st["length"] = pos + 1
        st["kv"].seq_lens.fill_(pos + 1)
        out = st["step"].step(q[:, :, 0].contiguous())          # [B, Hq, D]
        return self.c_proj(out.reshape(b, 1, c).to(x.dtype))

    def reset_cache(self):
        self._state = None

    @torch.no_grad()
    def forward(self, x, *args, **kwargs):
        if x.dim() != 3:
            raise ValueError("x is [batch, tokens, n_embd]")
        return self._decode(x) if x.shape[1] == 1 else self._prefill(x)


def create_attention(config, layer_index=None, fallback: Optional[Callable] = None):
    """``attention_factory.create_attention`` with the type ``condition_block_b200``; other
    types go to ``fallback`` (the factory being wrapped) or raise ``NotImplementedError``
    with the reference's message."""
    kind = config.attn.type
    if kind == ATTN_TYPE:
        return ConditionBlockSelfAttention(config, layer_index=layer_index)
    if fallback is not None:
        return fallback(config, layer_index)
    raise NotImplementedError(f"Attention type '{kind}' is not implemented")
