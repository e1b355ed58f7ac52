"""Batched Llama decode with block-sparse attention in every layer.

The reference generates one sequence at a time (``condition_block_triton_impl/
core.py:73-74``) either eagerly (``core.py:60-187``) or by replaying one
captured decode step (``core.py:190-316``).  This module is the batched form of
the same loop for a Hugging Face ``LlamaForCausalLM``:

* a ``StaticCache`` whose per-layer tensors ``[B, Hkv, T, D]`` (T a multiple of
  16) are addressed *in place* as a paged pool - page ``p`` of kv head ``h``
  starts at ``p * 16 * D + h * T * D``, sequence ``b`` owns the pages
  ``b * Hkv * T / 16 + j`` - so the attention kernels read the cache the model
  writes, no copy;
* prefill with dense SDPA, then block summaries per layer (once), then every
  decode step runs selection + paged sparse attention through
  ``ops.DecodeAttention`` from the attention hook;
* the decode step can be captured into a CUDA graph (token, position and
  sequence lengths live on the device and are advanced inside the graph).

    python -m interattn_b200.llama_decode --preset llama3-8b --batch 32 --prompt 8192 --steps 256

prints one JSON line with decode tokens/s (random-init weights, uniform-random
prompt ids: a throughput harness, not a quality one).
"""

from __future__ import annotations

import argparse
import contextlib
import json
import os
import time
from typing import Optional

import torch

from . import ops
from .reference_api import _sdpa_full, _sdpa_prefill

PAGE = 16


def cache_as_pool(k: torch.Tensor, v: torch.Tensor):
    """[B, Hkv, T, D] contiguous cache tensors -> ([n_pages, Hkv, 16, D] strided views, table int32 [B, T/16])."""
    b, hkv, t, d = (int(x) for x in k.shape)
    if t % PAGE != 0 or not k.is_contiguous() or not v.is_contiguous():
        raise ValueError("the static cache must be contiguous with a length that is a multiple of 16")
    pages_per_seq = t // PAGE
    n_pages = (b - 1) * hkv * pages_per_seq + pages_per_seq
    size, stride = (n_pages, hkv, PAGE, d), (PAGE * d, t * d, d, 1)
    table = (torch.arange(b, device=k.device, dtype=torch.int32)[:, None] * (hkv * pages_per_seq)
             + torch.arange(pages_per_seq, device=k.device, dtype=torch.int32)[None, :]).contiguous()
    return torch.as_strided(k, size, stride), torch.as_strided(v, size, stride), table


class BatchedBlockSparseDecoder:
    """Attention hook for batched single-token decode over a static cache."""

    def __init__(self, *, prompt_len: int, block_size: int = 64, top_k: Optional[int] = 64,
                 eps: Optional[float] = None, rep_mode: str = "sparse_only", full_attention_layers: int = 0,
                 device="cuda", reblock: bool = False, max_len: Optional[int] = None):
        # reblock: whenever the generated suffix has grown by a whole block, that block joins
        # the summarised prefix (ia_update_summaries) - the suffix stays shorter than a block
        # instead of growing with the generation.  The reference never re-blocks its suffix.
        self.reblock, self.max_len = bool(reblock), int(max_len or prompt_len)
        self.cur_prefix = int(prompt_len)
        self.prompt_len, self.block_size = int(prompt_len), int(block_size)
        self.top_k, self.eps, self.rep_mode = top_k, eps, rep_mode
        self.full_attention_layers = int(full_attention_layers)
        self.layers = {}
        self.device = torch.device(device)
        self.prefix_lens = None
        self.seq_lens = None      # shared by all layers, advanced once per step on the device

    def _layer(self, idx, key, value, n_q_heads):
        st = self.layers.get(idx)
        if st is None:
            b = int(key.shape[0])
            if self.prefix_lens is None:
                self.prefix_lens = torch.full((b,), self.prompt_len, dtype=torch.int32, device=key.device)
                self.seq_lens = torch.full((b,), self.prompt_len + 1, dtype=torch.int32, device=key.device)
            k_pool, v_pool, table = cache_as_pool(key, value)
            kv = ops.PagedKV(k_pool, v_pool, table, self.prefix_lens, self.seq_lens)
            span = self.max_len if self.reblock else self.prompt_len
            nb = max(1, (span + self.block_size - 1) // self.block_size)
            summ = ops.build_summaries(kv, self.block_size, max_blocks=nb)
            kw = dict(top_k=self.top_k) if self.top_k is not None else dict(eps=self.eps)
            st = ops.DecodeAttention(kv, summ, n_q_heads, rep_mode=self.rep_mode, **kw)
            self.layers[idx] = st
        return st

    def absorb_full_blocks(self, pos: int) -> None:
        """Before decoding the token at cache position ``pos``: move every complete block of
        generated tokens into the summarised prefix (all layers).  Runs between steps."""
        if not self.reblock or self.prefix_lens is None:
            return
        grown = (int(pos) - self.cur_prefix) // self.block_size * self.block_size
        if grown <= 0:
            return
        first = torch.full_like(self.prefix_lens, self.cur_prefix // self.block_size)
        self.cur_prefix += grown
        self.prefix_lens.fill_(self.cur_prefix)
        for st in self.layers.values():
            ops.build_summaries(st.kv, self.block_size, out=st.summ, first_blocks=first)

    def set_position(self, pos: int) -> None:
        """Eager loops: the token being decoded sits at cache position ``pos``."""
        if self.seq_lens is not None:
            self.seq_lens.fill_(int(pos) + 1)
        self._pos = int(pos)

    def hook(self, module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
        if query.shape[2] != 1:
            return _sdpa_prefill(query, key, value, scaling)
        idx = int(module.layer_idx)
        if idx < self.full_attention_layers:
            visible = self._pos + 1
            return _sdpa_full(query, key[:, :, :visible], value[:, :, :visible], scaling)
        b, hq, _, d = query.shape
        step = self._layer(idx, key, value, int(hq))
        out = step.step(query.reshape(b, hq, d).contiguous())
        return out.unsqueeze(1), None


@contextlib.contextmanager
def _decode_patches(decoder):
    """Install the hook and skip Hugging Face's causal-mask construction (every decode
    layer ignores the mask; building it costs a host round trip per step - the reference
    stubs it for the same reason, core.py:1356-1369)."""
    from transformers.models.llama import modeling_llama
    saved = modeling_llama.eager_attention_forward, modeling_llama.create_causal_mask
    modeling_llama.eager_attention_forward = decoder.hook
    modeling_llama.create_causal_mask = lambda *a, **k: None
    try:
        yield
    finally:
        modeling_llama.eager_attention_forward, modeling_llama.create_causal_mask = saved


@contextlib.contextmanager
def _attn_impl(model, name):
    old = model.config._attn_implementation
    model.config._attn_implementation = name
    try:
        yield
    finally:
        model.config._attn_implementation = old


def generate_batched(model, input_ids: torch.Tensor, max_new_tokens: int, *, block_size=64, top_k=64, eps=None,
                     rep_mode="sparse_only", full_attention_layers=0, cuda_graph=False, reblock=False,
                     fused_step=False, force_tokens=None, collect_logits=False, own_gemm=None):
    """Greedy batched generation.  Returns (tokens [B, max_new_tokens], stats dict with timings).

    fused_step: decode through ``llama_step.FusedLlamaStep`` (fused element-wise kernels and
    concatenated projection weights) instead of the Hugging Face modules around the hook.
    force_tokens [B, max_new_tokens]: feed these tokens instead of the greedy ones (teacher
    forcing, for comparing two decode paths step by step); collect_logits: keep every decode
    step's logits in ``stats["logits"]`` ([steps, B, vocab]).  Neither works with cuda_graph.
    own_gemm: passed to ``FusedLlamaStep`` (which projections use this library's GEMM kernel)."""
    from transformers import StaticCache
    b, prompt_len = (int(x) for x in input_ids.shape)
    dev = input_ids.device
    cache_len = (prompt_len + max_new_tokens + PAGE - 1) // PAGE * PAGE
    cache = StaticCache(config=model.config, max_cache_len=cache_len)
    stats = {}
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with torch.no_grad(), _attn_impl(model, "sdpa"):
        out = model(input_ids=input_ids, past_key_values=cache, use_cache=True, logits_to_keep=1,
                    cache_position=torch.arange(prompt_len, device=dev))
    tok = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)
    torch.cuda.synchronize()
    stats["prefill_s"] = time.perf_counter() - t0
    tokens = torch.empty((b, max_new_tokens), dtype=tok.dtype, device=dev)
    tokens[:, 0:1] = tok
    decoder = BatchedBlockSparseDecoder(prompt_len=prompt_len, block_size=block_size, top_k=top_k, eps=eps,
                                        rep_mode=rep_mode, full_attention_layers=full_attention_layers, device=dev,
                                        reblock=reblock, max_len=cache_len)
    tok_buf = tok.clone()
    pos_buf = torch.tensor([prompt_len], device=dev, dtype=torch.long)
    if cuda_graph and (force_tokens is not None or collect_logits):
        raise ValueError("force_tokens / collect_logits need the eager loop")
    if force_tokens is not None:
        tokens[:, 0:1] = force_tokens[:, 0:1]
        tok_buf.copy_(force_tokens[:, 0:1])
    kept_logits = []
    fused = None
    if fused_step:
        if full_attention_layers > 0:
            raise ValueError("the fused step needs every layer on the sparse path")
        from .llama_step import FusedLlamaStep
        n_q_heads = int(model.config.num_attention_heads)
        attention = [decoder._layer(i, cache.layers[i].keys, cache.layers[i].values, n_q_heads)
                     for i in range(int(model.config.num_hidden_layers))]
        fused = FusedLlamaStep(model, cache, attention, decoder.seq_lens, cache_len, own_gemm=own_gemm)

    def one_step():
        if fused is not None:
            fused.step(tok_buf)
            logits = fused.logits
        else:
            o = model(input_ids=tok_buf, past_key_values=cache, use_cache=True, logits_to_keep=1,
                      cache_position=pos_buf)
            logits = o.logits[:, -1, :]
            tok_buf.copy_(logits.argmax(dim=-1, keepdim=True))
        if collect_logits:
            kept_logits.append(logits.clone())

    def keep_token(i):
        if force_tokens is not None:
            tok_buf.copy_(force_tokens[:, i:i + 1])
        tokens[:, i:i + 1] = tok_buf

    n_decode = max_new_tokens - 1
    nvtx_steps = os.environ.get("INTERATTN_B200_NVTX", "") == "1"
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.no_grad(), _attn_impl(model, "eager"), _decode_patches(decoder):
        done = 0
        warm = min(3 if cuda_graph else 1, n_decode)   # builds the summaries and every workspace
        for _ in range(warm):
            decoder.set_position(prompt_len + done)
            one_step()
            done += 1
            keep_token(done)
            pos_buf.add_(1)
        torch.cuda.synchronize()
        stats["summaries_and_warmup_steps"] = warm
        graph = None
        if cuda_graph and done < n_decode:
            if full_attention_layers > 0:
                raise ValueError("the captured step needs every layer on the sparse path")
            graph = torch.cuda.CUDAGraph()
            decoder.seq_lens.fill_(prompt_len + done + 1)
            with torch.cuda.graph(graph):
                one_step()
                pos_buf.add_(1)
                decoder.seq_lens.add_(1)
            # the capture ran nothing: positions are still those of step `done`
        ev0.record()
        timed = 0
        while done < n_decode:
            decoder.absorb_full_blocks(prompt_len + done)
            if graph is not None:
                graph.replay()
            else:
                decoder.set_position(prompt_len + done)
                if nvtx_steps:  # a named range per eager step, for a profiler's range filter
                    torch.cuda.nvtx.range_push(f"decode_step_{timed}")
                one_step()
                if nvtx_steps:
                    torch.cuda.nvtx.range_pop()
                pos_buf.add_(1)
            done += 1
            timed += 1
            keep_token(done)
        ev1.record()
        torch.cuda.synchronize()
    stats["decode_steps_timed"] = timed
    stats["decode_s"] = ev0.elapsed_time(ev1) * 1e-3
    stats["tokens_per_s"] = b * timed / stats["decode_s"] if timed else float("nan")
    stats["cuda_graph"] = graph is not None
    stats["fused_step"] = fused is not None
    if collect_logits:
        stats["logits"] = torch.stack(kept_logits) if kept_logits else None
    return tokens, stats


PRESETS = {
    # Llama-3-8B architecture
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=500000.0,
                      max_position_embeddings=16384),
    "tiny": dict(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                 num_attention_heads=8, num_key_value_heads=2, head_dim=64, rope_theta=500000.0,
                 max_position_embeddings=4096),
}


def build_random_llama(preset: str, n_layers: Optional[int] = None, dtype=torch.bfloat16, device="cuda", seed=0):
    from transformers import LlamaConfig, LlamaForCausalLM
    kw = dict(PRESETS[preset])
    if n_layers is not None:
        kw["num_hidden_layers"] = int(n_layers)
    cfg = LlamaConfig(attn_implementation="eager", **kw)
    torch.manual_seed(seed)
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    return model.eval()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="llama3-8b", choices=sorted(PRESETS))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--block", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=64)
    ap.add_argument("--rep-mode", default="sparse_only", choices=["sparse_only", "hybrid"])
    ap.add_argument("--cuda-graph", action="store_true")
    ap.add_argument("--reblock", action="store_true", help="summarise generated tokens block by block")
    ap.add_argument("--fused-step", action="store_true",
                    help="fused element-wise kernels and concatenated projections instead of the model's modules")
    ap.add_argument("--full-attention-layers", type=int, default=0,
                    help="layers below this index decode with dense SDPA (all layers: the dense baseline)")
    a = ap.parse_args()
    model = build_random_llama(a.preset, a.layers)
    g = torch.Generator(device="cuda").manual_seed(0)
    ids = torch.randint(0, model.config.vocab_size, (a.batch, a.prompt), generator=g, device="cuda")
    tokens, stats = generate_batched(model, ids, a.steps, block_size=a.block, top_k=a.top_k, rep_mode=a.rep_mode,
                                     cuda_graph=a.cuda_graph, full_attention_layers=a.full_attention_layers,
                                     reblock=a.reblock, fused_step=a.fused_step)
    line = {"metric": "llama_decode_tokens_per_s", "value": stats["tokens_per_s"], "unit": "tok/s",
            "config": {"preset": a.preset, "layers": model.config.num_hidden_layers, "batch": a.batch,
                       "prompt": a.prompt, "new_tokens": a.steps, "block": a.block, "top_k": a.top_k,
                       "rep_mode": a.rep_mode, "cuda_graph": stats["cuda_graph"], "dtype": "bf16",
                       "full_attention_layers": a.full_attention_layers, "reblock": a.reblock, "fused_step": a.fused_step,
                       "weights": "random init", "data": "uniform random token ids"},
            "ms_per_decode_step": 1e3 * stats["decode_s"] / max(stats["decode_steps_timed"], 1),
            "prefill_s": stats["prefill_s"], "decode_steps_timed": stats["decode_steps_timed"]}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
