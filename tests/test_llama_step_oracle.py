"""The CPU restatement of the Llama step's element-wise ops against the Hugging Face
modules it restates (transformers' modeling_llama / cache_utils), bit for bit."""

import pytest
import torch

from oracle import llama_step_oracle as lo

transformers = pytest.importorskip("transformers")
from transformers import LlamaConfig, StaticCache  # noqa: E402
from transformers.models.llama import modeling_llama as ml  # noqa: E402


def _cfg():
    return LlamaConfig(vocab_size=64, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=500000.0,
                       max_position_embeddings=512)


def test_add_rmsnorm_is_the_module():
    g = torch.Generator().manual_seed(0)
    norm = ml.LlamaRMSNorm(256, eps=1e-5).to(torch.bfloat16)
    norm.weight.data = torch.randn(256, generator=g).to(torch.bfloat16)
    res = torch.randn(5, 256, generator=g).to(torch.bfloat16)
    delta = torch.randn(5, 256, generator=g).to(torch.bfloat16)
    x, y = lo.add_rmsnorm(res, delta, norm.weight.data, 1e-5)
    assert torch.equal(x, res + delta)
    assert torch.equal(y, norm(res + delta))
    x0, y0 = lo.add_rmsnorm(res, None, norm.weight.data, 1e-5)
    assert torch.equal(x0, res) and torch.equal(y0, norm(res))


def test_rope_append_is_the_module_and_the_cache_update():
    cfg = _cfg()
    g = torch.Generator().manual_seed(1)
    b, hq, hkv, d, t = 3, 4, 2, 64, 48
    rot = ml.LlamaRotaryEmbedding(cfg)
    cos_t, sin_t = rot(torch.empty(1, dtype=torch.bfloat16), torch.arange(t)[None])
    cos_t, sin_t = cos_t[0], sin_t[0]
    qkv = torch.randn(b, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16)
    seq_lens = torch.tensor([7, 33, 48], dtype=torch.int32)
    k_cache = torch.randn(b, hkv, t, d, generator=g).to(torch.bfloat16)
    v_cache = torch.randn(b, hkv, t, d, generator=g).to(torch.bfloat16)
    k_ref, v_ref = k_cache.clone(), v_cache.clone()
    q_out = lo.rope_append(qkv, cos_t, sin_t, seq_lens, k_cache, v_cache, hq)
    rows = qkv.view(b, hq + 2 * hkv, d)
    for i in range(b):   # the module path, one sequence at a time (its positions differ per sequence)
        pos = torch.tensor([int(seq_lens[i]) - 1])
        cos, sin = rot(torch.empty(1, dtype=torch.bfloat16), pos[None])
        q = rows[i:i + 1, :hq, None, :]                  # [1, Hq, 1, D]
        k = rows[i:i + 1, hq:hq + hkv, None, :]
        v = rows[i:i + 1, hq + hkv:, None, :]
        q_rot, k_rot = ml.apply_rotary_pos_emb(q, k, cos, sin)
        assert torch.equal(q_out[i], q_rot[0, :, 0])
        n = int(pos)                                     # rows already in the cache
        cache = StaticCache(config=cfg, max_cache_len=t)
        cache.update(k_ref[i:i + 1, :, :n].clone(), v_ref[i:i + 1, :, :n].clone(), 0)
        cache.update(k_rot, v, 0)                        # the layer appends at its own running length
        assert torch.equal(k_cache[i, :, :n + 1], cache.layers[0].keys[0, :, :n + 1])
        assert torch.equal(v_cache[i, :, :n + 1], cache.layers[0].values[0, :, :n + 1])
        assert torch.equal(k_cache[i, :, n + 1:], k_ref[i, :, n + 1:])
        assert torch.equal(v_cache[i, :, n + 1:], v_ref[i, :, n + 1:])


def test_silu_mul_is_the_mlp_expression():
    cfg = _cfg()
    mlp = ml.LlamaMLP(cfg).to(torch.bfloat16)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(6, 256, generator=g).to(torch.bfloat16)
    gate, up = mlp.gate_proj(x), mlp.up_proj(x)
    want = mlp.act_fn(gate) * up
    assert torch.equal(lo.silu_mul(torch.cat([gate, up], dim=-1)), want)
    assert torch.equal(mlp.down_proj(want), mlp(x))


def test_argmax_first_breaks_ties_low():
    logits = torch.tensor([[0.0, 3.0, 3.0, -1.0], [2.0, 2.0, 2.0, 2.0], [-5.0, -4.0, -3.0, -3.0]]).to(torch.bfloat16)
    assert lo.argmax_first(logits).tolist() == [1, 0, 2]
