"""The reference-named operators (interattn_b200.reference_api) on the GPU.

Cases follow the reference's own sanity scripts: Hkv 8 / G 4 / D 128 bf16 with
prompt 4096 and 4099 (padded tail), suffix 1 and 33, eps 0 (every block) and
1e6 (none)  - condition_block_triton_impl/block64_experiment/sanity.py:25-104 -
a strided (non-contiguous) cache view against its contiguous copy
(condition_block_triton_impl/README.md:531-536), and the attention hook inside
a small random Llama.  The checker is the CPU oracle.
"""

import pytest
import torch

from oracle import condition_block_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _api():
    from interattn_b200 import reference_api
    return reference_api


def _cache(hkv, total, d, dtype, seed, spare=7):
    """K/V laid out like a static Hugging Face cache: [Hkv, T_alloc, D] with T_alloc > T."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn((hkv, total + spare, d), generator=g).to(dtype)
    v = torch.randn((hkv, total + spare, d), generator=g).to(dtype)
    return k, v


def _oracle_step(q_grouped, k_all, v_all, prompt_len, block, *, eps=None, top_k=None, rep_mode="hybrid", summ=None):
    qg = q_grouped[:, :, 0].float().cpu()
    k_all, v_all = k_all.cpu(), v_all.cpu()
    if summ is None:
        summ = orc.block_summaries(k_all[:, :prompt_len], v_all[:, :prompt_len], block, storage="mixed")
    terms = orc.condition_terms(qg, summ)
    if top_k is not None:
        _, mask = orc.select_topk(terms["score"], summ.counts, top_k)
    else:
        mask = orc.select_threshold(terms["score"], summ.counts, eps)
    out = orc.decode_attention(qg, k_all, v_all, prompt_len, block, mask, rep_mode=rep_mode,
                               z=terms["z"], v_bar=summ.v_bar)
    return out, mask, terms, summ


def test_build_prompt_blocks_keys_values_and_strided_view():
    api = _api()
    hkv, d, block, length = 4, 128, 64, 1000
    k, v = _cache(hkv, length, d, torch.bfloat16, 1)
    kd, vd = k.to(DEV), v.to(DEV)
    prefix = api._build_prompt_blocks(kd[:, :length], vd[:, :length], block)      # strided view of the cache
    dense = api._build_prompt_blocks(kd[:, :length].contiguous(), vd[:, :length].contiguous(), block)
    want = orc.block_summaries(k[:, :length], v[:, :length], block)
    nb = want.n_blocks
    for key in ("k_block_attn", "v_block_attn", "token_idx", "valid_token", "k_bar", "v_bar", "k_max", "k_min",
                "v_norm_max", "v_norm_all", "block_valid_counts"):
        assert key in prefix
    assert prefix["k_block_attn"].shape == (hkv, nb, block, d)
    assert prefix["block_valid_counts"].dtype == torch.int64
    assert torch.equal(prefix["block_valid_counts"].cpu(), want.counts)
    assert torch.equal(prefix["k_max"].cpu().float(), want.k_max.float())
    assert torch.equal(prefix["k_min"].cpu().float(), want.k_min.float())
    assert torch.allclose(prefix["k_bar"].cpu(), want.k_bar, rtol=2e-6, atol=2e-6)
    assert torch.allclose(prefix["v_norm_max"].cpu(), want.v_norm_max, rtol=2e-6, atol=0)
    assert torch.allclose(prefix["v_norm_all"].cpu(), want.v_norm_max.amax(dim=-1), rtol=2e-6, atol=0)
    assert prefix["k_max"].dtype == torch.float32                    # reference default: fp32 summaries
    # the padded tail of the blocked view is zero, the body is the cache itself
    assert torch.equal(prefix["k_block_attn"].reshape(hkv, -1, d)[:, :length].cpu(), k[:, :length])
    assert bool((prefix["k_block_attn"].reshape(hkv, -1, d)[:, length:] == 0).all())
    # a strided view and its contiguous copy give bit-identical summaries
    for key in ("k_bar", "v_bar", "k_max", "k_min", "v_norm_max"):
        assert torch.equal(prefix[key], dense[key])


def test_select_and_stats_shims():
    api = _api()
    hkv, g, d, block, length = 4, 4, 128, 64, 1500
    k, v = _cache(hkv, length, d, torch.bfloat16, 2)
    kd, vd = k.to(DEV), v.to(DEV)
    prefix = api._build_prompt_blocks(kd[:, :length], vd[:, :length], block)
    q = torch.randn((hkv, g, 1, d), generator=torch.Generator().manual_seed(3)).bfloat16()
    _, mask0, terms, summ = _oracle_step(q, k[:, :length], v[:, :length], length, block, eps=0.0)
    eps = float(torch.quantile(terms["score"].flatten(), 0.7))
    selected, z_logits, v_bar, size, exists = api._select_prompt_blocks(q.to(DEV), prefix, eps)
    nb = summ.n_blocks
    assert selected.shape == (hkv, g, 1, nb) and z_logits.shape == (hkv, g, 1, nb)
    assert v_bar.shape == (hkv, g, 1, nb, d) and size.shape == (1, nb) and bool(exists.all())
    want = orc.select_threshold(terms["score"], summ.counts, eps)
    diff = (selected[:, 0, 0].cpu() ^ want)
    near = (terms["score"] - eps).abs() <= 3e-4 * terms["score"].abs() + 1e-8
    assert bool((~diff | near).all())
    assert torch.allclose(z_logits[:, :, 0].cpu(), terms["z"], rtol=1e-5, atol=1e-5)

    qq, s_cache, d_cache, partial, glob, n_blocks, n_chunks = api._run_condition_block_selection_stats(
        q.to(DEV), prefix, workspace={})
    assert (n_blocks, n_chunks) == (nb, 1) and partial.shape == (4, hkv * g, 1) and glob.shape == (4, hkv * g)
    assert torch.allclose(s_cache.cpu().reshape(hkv, g, nb), terms["s"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(d_cache.cpu().reshape(hkv, g, nb), terms["delta"], rtol=1e-4, atol=1e-5)
    z = terms["z"].reshape(hkv * g, nb).double()
    lse_z = torch.logsumexp(z, dim=1)
    lse_c = torch.logsumexp(z + torch.log(torch.cosh(terms["delta"].reshape(hkv * g, nb).double())), dim=1)
    gl = glob.cpu().double()
    assert torch.allclose(gl[0] + torch.log(gl[1]), lse_z, rtol=1e-5, atol=1e-5)
    assert torch.allclose(gl[2] + torch.log(gl[3]), lse_c, rtol=1e-5, atol=1e-4)
    # the term1-softmax variant: same s / delta, the second normaliser pair sums e^{z + delta}
    _, s2, d2, _, glob2, _, _ = api._run_condition_block_selection_stats(q.to(DEV), prefix, term1_mass_exp=True)
    assert torch.equal(s2, s_cache) and torch.equal(d2, d_cache)
    gl2 = glob2.cpu().double()
    lse_e = torch.logsumexp(z + terms["delta"].reshape(hkv * g, nb).double(), dim=1)
    assert torch.allclose(gl2[2] + torch.log(gl2[3]), lse_e, rtol=1e-5, atol=1e-4)
    with pytest.raises(ValueError):
        api._select_prompt_blocks(q.to(DEV), {"k_bar": None}, 0.1)


def test_packed_bounds_switch_of_the_reference(monkeypatch):
    """CONDITION_BLOCK_TMA_BOUNDS=1 (IMPL/core.py:490-499): the prefix carries ``k_bounds`` = stack((k_max, k_min),
    -1).flatten(2) and k_max / k_min become views into it; selection and the fused decode give what they give
    from two arrays."""
    api = _api()
    hkv, g, d, block, length = 4, 4, 128, 64, 1500
    k, v = _cache(hkv, length + 8, d, torch.bfloat16, 2)
    kd, vd = k.to(DEV), v.to(DEV)
    q = torch.randn((hkv, g, 1, d), generator=torch.Generator().manual_seed(3)).bfloat16().to(DEV)
    monkeypatch.setenv("CONDITION_BLOCK_MIXED_SUMMARIES", "1")
    plain = api._build_prompt_blocks(kd[:, :length], vd[:, :length], block)
    monkeypatch.setenv("CONDITION_BLOCK_TMA_BOUNDS", "1")
    packed = api._build_prompt_blocks(kd[:, :length], vd[:, :length], block)
    assert "k_bounds" in packed and "k_bounds" not in plain
    want = torch.stack((plain["k_max"], plain["k_min"]), dim=-1).flatten(2)
    assert torch.equal(packed["k_bounds"], want)
    assert torch.equal(packed["k_max"], plain["k_max"]) and torch.equal(packed["k_min"], plain["k_min"])
    assert packed["k_max"].data_ptr() == packed["k_bounds"].data_ptr()  # views, no duplicate storage
    eps = 1e-3
    sel_p = api._select_prompt_blocks(q, packed, eps)[0]
    sel = api._select_prompt_blocks(q, plain, eps)[0]
    assert torch.equal(sel_p, sel)
    n_suffix = torch.tensor(5, device=DEV, dtype=torch.int32)
    outs = [api._condition_block_decode_output_fused_triton(
        q_grouped=q, prompt_prefix=prefix, k_suffix=kd[:, length:], v_suffix=vd[:, length:], suffix_len_dev=n_suffix,
        eps=eps, page_size=block, store_selected=True, output_dtype=torch.bfloat16, workspace={})
        for prefix in (packed, plain)]
    torch.cuda.synchronize()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


SANITY = [(4096, 1, 0.0), (4099, 33, 0.0), (4096, 1, 1e6), (4099, 33, 1e6)]


@pytest.mark.parametrize("prompt_len,suffix_len,eps", SANITY)
@pytest.mark.parametrize("suffix_is_view", [True, False])
def test_fused_decode_sanity_cases(prompt_len, suffix_len, eps, suffix_is_view):
    api = _api()
    hkv, g, d, block = 8, 4, 128, 64
    k, v = _cache(hkv, prompt_len + suffix_len, d, torch.bfloat16, 1234, spare=40)
    kd, vd = k.to(DEV), v.to(DEV)
    q = torch.randn((hkv, g, 1, d), generator=torch.Generator().manual_seed(5)).bfloat16()
    prefix = api._build_prompt_blocks(kd[:, :prompt_len], vd[:, :prompt_len], block)
    total = prompt_len + suffix_len
    if suffix_is_view:       # static-cache style: full-size tail views, validity from the device scalar
        k_suffix, v_suffix = kd[:, prompt_len:], vd[:, prompt_len:]
    else:                    # unrelated suffix tensors, as the reference's sanity script passes them
        k_suffix, v_suffix = kd[:, prompt_len:total].clone(), vd[:, prompt_len:total].clone()
    suffix_len_dev = torch.tensor(suffix_len, device=DEV, dtype=torch.int32)
    out, selected = api._condition_block_decode_output_fused_triton(
        q_grouped=q.to(DEV), prompt_prefix=prefix, k_suffix=k_suffix, v_suffix=v_suffix,
        suffix_len_dev=suffix_len_dev, eps=eps, page_size=block, store_selected=True,
        output_dtype=torch.bfloat16, workspace={})
    want, mask, terms, summ = _oracle_step(q, k[:, :total], v[:, :total], prompt_len, block, eps=eps)
    assert out.shape == (hkv, g, 1, d) and out.dtype == torch.bfloat16
    nb = summ.n_blocks
    assert selected.shape == (hkv, g, 1, nb)
    if eps == 0.0:       # every block that holds a token (a one-token tail block has score 0: either way)
        assert bool(selected[..., : nb - 1].all())
    else:
        assert not bool(selected.any())
    got_mask = selected[:, 0, 0].cpu()
    want = orc.decode_attention(q[:, :, 0].float(), k[:, :total], v[:, :total], prompt_len, block, got_mask,
                                rep_mode="hybrid", z=terms["z"], v_bar=summ.v_bar)
    diff = (out[:, :, 0].float().cpu() - want).abs().max()
    assert float(diff) < 2e-2


def test_fused_decode_topk_and_workspace_reuse():
    api = _api()
    hkv, g, d, block, prompt_len = 2, 8, 128, 64, 2000
    k, v = _cache(hkv, prompt_len + 20, d, torch.bfloat16, 9, spare=12)
    kd, vd = k.to(DEV), v.to(DEV)
    prefix = api._build_prompt_blocks(kd[:, :prompt_len], vd[:, :prompt_len], block)
    ws = {}
    suffix_len_dev = torch.zeros((), device=DEV, dtype=torch.int32)
    for step in range(3):          # the suffix grows on the device, as in a captured decode loop
        suffix_len_dev.add_(5)
        total = prompt_len + 5 * (step + 1)
        q = torch.randn((hkv, g, 1, d), generator=torch.Generator().manual_seed(20 + step)).bfloat16()
        out, sel = api._condition_block_decode_output_fused_triton(
            q_grouped=q.to(DEV), prompt_prefix=prefix, k_suffix=kd[:, prompt_len:], v_suffix=vd[:, prompt_len:],
            suffix_len_dev=suffix_len_dev, eps=0.0, page_size=block, store_selected=True,
            output_dtype=torch.float32, workspace=ws, top_k=6, rep_mode="sparse_only")
        want, mask, _, _ = _oracle_step(q, k[:, :total], v[:, :total], prompt_len, block, top_k=6,
                                        rep_mode="sparse_only")
        assert torch.equal(sel[:, 0, 0].cpu(), mask)
        assert out.dtype == torch.float32
        torch.testing.assert_close(out[:, :, 0].cpu(), want, rtol=1e-2, atol=2e-2)
    assert "b200_step" in ws


def test_attention_hook_in_a_small_llama():
    """The runner installed as eager_attention_forward: decode logits of a random
    2-layer Llama (fp32) match the same model with a CPU oracle hook."""
    transformers = pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaForCausalLM
    from transformers.models.llama import modeling_llama
    api = _api()
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=128, hidden_size=512, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=8, num_key_value_heads=2, head_dim=64, max_position_embeddings=512,
                      rope_theta=500000.0, attn_implementation="eager")
    model = LlamaForCausalLM(cfg).float().eval()
    prompt_len, steps, block, eps = 200, 3, 64, 0.05
    ids = torch.randint(0, 128, (1, prompt_len + steps), generator=torch.Generator().manual_seed(1))

    class OracleRunner:
        def __init__(self):
            self.pos = prompt_len
            self.prefix = {}

        def hook(self, module, query, key, value, attention_mask, scaling, dropout=0.0, **kw):
            if query.shape[2] != 1:
                return api._sdpa_prefill(query, key, value, scaling)
            hkv, hq, d = key.shape[1], query.shape[1], query.shape[3]
            qg = query[0].reshape(hkv, hq // hkv, 1, d)
            k_all, v_all = key[0, :, : self.pos + 1], value[0, :, : self.pos + 1]
            layer = module.layer_idx
            if layer not in self.prefix:
                self.prefix[layer] = orc.block_summaries(k_all[:, :prompt_len], v_all[:, :prompt_len], block)
            out, *_ = _oracle_step(qg, k_all, v_all, prompt_len, block, eps=eps, summ=self.prefix[layer])
            return out.reshape(hq, 1, d).permute(1, 0, 2).unsqueeze(0).to(query.dtype), None

    def run(model, device, make_hook):
        logits = []
        with torch.no_grad():
            out = model(ids[:, :prompt_len].to(device), use_cache=True)
            cache = out.past_key_values
            runner = make_hook()
            original = modeling_llama.eager_attention_forward
            modeling_llama.eager_attention_forward = runner[1]
            try:
                for s in range(steps):
                    runner[0](prompt_len + s)
                    out = model(ids[:, prompt_len + s: prompt_len + s + 1].to(device), past_key_values=cache,
                                use_cache=True)
                    logits.append(out.logits[0, -1].float().cpu())
            finally:
                modeling_llama.eager_attention_forward = original
        return torch.stack(logits)

    def oracle_hook():
        r = OracleRunner()
        return (lambda pos: setattr(r, "pos", pos)), r.hook

    want = run(model, "cpu", oracle_hook)

    gpu_model = model.to(DEV)

    def gpu_hook():
        r = api.ConditionBlockDecodeRunner(model=gpu_model, model_config=cfg, full_attention_layers=0,
                                           block_size=block, eps=eps, prompt_len=prompt_len)
        return r.reset_step, r.hybrid_attention_forward

    got = run(gpu_model, DEV, gpu_hook)
    torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-3)
    # the context manager installs and restores the hook
    r = api.ConditionBlockDecodeRunner(model=gpu_model, block_size=block, eps=eps, prompt_len=prompt_len)
    before = modeling_llama.eager_attention_forward
    with api.condition_block_decode_context(r):
        assert modeling_llama.eager_attention_forward == r.hybrid_attention_forward
    assert modeling_llama.eager_attention_forward is before


def test_batched_static_cache_decode_matches_per_sequence_generation():
    """The batched decode loop (static cache addressed in place as a paged pool,
    eager and CUDA-graph replay) produces the tokens of the per-sequence
    generation entry point, which the test below pins to the CPU oracle."""
    pytest.importorskip("transformers")
    from types import SimpleNamespace
    from interattn_b200 import llama_decode
    api = _api()
    model = llama_decode.build_random_llama("tiny", dtype=torch.float32, device=DEV, seed=5)
    batch, prompt_len, new_tokens, block, top_k = 3, 200, 7, 64, 2
    ids = torch.randint(0, 512, (batch, prompt_len), generator=torch.Generator().manual_seed(6)).to(DEV)
    method = SimpleNamespace(condition_delta_mode="range_bound", max_new_tokens=new_tokens, full_attention_layers=0,
                             condition_block_size=block, condition_eps=0.0, condition_top_k=top_k,
                             condition_rep_mode="sparse_only")
    want = torch.cat([api.generate_condition_block_cached(
        model=model, tokenizer=None, input_ids=ids[b:b + 1], attention_mask=torch.ones_like(ids[b:b + 1]),
        method=method, device=DEV)[0] for b in range(batch)], dim=0)
    eager, stats = llama_decode.generate_batched(model, ids, new_tokens, block_size=block, top_k=top_k)
    assert torch.equal(eager, want)
    assert stats["decode_steps_timed"] > 0 and not stats["cuda_graph"]
    graphed, stats = llama_decode.generate_batched(model, ids, new_tokens, block_size=block, top_k=top_k,
                                                   cuda_graph=True)
    assert stats["cuda_graph"]
    assert torch.equal(graphed, want)


def test_generate_condition_block_cached_matches_oracle_greedy_tokens():
    """The generation entry point (greedy) against a hand-rolled loop whose decode
    attention is the CPU oracle, on a small random fp32 Llama."""
    pytest.importorskip("transformers")
    from types import SimpleNamespace
    from transformers import LlamaConfig, LlamaForCausalLM
    from transformers.models.llama import modeling_llama
    api = _api()
    torch.manual_seed(3)
    cfg = LlamaConfig(vocab_size=96, hidden_size=256, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=512,
                      attn_implementation="eager")
    model = LlamaForCausalLM(cfg).float().eval()
    prompt_len, new_tokens, block, top_k = 150, 5, 64, 2
    ids = torch.randint(0, 96, (1, prompt_len), generator=torch.Generator().manual_seed(4))
    method = SimpleNamespace(condition_delta_mode="range_bound", max_new_tokens=new_tokens, full_attention_layers=1,
                             condition_block_size=block, condition_eps=0.0, condition_top_k=top_k,
                             condition_rep_mode="hybrid")

    # reference loop on the CPU: layer 0 dense, layer 1 = oracle block-sparse attention
    state = {"pos": prompt_len, "summ": None, "hybrid_tokens": 0, "total_available": 0, "rows": 0,
             "selected_tokens": 0}

    def count(stats):
        for key in ("hybrid_tokens", "total_available", "rows", "selected_tokens"):
            state[key] += int(stats[key])

    def hook(module, query, key, value, attention_mask, scaling, dropout=0.0, **kw):
        if query.shape[2] != 1:
            return api._sdpa_prefill(query, key, value, scaling)
        if module.layer_idx < 1:
            count(api.full_attention_stats_for_heads(query.shape[1], [state["pos"]]))
            return api._sdpa_full(query, key[:, :, : state["pos"] + 1], value[:, :, : state["pos"] + 1], scaling)
        hkv, hq, d = key.shape[1], query.shape[1], query.shape[3]
        k_all, v_all = key[0, :, : state["pos"] + 1], value[0, :, : state["pos"] + 1]
        if state["summ"] is None:
            state["summ"] = orc.block_summaries(k_all[:, :prompt_len], v_all[:, :prompt_len], block)
        out, *_ = _oracle_step(query[0].reshape(hkv, hq // hkv, 1, d), k_all, v_all, prompt_len, block, top_k=top_k,
                               summ=state["summ"])
        terms = orc.condition_terms(query[0].reshape(hkv, hq // hkv, d), state["summ"])
        _, mask = orc.select_topk(terms["score"], state["summ"].counts, top_k)
        count(orc.condition_stats(mask, state["summ"].counts, hq // hkv, prompt_len, state["pos"] + 1 - prompt_len))
        return out.reshape(hq, 1, d).permute(1, 0, 2).unsqueeze(0).to(query.dtype), None

    want = []
    with torch.no_grad():
        out = model(ids, use_cache=True)
        cache, tok = out.past_key_values, out.logits[:, -1].argmax(-1, keepdim=True)
        want.append(tok)
        for _ in range(cfg.num_hidden_layers):      # the prefill step counts as dense in every layer
            count(api.full_attention_stats_for_heads(cfg.num_attention_heads, [prompt_len - 1]))
        original = modeling_llama.eager_attention_forward
        modeling_llama.eager_attention_forward = hook
        try:
            for s in range(new_tokens - 1):
                state["pos"] = prompt_len + s
                out = model(tok, past_key_values=cache, use_cache=True)
                tok = out.logits[:, -1].argmax(-1, keepdim=True)
                want.append(tok)
        finally:
            modeling_llama.eager_attention_forward = original
    want = torch.cat(want, dim=1)

    gpu_model = model.to(DEV)
    got, meta = api.generate_condition_block_cached(
        model=gpu_model, tokenizer=None, input_ids=ids.to(DEV), attention_mask=torch.ones_like(ids).to(DEV),
        method=method, device=DEV)
    assert got.shape == (1, new_tokens) and meta["decode_steps"] == new_tokens - 1
    assert torch.equal(got.cpu(), want)
    # the runner's statistics (lazy GPU scalars summed per step, read back once) against the oracle's
    budget = meta["condition_block_budget"]
    for key in ("hybrid_tokens", "total_available", "rows", "selected_tokens"):
        assert budget[key] == state[key], key
    assert meta["condition_block_equiv_budget"] == pytest.approx(state["hybrid_tokens"] / state["total_available"])
    assert len(budget["by_step"]) == new_tokens and 0 < budget["by_step"][-1]["equiv_budget"] <= 1
    # one more step by hand: summarize() per step, stats per compressed and per dense layer, no device read
    runner = api.ConditionBlockDecodeRunner(model=gpu_model, model_config=gpu_model.config, full_attention_layers=1,
                                            block_size=block, eps=0.0, prompt_len=prompt_len, top_k=top_k)
    assert runner.summarize() == {"aggregate": {}, "by_layer": {}} and not runner.skip_stats
    with pytest.raises(ValueError):
        api.generate_condition_block_cached(model=gpu_model, tokenizer=None, input_ids=ids.repeat(2, 1).to(DEV),
                                            attention_mask=None, method=method, device=DEV)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 3e-2)])
def test_factory_attention_module_prefills_densely_and_decodes_sparsely(dtype, tol):
    """attention_factory seam: forward(x[B, T, C]) -> y[B, T, C]; with every block selected a decode
    step equals dense causal attention of the last position, with top-2 it equals the oracle."""
    from types import SimpleNamespace
    from interattn_b200 import caller_surface as cs
    torch.manual_seed(21)
    cfg = SimpleNamespace(attn=SimpleNamespace(type=cs.ATTN_TYPE, select_block=64, top_k=64), n_embd=256, n_head=4,
                          n_kv_head=2, bias=False, block_size=512)
    mod = cs.create_attention(cfg, layer_index=0).to(DEV).to(dtype)
    b, t = 2, 300
    x = torch.randn(b, t + 1, 256, device=DEV, dtype=dtype)
    y_prefill = mod(x[:, :t])
    assert y_prefill.shape == (b, t, 256)
    y_step = mod(x[:, t:t + 1])
    assert y_step.shape == (b, 1, 256)
    mod.reset_cache()
    y_full = mod(x)                                       # dense causal attention over all T + 1 tokens
    assert torch.allclose(y_prefill.float(), y_full[:, :t].float(), atol=tol, rtol=tol)
    assert torch.allclose(y_step.float(), y_full[:, t:].float(), atol=tol, rtol=tol)
    # top-2 of the 5 prompt blocks: the selection must be what the oracle selects on the same K
    mod.reset_cache()
    mod.top_k = 2
    mod(x[:, :t])
    y_sparse = mod(x[:, t:t + 1])
    st = mod._state
    idx = st["step"].sel_idx.cpu()
    assert int(st["step"].sel_count.min()) == 2 and idx.shape[-1] >= 2
    assert not torch.allclose(y_sparse.float(), y_full[:, t:].float(), atol=tol, rtol=tol)


def test_generate_with_method_kind_b200_batch_1_and_batched():
    pytest.importorskip("transformers")
    from types import SimpleNamespace
    from interattn_b200 import caller_surface as cs, llama_decode
    api = _api()
    model = llama_decode.build_random_llama("tiny", dtype=torch.float32, device=DEV, seed=5)
    ids = torch.randint(0, 512, (3, 200), generator=torch.Generator().manual_seed(6)).to(DEV)
    method = SimpleNamespace(kind=cs.METHOD_KIND, condition_delta_mode="range_bound", max_new_tokens=6,
                             full_attention_layers=0, condition_block_size=64, condition_eps=0.0, condition_top_k=2,
                             condition_rep_mode="sparse_only")
    one, meta1 = cs.generate_with_method(model, None, ids[:1], torch.ones_like(ids[:1]), method, DEV)
    want, _ = api.generate_condition_block_cached(model=model, tokenizer=None, input_ids=ids[:1],
                                                  attention_mask=torch.ones_like(ids[:1]), method=method, device=DEV)
    assert torch.equal(one, want)
    many, meta = cs.generate_with_method(model, None, ids, torch.ones_like(ids), method, DEV)
    assert many.shape == (3, 6) and meta["batched"] and meta["method"] == cs.METHOD_KIND
    assert torch.equal(many[:1], one)
