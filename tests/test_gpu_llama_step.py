"""The fused element-wise kernels of the Llama decode step (through the C ABI) against
their CPU restatement, and the fused step against the module-by-module step."""

import pytest
import torch

from oracle import llama_step_oracle as lo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF = torch.bfloat16


def _step():
    from interattn_b200 import llama_step
    return llama_step


def _ulp_apart(a, b):
    """Largest distance between two bf16 tensors in units of the last place."""
    ia = a.contiguous().view(torch.int16).to(torch.int32)
    ib = b.contiguous().view(torch.int16).to(torch.int32)
    ia = torch.where(ia < 0, -(ia & 0x7fff), ia)
    ib = torch.where(ib < 0, -(ib & 0x7fff), ib)
    return int((ia - ib).abs().max())


@pytest.mark.parametrize("rows,hidden,with_delta", [(32, 4096, True), (5, 512, True), (3, 8192, False), (2, 136, True)])
def test_add_rmsnorm(rows, hidden, with_delta):
    ls = _step()
    g = torch.Generator().manual_seed(rows * 1000 + hidden)
    res = (torch.randn(rows, hidden, generator=g) * 3).to(BF)
    delta = torch.randn(rows, hidden, generator=g).to(BF) if with_delta else None
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(BF)
    want_x, want_y = lo.add_rmsnorm(res, delta, w, 1e-5)
    res_d, out = res.to(DEV), torch.empty(rows, hidden, dtype=BF, device=DEV)
    ls.add_rmsnorm(res_d, delta.to(DEV) if with_delta else None, w.to(DEV), 1e-5, out)
    assert torch.equal(res_d.cpu(), want_x)                       # the residual stream: bit-exact
    # the fp32 sum of squares is taken in another order: at most one unit in the last place
    assert _ulp_apart(out.cpu(), want_y) <= 1
    assert (out.cpu() != want_y).float().mean() < 0.01


@pytest.mark.parametrize("b,hq,hkv,d,t", [(3, 4, 2, 64, 48), (32, 32, 8, 128, 272)])
def test_rope_append(b, hq, hkv, d, t):
    ls = _step()
    g = torch.Generator().manual_seed(b + d)
    inv = 1.0 / (500000.0 ** (torch.arange(0, d, 2).float() / d))
    freqs = torch.arange(t).float()[:, None] * inv[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    cos_t, sin_t = emb.cos().to(BF), emb.sin().to(BF)
    qkv = torch.randn(b, (hq + 2 * hkv) * d, generator=g).to(BF)
    seq_lens = torch.randint(1, t + 1, (b,), generator=g).to(torch.int32)
    seq_lens[0], seq_lens[-1] = 1, t
    k_cache = torch.randn(b, hkv, t, d, generator=g).to(BF)
    v_cache = torch.randn(b, hkv, t, d, generator=g).to(BF)
    k_d, v_d = k_cache.to(DEV), v_cache.to(DEV)
    q_d = torch.empty(b, hq, d, dtype=BF, device=DEV)
    ls.rope_append(qkv.to(DEV), cos_t.to(DEV), sin_t.to(DEV), seq_lens.to(DEV), k_d, v_d, q_d)
    want_q = lo.rope_append(qkv, cos_t, sin_t, seq_lens, k_cache, v_cache, hq)
    assert torch.equal(q_d.cpu(), want_q)
    assert torch.equal(k_d.cpu(), k_cache) and torch.equal(v_d.cpu(), v_cache)


def test_rope_append_leaves_out_of_range_rows_alone():
    ls = _step()
    b, hq, hkv, d, t = 2, 2, 1, 64, 32
    qkv = torch.ones(b, (hq + 2 * hkv) * d, dtype=BF, device=DEV)
    cos_t = torch.ones(t, d, dtype=BF, device=DEV)
    sin_t = torch.zeros(t, d, dtype=BF, device=DEV)
    k_d = torch.zeros(b, hkv, t, d, dtype=BF, device=DEV)
    v_d = torch.zeros_like(k_d)
    q_d = torch.zeros(b, hq, d, dtype=BF, device=DEV)
    ls.rope_append(qkv, cos_t, sin_t, torch.tensor([0, t + 5], dtype=torch.int32, device=DEV), k_d, v_d, q_d)
    torch.cuda.synchronize()
    assert float(k_d.abs().sum()) == 0 and float(v_d.abs().sum()) == 0 and float(q_d.abs().sum()) == 0


@pytest.mark.parametrize("rows,inter", [(32, 14336), (3, 1024), (1, 8)])
def test_silu_mul(rows, inter):
    ls = _step()
    g = torch.Generator().manual_seed(inter)
    gu = (torch.randn(rows, 2 * inter, generator=g) * 2).to(BF)
    out = torch.empty(rows, inter, dtype=BF, device=DEV)
    ls.silu_mul(gu.to(DEV), out)
    want = lo.silu_mul(gu)
    # expf on the two machines may differ in the last fp32 bit: a rare flip of the bf16 rounding
    assert _ulp_apart(out.cpu(), want) <= 1
    assert (out.cpu() != want).float().mean() < 1e-3


def test_argmax_lowest_index_wins():
    ls = _step()
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(32, 128256, generator=g).to(BF)       # bf16 rounding makes exact ties likely
    logits[3, 77] = logits[3, 100000] = 50.0
    logits[4, 128255] = 60.0
    logits[5, :] = -1.0
    out = torch.empty(32, 1, dtype=torch.int64, device=DEV)
    ls.argmax(logits.to(DEV), out)
    assert torch.equal(out.cpu().view(-1), lo.argmax_first(logits))
    assert out[3, 0] == 77 and out[4, 0] == 128255 and out[5, 0] == 0
    odd = logits[:, 1:1001]                                     # rows off the 16-byte boundary, ragged length
    out2 = torch.empty(32, dtype=torch.int64, device=DEV)
    ls.argmax(logits.to(DEV)[:, 1:1001], out2)
    assert torch.equal(out2.cpu(), lo.argmax_first(odd))


@pytest.mark.parametrize("m,n,k", [(32, 6144, 4096), (32, 4096, 14336), (32, 28672, 4096), (5, 512, 512),
                                   (1, 1000, 72), (17, 130, 200), (32, 128256, 256)])
def test_skinny_gemm(m, n, k):
    ls = _step()
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).to(BF).to(DEV)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(BF).to(DEV)
    ws = ls.gemm_workspace(n, DEV)
    out = torch.full((m, n), float("nan"), dtype=BF, device=DEV)
    packed = ls.PackedWeight(w)
    ls.gemm(x, packed, out, ws)
    want = x.float() @ w.float().t()                              # fp32 accumulate of the same bf16 inputs
    err = (out.float() - want).abs()
    assert bool((err <= 2.0 ** -8 * want.abs() + 1e-3).all()), float(err.max())
    again = torch.empty_like(out)
    ls.gemm(x, packed, again, ws)                                 # the workspace is reusable as left behind,
    assert torch.equal(out, again)                                # and the result does not depend on timing
    assert int(ws[: ((n + 127) // 128) * 4].view(torch.int32).abs().sum()) == 0


def test_bad_arguments_raise():
    ls = _step()
    x = torch.zeros(2, 100, dtype=BF, device=DEV)               # hidden not a multiple of 8
    with pytest.raises(ValueError):
        ls.add_rmsnorm(x, None, torch.ones(100, dtype=BF, device=DEV), 1e-5, torch.empty_like(x))
    with pytest.raises(ValueError):
        ls.silu_mul(torch.zeros(2, 64, device=DEV), torch.zeros(2, 32, device=DEV))   # fp32
    with pytest.raises(ValueError):
        ls.add_rmsnorm(x.cpu(), None, torch.ones(100, dtype=BF), 1e-5, torch.empty(2, 100, dtype=BF))
    big = torch.zeros(33, 64, dtype=BF, device=DEV)               # more than 32 rows
    with pytest.raises(ValueError):
        ls.gemm(big, ls.PackedWeight(torch.zeros(128, 64, dtype=BF, device=DEV)),
                torch.zeros(33, 128, dtype=BF, device=DEV), ls.gemm_workspace(128, DEV))
    with pytest.raises(ValueError):                               # workspace too small
        ls.gemm(big[:4], ls.PackedWeight(torch.zeros(128, 64, dtype=BF, device=DEV)),
                torch.zeros(4, 128, dtype=BF, device=DEV), torch.zeros(16, dtype=torch.uint8, device=DEV))


@pytest.mark.parametrize("graph,own_gemm", [(False, "none"), (True, "none"), (False, "all"), (True, "w_down,lm_head")])
def test_fused_step_matches_the_module_by_module_step(graph, own_gemm):
    """Same weights, same prompts, the same tokens fed at every step: the logits of the fused
    step follow those of the Hugging Face modules around the attention hook."""
    pytest.importorskip("transformers")
    from interattn_b200 import llama_decode
    model = llama_decode.build_random_llama("tiny", dtype=BF, device=DEV, seed=11)
    batch, prompt_len, new_tokens, block, top_k = 3, 200, 9, 64, 2
    ids = torch.randint(0, 512, (batch, prompt_len), generator=torch.Generator().manual_seed(12)).to(DEV)
    forced = torch.randint(0, 512, (batch, new_tokens), generator=torch.Generator().manual_seed(13)).to(DEV)
    kw = dict(block_size=block, top_k=top_k, force_tokens=forced, collect_logits=True)
    _, ref = llama_decode.generate_batched(model, ids, new_tokens, **kw)
    _, got = llama_decode.generate_batched(model, ids, new_tokens, fused_step=True, own_gemm=own_gemm, **kw)
    assert got["fused_step"] and not ref["fused_step"]
    a, b = ref["logits"].float(), got["logits"].float()
    assert a.shape == b.shape == (new_tokens - 1, batch, 512)
    scale = float(a.abs().max())
    assert float((a - b).abs().max()) <= 0.03 * scale
    if graph:   # greedy tokens of the captured fused step == greedy tokens of the eager fused step
        t_eager, _ = llama_decode.generate_batched(model, ids, new_tokens, block_size=block, top_k=top_k,
                                                   fused_step=True, own_gemm=own_gemm)
        t_graph, st = llama_decode.generate_batched(model, ids, new_tokens, block_size=block, top_k=top_k,
                                                    fused_step=True, own_gemm=own_gemm, cuda_graph=True)
        assert st["cuda_graph"] and st["fused_step"]
        assert torch.equal(t_eager, t_graph)
