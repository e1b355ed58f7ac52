"""The two caller-side seams: method-kind dispatch and the attention factory (host logic, CPU)."""

import argparse
from types import SimpleNamespace

import pytest

from interattn_b200 import caller_surface as cs


def test_other_kinds_go_to_the_wrapped_dispatcher_or_raise():
    seen = []

    def original(model, tokenizer, input_ids, attention_mask, method, device, dataset=None):
        seen.append(method.kind)
        return "ids", {"method": method.kind}

    method = SimpleNamespace(kind="full")
    assert cs.generate_with_method(None, None, None, None, method, "cpu", fallback=original) == ("ids", {"method": "full"})
    assert seen == ["full"]
    with pytest.raises(NotImplementedError):
        cs.generate_with_method(None, None, None, None, method, "cpu")


def test_register_method_kind_patches_the_reference_modules():
    calls = []
    gen = SimpleNamespace(generate_with_method=lambda *a, **k: calls.append(a[4].kind) or ("x", {}))
    common = SimpleNamespace(LOCAL_PATCH_METHODS={"condition_block", "quest"})
    parser = argparse.ArgumentParser()
    parser.add_argument("--method", default="full", choices=["full", "condition_block_triton"])
    cs.register_method_kind(gen, common, parser)
    cs.register_method_kind(gen, common, parser)          # idempotent
    assert cs.METHOD_KIND in common.LOCAL_PATCH_METHODS
    assert parser.parse_args(["--method", cs.METHOD_KIND]).method == cs.METHOD_KIND
    assert gen.generate_with_method(None, None, None, None, SimpleNamespace(kind="quest"), "cpu") == ("x", {})
    assert calls == ["quest"]


def test_factory_raises_like_the_reference_for_unknown_types():
    cfg = SimpleNamespace(attn=SimpleNamespace(type="mamba"), n_embd=64, n_head=2, block_size=128)
    with pytest.raises(NotImplementedError, match="Attention type 'mamba' is not implemented"):
        cs.create_attention(cfg)
    assert cs.create_attention(cfg, fallback=lambda c, i: "theirs") == "theirs"


def test_factory_builds_the_module_and_it_refuses_cpu_decode():
    import torch
    cfg = SimpleNamespace(attn=SimpleNamespace(type=cs.ATTN_TYPE, select_block=64, top_k=2), n_embd=128, n_head=2,
                          bias=False, block_size=256)
    mod = cs.create_attention(cfg, layer_index=3)
    assert isinstance(mod, cs.ConditionBlockSelfAttention) and mod.layer == 3 and mod.capacity == 256
    with pytest.raises(ValueError):
        mod(torch.zeros(1, 1, 128))                       # decode before prefill
    with pytest.raises(ValueError):
        mod(torch.zeros(1, 300, 128))                     # longer than the context
