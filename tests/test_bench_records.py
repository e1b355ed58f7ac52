"""The bench line's per-kernel records, without a GPU: two-kernel and one-kernel forms carry the keys the
measurement contract names (roofline.bound / achieved / peak / unit / frac / traffic) and consistent arithmetic."""

import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_bytes_of_the_headline_workload(bench):
    from interattn_b200.workloads import CONFIGS
    cfg = CONFIGS["cfg2_llama8b_32k"]
    kv, sel = bench.algorithmic_bytes(cfg, "sparse_only", False)
    assert kv == 128 * 64 * 64 * 128 * 2 * 2          # pairs x blocks x tokens x D x (K, V) x bf16
    assert sel == 128 * 512 * (128 * 4 + 2 * 128 * 2 + 4)  # k_bar f32 + k_max, k_min bf16 + the value norm
    kv_h, _ = bench.algorithmic_bytes(cfg, "hybrid", False)
    assert kv_h - kv == 128 * (512 - 64) * 128 * 2       # one mean-value row per block that was not picked
    _, sel_ell = bench.algorithmic_bytes(cfg, "sparse_only", False, "diag_ell")
    assert sel - sel_ell == 128 * 512 * (128 * 2 - 4)     # w replaces (k_max, k_min); rho is one float more


@pytest.mark.parametrize("fused", [False, True])
def test_kernel_records(bench, fused):
    kernel_us, roof, roof_sel = bench.kernel_records(fused, 30.0, 50.0, 268435456, 67371008, "cfg2_llama8b_32k")
    for key in ("bound", "kernel", "achieved", "peak", "unit", "frac", "traffic", "bytes_per_launch"):
        assert key in roof
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s"
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-12
    if fused:
        assert roof_sel is None and roof["kernel"] == "condition_block_select_attend_kernel"
        assert kernel_us["select_attend"] == 80.0 and kernel_us["select"] == 0.0
        assert roof["bytes_per_launch"] == 268435456 + 67371008
        assert abs(roof["achieved"] - (268435456 + 67371008) / 80e-6 / 1e9) < 1e-6
        assert roof["duration_us"] == 80.0 and roof["isolated_us"] == 80.0
        # with the timed region's time per launch: that is the duration, the event-bracketed span stays beside it
        _, timed, _ = bench.kernel_records(True, 30.0, 50.0, 268435456, 67371008, "cfg2_llama8b_32k", region_us=73.0)
        assert timed["duration_us"] == 73.0 and timed["isolated_us"] == 80.0
        assert abs(timed["achieved"] - (268435456 + 67371008) / 73e-6 / 1e9) < 1e-6
        assert abs(timed["isolated_frac"] - roof["frac"]) < 1e-12
    else:
        assert roof["kernel"] == "condition_block_finalize_attention_kernel"
        assert abs(roof["achieved"] - 268435456 / 50e-6 / 1e9) < 1e-6
        assert abs(roof_sel["achieved"] - 67371008 / 30e-6 / 1e9) < 1e-6
        assert kernel_us == {"select": 30.0, "sparse_decode": 50.0, "finalize": 0.0}
    # the traffic figures come from the committed ncu summaries
    assert roof["traffic"] is not None and roof["traffic"] >= roof["bytes_per_launch"]


def test_fused_record_splits_into_phases(bench):
    _, roof, _ = bench.kernel_records(True, 30.0, 50.0, 268435456, 67371008, "cfg2_llama8b_32k", phases=(22.0, 45.0))
    ph = roof["phases"]
    assert abs(ph["attention"]["achieved"] - 268435456 / 45e-6 / 1e9) < 1e-6
    assert abs(ph["selection"]["frac"] - 67371008 / 22e-6 / 1e9 / roof["peak"]) < 1e-12
    assert ph["attention"]["bytes"] + ph["selection"]["bytes"] == roof["bytes_per_launch"]
