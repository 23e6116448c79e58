"""The C-ABI library loads and exports every symbol include/inferencequant_b200.h declares (no compute here)."""
import os
import re

import pytest

import inference_rs_b200 as pkg
from inference_rs_b200 import kernel_library as kl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "inferencequant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b((?:launch|b200q)_[A-Za-z0-9_]+)\s*\(", text))
    names |= set(re.findall(r"extern const char (\w+)\[\]", text))
    return names


def test_header_and_loader_agree():
    declared = _declared_symbols()
    assert declared, "no declarations parsed"
    known = set(kl.SYMBOLS) | set(kl.DATA_SYMBOLS)
    assert declared == known, (sorted(declared - known), sorted(known - declared))


def test_library_exports_every_declared_symbol():
    lib = pkg.library()  # raises if any symbol is missing
    for name in _declared_symbols():
        if name in kl.DATA_SYMBOLS:
            continue
        assert getattr(lib, name) is not None
    assert kl.build_id().startswith("b200q-sm100a")
    assert lib.b200q_version().decode().count(".") == 2


def test_missing_library_is_an_error_not_a_fallback(monkeypatch, tmp_path):
    monkeypatch.setattr(kl, "_lib", None)
    monkeypatch.setattr(kl, "HERE", str(tmp_path))
    monkeypatch.delenv("INFERENCE_KERNEL_DIR", raising=False)
    with pytest.raises(kl.KernelLibraryError, match="no CPU fallback"):
        kl.library()


def test_kernel_dir_env_takes_precedence(monkeypatch, tmp_path):
    monkeypatch.setenv("INFERENCE_KERNEL_DIR", str(tmp_path))
    assert kl.search_paths()[0] == os.path.join(str(tmp_path), "sm100a", kl.LIB_NAME)


def test_options_and_errors_round_trip():
    from inference_rs_b200 import ops
    ops.set_option("pdl", 0)
    assert ops.get_option("pdl") == 0
    with pytest.raises(kl.KernelLibraryError, match="unknown option"):
        ops.set_option("no_such_option", 1)
    assert ops.get_option("sm_count") > 0
    # the L2 prefetch size follows the launch mode until it is set, and again after -1
    assert ops.get_option("l2_prefetch_bytes") == 256 * 1024
    ops.set_option("pdl", 1)
    assert ops.get_option("l2_prefetch_bytes") == 64 * 1024
    ops.set_option("l2_prefetch_bytes", 4100)
    assert ops.get_option("l2_prefetch_bytes") == 4096
    ops.set_option("l2_prefetch_bytes", -1)
    ops.set_option("pdl", 0)
    assert ops.get_option("l2_prefetch_bytes") == 256 * 1024


@pytest.mark.parametrize("tag,k,n,b", [("Q4K", 4096, 4096, 1), ("Q6K", 14336, 4096, 4), ("Q8_0", 4096, 128256, 8),
                                       ("Q6K", 768, 100, 1), ("Q4K", 28672, 8192, 1)])
def test_gemv_plans_respect_hardware_limits(tag, k, n, b):
    from inference_rs_b200 import ops
    dt = pkg.GgmlDType[tag]
    plan = ops.gemv_plan(dt, k, n, b)
    if not plan["staged"]:
        return
    assert plan["smem"] <= 227 * 1024
    assert 2 <= plan["stages"] <= 16
    assert plan["rows_per_stage"] % plan["row_align"] == 0
    items = k // 128
    assert plan["warps_per_row"] * 32 * plan["items_per_lane"] >= items
    assert plan["stage_bytes"] >= plan["rows_per_stage"] * dt.row_bytes(k) + 16
    assert (plan["row_align"] * dt.row_bytes(k)) % 16 == 0
    assert 1 <= plan["grid"] <= 148


def test_short_launches_are_split_in_whole_stages_where_few_ctas_get_the_remainder():
    """The row partition's unit: a whole ring stage for ffn_gate / ffn_up of the 8B model (3 stages per CTA, 4 CTAs with a
    fourth), the 16-byte-aligned unit where half of the CTAs would get the extra stage (ffn_down) and for long launches
    (the output head), where a ragged last stage is amortised."""
    from inference_rs_b200 import ops
    if ops.get_option("sm_count") != 148:
        pytest.skip("the expectations are for 148 SMs")
    gate = ops.gemv_plan(pkg.GgmlDType.Q4K, 4096, 14336, 1)
    assert gate["staged"] and gate["row_align"] == gate["rows_per_stage"]
    down = ops.gemv_plan(pkg.GgmlDType.Q6K, 14336, 4096, 1)
    assert down["staged"] and down["row_align"] < down["rows_per_stage"]
    head = ops.gemv_plan(pkg.GgmlDType.Q6K, 4096, 128256, 1)
    assert head["staged"] and head["row_align"] < head["rows_per_stage"]
    small = ops.gemv_plan(pkg.GgmlDType.Q4K, 4096, 4096, 1)
    assert small["staged"] and small["row_align"] < small["rows_per_stage"]


def test_trace_buffer_needs_a_trace_build():
    """The launch timelines are a build option; the default library says so instead of silently ignoring the buffer."""
    import ctypes
    lib = pkg.library()
    assert lib.b200q_set_trace_buffer(None, 0) == 0
    rc = lib.b200q_set_trace_buffer(ctypes.c_void_p(4096), 4)
    assert rc in (0, -1)  # B200Q_ERR_UNSUPPORTED; 0 only in a library built with -DB200Q_GEMV_TRACE=1
    if rc != 0:
        assert b"B200Q_GEMV_TRACE" in lib.b200q_last_error()
    lib.b200q_set_trace_buffer(None, 0)
