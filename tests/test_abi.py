"""CPU tests of the C-ABI library: it loads, exports every symbol the header declares, refuses
to compute without a device (no fallback), and its host-only schedule logic is right."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def header_functions(name="gpt2_linear.h"):
    src = open(os.path.join(ROOT, "include", name)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(gpt2_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol(g):
    names = header_functions()
    assert len(names) >= 18
    for n in names:
        assert hasattr(g.lib, n), f"{n} declared in include/gpt2_linear.h but not exported"
    assert sorted(names) == sorted(g.EXPORTS)


def test_library_exports_every_model_symbol(g):
    names = header_functions("gpt2_model.h")  # the model calls and the step-schedule calls
    assert sorted(names) == sorted(g.MODEL_EXPORTS)
    for n in names:
        assert hasattr(g.lib, n)


def test_library_exports_every_attention_symbol(g):
    names = [n for n in header_functions("gpt2_attention.h") if n.startswith("gpt2_attention_")]
    assert sorted(names) == sorted(g.ATTENTION_EXPORTS)
    for n in names:
        assert hasattr(g.lib, n)
    # shape checks are host-only
    assert g.lib.gpt2_attention_supported(g.ATT_FLASH, 1024, 768, 12) == 1
    assert g.lib.gpt2_attention_supported(g.ATT_FLASH, 1000, 768, 12) == 0
    assert g.lib.gpt2_attention_supported(g.ATT_GEMM, 992, 768, 12) == 1
    assert g.lib.gpt2_attention_supported(g.ATT_SIMT, 7, 768, 12) == 1
    assert g.lib.gpt2_attention_supported(g.ATT_SIMT, 7, 768, 8) == 0


def test_version(g):
    assert g.lib.gpt2_linear_version() == 100


def test_no_device_means_error_not_fallback(g):
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    assert g.lib.gpt2_linear_init(0) == g.ERR_NO_DEVICE
    buf = (ctypes.c_float * 16)()
    p = ctypes.addressof(buf)
    assert g.forward(p, p, p, None, 1, 2, 2, 2) in (g.ERR_NO_DEVICE, g.ERR_NOT_INIT)
    assert g.backward_input(p, p, p, 1, 2, 2, 2) in (g.ERR_NO_DEVICE, g.ERR_NOT_INIT)
    assert g.backward_weight(p, None, p, p, 1, 2, 2, 2) in (g.ERR_NO_DEVICE, g.ERR_NOT_INIT)
    assert g.forward(p, p, p, None, 1, 2, 2, 2, host=True) in (g.ERR_NO_DEVICE, g.ERR_NOT_INIT)


def test_bad_arguments(g):
    buf = (ctypes.c_float * 16)()
    p = ctypes.addressof(buf)
    assert g.forward(p, p, p, None, 0, 2, 2, 2) == g.ERR_BAD_ARG
    assert g.backward_input(p, p, p, 1, -1, 2, 2) == g.ERR_BAD_ARG


# ---- schedule logic (host only; fake pointers are never dereferenced) ----
FAKE = 0x1000


def mlp_chain(g, B=2, S=256, C=64):
    """fc -> fc_proj forward, then their backward: the dependency pattern of one MLP block."""
    ops = [
        g.make_op(g.OP_FORWARD, B, S, C, 4 * C, FAKE, FAKE, FAKE, bias=FAKE),                       # 0 fc
        g.make_op(g.OP_FORWARD, B, S, 4 * C, C, FAKE, FAKE, FAKE, deps=[(0, g.DEP_ROWBLOCK)]),      # 1 fc_proj
        g.make_op(g.OP_BACKWARD_INPUT, B, S, 4 * C, C, FAKE, FAKE, FAKE, deps=[(1, g.DEP_ROWBLOCK)]),  # 2
        g.make_op(g.OP_BACKWARD_WEIGHT, B, S, 4 * C, C, FAKE, FAKE, FAKE, out_bias=FAKE,
                  deps=[(0, g.DEP_WHOLE_OP), (1, g.DEP_WHOLE_OP)]),                                  # 3
        g.make_op(g.OP_BACKWARD_INPUT, B, S, C, 4 * C, FAKE, FAKE, FAKE, deps=[(2, g.DEP_ROWBLOCK)]),  # 4
    ]
    return ops


@pytest.mark.parametrize("grid", [1, 2, 7, 148])
def test_schedule_validates_for_any_grid(g, grid):
    assert g.validate_schedule(mlp_chain(g), grid) == g.OK


def test_schedule_describe_counts(g):
    ops = mlp_chain(g, B=2, S=256, C=64)
    code, (tiles, counters, grid) = g.describe_schedule(ops, 148)
    assert code == g.OK
    # M = 512 -> 4 row blocks for the four M-row ops, K = 256 -> 2 row blocks for the weight gradient
    assert counters == (4 + 1) * 4 + (2 + 1)
    # default: single CTAs, 128-row tiles
    assert tiles >= 4 + 4 + 4 + 2 + 4 and grid == min(148, tiles)
    # the same list on CTA pairs (256-row tiles): at least 2 + 2 + 2 + 1 + 2 tiles on 148 / 2 pairs
    for op in ops:
        op.opts.cta_pair = 2
    code, (tiles2, counters2, grid2) = g.describe_schedule(ops, 148)
    assert code == g.OK and counters2 == counters
    assert 9 <= tiles2 < tiles and grid2 == min(74, tiles2)
    assert g.validate_schedule(ops, 148) == g.OK


def test_schedule_rejects_forward_pointing_dependency(g):
    ops = mlp_chain(g)
    ops[0].deps[0].producer = 1
    ops[0].deps[0].kind = g.DEP_ROWBLOCK
    assert g.validate_schedule(ops, 4) == g.ERR_SCHEDULE


def test_schedule_rejects_rowblock_dependency_between_different_row_counts(g):
    ops = mlp_chain(g)
    # the weight gradient's rows are K, not M: a row-block dependency on it is meaningless
    ops[4].deps[0].producer = 3
    assert g.validate_schedule(ops, 4) == g.ERR_SCHEDULE


def test_schedule_rejects_mixed_modes(g):
    ops = mlp_chain(g)
    ops[1].opts.mode = g.MODE_TF32X3
    assert g.validate_schedule(ops, 4) == g.ERR_SCHEDULE


def test_schedule_create_needs_device(g):
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    with pytest.raises(g.LinearError):
        g.Schedule(mlp_chain(g))
