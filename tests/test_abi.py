"""The C-ABI library loads and exports every symbol include/lact_b200.h declares; host-side
argument checks that need no GPU return the documented error codes."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from lact_b200 import build
    build.build()
    from lact_b200 import _lib
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "lact_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lact_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("lact_scan_fwd", "lact_scan_workspace_bytes", "lact_swiglu_ffn_fwd", "lact_fw_grad",
                 "lact_newton_schulz", "lact_l2_norm_add", "lact_prenorm_momentum_l2norm", "lact_bmm_bf16"):
        assert must in syms


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/lact_b200.h but not exported"


def test_version_and_error_strings(lib):
    assert lib.lact_version() >= 1000
    assert lib.lact_error_string(0) == b"ok"
    for code in range(-8, 0):
        assert lib.lact_error_string(code) != b"unknown code"


def test_null_arguments_are_rejected(lib):
    assert lib.lact_scan_fwd(None, None, 0, None, None, None, None, None, 0, None) == -1
    assert lib.lact_swiglu_ffn_fwd(None, None, None, None, 1, 128, 64, 64, None, 0, None) == -1
    assert lib.lact_newton_schulz(None, 0, None, 1, 64, 64, 5, 0, None, 0, None) == -1
    assert lib.lact_read_status(None, None) == -1


def test_workspace_queries_and_shape_checks(lib):
    from lact_b200._lib import ScanConfig
    n = C.c_size_t(0)
    assert lib.lact_swiglu_ffn_workspace_bytes(2, 100, 64, 128, C.byref(n)) == 0 and n.value >= 2 * 100 * 128 * 2
    assert lib.lact_swiglu_ffn_workspace_bytes(2, 100, 60, 128, C.byref(n)) == -2  # D not a multiple of 16
    assert lib.lact_fw_grad_workspace_bytes(2, 100, 64, 128, C.byref(n)) == 0 and n.value >= 2 * 100 * 3 * 128 * 2
    assert lib.lact_newton_schulz_workspace_bytes(2, 64, 128, C.byref(n)) == 0 and n.value > 0
    cfg = ScanConfig()
    cfg.B, cfg.L, cfg.D, cfg.H, cfg.out_len = 2, 256, 64, 64, 256
    cfg.act_dtype, cfg.renorm = 1, 1
    kind = (C.c_int32 * 3)(0, 1, 0)
    start = (C.c_int64 * 3)(0, 0, 128)
    end = (C.c_int64 * 3)(128, 128, 256)
    assert lib.lact_scan_workspace_bytes(C.byref(cfg), 3, kind, start, end, C.byref(n)) == 0 and n.value > 0
    base = n.value
    cfg.use_muon, cfg.ns_steps = 1, 5
    assert lib.lact_scan_workspace_bytes(C.byref(cfg), 3, kind, start, end, C.byref(n)) == 0 and n.value > base
    cfg.ns_steps = 3  # tuned table needs exactly 5 steps
    assert lib.lact_scan_workspace_bytes(C.byref(cfg), 3, kind, start, end, C.byref(n)) == -5
    cfg.ns_steps = 5
    end[1] = 0  # empty update range
    assert lib.lact_scan_workspace_bytes(C.byref(cfg), 3, kind, start, end, C.byref(n)) == -6
    end[1] = 300  # beyond L
    assert lib.lact_scan_workspace_bytes(C.byref(cfg), 3, kind, start, end, C.byref(n)) == -6
    cfg.act_dtype = 0  # fp32 activations are not supported by this build
    end[1] = 128
    assert lib.lact_scan_workspace_bytes(C.byref(cfg), 3, kind, start, end, C.byref(n)) == -3


def test_newton_schulz_trace_layout_queries(lib):
    """Host-only layout arithmetic of the Newton-Schulz trace: the result (iterate number `steps`) sits behind the
    norm partials, scale factors and completion counters and `steps` earlier iterates, inside the buffer."""
    for B, R, Cc, steps in ((2, 64, 128, 1), (4, 128, 64, 5), (3, 384, 384, 3)):
        off, need = C.c_size_t(0), C.c_size_t(0)
        assert lib.lact_ns_trace_result_offset(B, R, Cc, steps, C.byref(off)) == 0
        assert lib.lact_ns_trace_bytes(B, R, Cc, steps, C.byref(need)) == 0

        def up(x):
            return (x + 255) & ~255
        x0 = up(up(up(0) + B * 512 * 4) + B * 4)       # partial sums [B][512] fp32, then scale [B] fp32 ...
        x0 = up(x0 + (B + 64) * 4)                       # ... then completion counters [B + 64] u32, then the iterates
        assert off.value == x0 + B * R * Cc * steps * 2
        assert off.value % 16 == 0 and off.value + B * R * Cc * 2 <= need.value


def test_python_shim_rejects_cpu_tensors():
    import torch
    import lact_b200
    x = torch.zeros(1, 16, 16, dtype=torch.bfloat16)
    w = torch.zeros(1, 16, 16)
    lr = torch.zeros(1, 16, 1)
    with pytest.raises(RuntimeError):
        lact_b200.block_causal_lact_swiglu(w, w, w, x, x, x, lr, lr, lr, chunk_size=8)


def header_prototypes():
    """{name: number of parameters} for every function include/lact_b200.h declares."""
    text = open(os.path.join(ROOT, "include", "lact_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"\b(lact_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text, flags=re.S):
        params = m.group(2).strip()
        protos[m.group(1)] = 0 if params in ("", "void") else len(params.split(","))
    return protos


def test_ctypes_prototypes_match_the_header(lib):
    """Every entry point whose ctypes argument list the shim sets must list as many arguments as the header's
    prototype has parameters (a missing or extra argument would shift every later one silently)."""
    protos = header_prototypes()
    assert len(protos) >= 30
    checked = 0
    for name, n_params in protos.items():
        argtypes = getattr(getattr(lib, name), "argtypes", None)
        if argtypes is None:
            continue
        assert len(argtypes) == n_params, f"{name}: header has {n_params} parameters, the shim passes {len(argtypes)}"
        checked += 1
    assert checked >= 20
