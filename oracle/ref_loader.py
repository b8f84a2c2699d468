"""Loads the reference's own Python functions for this path, in place, on CPU, in eager mode.

TEST INFRASTRUCTURE ONLY (fixture generation and oracle pinning).  The reference tree is not
part of this repository and does not exist on a GPU box: callers must check `available()`.
Nothing is copied: modules are imported from where the reference lies.

* `torch.compile` cannot build on this image, so TORCHDYNAMO_DISABLE=1 is set before import
  (the decorated functions then run as plain eager PyTorch).
* The two autoregressive-video block modules import packages that are not installed, so only
  their four chunk functions are taken: the file is parsed with `ast`, the wanted
  `FunctionDef`s are compiled with their decorators stripped, and executed in a namespace that
  holds `torch`, `F` and the helpers from the reference's own `functions.py`.
"""
from __future__ import annotations

import ast
import importlib.util
import os
import sys
import types

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

# where the reference tree lives: LACT_REFERENCE_ROOT, else a `reference` directory beside this repository
REF_ROOT = os.environ.get("LACT_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def available() -> bool:
    return os.path.isdir(os.path.join(REF_ROOT, "lact_llm"))


def _load(name: str, rel: str) -> types.ModuleType:
    path = os.path.join(REF_ROOT, rel)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_cache: dict = {}


def llm_unfused():
    """lact_llm/lact_model/ttt_operation.py"""
    if "llm" not in _cache:
        _cache["llm"] = _load("_ref_ttt_operation", "lact_llm/lact_model/ttt_operation.py")
    return _cache["llm"]


def bidirectional():
    """minimal_implementations/bidirectional_lact_layer.py"""
    if "bidi" not in _cache:
        _cache["bidi"] = _load("_ref_bidirectional", "minimal_implementations/bidirectional_lact_layer.py")
    return _cache["bidi"]


def nvs():
    """lact_nvs/lact_ttt.py"""
    if "nvs" not in _cache:
        _cache["nvs"] = _load("_ref_lact_ttt", "lact_nvs/lact_ttt.py")
    return _cache["nvs"]


def ar_functions():
    """lact_ar_video/minVid/models/blocks/functions.py"""
    if "arf" not in _cache:
        _cache["arf"] = _load("_ref_ar_functions", "lact_ar_video/minVid/models/blocks/functions.py")
    return _cache["arf"]


def _extract(rel: str, names) -> dict:
    path = os.path.join(REF_ROOT, rel)
    with open(path) as fh:
        tree = ast.parse(fh.read(), filename=path)
    picked = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            node.decorator_list = []
            picked.append(node)
    module = ast.Module(body=picked, type_ignores=[])
    ast.fix_missing_locations(module)
    fn = ar_functions()
    ns = {"torch": torch, "F": F, "silu_backprop": fn.silu_backprop,
          "zeropower_via_newtonschulz5": fn.zeropower_via_newtonschulz5, "l2_norm": fn.l2_norm}
    exec(compile(module, path, "exec"), ns)
    return {n: ns[n] for n in names}


def ar_ops() -> dict:
    """The four autoregressive-video chunk functions (ar_lact_swa_repeat.py, ar_lact_swa_repeat_sp.py)."""
    if "ar" not in _cache:
        d = _extract("lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py",
                     ["ar_fast_weight_swish_glu_weight_norm_mini_batch",
                      "ar_fast_weight_swish_glu_weight_norm_mini_batch_inference"])
        d.update(_extract("lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat_sp.py",
                          ["ar_fast_weight_swish_glu_weight_norm_mini_batch_with_momentum",
                           "ar_fast_weight_swish_glu_weight_norm_mini_batch_inference_with_momentum"]))
        _cache["ar"] = d
    return _cache["ar"]


def fused_helpers() -> dict:
    """The in-file PyTorch reference functions of the fused sub-ops (lact_triton_kernels/*)."""
    if "fh" not in _cache:
        sys.path.insert(0, os.path.join(REF_ROOT, "lact_llm"))
        import lact_model.lact_triton_kernels.lact_swiglu_ffn as ffn
        import lact_model.lact_triton_kernels.lact_fw_grad as fg
        import lact_model.lact_triton_kernels.l2norm_triton_kernels as l2
        import lact_model.lact_triton_kernels.triton_prenorm_update_with_momentum as pm
        _cache["fh"] = dict(
            reference_swiglu_ffn_fwd=ffn.reference_swiglu_ffn_fwd,
            reference_lact_swiglu_ffn_fast_weight_grads=fg.reference_lact_swiglu_ffn_fast_weight_grads,
            reference_l2_norm_add_fused=l2.reference_l2_norm_add_fused,
            reference_l2_norm_add_fused_with_momentum=pm.reference_l2_norm_add_fused_with_momentum,
            pytorch_swiglu_bwd_bwd_fused_cat_inp_out=fg.pytorch_swiglu_bwd_bwd_fused_cat_inp_out,
        )
    return _cache["fh"]
