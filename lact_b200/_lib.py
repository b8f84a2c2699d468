"""ctypes binding of liblact_b200.so (the C ABI in include/lact_b200.h).

There is no fallback: if the shared library is missing, loading raises and every op fails.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import torch

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "liblact_b200.so")

LACT_F32, LACT_BF16 = 0, 1
RENORM_NONE, RENORM_EPS_OUTSIDE, RENORM_EPS_INSIDE = 0, 1, 2


class ScanConfig(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("B", "L", "D", "H", "out_len")] + [
        (n, C.c_int32) for n in ("act_dtype", "lr_dtype", "mom_dtype", "w_dtype", "use_momentum", "use_muon",
                                 "ns_steps", "ns_const_coeffs", "ns_concat", "ns_gram_right", "renorm", "prenorm",
                                 "prenorm_bf16", "overwrite_quirk")] + [("w_scale", C.c_float)] + [
        (n, C.c_int64) for n in ("q_bs", "q_ts", "k_bs", "k_ts", "v_bs", "v_ts", "o_bs", "o_ts")]


class ScanIO(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2", "momentum", "m0_in",
                                          "m1_in", "m2_in", "o", "w0_out", "w1_out", "w2_out", "m0_out", "m1_out",
                                          "m2_out", "state_dump", "ns_trace")]


ERR_CONFIG = -5  # LACT_ERR_CONFIG


class BmmDesc(C.Structure):
    """lact_bmm_desc of the C header."""
    _fields_ = ([(n, C.c_void_p) for n in ("a0", "b0", "a1", "b1", "c")] +
                [(n, C.c_int64) for n in ("a0_ld", "a0_bs", "b0_ld", "b0_bs", "a1_ld", "a1_bs", "b1_ld", "b1_bs",
                                          "c_ld", "c_bs", "batch", "M", "N", "K")] +
                [(n, C.c_int32) for n in ("a0_mn", "b0_mn", "a1_mn", "b1_mn", "c_dtype", "accumulate")])


class NsBwdGroup(C.Structure):
    """lact_ns_bwd_group of the C header."""
    _fields_ = [("du", C.c_void_p), ("g", C.c_void_p), ("dg", C.c_void_p), ("trace", C.c_void_p),
                ("trace_bytes", C.c_size_t), ("partials", C.c_void_p), ("nmat", C.c_int64), ("rows", C.c_int64),
                ("cols", C.c_int64)]


_lib: Optional[C.CDLL] = None


def _declare(lib: C.CDLL) -> None:
    vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
    szp = C.POINTER(C.c_size_t)
    lib.lact_version.restype = C.c_int
    lib.lact_error_string.restype = C.c_char_p
    lib.lact_error_string.argtypes = [C.c_int]
    lib.lact_read_status.argtypes = [vp, vp]
    lib.lact_stream_sync_count.restype = C.c_int64
    lib.lact_set_wait_limit_ns.argtypes = [C.c_uint64]
    lib.lact_debug_wait_timeout.argtypes = [vp, vp]
    lib.lact_static_status.argtypes = [vp]
    lib.lact_launch_count.restype = C.c_int64
    lib.lact_profile_enable.argtypes = [C.c_int]
    lib.lact_profile_enable.restype = C.c_int
    lib.lact_profile_num_classes.restype = C.c_int
    lib.lact_profile_class_name.argtypes = [C.c_int]
    lib.lact_profile_class_name.restype = C.c_char_p
    lib.lact_profile_read.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_int64)]
    lib.lact_profile_read.restype = C.c_int
    lib.lact_scan_workspace_bytes.argtypes = [C.POINTER(ScanConfig), i32, C.POINTER(i32), C.POINTER(i64),
                                              C.POINTER(i64), szp]
    lib.lact_scan_ns_trace_bytes.argtypes = [C.POINTER(ScanConfig), szp, szp]
    lib.lact_scan_ns_trace_bytes.restype = C.c_int
    lib.lact_ns_trace_result_offset.argtypes = [i64, i64, i64, i32, szp]
    lib.lact_ns_trace_result_offset.restype = C.c_int
    lib.lact_scan_fwd.argtypes = [C.POINTER(ScanConfig), C.POINTER(ScanIO), i32, C.POINTER(i32), C.POINTER(i64),
                                  C.POINTER(i64), C.POINTER(i64), vp, C.c_size_t, vp]
    lib.lact_swiglu_ffn_workspace_bytes.argtypes = [i64, i64, i64, i64, szp]
    lib.lact_swiglu_ffn_fwd.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, vp, C.c_size_t, vp]
    lib.lact_static_scratch_bytes.restype = C.c_size_t
    lib.lact_swiglu_ffn_fwd_static.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, vp]
    lib.lact_swiglu_ffn_fwd_static.restype = C.c_int
    lib.lact_fw_grad_workspace_bytes.argtypes = [i64, i64, i64, i64, szp]
    lib.lact_fw_grad.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, i64, i64, i64, i64, vp, C.c_size_t, vp]
    lib.lact_newton_schulz_workspace_bytes.argtypes = [i64, i64, i64, szp]
    lib.lact_newton_schulz.argtypes = [vp, i32, vp, i64, i64, i64, i32, i32, vp, C.c_size_t, vp]
    lib.lact_l2_norm_add.argtypes = [vp, i32, vp, i32, vp, vp, i32, i64, i64, i64, f32, vp]
    lib.lact_prenorm_momentum_l2norm.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, f32, vp]
    lib.lact_bmm_bf16.argtypes = [vp, i32, vp, i32, vp, i32, i64, i64, i64, i64, vp, vp]
    lib.lact_bmm2_bf16.argtypes = [vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, i64, i64, i64, i64, vp, vp]
    lib.lact_bmm2_strided_bf16.argtypes = [vp, i32, i64, i64, vp, i32, i64, i64, vp, i32, i64, i64, vp, i32, i64, i64, vp,
                                           i32, i64, i64, i32, i64, i64, i64, i64, vp, vp]
    lib.lact_qkv_prologue.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp]
    lib.lact_qkv_prologue_rope.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, vp, vp, vp, i64, i64, i64, i64, i32, i32,
                                           vp, vp, i64, i64, i64, vp, vp]
    lib.lact_qkv_prologue_rope.restype = C.c_int
    lib.lact_lr_prologue.argtypes = [vp, i32, i64, f32, vp, i32, i64, vp, vp, vp, vp, i64, i64, i64, vp]
    lib.lact_out_epilogue.argtypes = [vp, vp, vp, i64, vp, i64, vp, i64, i64, i64, i64, i64, f32, vp]
    lib.lact_swiglu_bwd_planes.argtypes = [vp, vp, vp, vp, vp, i32, f32, vp, vp, i64, i64, vp]
    lib.lact_fw_grad_bwd_pointwise.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, f32, vp, vp, vp, vp, vp, vp, vp, i64,
                                               i64, vp]
    lib.lact_renorm_bwd.argtypes = [vp, vp, i32, vp, vp, vp, vp, vp, i64, i64, i32, vp]
    lib.lact_ns_norm_bwd.argtypes = [vp, vp, vp, i64, i64, vp]
    lib.lact_momentum_bwd_slices.restype = C.c_int
    lib.lact_qkv_prologue_bwd.argtypes = [vp] * 3 + [i64] * 6 + [vp] * 6 + [i64] * 4 + [i32, i32, vp, vp, i64, i64, i64, vp, vp]
    lib.lact_out_epilogue_bwd_blocks.restype = C.c_int
    lib.lact_out_epilogue_bwd.argtypes = [vp, vp, vp, i64, vp, i64, vp, vp, vp, i64, i64, i64, i64, f32, vp]
    lib.lact_swa_fwd.argtypes = [vp, vp, vp, vp] + [i64] * 14 + [f32, vp, vp, vp, vp]
    lib.lact_swa_bwd.argtypes = [vp] * 10 + [i64] * 16 + [f32, vp, vp, vp]
    lib.lact_bmm_group_bf16.argtypes = [C.POINTER(BmmDesc), i32, vp, vp]
    lib.lact_fw_grad_pointwise.argtypes = [vp, vp, vp, i64, i64, vp, i64, i64, vp, vp, vp, i32, i64, f32, vp, vp, i64, i64,
                                           i64, i64, vp, vp]
    lib.lact_ns_trace_bwd_fused.argtypes = [C.POINTER(NsBwdGroup), i32, i32, i32, i32, vp, vp]
    lib.lact_ns_norm_bwd.restype = C.c_int
    lib.lact_momentum_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, vp]
    lib.lact_momentum_bwd.restype = C.c_int
    lib.lact_ns_trace_bytes.argtypes = [i64, i64, i64, i32, C.POINTER(C.c_size_t)]
    lib.lact_ns_trace_fwd.argtypes = [vp, i32, vp, i64, i64, i64, i32, i32, i32, vp, C.c_size_t, vp, vp]
    lib.lact_ns_trace_bwd.argtypes = [vp, vp, i64, i64, i64, i32, i32, i32, vp, C.c_size_t, vp, vp]
    lib.lact_sgemm_f32.argtypes = [vp, i32, vp, i32, vp, i32, vp, i64, i64, i64, i64, vp]
    lib.lact_swiglu_planes_f32.argtypes = [vp, vp, vp, vp, vp, i32, f32, vp, vp, i64, i64, vp]
    lib.lact_add_renorm.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, i32, vp]
    for name in ("lact_read_status", "lact_set_wait_limit_ns", "lact_debug_wait_timeout", "lact_static_status",
                 "lact_scan_workspace_bytes", "lact_scan_fwd", "lact_swiglu_ffn_workspace_bytes",
                 "lact_swiglu_ffn_fwd", "lact_fw_grad_workspace_bytes", "lact_fw_grad",
                 "lact_newton_schulz_workspace_bytes", "lact_newton_schulz", "lact_l2_norm_add",
                 "lact_prenorm_momentum_l2norm", "lact_bmm_bf16", "lact_bmm2_bf16", "lact_bmm2_strided_bf16", "lact_swiglu_bwd_planes",
                 "lact_fw_grad_bwd_pointwise", "lact_renorm_bwd", "lact_sgemm_f32", "lact_swiglu_planes_f32",
                 "lact_add_renorm", "lact_qkv_prologue", "lact_lr_prologue", "lact_out_epilogue", "lact_ns_trace_bytes", "lact_ns_trace_fwd", "lact_ns_trace_bwd"):
        getattr(lib, name).restype = C.c_int


def lib() -> C.CDLL:
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m lact_b200.build` "
                              "(there is no fallback implementation)")
        handle = C.CDLL(LIB_PATH)
        _declare(handle)
        _lib = handle
    return _lib


class LactError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = lib().lact_error_string(rc).decode()
    if rc in (-1, -2, -3, -5, -6):
        raise ValueError(f"{what}: {msg} (code {rc})")
    raise LactError(f"{what}: {msg} (code {rc})")


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return LACT_F32
    if t.dtype == torch.bfloat16:
        return LACT_BF16
    raise TypeError(f"unsupported dtype {t.dtype}: expected float32 or bfloat16")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


# One growing scratch buffer per (device, stream), taken from PyTorch's caching allocator.  Kernels
# of consecutive calls on one stream are ordered, so reuse is safe.
_workspaces: Dict[tuple, torch.Tensor] = {}
SYNC_CHECK = os.environ.get("LACT_B200_SYNC_CHECK", "0") == "1"


def _key(device: torch.device) -> tuple:
    return (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr())


def workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    """Scratch for one call on the current stream.  Never waits for the device."""
    key = _key(device)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


class _StatusRing:
    """Device status words of finished calls, copied to pinned host memory WITHOUT waiting.

    Every call's kernels leave a status word at the head of its workspace (0 = ok, 101 = a bounded
    wait ran out).  The next call on the stream clears that word, so right after a call has been
    enqueued an asynchronous 4-byte copy into the next slot of a pinned ring is enqueued behind
    it.  The host looks at slots whose copy has completed (an event query, no wait) whenever a
    later call is made, and at all of them in `synchronize_and_check`.  A slot is waited for only
    when the ring wraps around while its copy is still in flight (256 calls ahead of the device).
    """
    SLOTS = 256

    def __init__(self):
        self.host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
        self.events = [None] * self.SLOTS
        self.head = 0  # next slot to use
        self.tail = 0  # oldest slot not yet examined

    def _examine(self, slot: int) -> None:
        self.events[slot] = None
        st = int(self.host[slot])
        if st != 0:
            self.host[slot] = 0
            raise LactError("device status: " + lib().lact_error_string(st).decode() + f" (code {st})")

    def poll(self, wait: bool = False) -> None:
        """Examines finished slots in order; with `wait`, all of them."""
        while self.tail != self.head:
            slot = self.tail % self.SLOTS
            ev = self.events[slot]
            if ev is not None:
                if wait:
                    ev.synchronize()
                elif not ev.query():
                    return
            self.tail += 1
            self._examine(slot)

    def post(self, ws: torch.Tensor) -> None:
        if self.head - self.tail >= self.SLOTS:  # the ring is full: the oldest copy must have landed
            slot = self.tail % self.SLOTS
            if self.events[slot] is not None:
                self.events[slot].synchronize()
            self.tail += 1
            self._examine(slot)
        slot = self.head % self.SLOTS
        self.host[slot:slot + 1].copy_(ws[:4].view(torch.int32), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[slot] = ev
        self.head += 1


_rings: Dict[int, _StatusRing] = {}


def mark_pending(ws: torch.Tensor) -> None:
    """Called after a library call has been enqueued with `ws` as its workspace: arranges for the
    call's device status word to reach the host without blocking (see `_StatusRing`), and raises
    for any EARLIER call whose word has arrived non-zero.  Inside CUDA-graph stream capture
    nothing is recorded.  LACT_B200_SYNC_CHECK=1 checks synchronously instead (debugging)."""
    if torch.cuda.is_current_stream_capturing():
        return
    if SYNC_CHECK:
        read_status(ws)
        return
    idx = ws.device.index
    ring = _rings.get(idx)
    if ring is None:
        ring = _rings[idx] = _StatusRing()
    with torch.cuda.device(ws.device):
        ring.post(ws)
        ring.poll()


def read_status(ws: torch.Tensor) -> None:
    """Synchronises the current stream and raises if the workspace's status word is non-zero."""
    rc = lib().lact_read_status(ws.data_ptr(), stream_ptr())
    if rc != 0:
        raise LactError("device status: " + lib().lact_error_string(rc).decode() + f" (code {rc})")


def synchronize_and_check() -> None:
    """Waits for every status word posted so far and raises if any call recorded a device-side
    error (a bounded wait that ran out).  The op calls themselves never wait."""
    for idx, ring in list(_rings.items()):
        with torch.cuda.device(idx):
            ring.poll(wait=True)


def stream_sync_count() -> int:
    """cudaStreamSynchronize calls made inside the library in this process so far."""
    return int(lib().lact_stream_sync_count())


def nvtx_enable(on: bool = True) -> None:
    """NVTX ranges around every kernel launch of the library (named after the kernel class) on / off."""
    check(lib().lact_nvtx_enable(1 if on else 0), "lact_nvtx_enable")


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib().lact_launch_count())


def profile_enable(on: bool) -> None:
    lib().lact_profile_enable(int(on))


def profile_read() -> dict:
    """{class name: (total ms, launches)} for launches recorded since the last read."""
    n = lib().lact_profile_num_classes()
    ms = (C.c_double * n)()
    cnt = (C.c_int64 * n)()
    check(lib().lact_profile_read(ms, cnt), "lact_profile_read")
    return {lib().lact_profile_class_name(i).decode(): (ms[i], int(cnt[i])) for i in range(n) if cnt[i]}
