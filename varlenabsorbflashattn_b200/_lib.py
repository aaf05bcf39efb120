"""ctypes binding of libvafa_b200.so (the C ABI declared in include/vafa.h).

There is no fallback: if the shared library is missing or a call fails, a RuntimeError is
raised.  Nothing here computes anything.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# VAFA_LIB_PATH points at a library built elsewhere (another build variant, an installed copy)
LIB_PATH = os.environ.get("VAFA_LIB_PATH") or os.path.join(_PKG, "libvafa_b200.so")

VAFA_F32, VAFA_BF16, VAFA_F16 = 0, 1, 2
IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05 = 0, 1, 2
IMPL_NAMES = {"auto": IMPL_AUTO, "simt": IMPL_SIMT, "tcgen05": IMPL_TCGEN05}
STATUS_WORDS = 4

DTYPE_CODE = {torch.float32: VAFA_F32, torch.bfloat16: VAFA_BF16, torch.float16: VAFA_F16}

EXPORTS = (
    "vafa_abi_version", "vafa_last_error", "vafa_check_status", "vafa_cast_from_f32",
    "vafa_varlen_fwd_workspace_bytes", "vafa_varlen_bwd_workspace_bytes", "vafa_varlen_fwd", "vafa_varlen_bwd",
    "vafa_varlen_fwd_noalloc",
    "vafa_absorb_saved_bytes", "vafa_absorb_fwd_workspace_bytes", "vafa_absorb_bwd_workspace_bytes",
    "vafa_absorb_fwd", "vafa_absorb_bwd", "vafa_absorb_bwd_phase", "vafa_absorb_inner_fwd", "vafa_absorb_inner_bwd",
    "vafa_profile_enable", "vafa_profile_kernel_count", "vafa_profile_kernel_name", "vafa_profile_read",
    "vafa_profile_reset", "vafa_set_wait_limit_cycles", "vafa_selftest_bounded_wait", "vafa_set_varlen_bwd_mode",
)


class VarlenArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("lse", C.c_void_p),
        ("d_o", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("n_seg", C.c_int32), ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("num_heads", C.c_int32), ("head_dim", C.c_int32), ("dtype", C.c_int32), ("causal", C.c_int32),
        ("scale", C.c_float), ("impl", C.c_int32), ("split_k_block", C.c_int32), ("sm_count", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
        ("num_kv_heads", C.c_int32),
    ]


class AbsorbArgs(C.Structure):
    _fields_ = [
        ("q_raw", C.c_void_p), ("x", C.c_void_p), ("w_q", C.c_void_p), ("w_k", C.c_void_p), ("w_v", C.c_void_p),
        ("o", C.c_void_p), ("lse", C.c_void_p), ("saved", C.c_void_p), ("d_o", C.c_void_p),
        ("dq_raw", C.c_void_p), ("dx", C.c_void_p), ("dw", C.c_void_p),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("n_seg", C.c_int32), ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("d_q", C.c_int32), ("d_kv", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("scale", C.c_float), ("impl", C.c_int32), ("sm_count", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
        ("x_width", C.c_int32),
    ]


_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m varlenabsorbflashattn_b200.build` "
                "(there is no fallback implementation)")
        lib = C.CDLL(LIB_PATH)
        lib.vafa_abi_version.restype = C.c_int
        lib.vafa_last_error.restype = C.c_char_p
        lib.vafa_check_status.argtypes = [C.c_void_p, C.c_void_p]
        lib.vafa_check_status.restype = C.c_int
        lib.vafa_cast_from_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int32, C.c_void_p]
        lib.vafa_cast_from_f32.restype = C.c_int
        for name in ("vafa_varlen_fwd_workspace_bytes", "vafa_varlen_bwd_workspace_bytes"):
            getattr(lib, name).argtypes = [C.POINTER(VarlenArgs)]
            getattr(lib, name).restype = C.c_size_t
        for name in ("vafa_varlen_fwd", "vafa_varlen_bwd", "vafa_varlen_fwd_noalloc"):
            getattr(lib, name).argtypes = [C.POINTER(VarlenArgs), C.c_void_p]
            getattr(lib, name).restype = C.c_int
        for name in ("vafa_absorb_saved_bytes", "vafa_absorb_fwd_workspace_bytes", "vafa_absorb_bwd_workspace_bytes"):
            getattr(lib, name).argtypes = [C.POINTER(AbsorbArgs)]
            getattr(lib, name).restype = C.c_size_t
        for name in ("vafa_absorb_fwd", "vafa_absorb_bwd", "vafa_absorb_inner_fwd", "vafa_absorb_inner_bwd"):
            getattr(lib, name).argtypes = [C.POINTER(AbsorbArgs), C.c_void_p]
            getattr(lib, name).restype = C.c_int
        lib.vafa_absorb_bwd_phase.argtypes = [C.POINTER(AbsorbArgs), C.c_int32, C.c_void_p]
        lib.vafa_absorb_bwd_phase.restype = C.c_int
        lib.vafa_set_varlen_bwd_mode.argtypes = [C.c_int]
        lib.vafa_set_varlen_bwd_mode.restype = C.c_int
        lib.vafa_set_wait_limit_cycles.argtypes = [C.c_longlong]
        lib.vafa_set_wait_limit_cycles.restype = C.c_longlong
        lib.vafa_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_void_p]
        lib.vafa_selftest_bounded_wait.restype = C.c_int
        lib.vafa_profile_enable.argtypes = [C.c_int]
        lib.vafa_profile_kernel_name.argtypes = [C.c_int]
        lib.vafa_profile_kernel_name.restype = C.c_char_p
        lib.vafa_profile_read.argtypes = [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_longlong),
                                          C.POINTER(C.c_longlong)]
        if lib.vafa_abi_version() != 3:
            raise RuntimeError("libvafa_b200.so: ABI version mismatch; rebuild")
        _lib = lib
    return _lib


def last_error() -> str:
    return load().vafa_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")


_status = {}
_sm_count = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] that kernels write error codes into (zeroed once)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    t = _status.get(key)
    if t is None:
        t = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _sm_count.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _sm_count[idx] = n
    return n


def check_status(device: torch.device) -> None:
    """Synchronise the current stream and raise if a kernel reported an error."""
    st = status_word(device)
    rc = load().vafa_check_status(st.data_ptr(), torch.cuda.current_stream(device).cuda_stream)
    if rc != 0:
        msg = last_error()
        st.zero_()
        raise RuntimeError(f"device-side error: {msg}")


_check_after_each_op = os.environ.get("VAFA_CHECK_STATUS", "0").lower() in ("1", "true", "on", "yes")


def set_check_status(enabled: bool) -> None:
    """Read the device status word after every operator call (off by default; also VAFA_CHECK_STATUS=1).

    The kernels report device-side failures -- a bounded wait that ran out, a tile list that did not fit
    its buffers -- by writing a code to a status word instead of trapping, and the outputs of such a call
    are undefined.  Reading the word needs a stream synchronisation, which is why it is opt-in: with it on,
    every `packed_varlen_attn` / `packed_target_attn` call (forward and backward) synchronises and raises
    RuntimeError on a reported failure, much as the reference's cu_seqlens validation synchronises.  With it
    off, call `check_status(device)` yourself at a point where a synchronisation is acceptable (once per
    step, say)."""
    global _check_after_each_op
    _check_after_each_op = bool(enabled)


def maybe_check_status(device: torch.device) -> None:
    if _check_after_each_op:
        check_status(device)


def workspace(nbytes: int, device: torch.device) -> torch.Tensor | None:
    if nbytes <= 0:
        return None
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def profile_enable(on: bool) -> None:
    load().vafa_profile_enable(1 if on else 0)


def profile_reset() -> None:
    load().vafa_profile_reset()


def profile_read() -> dict:
    """{kernel name: (total_ms over timed launches, timed launches, all launches)}; waits for the events."""
    lib = load()
    out = {}
    for i in range(lib.vafa_profile_kernel_count()):
        ms, nt, na = C.c_double(0), C.c_longlong(0), C.c_longlong(0)
        lib.vafa_profile_read(i, C.byref(ms), C.byref(nt), C.byref(na))
        if na.value:
            out[lib.vafa_profile_kernel_name(i).decode()] = (ms.value, nt.value, na.value)
    return out
