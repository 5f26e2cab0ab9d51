"""ctypes binding of librtp_b200.so (the hand-written sm_100a kernels).

The shared library is built in-tree by ``rtp_b200/csrc/build.py`` and loaded lazily.  On a machine
with a GPU the library is mandatory: :func:`lib` raises instead of falling back to PyTorch kernels.
"""
import ctypes as C
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "librtp_b200.so")
MAX_WORLD = 8

_lock = threading.Lock()
_lib = None


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("lda", C.c_longlong), ("a_mn", C.c_int),
        ("b", C.c_void_p), ("ldb", C.c_longlong), ("b_mn", C.c_int),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("d", C.c_void_p), ("ldd", C.c_longlong), ("d_fp32", C.c_int),
        ("c", C.c_void_p), ("ldc", C.c_longlong), ("c_fp32", C.c_int),
        ("bias", C.c_void_p), ("act", C.c_int),
        ("mask", C.c_void_p), ("ldmask", C.c_longlong), ("mask_scale", C.c_float),
        ("drop_p", C.c_float), ("seed", C.c_ulonglong), ("offset", C.c_ulonglong), ("step_ptr", C.c_void_p),
        ("status", C.c_void_p), ("num_ctas", C.c_int), ("bn", C.c_int),
    ]


class GemmBatched(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("lda", C.c_longlong), ("a_mn", C.c_int), ("a_rows", C.c_longlong), ("a_cols", C.c_longlong),
        ("b", C.c_void_p), ("ldb", C.c_longlong), ("b_mn", C.c_int), ("b_rows", C.c_longlong), ("b_cols", C.c_longlong),
        ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("batch", C.c_int), ("batch_inner", C.c_int),
        ("a_bo_mn", C.c_int), ("a_bo_k", C.c_int), ("a_bi_mn", C.c_int), ("a_bi_k", C.c_int),
        ("b_bo_mn", C.c_int), ("b_bo_k", C.c_int), ("b_bi_mn", C.c_int), ("b_bi_k", C.c_int),
        ("d", C.c_void_p), ("ldd", C.c_longlong), ("d_bo", C.c_longlong), ("d_bi", C.c_longlong),
        ("alpha", C.c_float), ("causal", C.c_int), ("bn", C.c_int), ("status", C.c_void_p),
    ]


class Ring(C.Structure):
    _fields_ = [
        ("rank", C.c_int), ("world", C.c_int),
        ("ws", C.c_void_p * MAX_WORLD),
        ("slot_bytes", C.c_ulonglong),
        ("ctas", C.c_int),
        ("timeout_ns", C.c_ulonglong),
    ]


class LinearFwd(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("M", C.c_int), ("in_features", C.c_int), ("out_features", C.c_int),
        ("home", C.c_void_p), ("bias_off", C.c_longlong), ("shard_bytes", C.c_ulonglong),
        ("x", C.c_void_p), ("ldx", C.c_longlong),
        ("y", C.c_void_p), ("ldy", C.c_longlong),
        ("act", C.c_int),
        ("drop_p", C.c_float), ("seed", C.c_ulonglong), ("offset", C.c_ulonglong), ("step_ptr", C.c_void_p),
        ("bank", C.c_int), ("no_self_push", C.c_int),
        ("next_home", C.c_void_p), ("next_bytes", C.c_ulonglong), ("next_kind", C.c_int),
    ]


class LinearBwd(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("M", C.c_int), ("in_features", C.c_int), ("out_features", C.c_int),
        ("home", C.c_void_p), ("bias_off", C.c_longlong), ("shard_bytes", C.c_ulonglong),
        ("x", C.c_void_p), ("ldx", C.c_longlong),
        ("dy", C.c_void_p), ("ldy", C.c_longlong),
        ("dx", C.c_void_p), ("lddx", C.c_longlong),
        ("grad_home", C.c_void_p),
        ("dbias_full", C.c_void_p),
        ("mask", C.c_void_p), ("ldmask", C.c_longlong), ("mask_scale", C.c_float),
        ("dx_accumulate", C.c_int), ("grad_accumulate", C.c_int),
        ("bank", C.c_int), ("no_self_push", C.c_int),
        ("next_home", C.c_void_p), ("next_bytes", C.c_ulonglong), ("next_kind", C.c_int),
        ("ones", C.c_void_p),
    ]


class EmbedFwd(C.Structure):
    _fields_ = [
        ("home", C.c_void_p), ("shard_bytes", C.c_ulonglong),
        ("V", C.c_int), ("Ds", C.c_int), ("D", C.c_int),
        ("ids", C.c_void_p), ("T", C.c_int),
        ("out", C.c_void_p), ("ld_out", C.c_longlong),
        ("scale", C.c_float),
        ("pe", C.c_void_p), ("ld_pe", C.c_longlong), ("tokens_per_pos", C.c_int),
        ("drop_p", C.c_float), ("seed", C.c_ulonglong), ("offset", C.c_ulonglong), ("step_ptr", C.c_void_p),
    ]


class ExpertFwd(C.Structure):
    _fields_ = [
        ("cap", C.c_int), ("n_local", C.c_int), ("in_features", C.c_int), ("out_features", C.c_int),
        ("home", C.c_void_p), ("expert_stride", C.c_longlong), ("bias_off", C.c_longlong), ("shard_bytes", C.c_ulonglong),
        ("x", C.c_void_p), ("ldx", C.c_longlong), ("y", C.c_void_p), ("ldy", C.c_longlong), ("act", C.c_int),
    ]


class ExpertBwd(C.Structure):
    _fields_ = [
        ("cap", C.c_int), ("n_local", C.c_int), ("in_features", C.c_int), ("out_features", C.c_int),
        ("home", C.c_void_p), ("expert_stride", C.c_longlong), ("bias_off", C.c_longlong), ("shard_bytes", C.c_ulonglong),
        ("x", C.c_void_p), ("ldx", C.c_longlong), ("dy", C.c_void_p), ("ldy", C.c_longlong),
        ("dx", C.c_void_p), ("lddx", C.c_longlong), ("grad_home", C.c_void_p), ("dbias_full", C.c_void_p),
        ("mask", C.c_void_p), ("ldmask", C.c_longlong), ("mask_scale", C.c_float),
    ]


class FlashRef(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("sb", C.c_longlong), ("ss", C.c_longlong), ("width", C.c_longlong),
                ("col_base", C.c_int), ("hpg", C.c_int), ("gstride", C.c_int), ("hstride", C.c_int)]


class FlashArgs(C.Structure):
    _fields_ = [
        ("q", FlashRef), ("k", FlashRef), ("v", FlashRef), ("o", FlashRef),
        ("dout", FlashRef), ("dq", FlashRef), ("dk", FlashRef), ("dv", FlashRef),
        ("lse", C.c_void_p), ("delta", C.c_void_p),
        ("B", C.c_int), ("H", C.c_int), ("Sq", C.c_int), ("Sk", C.c_int), ("head_dim", C.c_int), ("causal", C.c_int),
        ("mask", C.c_void_p), ("mask_ld", C.c_longlong), ("mask_fp32", C.c_int),
        ("kpm", C.c_void_p), ("kpm_ld", C.c_longlong),
        ("sm_scale", C.c_float),
        ("drop_p", C.c_float), ("seed", C.c_ulonglong), ("offset", C.c_ulonglong), ("step_ptr", C.c_void_p),
        ("status", C.c_void_p),
    ]


class ReduceBlocks(C.Structure):
    _fields_ = [("src", C.c_void_p), ("block_elems", C.c_longlong), ("out", C.c_void_p)]


class ReduceScatter(C.Structure):
    _fields_ = [("src", C.c_void_p), ("ld", C.c_longlong), ("rows", C.c_int), ("cols", C.c_int), ("out", C.c_void_p)]


def available() -> bool:
    """True when the compiled library exists and a CUDA device is present."""
    return os.path.exists(LIB_PATH) and torch.cuda.is_available()


def lib():
    """Load (once) and return the ctypes handle. Raises if the library is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m rtp_b200.csrc.build` "
                "(the CUDA kernels are mandatory on a GPU machine; there is no PyTorch fallback)")
        L = C.CDLL(LIB_PATH)
        L.rtp_last_error.restype = C.c_char_p
        L.rtp_ws_bytes_world.restype = C.c_ulonglong
        L.rtp_ws_bytes_world.argtypes = [C.c_ulonglong, C.c_int]
        L.rtp_ws_wslot.restype = C.c_void_p
        L.rtp_ws_wslot.argtypes = [C.c_void_p, C.c_ulonglong, C.c_int, C.c_int]
        L.rtp_ws_gslot.restype = C.c_void_p
        L.rtp_ws_gslot.argtypes = [C.c_void_p, C.c_ulonglong, C.c_int, C.c_int]
        L.rtp_ws_create_world.argtypes = [C.c_ulonglong, C.c_int, C.POINTER(C.c_void_p)]
        L.rtp_ws_destroy.argtypes = [C.c_void_p]
        L.rtp_ws_reset.argtypes = [C.c_void_p, C.c_void_p]
        L.rtp_ws_ipc_get.argtypes = [C.c_void_p, C.c_void_p]
        L.rtp_ws_ipc_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        L.rtp_ws_ipc_close.argtypes = [C.c_void_p]
        L.rtp_ws_status.argtypes = [C.c_void_p, C.POINTER(C.c_ulonglong), C.c_void_p]
        L.rtp_ws_counters.argtypes = [C.c_void_p, C.POINTER(C.c_ulonglong), C.c_void_p]
        L.rtp_ws_num_counters.restype = C.c_int
        L.rtp_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        L.rtp_gemm_batched.argtypes = [C.POINTER(GemmBatched), C.c_void_p]
        L.rtp_linear_fwd.argtypes = [C.POINTER(Ring), C.POINTER(LinearFwd), C.c_void_p]
        L.rtp_linear_bwd.argtypes = [C.POINTER(Ring), C.POINTER(LinearBwd), C.c_void_p]
        L.rtp_embed_fwd_rot.argtypes = [C.POINTER(Ring), C.POINTER(EmbedFwd), C.c_void_p]
        L.rtp_reduce_scatter_cols.argtypes = [C.POINTER(Ring), C.POINTER(ReduceScatter), C.c_void_p]
        L.rtp_embed_fwd_rot_emu.argtypes = [C.POINTER(Ring), C.POINTER(EmbedFwd), C.c_int, C.c_void_p]
        L.rtp_reduce_blocks.argtypes = [C.POINTER(Ring), C.POINTER(ReduceBlocks), C.c_void_p]
        L.rtp_reduce_blocks_emu.argtypes = [C.POINTER(Ring), C.POINTER(ReduceBlocks), C.c_int, C.c_void_p]
        L.rtp_reduce_scatter_cols_emu.argtypes = [C.POINTER(Ring), C.POINTER(ReduceScatter), C.c_int, C.c_void_p]
        L.rtp_expert_fwd.argtypes = [C.POINTER(Ring), C.POINTER(ExpertFwd), C.c_void_p]
        L.rtp_expert_bwd.argtypes = [C.POINTER(Ring), C.POINTER(ExpertBwd), C.c_void_p]
        L.rtp_expert_fwd_emu.argtypes = [C.POINTER(Ring), C.POINTER(ExpertFwd), C.c_int, C.c_void_p]
        L.rtp_expert_bwd_emu.argtypes = [C.POINTER(Ring), C.POINTER(ExpertBwd), C.c_int, C.c_void_p]
        L.rtp_set_pair_mode.argtypes = [C.c_int]
        L.rtp_shift_staging_bytes.restype = C.c_ulonglong
        L.rtp_shift_staging_bytes.argtypes = [C.c_int]
        L.rtp_shift_staging_create.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
        L.rtp_shift_staging_destroy.argtypes = [C.c_void_p]
        L.rtp_ring_shift.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.c_ulonglong, C.POINTER(C.c_void_p),
                                     C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_int,
                                     C.POINTER(C.c_void_p), C.c_ulonglong, C.c_void_p]
        L.rtp_shift_last_error.restype = C.c_char_p
        L.rtp_flash_fwd.argtypes = [C.POINTER(FlashArgs), C.c_void_p]
        L.rtp_flash_bwd.argtypes = [C.POINTER(FlashArgs), C.c_void_p]
        L.rtp_flash_last_error.restype = C.c_char_p
        L.rtp_linear_fwd_emu.argtypes = [C.POINTER(Ring), C.POINTER(LinearFwd), C.c_int, C.c_void_p]
        L.rtp_linear_bwd_emu.argtypes = [C.POINTER(Ring), C.POINTER(LinearBwd), C.c_int, C.c_void_p]
        L.rtp_linear_bwd_folds_bias.argtypes = [C.POINTER(Ring), C.POINTER(LinearBwd)]
        _lib = L
    return _lib


launches = 0      # calls into the library that launched kernels (every entry point launches at least one)
_serialize = os.environ.get("RTP_SERIALIZE", "0") not in ("", "0")
_after_launch_hooks = []     # callables run after every launch in serialised mode (the engines register their checks)
_checking = False            # the checks themselves call into the library: no nesting


def set_serialize(on: bool) -> bool:
    """Serialised (bisect) mode: after every library launch the stream is synchronised and every status word is
    read, so the first launch whose bounded wait ran out is named in the exception instead of surfacing at the next
    ``check``.  Also switched on by ``RTP_SERIALIZE=1``.  Has no effect while a CUDA graph is being captured."""
    global _serialize
    old, _serialize = _serialize, bool(on)
    return old


def check(rc: int, what: str):
    global launches, _checking
    launches += 1
    if rc != 0:
        msg = lib().rtp_last_error()
        raise RuntimeError(f"{what} failed: {msg.decode() if msg else rc}")
    if _serialize and not _checking and not torch.cuda.is_current_stream_capturing():
        torch.cuda.synchronize()
        _checking = True
        try:
            for w in list(_status_words.values()):
                v = int(w.item())
                if v:
                    w.zero_()
                    raise RotationTimeout(status_text(v))
            for hook in _after_launch_hooks:
                hook()
        except RotationTimeout as e:
            raise RotationTimeout(f"{what}: {e}") from None
        finally:
            _checking = False


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_status_words = {}


def status_word(device=None) -> torch.Tensor:
    """A per-device int64 word that kernels outside a ring use to report bounded-wait expiries."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index)
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int64, device=dev)
        _status_words[key] = w
    return w


STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "wait for a peer's data timed out",
                3: "wait for a peer's free slot timed out", 4: "bad argument"}


def status_text(v: int) -> str:
    """Status word of a kernel in words.  A bad-argument code from the rotation GEMM's producer carries the phase and the
    two offending copy coordinates in its upper bits."""
    if (v & 0xff) == 4 and v > 0xff:
        return (f"bad argument: unaligned copy coordinate in phase {(v >> 8) & 0xff} "
                f"(A x = {(v >> 16) & 0xfffff}, B x = {(v >> 40) & 0xfffff})")
    return STATUS_NAMES.get(v, f"status {v}")


class RotationTimeout(RuntimeError):
    """A bounded device-side wait expired; the kernel returned early and its outputs are invalid."""


def check_status(device=None):
    """Synchronously read the status word and raise RotationTimeout if a kernel reported an error."""
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RotationTimeout(status_text(v))
