"""ctypes binding of the C ABI declared in include/flashmhf.h.

There is no fallback: if the shared library is missing or its ABI version differs, loading raises."""
import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLASHMHF_LIB") or os.path.join(_PKG, "lib", "libflashmhf_b200.so")   # FLASHMHF_LIB: another build of the same ABI
ABI_VERSION = 3

BF16, F32_CHECK = 0, 1
BWD_INPUTS, BWD_WEIGHTS = 1, 2      # flashmhf_bwd_params.parts
SELFTEST_CODE = 9901                # status code of flashmhf_selftest_bounded_wait
STATIC_SCRATCH_BYTES = 72 << 20

EXPORTS = ("flashmhf_abi_version", "flashmhf_forward_workspace_bytes", "flashmhf_strerror", "flashmhf_last_cuda_error", "flashmhf_forward", "flashmhf_forward_chained",
           "flashmhf_backward_workspace_bytes", "flashmhf_backward", "flashmhf_device_status",
           "flashmhf_launch_count", "flashmhf_profile_begin", "flashmhf_profile_end",
           "flashmhf_backward_static_scratch", "flashmhf_prologue_forward",
           "flashmhf_prologue_backward_workspace_bytes", "flashmhf_prologue_backward", "flashmhf_lm_rope",
           "flashmhf_lm_rmsnorm_forward", "flashmhf_lm_rmsnorm_backward_workspace_bytes", "flashmhf_lm_rmsnorm_backward",
           "flashmhf_selftest_bounded_wait")


class Tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride", C.c_int64 * 3)]


class Dims(C.Structure):
    _fields_ = [("B", C.c_int32), ("H", C.c_int32), ("S", C.c_int32), ("Dh", C.c_int32),
                ("Hkuv", C.c_int32), ("E", C.c_int32), ("De", C.c_int32), ("dtype", C.c_int32)]


class Scaling(C.Structure):
    _fields_ = [("head_scaling", C.c_float), ("up_scaling", C.c_float), ("final_scaling", C.c_float)]


NO_SCALING = (1.0, 1.0, 1.0)


class FwdParams(C.Structure):
    _fields_ = [("d", Dims), ("Q", Tensor), ("K", Tensor), ("U", Tensor), ("V", Tensor), ("R", Tensor), ("O", Tensor),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("scale", Scaling)]


class BwdParams(C.Structure):
    _fields_ = [("d", Dims), ("Q", Tensor), ("K", Tensor), ("U", Tensor), ("V", Tensor), ("R", Tensor),
                ("dO", Tensor), ("dQ", Tensor), ("dK", Tensor), ("dU", Tensor), ("dV", Tensor), ("dR", Tensor),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("scale", Scaling), ("parts", C.c_uint32)]


class PrologueParams(C.Structure):
    _fields_ = [("B", C.c_int32), ("S", C.c_int32), ("H", C.c_int32), ("Dh", C.c_int32), ("E", C.c_int32),
                ("eps", C.c_float), ("X", C.c_void_p), ("x_token_stride", C.c_int64), ("norm_weight", C.c_void_p),
                ("router", C.c_void_p), ("Q", C.c_void_p), ("R", C.c_void_p)]


class PrologueBwdParams(C.Structure):
    _fields_ = [("fwd", PrologueParams), ("dQ", C.c_void_p), ("dq_stride", C.c_int64 * 3), ("dR", C.c_void_p),
                ("dX", C.c_void_p), ("d_router", C.c_void_p), ("d_norm_weight", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class FlashMHFError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"flashmhf status {status}: {msg}")
        self.status = status


_lock = threading.Lock()
_lib = None


def load():
    """Load (once) and return the library handle with argtypes set."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is not built; run `python -m flashmhf_b200.build` "
                              "(there is no non-CUDA fallback)")
        lib = C.CDLL(LIB_PATH)
        lib.flashmhf_abi_version.restype = C.c_int
        if lib.flashmhf_abi_version() != ABI_VERSION:
            raise ImportError(f"{LIB_PATH}: ABI version {lib.flashmhf_abi_version()} != {ABI_VERSION}; rebuild")
        lib.flashmhf_strerror.restype = C.c_char_p
        lib.flashmhf_strerror.argtypes = [C.c_int]
        lib.flashmhf_last_cuda_error.restype = C.c_char_p
        lib.flashmhf_forward.restype = C.c_int
        lib.flashmhf_forward.argtypes = [C.POINTER(FwdParams), C.c_void_p]
        lib.flashmhf_forward_chained.restype = C.c_int
        lib.flashmhf_forward_chained.argtypes = [C.POINTER(FwdParams), C.c_void_p]
        lib.flashmhf_forward_workspace_bytes.restype = C.c_size_t
        lib.flashmhf_forward_workspace_bytes.argtypes = [C.POINTER(Dims)]
        lib.flashmhf_backward_workspace_bytes.restype = C.c_size_t
        lib.flashmhf_backward_workspace_bytes.argtypes = [C.POINTER(Dims)]
        lib.flashmhf_backward.restype = C.c_int
        lib.flashmhf_backward.argtypes = [C.POINTER(BwdParams), C.c_void_p]
        lib.flashmhf_backward_static_scratch.restype = C.c_int
        lib.flashmhf_backward_static_scratch.argtypes = [C.POINTER(BwdParams), C.c_void_p]
        lib.flashmhf_prologue_forward.restype = C.c_int
        lib.flashmhf_prologue_forward.argtypes = [C.POINTER(PrologueParams), C.c_void_p]
        lib.flashmhf_prologue_backward_workspace_bytes.restype = C.c_size_t
        lib.flashmhf_prologue_backward_workspace_bytes.argtypes = [C.POINTER(PrologueParams)]
        lib.flashmhf_prologue_backward.restype = C.c_int
        lib.flashmhf_prologue_backward.argtypes = [C.POINTER(PrologueBwdParams), C.c_void_p]
        lib.flashmhf_lm_rope.restype = C.c_int
        lib.flashmhf_lm_rope.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]
        lib.flashmhf_lm_rmsnorm_forward.restype = C.c_int
        lib.flashmhf_lm_rmsnorm_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_void_p]
        lib.flashmhf_lm_rmsnorm_backward_workspace_bytes.restype = C.c_size_t
        lib.flashmhf_lm_rmsnorm_backward_workspace_bytes.argtypes = [C.c_int64, C.c_int32]
        lib.flashmhf_lm_rmsnorm_backward.restype = C.c_int
        lib.flashmhf_lm_rmsnorm_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                     C.c_size_t, C.c_int64, C.c_int32, C.c_float, C.c_void_p]
        lib.flashmhf_selftest_bounded_wait.restype = C.c_int
        lib.flashmhf_selftest_bounded_wait.argtypes = [C.c_longlong, C.c_void_p]
        lib.flashmhf_device_status.restype = C.c_int
        lib.flashmhf_device_status.argtypes = [C.POINTER(C.c_int)]
        lib.flashmhf_launch_count.restype = C.c_uint64
        lib.flashmhf_profile_begin.restype = C.c_int
        lib.flashmhf_profile_begin.argtypes = [C.c_int]
        lib.flashmhf_profile_end.restype = C.c_int
        lib.flashmhf_profile_end.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int)]
        _lib = lib
        return lib


def check(status):
    """Raise FlashMHFError for a non-zero status."""
    if status != 0:
        lib = load()
        msg = lib.flashmhf_strerror(status).decode()
        if status == -8:
            msg += ": " + lib.flashmhf_last_cuda_error().decode()
        raise FlashMHFError(status, msg)


def device_status():
    """Synchronise the current device and raise if a kernel gave up on a bounded wait since the last call.

    The launch whose wait ran out left its outputs unwritten; later launches ran normally.  Reading clears the word."""
    code = C.c_int(0)
    st = load().flashmhf_device_status(C.byref(code))
    if st != 0:
        lib = load()
        err = FlashMHFError(st, lib.flashmhf_strerror(st).decode() + f" (kernel/wait code {code.value})")
        err.code = code.value
        raise err


def launch_count():
    return int(load().flashmhf_launch_count())


PROFILE_TAGS = {1: "fwd_kernel", 2: "bwd_dq_kernel", 3: "bwd_dw_kernel", 4: "dw_reduce_kernel", 5: "o_reduce_kernel",
                6: "prologue_fwd_kernel", 7: "prologue_bwd_kernel", 8: "prologue_reduce_kernel"}


def profile_begin(max_marks=4096):
    check(load().flashmhf_profile_begin(max_marks))


def profile_end(capacity=4096):
    """Synchronise and return {kernel name: [durations in ms]} for every kernel launched since profile_begin."""
    ms = (C.c_float * capacity)()
    tags = (C.c_int * capacity)()
    n = C.c_int(0)
    check(load().flashmhf_profile_end(ms, tags, capacity, C.byref(n)))
    out = {}
    for i in range(n.value):
        out.setdefault(PROFILE_TAGS.get(tags[i], str(tags[i])), []).append(float(ms[i]))
    return out
