"""ctypes loader for the C-ABI library.  Fails loudly when the library is not built."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
lib_path = os.path.join(_HERE, "liblancelot_b200.so")

LB_OK, LB_ERR_INVALID_ARG, LB_ERR_LOGIC, LB_ERR_CUDA, LB_ERR_NO_MEMORY = range(5)


class LancelotError(RuntimeError):
    """A C-ABI call failed.  ``code`` is one of the LB_ERR_* values."""

    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


class InvalidArgument(LancelotError, ValueError):
    """Raised where the reference throws std::invalid_argument (pybind maps it to ValueError)."""


def _load():
    if not os.path.exists(lib_path):
        raise ImportError(
            "liblancelot_b200.so is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU fallback)")
    return C.CDLL(lib_path, mode=C.RTLD_GLOBAL)


lib = _load()
lib.lb_last_error.restype = C.c_char_p
lib.lb_minimal_primitive_root.restype = C.c_uint64
lib.lb_minimal_primitive_root.argtypes = [C.c_uint64, C.c_uint64]
lib.lb_max_bit_count_tc128.argtypes = [C.c_uint64]
lib.lb_keyswitch_workspace_bytes.restype = C.c_size_t
lib.lb_keyswitch_workspace_bytes.argtypes = [C.c_void_p, C.c_int]
lib.lb_context_destroy.restype = None
lib.lb_context_destroy.argtypes = [C.c_void_p]


def check(code):
    """Translate a status code into the exception class the reference's binding would raise."""
    if code == LB_OK:
        return
    msg = lib.lb_last_error().decode("utf-8", "replace")
    if code == LB_ERR_INVALID_ARG:
        raise InvalidArgument(code, msg)
    raise LancelotError(code, msg)
