"""ctypes binding of librsfa_b200.so (the C ABI declared in include/rsfa.h).

There is no fallback: if the shared library is missing the import of the
operator module fails with instructions to build it.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librsfa_b200.so")

RSFA_OK = 0
RSFA_ERR_INVALID_ARGUMENT = -1
RSFA_ERR_UNSUPPORTED = -2
RSFA_ERR_CUDA = -3
RSFA_ERR_DEVICE_STATUS = -4
RSFA_ERR_NO_DEVICE = -5
RSFA_ERR_TOO_LARGE = -6
RSFA_DTYPE_F16 = 0
RSFA_DTYPE_BF16 = 1
RSFA_PATH_GENERIC = 0
RSFA_PATH_TCGEN05 = 1

# name -> (restype, argtypes); mirrors include/rsfa.h one to one
_c = ctypes
SIGNATURES = {
    "rsfa_fwd": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                            _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_int64),
                            _c.c_int, _c.c_float, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "rsfa_fwd_host": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                 _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_float,
                                 _c.c_int, _c.c_int, _c.c_int, _c.c_int]),
    "rsfa_fwd_noalloc": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                    _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_int64),
                                    _c.c_int, _c.c_float, _c.c_int, _c.c_void_p]),
    "rsfa_get_tiling": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                   _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "rsfa_select_path": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.c_float, _c.c_int, _c.c_int,
                                    _c.c_int, _c.POINTER(_c.c_int), _c.POINTER(_c.c_int),
                                    _c.POINTER(_c.c_int)]),
    "rsfa_work_items": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_float,
                                   _c.POINTER(_c.c_longlong)]),
    "rsfa_sm_count": (_c.c_int, [_c.c_int]),
    "rsfa_device_status": (_c.c_int, [_c.c_int, _c.POINTER(_c.c_int)]),
    "rsfa_launch_count": (_c.c_longlong, []),
    "rsfa_set_option": (_c.c_int, [_c.c_char_p, _c.c_longlong]),
    "rsfa_get_option": (_c.c_longlong, [_c.c_char_p]),
    "rsfa_strerror": (_c.c_char_p, [_c.c_int]),
    "rsfa_version": (_c.c_int, []),
}

_lib = None


def load():
    """Load the library once and attach the prototypes."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "librsfa_b200.so is not built: run `python ascend-rsfa_b200/build.py` "
                "(needs nvcc with sm_100a support); there is no CPU or PyTorch fallback")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def strerror(code):
    return load().rsfa_strerror(int(code)).decode()


def check(code, what="rsfa call"):
    """Map a C return code to the Python exception the operator documents."""
    if code == RSFA_OK:
        return
    msg = "%s failed: %s (code %d)" % (what, strerror(code), code)
    if code in (RSFA_ERR_INVALID_ARGUMENT, RSFA_ERR_TOO_LARGE):
        raise ValueError(msg)
    if code == RSFA_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)
