"""Loader of libwein_b200.so.  There is no CPU fallback: a missing library is an error."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwein_b200.so")


class LibraryMissing(RuntimeError):
    pass


class WeinB200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"wein_b200 status {code}: {msg}")
        self.code = code


_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m inferulm_b200.build` (needs nvcc); "
                "there is no CPU or PyTorch fallback for these operators")
        try:
            import torch  # noqa: F401  (brings in the CUDA runtime / cuBLASLt the library links against)
        except Exception:
            pass
        _lib = C.CDLL(LIB_PATH)
        _lib.wein_b200_last_error.restype = C.c_char_p
        _lib.wein_b200_abi_version.restype = C.c_uint32
    return _lib


def check(code):
    if code != 0:
        raise WeinB200Error(code, load().wein_b200_last_error().decode())
    return code
