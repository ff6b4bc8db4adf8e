"""TEST INFRASTRUCTURE ONLY.  ctypes access to oracle/_ref/libinsignia_ref.so: the reference's own CUDA engine, compiled
unmodified for sm_100a by oracle/Makefile.  Used by the GPU tests as a second checker."""
import ctypes as C
import os

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libinsignia_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(_PATH)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(_PATH)
        L.ref_last_error.restype = C.c_char_p
        L.ref_engine_create.restype = C.c_void_p
        L.ref_engine_create.argtypes = [C.c_char_p, C.c_ulonglong, C.c_int]
        for n in ("ref_engine_destroy",):
            getattr(L, n).argtypes = [C.c_void_p]
            getattr(L, n).restype = None
        for n in ("ref_engine_embed", "ref_engine_layer", "ref_engine_forward_token", "ref_engine_decode_token",
                  "ref_engine_mtp_draft"):
            getattr(L, n).argtypes = [C.c_void_p, C.c_int]
        L.ref_engine_logits_argmax.argtypes = [C.c_void_p]
        L.ref_engine_position.argtypes = [C.c_void_p]
        L.ref_engine_set_position.argtypes = [C.c_void_p, C.c_int]
        L.ref_engine_set_position.restype = None
        L.ref_engine_read.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_ulonglong]
        _lib = L
    return _lib


def call(name, *args):
    """Kernel-level entry: device pointers as ints, ints as ints."""
    fn = getattr(lib(), name)
    cargs = [C.c_void_p(a) if isinstance(a, int) and a > (1 << 20) else a for a in args]
    rc = fn(*cargs)
    if rc != 0:
        raise RuntimeError(f"{name}: {lib().ref_last_error().decode()}")


class RefEngine:
    def __init__(self, index_path, max_context=512, budget=16 << 30):
        self.h = lib().ref_engine_create(index_path.encode(), budget, max_context)
        if not self.h:
            raise RuntimeError(lib().ref_last_error().decode())

    def _chk(self, rc):
        if rc < 0:
            raise RuntimeError(lib().ref_last_error().decode())
        return rc

    def embed(self, t):
        self._chk(lib().ref_engine_embed(self.h, t))

    def layer(self, l):
        self._chk(lib().ref_engine_layer(self.h, l))

    def forward_token(self, t):
        self._chk(lib().ref_engine_forward_token(self.h, t))

    def logits_argmax(self):
        return self._chk(lib().ref_engine_logits_argmax(self.h))

    def decode_token(self, t):
        return self._chk(lib().ref_engine_decode_token(self.h, t))

    def mtp_draft(self, t):
        return self._chk(lib().ref_engine_mtp_draft(self.h, t))

    @property
    def position(self):
        return lib().ref_engine_position(self.h)

    @position.setter
    def position(self, p):
        lib().ref_engine_set_position(self.h, p)

    def read(self, field, n):
        import numpy as np

        out = np.empty(n, np.float32)
        self._chk(lib().ref_engine_read(self.h, field.encode(), out.ctypes.data, n))
        return out

    def close(self):
        if self.h:
            lib().ref_engine_destroy(self.h)
            self.h = None
