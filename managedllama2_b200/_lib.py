"""ctypes loader for libml2b200.so. There is no fallback: a missing library or symbol raises."""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libml2b200.so")
HEADER_PATH = os.path.join(os.path.dirname(HERE), "include", "ml2b200.h")

_lib = None


class Ml2Error(RuntimeError):
    def __init__(self, code, text):
        super().__init__("ml2b200 error %d: %s" % (code, text))
        self.code = code


def declared_symbols():
    """Names of every function include/ml2b200.h declares."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ml2_[a-z0-9_]+)\s*\(", text)))


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m managedllama2_b200.build` "
                              "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        lib.ml2_last_error.restype = ctypes.c_char_p
        lib.ml2_ctx_launch_count.restype = ctypes.c_longlong
        _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise Ml2Error(rc, load().ml2_last_error().decode("utf-8", "replace"))


class QWeightStruct(ctypes.Structure):
    _fields_ = [("weight", ctypes.c_void_p), ("zeros", ctypes.c_void_p), ("scales", ctypes.c_void_p)]


class ConfigStruct(ctypes.Structure):
    _fields_ = [("dim", ctypes.c_int32), ("hidden_dim", ctypes.c_int32), ("n_layers", ctypes.c_int32),
                ("n_heads", ctypes.c_int32), ("n_kv_heads", ctypes.c_int32), ("vocab_size", ctypes.c_int32),
                ("seq_len", ctypes.c_int32), ("rope_theta", ctypes.c_float)]
