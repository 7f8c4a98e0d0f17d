"""ctypes binding of libblum.so (the C ABI declared in include/blum.h, plus the development hooks of include/blum_dev.h).

The library is the product; this module only loads it and declares argument types.
There is no fallback: if the shared library is missing, importing raises.
"""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libblum.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "blum.h")
DEV_HEADER_PATH = os.path.join(HERE, "..", "include", "blum_dev.h")

F32, F16, BF16 = 0, 1, 2
DTYPE_SIZE = {F32: 4, F16: 2, BF16: 2}

OK = 0
ERR_INVALID, ERR_CUDA, ERR_OOM, ERR_STATE, ERR_DEVICE, ERR_COMM = -1, -2, -3, -4, -5, -6


class BlumError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("blum error %d: %s" % (code, message))
        self.code = code
        self.message = message


class LlamaCfg(C.Structure):
    _fields_ = [
        ("layers", C.c_int32), ("hidden", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float),
        ("act_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("page_size", C.c_int32),
        ("max_seqs", C.c_int32), ("max_ctx", C.c_int32), ("kv_pages", C.c_int64),
        ("embed_q8", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
        ("rope_mode", C.c_int32), ("qk_norm", C.c_int32), ("tie_head", C.c_int32),
    ]


_CTYPE = {
    "int": C.c_int, "int32_t": C.c_int32, "int64_t": C.c_int64, "uint64_t": C.c_uint64, "size_t": C.c_size_t,
    "float": C.c_float, "blum_dtype": C.c_int, "void": None,
}


def declared_functions(header_path=HEADER_PATH):
    """Parses the prototypes of include/blum.h: {name: (restype, [argtypes])}."""
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    protos = {}
    pat = re.compile(r"(?:^|[;}\n])\s*((?:const\s+)?[A-Za-z_][A-Za-z0-9_]*\s*\**)\s*(blum_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", re.S)
    for ret, name, args in pat.findall(text):
        ret = ret.strip()
        argl = []
        args = args.strip()
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    argl.append(C.c_void_p)
                else:
                    base = a.replace("const", "").split()[0]
                    argl.append(_CTYPE[base])
        if "*" in ret:
            restype = C.c_char_p if "char" in ret else C.c_void_p
        else:
            restype = _CTYPE[ret.replace("const", "").strip()]
        protos[name] = (restype, argl)
    return protos


def all_declared_functions():
    """The product ABI (blum.h) plus the development hooks (blum_dev.h)."""
    protos = declared_functions(HEADER_PATH)
    protos.update(declared_functions(DEV_HEADER_PATH))
    return protos


def load(path=LIB_PATH):
    if not os.path.exists(path):
        raise ImportError(
            "libblum.so not found at %s: build it with `python -m luminal_b200.build` "
            "(there is no CPU fallback)" % path)
    lib = C.CDLL(path)
    for name, (restype, argtypes) in all_declared_functions().items():
        fn = getattr(lib, name)   # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib
