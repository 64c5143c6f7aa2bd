"""ctypes binding of libnsa_sm100.so.

The parameter structs are mirrored from include/nsa_sm100.h by parsing the header (one source of truth);
`nsa_struct_size` cross-checks every mirror against the compiled library at load time.  There is no
fallback: if the library is missing the import of any op fails with the build command to run.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG_ROOT = os.path.dirname(_HERE)
_HEADER = os.path.join(os.path.dirname(_PKG_ROOT), "include", "nsa_sm100.h")
_LIB_PATH = os.path.join(_PKG_ROOT, "csrc", "libnsa_sm100.so")

_SCALARS = {"int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64, "float": ctypes.c_float}

structs = {}
functions = []


def _parse_header(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for m in re.finditer(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        name, body = m.group(3), m.group(2)
        fields = []
        for decl in body.split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            is_ptr_type = False
            base = decl
            mm = re.match(r"^(const\s+)?(\w+)\s*(.*)$", decl)
            base_t, rest = mm.group(2), mm.group(3)
            for d in rest.split(","):
                d = d.strip()
                ptr = d.startswith("*")
                fname = d.lstrip("* ").strip()
                if ptr:
                    ctype = ctypes.c_void_p
                elif base_t in structs:
                    ctype = structs[base_t]
                else:
                    ctype = _SCALARS[base_t]
                fields.append((fname, ctype))
        structs[name] = type(name, (ctypes.Structure,), {"_fields_": fields})
    for m in re.finditer(r"^\s*(?:const\s+char\s*\*|int)\s+(nsa_\w+)\s*\(", text, flags=re.M):
        functions.append(m.group(1))


with open(_HEADER) as _f:
    _parse_header(_f.read())

_LIB_PATH_F16 = os.path.join(_PKG_ROOT, "csrc", "libnsa_sm100_f16.so")
_libs = {}


def lib(f16=False):
    """The kernel library: the bf16 build, or (f16=True) the build of the same sources for IEEE-half tensors."""
    if f16 in _libs:
        return _libs[f16]
    path = _LIB_PATH_F16 if f16 else _LIB_PATH
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python {os.path.join(_PKG_ROOT, 'build.py')}` "
            "(nvcc, sm_100a).  flash_nsa has no CPU or PyTorch fallback.")
    L = ctypes.CDLL(path)
    L.nsa_last_error.restype = ctypes.c_char_p
    L.nsa_struct_size.argtypes = [ctypes.c_char_p]
    for name, st in structs.items():
        n = L.nsa_struct_size(name.encode())
        if n != ctypes.sizeof(st):
            raise ImportError(f"ABI mismatch for {name}: header mirror {ctypes.sizeof(st)} bytes, library {n} bytes")
    for fn in functions:
        if not hasattr(L, fn):
            raise ImportError(f"{path} does not export {fn}")
    if L.nsa_element_type() != (1 if f16 else 0):
        raise ImportError(f"{path} computes in the other 16-bit element type")
    _libs[f16] = L
    return L


class NsaError(RuntimeError):
    pass


# kernels launched by one call of each entry point (used by the benchmark's launch counter)
KERNELS_PER_CALL = {
    "nsa_cmp_attn_bwd": 3, "nsa_swa_bwd": 3, "nsa_slc_attn_bwd": 3, "nsa_k2q_index": 4,
}
launch_count = 0


def call(fn_name, params, stream, f16=False):
    """Invoke an entry point `int fn(const Params*, void* stream)`; raise on a non-zero status."""
    global launch_count
    L = lib(f16)
    n = KERNELS_PER_CALL.get(fn_name, 1)
    ph = getattr(params, "phases", 0) if fn_name.endswith("_bwd") else 0
    if ph:   # a backward entry point asked for a subset of {delta, dK/dV, dQ}
        n = bin(ph & 7).count("1")
    if fn_name == "nsa_slc_attn_bwd" and (ph & 6) in (0, 6) and os.environ.get("NSA_SLC_BWD_UNFUSED", "0")[:1] != "1":
        n -= 1   # dK/dV and dQ of the selected branch are one kernel when asked for together
    launch_count += n
    rc = getattr(L, fn_name)(ctypes.byref(params), ctypes.c_void_p(stream))
    if rc != 0:
        raise NsaError(f"{fn_name} failed ({rc}): {L.nsa_last_error().decode()}")
