"""The C-ABI library on a machine without a GPU: it loads, exports every entry point that include/nsa_sm100.h declares,
its parameter structs have the sizes of the header's mirrors, and argument checking answers with error codes before any
CUDA call (no compute is launched here)."""
import ctypes
import importlib.util
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
PKG = os.path.join(ROOT, "scalable-flash-native-sparse-attention_b200")
HEADER = os.path.join(ROOT, "include", "nsa_sm100.h")
LIB = os.path.join(PKG, "csrc", "libnsa_sm100.so")


def _lib_module():
    if not os.path.exists(LIB):   # build in tree (nvcc cross-compiles sm_100a without a GPU)
        subprocess.run([sys.executable, os.path.join(PKG, "build.py")], check=True)
    spec = importlib.util.spec_from_file_location("nsa_lib_binding", os.path.join(PKG, "flash_nsa", "_lib.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _declared():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    fns = re.findall(r"^\s*(?:const\s+char\s*\*|int)\s+(nsa_\w+)\s*\(", text, flags=re.M)
    structs = re.findall(r"typedef\s+struct\s+\w+\s*\{.*?\}\s*(\w+)\s*;", text, flags=re.S)
    return fns, structs


def test_every_declared_entry_point_is_exported():
    fns, _ = _declared()
    assert len(fns) >= 25 and "nsa_cmp_attn_fwd" in fns and "nsa_decode_fused" in fns and "nsa_rope" in fns
    L = ctypes.CDLL(LIB) if os.path.exists(LIB) else _lib_module().lib()
    missing = [f for f in fns if not hasattr(L, f)]
    assert not missing, missing


def test_the_half_build_exports_the_same_entry_points():
    """libnsa_sm100_f16.so: the same sources with IEEE half as the 16-bit element type; same symbols, same structs."""
    m = _lib_module()
    L, H = m.lib(), m.lib(f16=True)          # raises on a missing symbol, a struct size mismatch or the wrong element type
    assert L.nsa_element_type() == 0 and H.nsa_element_type() == 1
    fns, _ = _declared()
    assert not [f for f in fns if not hasattr(H, f)]


def test_struct_mirrors_match_the_library():
    m = _lib_module()
    L = m.lib()                      # raises on any size mismatch or missing symbol
    _, structs = _declared()
    assert set(structs) == set(m.structs)
    for name in structs:
        assert L.nsa_struct_size(name.encode()) == ctypes.sizeof(m.structs[name]) > 0
    assert L.nsa_struct_size(b"NoSuchStruct") == 0
    assert L.nsa_version() > 0


def test_argument_errors_come_back_as_codes_and_messages():
    m = _lib_module()
    L = m.lib()
    # null parameter block and zeroed parameter blocks are rejected before anything touches the GPU
    assert L.nsa_combine_fwd(None, None) < 0
    assert b"combine" in L.nsa_last_error()
    p = m.structs["NsaRopeParams"]()
    assert L.nsa_rope(ctypes.byref(p), None) < 0
    assert b"rope" in L.nsa_last_error()
    k = m.structs["NsaK2qParams"]()
    assert L.nsa_k2q_index(ctypes.byref(k), None) < 0
    s = m.structs["NsaStoreKvParams"]()
    assert L.nsa_store_kvcache(ctypes.byref(s), None) < 0
