"""The ctypes declarations in `ops/native.py` against the `extern "C"` prototypes in `csrc/`: same number of
arguments and the same C types, for every bound entry point. A mismatch would corrupt the argument list of a launch
that only runs on a GPU, so it is checked on the host."""
import ctypes
import glob
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "popxl_addons_b200", "csrc")

_C_TYPES = {"int": "i", "long long": "q", "float": "f", "unsigned int": "I", "unsigned": "I", "double": "d"}
_PY_TYPES = {ctypes.c_int: "i", ctypes.c_longlong: "q", ctypes.c_float: "f", ctypes.c_void_p: "p", ctypes.c_uint: "I",
             ctypes.c_double: "d"}


def _prototypes():
    protos = {}
    for path in glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.h")):
        for m in re.finditer(r"XL_API\s+[\w\s\*]+?\s+(xl_\w+)\s*\(([^)]*)\)", open(path).read(), re.S):
            args = [a.strip() for a in m.group(2).replace("\n", " ").split(",") if a.strip() and a.strip() != "void"]
            protos[m.group(1)] = args
    return protos


def _c_code(arg: str) -> str:
    arg = re.sub(r"\s+", " ", arg)
    if "*" in arg or "cudaStream_t" in arg:
        return "p"
    return _C_TYPES.get(arg.rsplit(" ", 1)[0].replace("const ", "").strip(), "?")


def test_ctypes_signatures_match_the_c_prototypes():
    from popxl_addons_b200.ops import native

    protos = _prototypes()
    assert len(protos) > 40
    checked = 0
    for attr in dir(native):
        fn = getattr(native, attr)
        if not isinstance(fn, ctypes._CFuncPtr) or getattr(fn, "argtypes", None) is None:
            continue
        name = fn.__name__
        assert name in protos, f"{name} is bound in native.py but has no XL_API prototype in csrc/"
        want = "".join(_c_code(a) for a in protos[name])
        got = "".join(_PY_TYPES.get(t, "?") for t in fn.argtypes)
        assert "?" not in want, f"unrecognised C type in the prototype of {name}: {protos[name]}"
        assert want == got, f"{name}: C prototype takes {want}, ctypes declares {got}"
        checked += 1
    assert checked >= 45
