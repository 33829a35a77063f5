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


def test_every_call_site_passes_as_many_arguments_as_the_binding_declares():
    """Most launches sit on GPU-only branches: a wrong argument count there would first show as a TypeError on the GPU
    box. The call sites are counted from the source instead."""
    import ast

    from popxl_addons_b200.ops import native

    root = os.path.dirname(HERE)
    files = ["popxl_addons_b200/ops/native.py", "popxl_addons_b200/parallel/fused.py",
             "popxl_addons_b200/models/generator.py", "popxl_addons_b200/xl/session.py",
             "popxl_addons_b200/utils/kernel_bench.py", "tests/test_gpu_kernels.py", "tests/test_gpu_decode.py",
             "tests/test_gpu_misc.py", "tests/dist_worker.py", "bench.py"]
    calls = 0
    for rel in files:
        tree = ast.parse(open(os.path.join(root, rel)).read())
        for node in ast.walk(tree):
            if not isinstance(node, ast.Call):
                continue
            f = node.func
            name = f.id if isinstance(f, ast.Name) else (
                f.attr if isinstance(f, ast.Attribute) and isinstance(f.value, ast.Name)
                and f.value.id in ("nat", "native", "_native") else None)
            fn = getattr(native, name, None) if name else None
            if not isinstance(fn, ctypes._CFuncPtr) or fn.argtypes is None:
                continue
            if any(isinstance(a, ast.Starred) for a in node.args):
                continue
            calls += 1
            assert not node.keywords and len(node.args) == len(fn.argtypes), \
                f"{rel}:{node.lineno}: {name} is called with {len(node.args)} arguments, declared with {len(fn.argtypes)}"
    assert calls >= 50
