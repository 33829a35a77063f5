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


def test_gemm_entry_points_reject_unsupported_arguments_on_the_host():
    """Shapes and alignments a kernel does not take are refused before any CUDA call (return -1), so the caller can
    fall back; nothing here touches a device."""
    from popxl_addons_b200.ops import native

    ok = dict(a=256, b=512, c=1024, M=256, N=256, K=64, batch=1, a_mn=0, b_mn=0, lda=64, ldb=64, ldc=256, sa=0, sb=0,
              sc=0, fp16=0, cdt=2)

    def pair(**kw):
        v = {**ok, **kw}
        return native._gemm_pair(v["a"], v["b"], v["c"], v["M"], v["N"], v["K"], v["batch"], v["a_mn"], v["b_mn"],
                                 v["lda"], v["ldb"], v["ldc"], v["sa"], v["sb"], v["sc"], v["fp16"], v["cdt"], None, 0, 0,
                                 v.get("accumulate", 0), None, 1.0, None, 0, v.get("tile_n", 0), None)

    assert pair(N=64) == -1               # narrow outputs stay on the single-CTA kernel
    assert pair(tile_n=192) == -1         # tiles are 256 or 128 columns wide
    assert pair(M=0) == -1
    assert pair(a=260) == -1              # operand not 16-byte aligned
    assert pair(lda=60) == -1             # leading dimension not a multiple of 8 elements
    assert pair(batch=2, sa=12) == -1
    assert pair(accumulate=3) == -1       # collective epilogues are not implemented on CTA pairs
    assert pair(accumulate=2) == -1       # running mean without a step counter

    def single(**kw):
        v = {**ok, **kw}
        return native._gemm(v["a"], v["b"], v["c"], v["M"], v["N"], v["K"], v["batch"], v["a_mn"], v["b_mn"], v["lda"],
                            v["ldb"], v["ldc"], v["sa"], v["sb"], v["sc"], v["fp16"], v["cdt"], None, 0, 0,
                            v.get("accumulate", 0), None, 1.0, None, 148, None, 0, 1, None, None)

    assert single(K=0) == -1
    assert single(b=516) == -1
    assert single(accumulate=4) == -1     # reduce-scatter needs the full entry point
    assert single(accumulate=3) < 0       # all-reduce without signal pads (or no driver to encode tensor maps)


def test_attention_key_split_planner_on_the_host():
    """The planner that divides a query block's keys over CTAs is host code: many heads keep one CTA per query block,
    few heads are split so that the launch fills the SMs, and the split never produces an empty part."""
    import ctypes

    from popxl_addons_b200.ops import native

    def plan(fn, B, S, H, D, sms=148):
        items = ctypes.c_int(0)
        chunk = fn(B, S, H, D, 1, sms, ctypes.byref(items))
        return chunk, items.value

    for fn, bkv in ((native._attn_plan, 64), (native._attn_bwd_plan, 32)):
        chunk, items = plan(fn, 1, 2048, 16, 256)
        assert chunk == 0 and items == 16                      # 256 CTAs already: no splitting
        chunk, items = plan(fn, 1, 2048, 4, 256)
        assert chunk >= 2 and 16 < items and 4 * items <= 2 * 148   # about one wave of CTAs
        n_last = 2048 // bkv
        assert -(-n_last // chunk) <= n_last                   # every part of the longest block has at least one key block
        chunk, items = plan(fn, 1, 128, 1, 64)
        assert chunk == 0 and items == 1                       # a single query block with two key blocks stays whole
        assert fn(1, 2048, 4, 96, 1, 148, None) == -1          # unsupported head dimension
