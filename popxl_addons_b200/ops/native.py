"""Bridge between the op registry and the hand-written sm_100a kernels in `lib/libxlb200.so`.

Importing this module loads the library (building it first if the sources are newer and nvcc is available) and
attaches a CUDA implementation to every op that has one. A CUDA implementation returns `NotImplemented` for operands it
does not cover (odd alignment, unsupported dtype); the session then runs the op's torch reference. If the library is
missing on a machine with a GPU the import fails loudly rather than silently running the reference everywhere.
"""
import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from ..xl.opdef import FALLBACKS, OPS, STRICT, NativeFallback, native, note_fallback  # noqa: F401  (re-exported)

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libxlb200.so")

F32, F16, BF16 = 0, 1, 2
_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

LAUNCHES = {"count": 0, "by_kernel": {}}


def _load():
    if not os.path.exists(_LIB_PATH):
        try:
            from .. import build as _build

            _build.build()
        except Exception as e:  # pragma: no cover
            raise ImportError(f"Native library {_LIB_PATH} is missing and could not be built: {e}") from e
    return ctypes.CDLL(_LIB_PATH)


LIB = _load()
_c_int, _c_ll, _c_f, _c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _sig(name, *argtypes, restype=_c_int):
    fn = getattr(LIB, name)
    fn.argtypes = list(argtypes)
    fn.restype = restype
    return fn


_gelu_fwd = _sig("xl_gelu_fwd", _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p)
_gelu_bwd = _sig("xl_gelu_bwd", _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p)
_silu_fwd = _sig("xl_silu_fwd", _c_p, _c_p, _c_ll, _c_int, _c_p)
_silu_bwd = _sig("xl_silu_bwd", _c_p, _c_p, _c_p, _c_ll, _c_int, _c_p)
_swiglu_fwd = _sig("xl_swiglu_fwd", _c_p, _c_p, _c_p, _c_ll, _c_int, _c_p)
_swiglu_bwd = _sig("xl_swiglu_bwd", _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_p)
_ln_fwd = _sig("xl_layer_norm_fwd", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_f, _c_int, _c_p)
_ln_bwd = _sig("xl_layer_norm_bwd", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p)
_rms_fwd = _sig("xl_rms_norm_fwd", _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_f, _c_int, _c_p)
_rms_bwd = _sig("xl_rms_norm_bwd", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p)
_norm_parts = _sig("xl_norm_bwd_parts", _c_ll)
_adam = _sig("xl_adam_step", _c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_p, _c_f, _c_f, _c_f, _c_f, _c_f,
             _c_f, _c_int, _c_ll, _c_p)
_sgd = _sig("xl_sgd_step", _c_p, _c_int, _c_p, _c_int, _c_p, _c_f, _c_f, _c_f, _c_f, _c_ll, _c_p)
_col_sum = _sig("xl_col_sum", _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p)
_col_sum_parts = _sig("xl_col_sum_parts", _c_ll, _c_int, _c_int)
_acc_mean = _sig("xl_accumulate_mean", _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_p)
_sumsq_parts = _sig("xl_sumsq_parts", _c_ll)
_sumsq = _sig("xl_grad_sumsq", _c_p, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_p)
_rotary = _sig("xl_rotary", _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll,
               _c_ll, _c_ll, _c_ll, _c_ll, _c_ll, _c_p)
_gq = _sig("xl_gq_decompress", _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p)
_sm_fwd = _sig("xl_attn_softmax_fwd", _c_p, _c_p, _c_ll, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p)
_attn_flash = _sig("xl_attn_fwd_tcgen05", _c_p, _c_ll, _c_ll, _c_p, _c_ll, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                   _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p)
_attn_plan = _sig("xl_attn_fwd_plan", _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p)
_attn_bwd_dq = _sig("xl_attn_bwd_dq_tcgen05", _c_p, _c_ll, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int,
                    _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_int, _c_p, _c_p, _c_p,
                    _c_p)
_attn_bwd_plan = _sig("xl_attn_bwd_plan", _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p)
_sm_bwd = _sig("xl_attn_softmax_bwd", _c_p, _c_p, _c_ll, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p)
_ce = _sig("xl_ce_fwd_bwd", _c_p, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p, _c_f, _c_int, _c_p)
_gemm = _sig("xl_gemm_tcgen05", _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll,
             _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_f, _c_p, _c_int, _c_p, _c_int,
             _c_int, _c_p, _c_p)
_gemm_fused = _sig("xl_gemm_tcgen05_fused", _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll,
                   _c_ll, _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_f, _c_p, _c_int, _c_p,
                   _c_int, _c_int, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p)
_gemm_pair = _sig("xl_gemm2cta_tcgen05", _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll,
                  _c_ll, _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_f, _c_p, _c_int, _c_int,
                  _c_p)
_rts_multi_grid = _sig("xl_rts_adam_multi_grid", _c_int)
_rts_adam_multi = _sig("xl_rts_adam_multi", _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p,
                       _c_p, _c_p, _c_f, _c_f, _c_f, _c_f, _c_f, _c_int, _c_p)
_gemm_ar_pull = _sig("xl_gemm_tcgen05_ar_pull", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
                     _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_f, _c_p, _c_int, _c_p, _c_int,
                     _c_int, _c_p, _c_p, _c_int, _c_int, _c_p, _c_p)
_symm_all_gather_mc = _sig("xl_symm_all_gather_mc", _c_p, _c_p, _c_ll, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p)
_gq_small = _sig("xl_gq_gemm_small_m", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll,
                 _c_int, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p)
_rot_append = _sig("xl_rotary_append", _c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                   _c_int, _c_p)
_attn_dec = _sig("xl_attn_decode", _c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
                 _c_f, _c_int, _c_int, _c_p)
_ar_add_ln = _sig("xl_ar_add_layer_norm", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p, _c_ll,
                  _c_p, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p)
_add_ln = _sig("xl_add_layer_norm", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_f, _c_int, _c_p)
_argmax = _sig("xl_argmax_rows", _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p)
_advance = _sig("xl_advance_position", _c_p, _c_p)
_store_row = _sig("xl_store_row", _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_p)
_symm_all_reduce_mc = _sig("xl_symm_all_reduce_mc", _c_p, _c_p, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int,
                           _c_int, _c_p, _c_p)
_gemm_fp8 = _sig("xl_gemm_tcgen05_fp8", _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_int, _c_int, _c_int,
                 _c_p, _c_int, _c_f, _c_p, _c_p, _c_int, _c_p)
_to_fp8 = _sig("xl_pow2_cast_to_fp8", _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_p)
_from_fp8 = _sig("xl_pow2_cast_from_fp8", _c_p, _c_p, _c_int, _c_p, _c_int, _c_ll, _c_int, _c_p)
_mse_scale = _sig("xl_fp8_mse_scale", _c_p, _c_int, _c_ll, _c_p, _c_int, _c_int, ctypes.c_double, _c_p, _c_p)
_csr_mm = _sig("xl_dense_csr_matmul", _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p)
_gather_rows = _sig("xl_gather_rows", _c_p, _c_int, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p)
_scatter_rows = _sig("xl_scatter_add_rows", _c_p, _c_int, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_p)
_row_sum_sumsq = _sig("xl_row_sum_sumsq", _c_p, _c_int, _c_p, _c_int, _c_int, _c_p)
_ln_apply_stats = _sig("xl_ln_apply_stats", _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_f, _c_f, _c_p)
_ce_stats = _sig("xl_ce_shard_stats", _c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_int, _c_p)
_ce_rescale = _sig("xl_ce_shard_rescale", _c_p, _c_p, _c_p, _c_int, _c_p)
_ce_combine = _sig("xl_ce_shard_combine", _c_p, _c_p, _c_int, _c_int, _c_p)
_ce_grad_loss = _sig("xl_ce_shard_grad_loss", _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int,
                     _c_int, _c_p)
_ce_nls = _sig("xl_ce_shard_nls", _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p)
_ce_nls_grad = _sig("xl_ce_nls_grad", _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int, _c_p)
_ln_shard_bwd_stats = _sig("xl_ln_shard_bwd_stats", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_p)
_ln_shard_bwd_parts = _sig("xl_ln_shard_bwd_parts", _c_int)
_ln_shard_bwd_apply = _sig("xl_ln_shard_bwd_apply", _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int,
                           _c_int, _c_f, _c_int, _c_p)
_set_spin = _sig("xl_set_comm_spin_limit", ctypes.c_uint)
_symm_barrier = _sig("xl_symm_barrier", _c_p, _c_int, _c_int, _c_int, _c_p, _c_p)
_symm_all_reduce = _sig("xl_symm_all_reduce", _c_p, _c_p, _c_ll, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p,
                        _c_p)
_rts_adam = _sig("xl_rts_adam", _c_p, _c_p, _c_int, _c_p, _c_p, _c_int, _c_p, _c_p, _c_ll, _c_ll, _c_int, _c_f, _c_f,
                 _c_f, _c_f, _c_f, _c_f, _c_int, _c_p)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_RECORDING = []  # stack of lists: kernels launched while a CUDA graph is being captured


def _count(name: str):
    LAUNCHES["count"] += 1
    LAUNCHES["by_kernel"][name] = LAUNCHES["by_kernel"].get(name, 0) + 1
    if _RECORDING:
        _RECORDING[-1].append(name)


def count_replay(names):
    """Account for the kernels of a captured graph each time it is replayed."""
    LAUNCHES["count"] += len(names)
    by = LAUNCHES["by_kernel"]
    for n in names:
        by[n] = by.get(n, 0) + 1


def _check(rc: int, name: str):
    if rc != 0:
        raise RuntimeError(f"CUDA kernel launcher {name} failed with code {rc} "
                           f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _ok(*ts) -> bool:
    """Operands the vectorised kernels accept: CUDA, contiguous, 16-byte aligned, fp32 / fp16 / bf16."""
    for t in ts:
        if t is None:
            continue
        if not (t.is_cuda and t.is_contiguous() and t.dtype in _CODE and t.data_ptr() % 16 == 0):
            return False
    return True


# ---- scratch memory ------------------------------------------------------------------------------------------------
_WORKSPACE: Dict[Tuple[int, str], torch.Tensor] = {}
_ERR: Dict[int, torch.Tensor] = {}


def workspace(nbytes: int, device: torch.device, tag: str = "default") -> torch.Tensor:
    """Per-device scratch buffer (fp32 view), grown on demand and reused by later launches on the same stream."""
    key = (device.index or 0, tag)
    buf = _WORKSPACE.get(key)
    n = (nbytes + 3) // 4
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 1 << 18), dtype=torch.float32, device=device)
        _WORKSPACE[key] = buf
    return buf


def gemm_error_flag(device: torch.device) -> torch.Tensor:
    """Device int that the GEMM kernels set when one of their bounded waits gave up."""
    idx = device.index or 0
    if idx not in _ERR:
        _ERR[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _ERR[idx]


def check_gemm_errors():
    """Raise if any GEMM launched so far reported a wait that ran out (synchronises the device)."""
    for idx, flag in _ERR.items():
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            names = {1: "operand tiles never arrived (TMA)", 2: "shared-memory stage was never released",
                     3: "accumulator never completed", 4: "accumulator buffer was never drained",
                     11: "attention: query tile never arrived", 12: "attention: key / value block never arrived",
                     13: "attention: key / value stage was never released", 14: "attention: scores never completed",
                     15: "attention: score buffer was never drained", 16: "attention: probabilities never arrived",
                     17: "attention: output accumulation never completed",
                     21: "CTA-pair GEMM: operand tiles never arrived (TMA)",
                     22: "CTA-pair GEMM: shared-memory stage was never released",
                     23: "CTA-pair GEMM: accumulator never completed",
                     24: "CTA-pair GEMM: accumulator buffer was never drained"}
            raise RuntimeError(f"tcgen05 GEMM on cuda:{idx} gave up waiting: {names.get(code, code)}")


# ---- elementwise ---------------------------------------------------------------------------------------------------
@native("gelu")
def gelu_cuda(x, approximate="none"):
    if not _ok(x):
        return NotImplemented
    y = torch.empty_like(x)
    _check(_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), _CODE[x.dtype], int(approximate == "tanh"), _stream()),
           "gelu_fwd")
    _count("gelu_fwd")
    return y


@native("gelu_grad")
def gelu_grad_cuda(x, g, approximate="none"):
    if not _ok(x, g) or x.dtype != g.dtype:
        return NotImplemented
    dx = torch.empty_like(x)
    _check(_gelu_bwd(x.data_ptr(), g.data_ptr(), dx.data_ptr(), x.numel(), _CODE[x.dtype],
                     int(approximate == "tanh"), _stream()), "gelu_bwd")
    _count("gelu_bwd")
    return dx


@native("swish")
def swish_cuda(x):
    if not _ok(x):
        return NotImplemented
    y = torch.empty_like(x)
    _check(_silu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), _CODE[x.dtype], _stream()), "silu_fwd")
    _count("silu_fwd")
    return y


@native("swish_grad")
def swish_grad_cuda(x, g):
    if not _ok(x, g) or x.dtype != g.dtype:
        return NotImplemented
    dx = torch.empty_like(x)
    _check(_silu_bwd(x.data_ptr(), g.data_ptr(), dx.data_ptr(), x.numel(), _CODE[x.dtype], _stream()), "silu_bwd")
    _count("silu_bwd")
    return dx


@native("swiglu")
def swiglu_cuda(gate, up):
    if not _ok(gate, up) or gate.dtype != up.dtype or gate.shape != up.shape:
        return NotImplemented
    y = torch.empty_like(gate)
    _check(_swiglu_fwd(gate.data_ptr(), up.data_ptr(), y.data_ptr(), gate.numel(), _CODE[gate.dtype], _stream()),
           "swiglu_fwd")
    _count("swiglu_fwd")
    return y


@native("swiglu_grad")
def swiglu_grad_cuda(gate, up, g):
    if not _ok(gate, up, g) or not (gate.dtype == up.dtype == g.dtype):
        return NotImplemented
    dg, du = torch.empty_like(gate), torch.empty_like(up)
    _check(_swiglu_bwd(gate.data_ptr(), up.data_ptr(), g.data_ptr(), dg.data_ptr(), du.data_ptr(), gate.numel(),
                       _CODE[gate.dtype], _stream()), "swiglu_bwd")
    _count("swiglu_bwd")
    return dg, du


# ---- normalisation -------------------------------------------------------------------------------------------------
@native("layer_norm")
def layer_norm_cuda(x, w, b, eps):
    if x.is_cuda and not x.is_contiguous():
        x = x.contiguous()  # e.g. the last position of every sequence: a strided slice of the activations
    if not _ok(x, w, b) or not (x.dtype == w.dtype == b.dtype):
        return NotImplemented
    cols = x.shape[-1]
    rows = x.numel() // cols
    y = torch.empty_like(x)
    mean = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    rc = _ln_fwd(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, cols,
                 float(eps), _CODE[x.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "layer_norm_fwd")
    _count("layer_norm_fwd")
    return y, mean, rstd


@native("layer_norm_grad")
def layer_norm_grad_cuda(x, w, mean, rstd, g):
    if not _ok(x, w, g, mean, rstd) or not (x.dtype == w.dtype == g.dtype):
        return NotImplemented
    cols = x.shape[-1]
    rows = x.numel() // cols
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    ws = workspace(_norm_parts(rows) * 2 * cols * 4, x.device, "norm")
    rc = _ln_bwd(x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), g.data_ptr(), dx.data_ptr(),
                 dw.data_ptr(), db.data_ptr(), ws.data_ptr(), rows, cols, _CODE[x.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "layer_norm_bwd")
    _count("layer_norm_bwd")
    return dx, dw, db


@native("rms_norm")
def rms_norm_cuda(x, w, eps):
    if not _ok(x, w) or x.dtype != w.dtype:
        return NotImplemented
    cols = x.shape[-1]
    rows = x.numel() // cols
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    rc = _rms_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols, float(eps), _CODE[x.dtype],
                  _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "rms_norm_fwd")
    _count("rms_norm_fwd")
    return y, rstd


@native("rms_norm_grad")
def rms_norm_grad_cuda(x, w, rstd, g):
    if not _ok(x, w, g, rstd) or not (x.dtype == w.dtype == g.dtype):
        return NotImplemented
    cols = x.shape[-1]
    rows = x.numel() // cols
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    ws = workspace(_norm_parts(rows) * 2 * cols * 4, x.device, "norm")
    rc = _rms_bwd(x.data_ptr(), w.data_ptr(), rstd.data_ptr(), g.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                  ws.data_ptr(), rows, cols, _CODE[x.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "rms_norm_bwd")
    _count("rms_norm_bwd")
    return dx, dw


# ---- optimizer -----------------------------------------------------------------------------------------------------
def _scalars(extra, attrs):
    """Resolve op scalars to floats; tensor-valued scalars make the native path decline (they stay on device)."""
    vals = dict(attrs)
    if vals.pop("_tensor_scalars"):
        return None
    return vals


@native("adam_fused_")
def adam_cuda(w, g, m, v, *rest, has_step, has_master, bias_correction, **attrs):
    rest = list(rest)
    step = rest.pop(0) if has_step else None
    master = rest.pop(0) if has_master else None
    s = _scalars(rest, attrs)
    if s is None or not _ok(w, g, m, v, master) or v.dtype != torch.float32:
        return NotImplemented
    if g.dtype != w.dtype and g.dtype != torch.float32:
        return NotImplemented
    if step is not None and step.dtype != torch.float32:
        return NotImplemented
    rc = _adam(w.data_ptr(), _CODE[w.dtype], g.data_ptr(), _CODE[g.dtype], m.data_ptr(), _CODE[m.dtype], v.data_ptr(),
               master.data_ptr() if master is not None else None, step.data_ptr() if step is not None else None,
               float(s["lr"]), float(s["beta1"]), float(s["beta2"]), float(s["epsilon"]), float(s["weight_decay"]),
               float(s["grad_scale"]), int(bool(bias_correction)), w.numel(), _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "adam_step")
    _count("adam_step")
    return w


@native("sgd_fused_")
def sgd_cuda(w, g, *rest, has_momentum, **attrs):
    rest = list(rest)
    buf = rest.pop(0) if has_momentum else None
    s = _scalars(rest, attrs)
    if s is None or not _ok(w, g, buf) or (buf is not None and buf.dtype != torch.float32):
        return NotImplemented
    rc = _sgd(w.data_ptr(), _CODE[w.dtype], g.data_ptr(), _CODE[g.dtype], buf.data_ptr() if buf is not None else None,
              float(s["lr"]), float(s["momentum"]), float(s["weight_decay"]), float(s["grad_scale"]), w.numel(),
              _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "sgd_step")
    _count("sgd_step")
    return w


@native("sum")
def sum_cuda(a, axis, keepdims):
    """Sum over the leading axes of a contiguous tensor (bias gradients: over the token rows): column sums in fp32,
    added in a fixed order."""
    if axis is None or keepdims or not _ok(a) or a.dim() < 2:
        return NotImplemented
    axes = sorted(int(x) % a.dim() for x in axis)
    if axes != list(range(len(axes))) or len(axes) == a.dim():
        return NotImplemented
    cols = 1
    for d in a.shape[len(axes):]:
        cols *= d
    rows = a.numel() // max(cols, 1)
    n = 4 if a.dtype == torch.float32 else 8
    if rows < 64 or cols % n or a.dtype not in _CODE:
        return NotImplemented
    out = torch.empty(a.shape[len(axes):], dtype=a.dtype, device=a.device)
    ws = workspace(_col_sum_parts(rows, cols, _CODE[a.dtype]) * cols * 4, a.device, "col_sum")
    rc = _col_sum(a.data_ptr(), out.data_ptr(), ws.data_ptr(), rows, cols, _CODE[a.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "col_sum")
    _count("col_sum")
    return out


@native("accumulate_mean_")
def accumulate_mean_cuda(acc, x, *extra, **attrs):
    if attrs.get("_tensor_scalars") != ("step",) or not _ok(acc, x) or extra[0].dtype != torch.float32:
        return NotImplemented
    _check(_acc_mean(acc.data_ptr(), _CODE[acc.dtype], x.data_ptr(), _CODE[x.dtype], extra[0].data_ptr(), acc.numel(),
                     _stream()), "accumulate_mean")
    _count("accumulate_mean")
    return acc


@native("matmul_accumulate_mean_")
def matmul_accumulate_mean_cuda(acc, a, b, step):
    if step.dtype != torch.float32 or not acc.is_contiguous():
        return NotImplemented
    res = gemm(a, b, out=acc, accumulate=2, step=step)
    return res


def grad_sumsq_cuda(t, scale):
    if not _ok(t) or not (scale.is_cuda and scale.dtype == torch.float32):
        return NotImplemented
    out = torch.empty((), dtype=torch.float32, device=t.device)
    ws = workspace(_sumsq_parts(t.numel()) * 4, t.device, "sumsq")
    _check(_sumsq(t.data_ptr(), _CODE[t.dtype], scale.data_ptr(), out.data_ptr(), ws.data_ptr(), t.numel(), _stream()),
           "grad_sumsq")
    _count("grad_sumsq")
    return out


# ---- rotary / int4 -------------------------------------------------------------------------------------------------
def rotary_launch(x, sin, cos, y, rotary_dim, inverse):
    """Rotate `x (B,H,S,D)` into `y` (may alias `x`); both may be strided views whose last axis is contiguous."""
    B, H, S, D = x.shape
    _check(_rotary(x.data_ptr(), sin.data_ptr(), cos.data_ptr(), y.data_ptr(), B, H, S, D, rotary_dim, sin.shape[0],
                   int(bool(inverse)), _CODE[x.dtype], x.stride(0), x.stride(1), x.stride(2), y.stride(0), y.stride(1),
                   y.stride(2), _stream()), "rotary")
    _count("rotary")


@native("rotary_pos_embed")
def rotary_cuda(x, sin, cos, rotary_dim, inverse):
    if not (x.is_cuda and x.dtype in _CODE and x.dim() == 4 and x.stride(-1) == 1) or not _ok(sin, cos):
        return NotImplemented
    if not (x.dtype == sin.dtype == cos.dtype) or x.shape[-1] % 2 or rotary_dim % 2:
        return NotImplemented
    y = torch.empty_like(x)  # keeps the strides of a dense permuted view
    if y.stride(-1) != 1:
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    rotary_launch(x, sin, cos, y, rotary_dim, inverse)
    return y


def gq_decompress_cuda(packed, scale, bias, out_dtype=None):
    if not (packed.is_cuda and packed.is_contiguous() and packed.dtype == torch.uint16) or not _ok(scale, bias):
        return NotImplemented
    if scale.dtype != bias.dtype:
        return NotImplemented
    r, g, w = packed.shape
    out = torch.empty((r, g * w * 4), dtype=out_dtype or scale.dtype, device=packed.device)
    rc = _gq(packed.data_ptr(), scale.data_ptr(), bias.data_ptr(), out.data_ptr(), packed.numel(), w, _CODE[out.dtype],
             _CODE[scale.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "gq_decompress")
    _count("gq_decompress")
    return out


# ---- GEMM ----------------------------------------------------------------------------------------------------------
_SM_COUNT: Dict[int, int] = {}


def _sms(device) -> int:
    idx = device.index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[idx]


def _major(t: torch.Tensor, contraction_last: bool):
    """(is_mn_major, leading dimension) of a 2-D (or batched 3-D) operand view, or None if neither axis is dense.
    `contraction_last`: the reduction dimension is the last axis (A operand) rather than the second-to-last (B)."""
    s_row, s_col = t.stride(-2), t.stride(-1)
    rows, cols = t.shape[-2], t.shape[-1]
    if s_col == 1 and (s_row >= cols):
        # last axis contiguous
        return (0 if contraction_last else 1), s_row
    if s_row == 1 and (s_col >= rows):
        return (1 if contraction_last else 0), s_col
    if cols == 1 and s_row == 1:
        return (1 if contraction_last else 0), max(s_col, rows)
    return None


# Plain GEMMs with N > 128 run on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles: measured 1.15 to 1.22x the single-CTA
# kernel on the transformer shapes); collective epilogues, the all-gather prologue and causal products keep the
# single-CTA kernel. XL_GEMM_CTA_PAIRS=0 switches the pairs off.
_GEMM_CTA_PAIRS = os.environ.get("XL_GEMM_CTA_PAIRS", "1") != "0"
# columns of C per tile of the CTA-pair kernel: 0 lets the library pick 256 or 128 per shape (fewer waves of CTA pairs)
_GEMM_PAIR_TILE_N = [int(os.environ.get("XL_GEMM_PAIR_TILE_N", "0"))]


def gemm(a: torch.Tensor, b: torch.Tensor, *, bias: Optional[torch.Tensor] = None, act: int = 0,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, accumulate: int = 0,
         step: Optional[torch.Tensor] = None, alpha: float = 1.0, comm=None, rs_dst: Optional[torch.Tensor] = None,
         gather: Optional[tuple] = None, causal: int = 0):
    """`out = act(alpha * a @ b + bias)` on the tcgen05 kernel. `a`: (M,K) or (B,M,K); `b`: (K,N) or (B,K,N); either may
    be a transposed view. With `accumulate=1` the result is added to `out`, with `accumulate=2` it is folded into `out`
    as a running mean with count `step`. `accumulate=3` with `comm` (a group context owning `out` in symmetric memory)
    all-reduces the product over the group inside the kernel: `out` must have been zeroed on this stream.
    `accumulate=4` with `comm` and `rs_dst` (int64 device tensor: every rank's zeroed output shard, `out` being this
    rank's) reduce-scatters the product over the rows instead. `gather=(mode, src_ptrs, flags, blocks_per_shard,
    n_copy)` pulls the remote row blocks of the sharded operand (mode 1: `a`, mode 2: `b`) from the peers inside the
    kernel. `causal` (1, 2, 3) skips the masked half of square attention products: 1 = output tiles above the diagonal
    (Q K^T), 2 = contraction up to the row (P V), 3 = contraction from the row (P^T dO).
    Returns NotImplemented for operands the kernel cannot take."""
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16) or not (a.is_cuda and b.is_cuda):
        return NotImplemented
    batched = a.dim() == 3
    if a.dim() not in (2, 3) or b.dim() != a.dim():
        return NotImplemented
    ma, mb = _major(a, True), _major(b, False)
    if ma is None or mb is None:
        return NotImplemented
    (a_mn, lda), (b_mn, ldb) = ma, mb
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-1]
    if b.shape[-2] != K:
        raise ValueError(f"gemm shape mismatch {tuple(a.shape)} x {tuple(b.shape)}")
    batch = a.shape[0] if batched else 1
    sa = a.stride(0) if batched else 0
    sb = b.stride(0) if batched else 0
    if batched and b.shape[0] != batch:
        return NotImplemented
    if lda % 8 or ldb % 8 or a.data_ptr() % 16 or b.data_ptr() % 16 or (batched and (sa % 8 or sb % 8)):
        return NotImplemented
    if out is None:
        out_dtype = out_dtype or a.dtype
        out = torch.empty((batch, M, N) if batched else (M, N), dtype=out_dtype, device=a.device)
    if out.dtype not in _CODE or out.stride(-1) != 1 or out.dim() != a.dim():
        return NotImplemented
    if accumulate == 4 and (rs_dst is None or comm is None or out.shape[-2] * comm.world != M):
        return NotImplemented
    ldc = out.stride(-2)
    stride_c = out.stride(0) if batched else 0
    esz = out.element_size()
    if (ldc * esz) % 16 or out.data_ptr() % 16 or (batched and (stride_c * esz) % 16):
        return NotImplemented
    if bias is not None and not (bias.is_cuda and bias.is_contiguous() and bias.dtype in _CODE and bias.numel() == N):
        return NotImplemented
    err = gemm_error_flag(a.device)
    out_ptr, pads, crank, cworld, lsync = out.data_ptr(), None, 0, 1, None
    if accumulate == 3:
        if comm is None or batched:
            return NotImplemented
        out_ptr = comm.arena.multicast_ptr(out)
        if not out_ptr:
            return NotImplemented
        pads, crank, cworld = comm.arena.pads_dev.data_ptr(), comm.rank, comm.world
        lsync = comm.arena.local_sync.data_ptr()
        err = comm.err
    rs_ptr, rs_rows = None, 0
    g_mode, g_src, g_dst, g_flags, g_bps, g_copy = 0, None, None, None, 0, 0
    if accumulate == 4 or gather is not None:
        if comm is None or batched:
            return NotImplemented
        pads, crank, cworld = comm.arena.pads_dev.data_ptr(), comm.rank, comm.world
        lsync = comm.arena.local_sync.data_ptr()
        err = comm.err
        if accumulate == 4:
            rs_ptr, rs_rows = rs_dst.data_ptr(), out.shape[-2]
        if gather is not None:
            g_mode, src_ptrs, flags, g_bps, g_copy = gather
            g_src, g_flags = src_ptrs.data_ptr(), flags.data_ptr()
            g_dst = a.data_ptr() if g_mode == 1 else b.data_ptr()
    if _GEMM_CTA_PAIRS and accumulate <= 2 and gather is None and not causal and N > 128:
        rc = _gemm_pair(a.data_ptr(), b.data_ptr(), out_ptr, M, N, K, batch, a_mn, b_mn, lda, ldb, ldc, sa, sb, stride_c,
                        int(a.dtype == torch.float16), _CODE[out.dtype], bias.data_ptr() if bias is not None else None,
                        _CODE[bias.dtype] if bias is not None else 0, act, accumulate,
                        step.data_ptr() if step is not None else None, float(alpha), err.data_ptr(), 0, _GEMM_PAIR_TILE_N[0],
                        _stream())
        if rc >= 0:
            _check(rc, "gemm2cta_tcgen05")
            _count("gemm2cta_tcgen05")
            return out
    rc = _gemm_fused(a.data_ptr(), b.data_ptr(), out_ptr, M, N, K, batch, a_mn, b_mn, lda, ldb, ldc, sa, sb, stride_c,
                     int(a.dtype == torch.float16), _CODE[out.dtype], bias.data_ptr() if bias is not None else None,
                     _CODE[bias.dtype] if bias is not None else 0, act, accumulate,
                     step.data_ptr() if step is not None else None, float(alpha), err.data_ptr(), _sms(a.device), pads,
                     crank, cworld, lsync, rs_ptr, rs_rows, g_mode, g_src, g_dst, g_flags, g_bps, g_copy, int(causal),
                     _stream())
    if rc < 0:
        return NotImplemented
    _check(rc, "gemm_tcgen05")
    _count("gemm_tcgen05")
    return out


def gemm_all_reduce_pull(pairs, comm, partial: torch.Tensor, result: torch.Tensor, flags_ptrs: torch.Tensor,
                         n_red: int = 8, alpha: float = 1.0, scatter: bool = False, timestamps: Optional[torch.Tensor] = None):
    """`result <- all_reduce over the group of (sum of a @ b over pairs)` in one kernel (one or two operand pairs, all
    with the same layouts). Every rank's GEMM CTAs store the partial product into `partial` (symmetric memory) and flag
    each tile at the rank that owns its rows; that rank adds the copies of the tile inside NVSwitch
    (`multimem.ld_reduce`) and writes the sum into every rank's `result` (`multimem.st`), tile by tile while the
    remaining tiles are still being multiplied. `partial`, `result`: `(M, N)` arena tensors of the group `comm`;
    `flags_ptrs`: int64 device tensor with every rank's address of the (zeroed) flag words (2 * tiles int32).
    `scatter=True` is the reduce-scatter form: `result` is `(M / world, N)` (any device memory) and receives only the
    sums of this rank's rows. Returns `result` (valid once the kernel has finished) or NotImplemented."""
    (a, b) = pairs[0]
    a2, b2 = pairs[1] if len(pairs) > 1 else (None, None)
    if len(pairs) > 2 or a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16) or a.dim() != 2 or b.dim() != 2:
        return NotImplemented
    ma, mb = _major(a, True), _major(b, False)
    if ma is None or mb is None:
        return NotImplemented
    (a_mn, lda), (b_mn, ldb) = ma, mb
    M, K = a.shape
    N = b.shape[1]
    K2, lda2, ldb2 = 0, 0, 0
    if a2 is not None:
        m2, n2 = _major(a2, True), _major(b2, False)
        if m2 is None or n2 is None or m2[0] != a_mn or n2[0] != b_mn or a2.dtype != a.dtype or b2.dtype != a.dtype \
                or a2.shape[0] != M or b2.shape[1] != N or a2.shape[1] != b2.shape[0]:
            return NotImplemented
        K2, lda2, ldb2 = a2.shape[1], m2[1], n2[1]
    rows_out = M // comm.world if scatter else M
    if partial.shape != (M, N) or result.shape != (rows_out, N) or partial.dtype != a.dtype or result.dtype != a.dtype \
            or partial.stride(1) != 1 or result.stride() != partial.stride():
        return NotImplemented
    mc_p = comm.arena.multicast_ptr(partial)
    mc_r = result.data_ptr() if scatter else comm.arena.multicast_ptr(result)
    if not mc_p or not mc_r or M % (128 * comm.world):
        return NotImplemented
    rc = _gemm_ar_pull(a.data_ptr(), b.data_ptr(), a2.data_ptr() if a2 is not None else None,
                       b2.data_ptr() if b2 is not None else None, partial.data_ptr(), mc_p, mc_r, M, N, K, K2, a_mn, b_mn,
                       lda, ldb, lda2, ldb2, partial.stride(0), int(a.dtype == torch.float16), _CODE[a.dtype], float(alpha),
                       comm.err.data_ptr(), _sms(a.device), comm.arena.pads_dev.data_ptr(), comm.rank, comm.world,
                       comm.arena.local_sync.data_ptr(), flags_ptrs.data_ptr(), int(n_red), int(bool(scatter)),
                       timestamps.data_ptr() if timestamps is not None else None, _stream())
    if rc < 0:
        return NotImplemented
    _check(rc, "gemm_rs_pull_tcgen05" if scatter else "gemm_ar_pull_tcgen05")
    _count("gemm_rs_pull_tcgen05" if scatter else "gemm_ar_pull_tcgen05")
    return result


def _flatten_batch(t: torch.Tensor) -> Optional[torch.Tensor]:
    """View an N-D operand as 3-D (batch, rows, cols) without copying, if its batch axes are jointly dense."""
    if t.dim() == 3:
        return t
    if t.is_contiguous():
        return t.view(-1, t.shape[-2], t.shape[-1])
    # batch axes must collapse to one stride
    stride = t.stride(-3)
    expected = stride
    for d in range(t.dim() - 3, -1, -1):
        if t.shape[d] != 1 and t.stride(d) != expected:
            return None
        expected = t.stride(d) * t.shape[d] if t.shape[d] != 1 else expected
        if d > 0:
            expected = t.stride(d) * t.shape[d]
    n = 1
    for sdim in t.shape[:-2]:
        n *= sdim
    return torch.as_strided(t, (n, t.shape[-2], t.shape[-1]), (stride, t.stride(-2), t.stride(-1)), t.storage_offset())


@native("matmul")
def matmul_cuda(a, b):
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        return NotImplemented
    if b.dim() == 2 and a.dim() >= 2:
        a2 = a.reshape(-1, a.shape[-1]) if a.dim() > 2 else a
        res = gemm(a2, b)
        if res is NotImplemented:
            return res
        return res.view(*a.shape[:-1], b.shape[-1])
    if a.dim() == b.dim() and a.dim() >= 3 and a.shape[:-2] == b.shape[:-2]:
        a3, b3 = _flatten_batch(a), _flatten_batch(b)
        if a3 is None or b3 is None:
            return NotImplemented
        res = gemm(a3, b3)
        if res is NotImplemented:
            return res
        return res.view(*a.shape[:-2], a.shape[-2], b.shape[-1])
    return NotImplemented


_ACT = {"none": 0, "gelu": 1, "gelu_tanh": 2, "relu": 3}


@native("linear_bias_act")
def linear_bias_act_cuda(x, w, *b, act):
    if x.dtype != w.dtype or x.dtype not in (torch.bfloat16, torch.float16) or not x.is_contiguous():
        return NotImplemented
    res = gemm(x.reshape(-1, x.shape[-1]), w, bias=b[0] if b else None, act=_ACT[act])
    if res is NotImplemented:
        return res
    return res.view(*x.shape[:-1], w.shape[-1])


# ---- attention: two batched tcgen05 GEMMs around a fused scale + causal-mask + softmax kernel ---------------------------
@native("attention")
def attention_cuda(q, k, v, causal, scale):
    if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.bfloat16, torch.float16) or q.dim() != 4:
        return NotImplemented
    B, H, Sq, D = q.shape
    Sk = k.shape[-2]
    q3, k3, v3 = (_flatten_batch(t) for t in (q, k, v))
    if q3 is None or k3 is None or v3 is None:
        return NotImplemented
    scores = gemm(q3, k3.transpose(-1, -2))
    if scores is NotImplemented:
        return NotImplemented
    lse = torch.empty((B * H, Sq), dtype=torch.float32, device=q.device)
    rc = _sm_fwd(scores.data_ptr(), lse.data_ptr(), B * H * Sq, Sq, Sk, float(scale), int(bool(causal)),
                 _CODE[scores.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "attn_softmax_fwd")
    _count("attn_softmax_fwd")
    o = gemm(scores, v3)
    if o is NotImplemented:
        return NotImplemented
    return o.view(B, H, Sq, D), lse.view(B, H, Sq)


@native("attention_grad")
def attention_grad_cuda(q, k, v, o, lse, do, causal, scale):
    if not (q.dtype == k.dtype == v.dtype == do.dtype) or q.dtype not in (torch.bfloat16, torch.float16):
        return NotImplemented
    B, H, Sq, D = q.shape
    Sk = k.shape[-2]
    q3, k3, v3, do3 = (_flatten_batch(t) for t in (q, k, v, do))
    if any(t is None for t in (q3, k3, v3, do3)):
        return NotImplemented
    # probabilities are recomputed from q, k (they are not kept between forward and backward)
    p = gemm(q3, k3.transpose(-1, -2))
    if p is NotImplemented:
        return NotImplemented
    tmp_lse = torch.empty((B * H, Sq), dtype=torch.float32, device=q.device)
    rc = _sm_fwd(p.data_ptr(), tmp_lse.data_ptr(), B * H * Sq, Sq, Sk, float(scale), int(bool(causal)),
                 _CODE[p.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "attn_softmax_fwd")
    _count("attn_softmax_fwd")
    dv = gemm(p.transpose(-1, -2), do3)
    dp = gemm(do3, v3.transpose(-1, -2))
    if dv is NotImplemented or dp is NotImplemented:
        return NotImplemented
    rc = _sm_bwd(p.data_ptr(), dp.data_ptr(), B * H * Sq, Sq, Sk, float(scale), int(bool(causal)), _CODE[p.dtype],
                 _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "attn_softmax_bwd")
    _count("attn_softmax_bwd")
    dq = gemm(dp, k3)
    dk = gemm(dp.transpose(-1, -2), q3)
    if dq is NotImplemented or dk is NotImplemented:
        return NotImplemented
    return dq.view_as(q), dk.view_as(k), dv.view_as(v)


def _heads_view(mat, col0, B, S, H, D):
    """(B, H, S, D) strided view of columns [col0, col0 + H*D) of a (B*S, ld) row-major matrix."""
    ld = mat.stride(0)
    return torch.as_strided(mat, (B, H, S, D), (S * ld, D, ld, 1), mat.storage_offset() + col0)


# the masked half of causal attention products is not computed (XL_CAUSAL_SKIP=0 computes the full products)
_CAUSAL_SKIP = os.environ.get("XL_CAUSAL_SKIP", "1") != "0"
# The forward pass of `attention_qkv` runs as one kernel that keeps the scores on chip (measured 2.7x the GEMM + softmax +
# GEMM path at 16 heads x 2048 x 256 and 1.8x at 4 heads, where the keys of a query block are divided over CTAs). Only
# with very little work (short sequences of few heads) the batched GEMM path is used. XL_FLASH_ATTENTION=0 / 1 forces it.
_FLASH_ATTENTION = os.environ.get("XL_FLASH_ATTENTION", "auto")
_FLASH_MIN_CTAS = 16


def _use_flash(B, S, H):
    if _FLASH_ATTENTION in ("0", "1"):
        return _FLASH_ATTENTION == "1"
    if _FLASH_ATTENTION is True or _FLASH_ATTENTION is False:  # set by tools
        return bool(_FLASH_ATTENTION)
    return B * H * ((S + 127) // 128) >= _FLASH_MIN_CTAS


_ATTN_SPLIT = os.environ.get("XL_ATTENTION_SPLIT_KEYS", "1") != "0"
_ATTN_PLANS: dict = {}


def _attention_split(kind, plan_fn, B, S, H, D, causal, device):
    """Key-range splitting of an attention kernel for this shape: `(chunk, items)` as planned by the library for the
    device's SM count (chunk 0: every query block keeps all its keys)."""
    key = (kind, B, S, H, D, bool(causal), device.index or 0)
    plan = _ATTN_PLANS.get(key)
    if plan is None:
        items = ctypes.c_int(0)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        chunk = plan_fn(B, S, H, D, int(bool(causal)), sms, ctypes.byref(items)) if _ATTN_SPLIT else 0
        plan = _ATTN_PLANS[key] = (max(int(chunk), 0), int(items.value))
    return plan


def flash_attention_fwd(packed, q_col, k_col, v_col, B, S, H, D, scale, causal, out=None, trace=None):
    """softmax(scale * Q K^T [+ causal mask]) V for the heads stored as column windows of `packed (B*S, cols)`; one
    tcgen05 kernel, scores never leave the chip. Returns `(out (B*S, H*D), lse (B, H, S))` or NotImplemented."""
    if packed.dtype not in (torch.bfloat16, torch.float16) or not packed.is_cuda or packed.dim() != 2 \
            or packed.stride(1) != 1 or D not in (64, 128, 256) or packed.shape[0] != B * S:
        return NotImplemented
    if out is None:
        out = torch.empty((B * S, H * D), dtype=packed.dtype, device=packed.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=packed.device)
    chunk, items = _attention_split("fwd", _attn_plan, B, S, H, D, causal, packed.device)
    part_o = part_lse = None
    if chunk > 0:
        slots = B * H * items * 128
        ws = workspace(slots * (D * 2 + 4), packed.device, "attn_split")
        part_o, part_lse = ws.data_ptr(), ws.data_ptr() + slots * D * 2
    rc = _attn_flash(packed.data_ptr(), packed.stride(0), packed.shape[1], out.data_ptr(), out.stride(0), lse.data_ptr(),
                     B, S, H, D, q_col, k_col, v_col, float(scale), int(bool(causal)),
                     int(packed.dtype == torch.float16), gemm_error_flag(packed.device).data_ptr(),
                     trace.data_ptr() if trace is not None else None, chunk, part_o, part_lse, _stream())
    if rc < 0:
        return NotImplemented
    _check(rc, "attn_fwd_tcgen05")
    _count("attn_fwd_tcgen05")
    return out, lse


@native("attention_qkv")
def attention_qkv_cuda(qkv, sin, cos, seq_len, n_heads, head_dim, rotary_dim, causal, scale, inplace):
    if qkv.dtype not in (torch.bfloat16, torch.float16) or not (qkv.is_cuda and qkv.is_contiguous()):
        return NotImplemented
    T = qkv.shape[0]
    B, S, H, D = T // seq_len, seq_len, n_heads, head_dim
    hd = H * D
    rot = qkv if inplace else qkv.clone()
    q, k, v = (_heads_view(rot, i * hd, B, S, H, D) for i in range(3))
    if rotary_dim:
        if sin.dtype != qkv.dtype or not _ok(sin, cos):
            return NotImplemented
        qk = _heads_view(rot, 0, B, S, 2 * H, D)  # q and k heads are adjacent column windows: one launch rotates both
        rotary_launch(qk, sin, cos, qk, rotary_dim, False)
    if _use_flash(B, S, H):
        res = flash_attention_fwd(rot, 0, hd, 2 * hd, B, S, H, D, scale, causal)
        if res is not NotImplemented:
            return res[0], rot, res[1]
    out = torch.empty((T, hd), dtype=qkv.dtype, device=qkv.device)
    o = _heads_view(out, 0, B, S, H, D)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=qkv.device)
    c1, c2, c3 = (1, 2, 3) if causal and _CAUSAL_SKIP else (0, 0, 0)
    for b in range(B):
        scores = gemm(q[b], k[b].transpose(-1, -2), causal=c1)
        if scores is NotImplemented:
            return NotImplemented
        rc = _sm_fwd(scores.data_ptr(), lse[b].data_ptr(), H * S, S, S, float(scale), int(bool(causal)),
                     _CODE[scores.dtype], _stream())
        if rc == -1:
            return NotImplemented
        _check(rc, "attn_softmax_fwd")
        _count("attn_softmax_fwd")
        if gemm(scores, v[b], out=o[b], causal=c2) is NotImplemented:
            return NotImplemented
    return out, rot, lse


# XL_FLASH_ATTENTION_BWD=0: the backward pass recomputes the scores with a GEMM and runs the two softmax kernels instead
# of the single kernel that keeps the scores on chip
_FLASH_ATTENTION_BWD = os.environ.get("XL_FLASH_ATTENTION_BWD", "1") != "0"


def flash_attention_bwd_dq(qkv_rot, out, dout, lse, dqkv, B, S, H, D, scale, causal, trace=None):
    """First pass of the attention backward as one tcgen05 kernel: recomputes P from q, k and `lse`, forms dP = dO V^T and
    dS = P o (dP - dO . O) * scale on chip, accumulates dQ = dS K into the q window of `dqkv`, and writes P and dS once
    as `(B*H, S, S)` 16-bit matrices for the two remaining products. Returns `(P, dS)` or NotImplemented."""
    hd = H * D
    if D not in (64, 128, 256) or S % 8 or qkv_rot.dtype not in (torch.bfloat16, torch.float16) or lse.dtype != torch.float32:
        return NotImplemented
    if not (out.is_cuda and out.stride(1) == 1 and dout.stride(1) == 1 and lse.is_contiguous()):
        return NotImplemented
    P = torch.empty((B * H, S, S), dtype=qkv_rot.dtype, device=qkv_rot.device)
    dS = torch.empty_like(P)
    chunk, items = _attention_split("bwd", _attn_bwd_plan, B, S, H, D, causal, qkv_rot.device)
    part_dq = None
    if chunk > 0:
        part_dq = workspace(B * H * items * 128 * D * 4, qkv_rot.device, "attn_split").data_ptr()
    rc = _attn_bwd_dq(qkv_rot.data_ptr(), qkv_rot.stride(0), qkv_rot.shape[1], out.data_ptr(), out.stride(0),
                      dout.data_ptr(), dout.stride(0), lse.data_ptr(), P.data_ptr(), dS.data_ptr(), dqkv.data_ptr(),
                      dqkv.stride(0), 0, B, S, H, D, 0, hd, 2 * hd, float(scale), int(bool(causal)),
                      int(qkv_rot.dtype == torch.float16), gemm_error_flag(qkv_rot.device).data_ptr(), chunk, part_dq,
                      workspace(B * H * S * 4, qkv_rot.device, "attn_delta").data_ptr(),
                      trace.data_ptr() if trace is not None else None, _stream())
    if rc < 0:
        return NotImplemented
    _check(rc, "attn_bwd_dq_tcgen05")
    _count("attn_bwd_dq_tcgen05")
    return P, dS


@native("attention_qkv_grad")
def attention_qkv_grad_cuda(qkv_rot, lse, dout, sin, cos, *fwd_out, seq_len, n_heads, head_dim, rotary_dim, causal, scale):
    if qkv_rot.dtype not in (torch.bfloat16, torch.float16) or not (qkv_rot.is_contiguous() and dout.is_contiguous()):
        return NotImplemented
    if dout.dtype != qkv_rot.dtype:
        return NotImplemented
    T = qkv_rot.shape[0]
    B, S, H, D = T // seq_len, seq_len, n_heads, head_dim
    hd = H * D
    q, k, v = (_heads_view(qkv_rot, i * hd, B, S, H, D) for i in range(3))
    do = _heads_view(dout, 0, B, S, H, D)
    dqkv = torch.empty_like(qkv_rot)
    dq, dk, dv = (_heads_view(dqkv, i * hd, B, S, H, D) for i in range(3))
    c1, c2, c3 = (1, 2, 3) if causal and _CAUSAL_SKIP else (0, 0, 0)
    fused = NotImplemented
    if _FLASH_ATTENTION_BWD and fwd_out and causal and fwd_out[0].dtype == qkv_rot.dtype:
        fused = flash_attention_bwd_dq(qkv_rot, fwd_out[0], dout, lse, dqkv, B, S, H, D, scale, causal)
    if fused is not NotImplemented:
        # dQ is done; the two remaining products read P and dS over the causal half (contraction from the tile's first row)
        P, dS = (t.view(B, H, S, S) for t in fused)
        for b in range(B):
            if gemm(P[b].transpose(-1, -2), do[b], out=dv[b], causal=c3) is NotImplemented \
                    or gemm(dS[b].transpose(-1, -2), q[b], out=dk[b], causal=c3) is NotImplemented:
                return NotImplemented
    else:
        tmp_lse = torch.empty((H, S), dtype=torch.float32, device=qkv_rot.device)
        for b in range(B):
            p = gemm(q[b], k[b].transpose(-1, -2), causal=c1)
            if p is NotImplemented:
                return NotImplemented
            rc = _sm_fwd(p.data_ptr(), tmp_lse.data_ptr(), H * S, S, S, float(scale), int(bool(causal)), _CODE[p.dtype],
                         _stream())
            if rc == -1:
                return NotImplemented
            _check(rc, "attn_softmax_fwd")
            _count("attn_softmax_fwd")
            if gemm(p.transpose(-1, -2), do[b], out=dv[b], causal=c3) is NotImplemented:
                return NotImplemented
            dp = gemm(do[b], v[b].transpose(-1, -2), causal=c1)
            if dp is NotImplemented:
                return NotImplemented
            _check(_sm_bwd(p.data_ptr(), dp.data_ptr(), H * S, S, S, float(scale), int(bool(causal)), _CODE[p.dtype],
                           _stream()), "attn_softmax_bwd")
            _count("attn_softmax_bwd")
            if gemm(dp, k[b], out=dq[b], causal=c2) is NotImplemented \
                    or gemm(dp.transpose(-1, -2), q[b], out=dk[b], causal=c3) is NotImplemented:
                return NotImplemented
    if rotary_dim:
        dqk = _heads_view(dqkv, 0, B, S, 2 * H, D)
        rotary_launch(dqk, sin, cos, dqk, rotary_dim, True)
    return dqkv


# ---- fused cross-entropy -------------------------------------------------------------------------------------------------
@native("ce_with_grad")
def ce_with_grad_cuda(logits, labels, loss_grad, ignore_index, reduction):
    if not _ok(logits) or not labels.is_cuda:
        return NotImplemented
    V = logits.shape[-1]
    rows = logits.numel() // V
    lab = labels.reshape(-1)
    if lab.dtype != torch.int32:
        lab = lab.to(torch.int32)
    ii = -100 if ignore_index is None else int(ignore_index)
    loss_row = torch.empty(rows, dtype=torch.float32, device=logits.device)
    dlogits = torch.empty_like(logits)
    lg = loss_grad.float().reshape(())
    if reduction == "mean":
        count = (lab != ii).sum().clamp(min=1).float()
        scale_t = (lg / count).reshape(1)
    else:
        count = None
        scale_t = lg.reshape(1)
    rc = _ce(logits.data_ptr(), lab.data_ptr(), loss_row.data_ptr(), dlogits.data_ptr(), rows, V, ii,
             scale_t.data_ptr(), 1.0, _CODE[logits.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "ce_fwd_bwd")
    _count("ce_fwd_bwd")
    if reduction == "mean":
        loss = loss_row.sum() / count
    elif reduction == "sum":
        loss = loss_row.sum()
    else:
        loss = loss_row.reshape(labels.shape)
    return loss.to(logits.dtype), dlogits


# ---- decoding path -------------------------------------------------------------------------------------------------------
def set_comm_spin_limit(polls: int) -> None:
    """Poll budget of every bounded wait on a peer in kernels launched from now on (0 restores the default)."""
    _set_spin(int(polls))


if os.environ.get("XL_COMM_SPIN_LIMIT"):  # e.g. first runs of a new collective kernel: give up after seconds, not minutes
    set_comm_spin_limit(int(os.environ["XL_COMM_SPIN_LIMIT"]))


def _row_window_ok(t) -> bool:
    """2-D, CUDA, unit column stride, 16-byte aligned rows (a column window of a wider row-major matrix is fine)."""
    return (t.is_cuda and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0
            and t.dtype in (torch.bfloat16, torch.float16))


@native("rotary_kv_append_")
def rotary_kv_append_cuda(qkv, sin_tab, cos_tab, k_cache, v_cache, pos, n_heads, head_dim, rotary_dim):
    if not _row_window_ok(qkv) or not _ok(k_cache, v_cache) or pos.dtype != torch.int32 or qkv.dtype != k_cache.dtype:
        return NotImplemented
    if rotary_dim and not (_ok(sin_tab, cos_tab) and sin_tab.dtype == qkv.dtype):
        return NotImplemented
    B = qkv.shape[0]
    rc = _rot_append(qkv.data_ptr(), qkv.stride(0), sin_tab.data_ptr(), cos_tab.data_ptr(), k_cache.data_ptr(),
                     v_cache.data_ptr(), pos.data_ptr(), B, n_heads, head_dim, rotary_dim, k_cache.shape[2],
                     _CODE[qkv.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "rotary_append")
    _count("rotary_append")
    return qkv


_AD_SCRATCH: Dict[int, torch.Tensor] = {}


def _attn_decode_launch(qkv, k_cache, v_cache, pos, n_heads, head_dim, scale, out):
    if not (_row_window_ok(qkv) and _row_window_ok(out)) or not _ok(k_cache, v_cache) or pos.dtype != torch.int32:
        return NotImplemented
    if head_dim not in (64, 128, 256) or k_cache.dtype != qkv.dtype or out.dtype != qkv.dtype:
        return NotImplemented
    B, smax = qkv.shape[0], k_cache.shape[2]
    bh = B * n_heads
    # enough CTAs to fill the machine, at least 32 cache positions per CTA
    splits = max(1, min((8 * _sms(qkv.device) + bh - 1) // bh, (smax + 31) // 32, 64))
    ws = workspace(bh * splits * (head_dim + 2) * 4, qkv.device, "attn_decode")
    idx = qkv.device.index or 0
    counters = _AD_SCRATCH.get(idx)
    if counters is None or counters.numel() < bh:
        counters = _AD_SCRATCH[idx] = torch.zeros(max(bh, 4096), dtype=torch.int32, device=qkv.device)
    rc = _attn_dec(qkv.data_ptr(), qkv.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), out.stride(0),
                   ws.data_ptr(), counters.data_ptr(), pos.data_ptr(), B, n_heads, head_dim, smax, float(scale), splits,
                   _CODE[qkv.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "attn_decode")
    _count("attn_decode")
    return out


@native("attention_decode_packed")
def attention_decode_packed_cuda(qkv, k_cache, v_cache, pos, n_heads, head_dim, scale):
    out = torch.empty((qkv.shape[0], n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    return _attn_decode_launch(qkv, k_cache, v_cache, pos, n_heads, head_dim, scale, out)


@native("attention_decode_into_")
def attention_decode_into_cuda(buf, k_cache, v_cache, pos, n_heads, head_dim, out_col, scale):
    hd = n_heads * head_dim
    res = _attn_decode_launch(buf, k_cache, v_cache, pos, n_heads, head_dim, scale, buf[:, out_col:out_col + hd])
    return buf if res is not NotImplemented else NotImplemented


@native("add_layer_norm_")
def add_layer_norm_cuda(x, *rest, has_delta, has_bias, eps):
    rest = list(rest)
    delta = rest.pop(0) if has_delta else None
    bias = rest.pop(0) if has_bias else None
    w, b = rest
    if not _ok(x, delta, bias, w, b) or x.dim() != 2 or x.shape[1] > 8192:
        return NotImplemented
    if any(t is not None and t.dtype != x.dtype for t in (delta, bias, w, b)):
        return NotImplemented
    h = torch.empty_like(x)
    rc = _add_ln(x.data_ptr(), delta.data_ptr() if delta is not None else None,
                 bias.data_ptr() if bias is not None else None, w.data_ptr(), b.data_ptr(), h.data_ptr(), x.shape[0],
                 x.shape[1], float(eps), _CODE[x.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "add_layer_norm")
    _count("add_layer_norm")
    return h


@native("argmax_rows")
def argmax_rows_cuda(logits, valid, index_offset):
    if not _ok(logits) or logits.dim() != 2:
        return NotImplemented
    rows, V = logits.shape
    m = torch.empty(rows, dtype=torch.float32, device=logits.device)
    i = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(_argmax(logits.data_ptr(), m.data_ptr(), i.data_ptr(), rows, V, valid, index_offset, _CODE[logits.dtype],
                   _stream()), "argmax_rows")
    _count("argmax_rows")
    return m, i


@native("advance_position_")
def advance_position_cuda(pos):
    if pos.dtype != torch.int32:
        return NotImplemented
    _check(_advance(pos.data_ptr(), _stream()), "advance_position")
    _count("advance_position")
    return pos


@native("store_row_")
def store_row_cuda(buf, pos, vals, base):
    if buf.dtype != torch.int32 or vals.dtype != torch.int32 or pos.dtype != torch.int32 or not buf.is_contiguous():
        return NotImplemented
    _check(_store_row(buf.data_ptr(), pos.data_ptr(), base, vals.data_ptr(), vals.numel(), buf.shape[0], _stream()),
           "store_row")
    _count("store_row")
    return buf


_GQ_SCRATCH: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}


def _gq_scratch(device, n_tiles: int):
    """Zero-initialised split-K scratch of the small-M GEMM (the kernel hands it back zeroed after every launch)."""
    idx = device.index or 0
    cur = _GQ_SCRATCH.get(idx)
    if cur is None or cur[1].numel() < n_tiles:
        n = max(n_tiles, 2048)
        cur = (torch.zeros(n * 512, dtype=torch.float32, device=device), torch.zeros(n, dtype=torch.int32, device=device))
        _GQ_SCRATCH[idx] = cur
    return cur


def gq_gemm_small_m(x, packed, scale, zero, bias, out=None, act_from_col=None, ctas=None):
    """`x (M<=16, K) @ dequant(packed (N, K/gs, gs/4))^T + bias` with the de-quantisation fused into the GEMM; GELU on
    the output columns `>= act_from_col` if given. `x` and `out` may be column windows of wider row-major matrices.
    With `zero=None`, `scale` holds (scale, zero) pairs laid out `(K/gs, N, 2)` (see `interleave_scale_zero`)."""
    M, K = x.shape
    N, groups, words = packed.shape
    gs = words * 4
    transposed = zero is None
    if transposed:
        if scale.shape != (groups, N, 2) or not scale.is_contiguous():
            return NotImplemented
        zero = scale
    if M > 16 or not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16) or x.stride(1) != 1:
        return NotImplemented
    if x.stride(0) % 8 or x.data_ptr() % 16 or not _ok(scale, zero, bias):
        return NotImplemented
    if scale.dtype != zero.dtype or scale.dtype not in (torch.bfloat16, torch.float16) or groups * gs != K \
            or not packed.is_contiguous() or (bias is not None and bias.dtype != x.dtype):
        return NotImplemented
    y = out if out is not None else torch.empty((M, N), dtype=x.dtype, device=x.device)
    if y.shape != (M, N) or y.dtype != x.dtype or y.stride(1) != 1:
        return NotImplemented
    n_tiles = (N + 31) // 32
    ws, counters = _gq_scratch(x.device, n_tiles)
    rc = _gq_small(x.data_ptr(), packed.data_ptr(), scale.data_ptr(), zero.data_ptr(),
                   bias.data_ptr() if bias is not None else None, y.data_ptr(), M, N, K, gs, x.stride(0), y.stride(0),
                   N if act_from_col is None else int(act_from_col), int(ctas or 2 * _sms(x.device)),
                   ws.data_ptr(), counters.data_ptr(), _CODE[x.dtype], _CODE[scale.dtype], int(transposed), _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "gq_gemm_small_m")
    _count("gq_gemm_small_m")
    return y


# ---- FP8 ---------------------------------------------------------------------------------------------------------------------
_FP8_TORCH = {"float8_143": torch.float8_e4m3fn, "float8_152": torch.float8_e5m2}
_FP8_E5M2 = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}


def _log2_arg(log2_scale):
    """(pointer, is_int) of a device scalar holding a power-of-two exponent."""
    if log2_scale.dtype == torch.int32:
        return log2_scale, 1
    if log2_scale.dtype == torch.float32:
        return log2_scale, 0
    return log2_scale.float(), 0


@native("pow2scale_cast_to_fp8")
def pow2scale_cast_to_fp8_cuda(x, log2_scale, dt):
    if not _ok(x) or not log2_scale.is_cuda or log2_scale.numel() != 1 or dt.name not in _FP8_TORCH:
        return NotImplemented
    tdt = _FP8_TORCH[dt.name]
    y = torch.empty(x.shape, dtype=tdt, device=x.device)
    ls, is_int = _log2_arg(log2_scale)
    _check(_to_fp8(x.data_ptr(), _CODE[x.dtype], ls.data_ptr(), is_int, y.data_ptr(), x.numel(), _FP8_E5M2[tdt], _stream()),
           "pow2_cast_to_fp8")
    _count("pow2_cast_to_fp8")
    return y


@native("pow2scale_cast_from_fp8")
def pow2scale_cast_from_fp8_cuda(x, log2_scale, dt):
    if x.dtype not in _FP8_E5M2 or not (x.is_cuda and x.is_contiguous()) or log2_scale.numel() != 1:
        return NotImplemented
    out_dt = dt.as_torch()
    if out_dt not in _CODE:
        return NotImplemented
    y = torch.empty(x.shape, dtype=out_dt, device=x.device)
    ls, is_int = _log2_arg(log2_scale)
    _check(_from_fp8(x.data_ptr(), ls.data_ptr(), is_int, y.data_ptr(), _CODE[out_dt], x.numel(), _FP8_E5M2[x.dtype],
                     _stream()), "pow2_cast_from_fp8")
    _count("pow2_cast_from_fp8")
    return y


def gemm_fp8(a, b_t, out_dtype=torch.bfloat16, alpha: float = 1.0, log2_scale=None, bias=None):
    """`2^log2_scale * alpha * a @ b_t^T` on the tcgen05 8-bit float path: `a (M, K)`, `b_t (N, K)`, both row-major fp8
    (e4m3 / e5m2, may differ), fp32 accumulation. `log2_scale`: optional device scalar."""
    if a.dtype not in _FP8_E5M2 or b_t.dtype not in _FP8_E5M2 or a.dim() != 2 or b_t.dim() != 2:
        return NotImplemented
    if not (a.is_cuda and a.is_contiguous() and b_t.is_contiguous()) or a.shape[1] != b_t.shape[1]:
        return NotImplemented
    M, K = a.shape
    N = b_t.shape[0]
    if K % 16 or a.data_ptr() % 16 or b_t.data_ptr() % 16 or out_dtype not in _CODE:
        return NotImplemented
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if (N * out.element_size()) % 16:
        return NotImplemented
    ls = None
    if log2_scale is not None:
        ls = log2_scale.float().reshape(1) if log2_scale.dtype != torch.float32 else log2_scale.reshape(1)
    err = gemm_error_flag(a.device)
    rc = _gemm_fp8(a.data_ptr(), b_t.data_ptr(), out.data_ptr(), M, N, K, K, K, N, _FP8_E5M2[a.dtype], _FP8_E5M2[b_t.dtype],
                   _CODE[out_dtype], bias.data_ptr() if bias is not None else None,
                   _CODE[bias.dtype] if bias is not None else 0, float(alpha), ls.data_ptr() if ls is not None else None,
                   err.data_ptr(), _sms(a.device), _stream())
    if rc < 0:
        return NotImplemented
    _check(rc, "gemm_tcgen05_fp8")
    _count("gemm_tcgen05_fp8")
    return out


@native("matmul_pow2scaled")
def matmul_pow2scaled_cuda(a, b, log2_scale, out_dt):
    if a.dtype not in _FP8_E5M2 or b.dtype not in _FP8_E5M2 or b.dim() != 2 or log2_scale.numel() != 1:
        return NotImplemented
    out_dtype = out_dt.as_torch()
    a2 = a.reshape(-1, a.shape[-1])
    if not a2.is_contiguous():
        a2 = a2.contiguous()
    # the kernel takes both operands with the contraction index contiguous: B as (N, K)
    b_t = b.t().contiguous() if b.stride(-1) == 1 else b.t()
    res = gemm_fp8(a2, b_t, out_dtype=out_dtype, log2_scale=log2_scale)
    if res is NotImplemented:
        return res
    return res.view(*a.shape[:-1], b.shape[-1])


_MSE_SCRATCH: Dict[int, torch.Tensor] = {}


def fp8_mse_scale_cuda(x, fmt_name, src_mantissa_bits):
    from .fp8_mse_scale import _format_window
    from .fp8_utils import FP8_FORMATS

    if not _ok(x):
        return NotImplemented
    fmt = FP8_FORMATS[fmt_name]
    lo, span = _format_window(fmt)
    qerr = 2.0 ** (-2.0 * (src_mantissa_bits - fmt["mantissa_bits"]))
    idx = x.device.index or 0
    scratch = _MSE_SCRATCH.get(idx)
    if scratch is None:
        scratch = _MSE_SCRATCH[idx] = torch.zeros(256, dtype=torch.int32, device=x.device)
    out = torch.empty((), dtype=torch.int32, device=x.device)
    _check(_mse_scale(x.data_ptr(), _CODE[x.dtype], x.numel(), scratch.data_ptr(), int(lo), int(span), float(qerr),
                      out.data_ptr(), _stream()), "fp8_mse_scale")
    _count("fp8_mse_scale")
    return out


def dense_csr_matmul_cuda(lhs, indptr, indices, values, n_rows, n_cols):
    if not _ok(lhs) or not (indptr.is_cuda and indices.is_cuda and values.is_cuda) or values.dtype != torch.float32:
        return NotImplemented
    if indptr.dtype != torch.int32 or indices.dtype != torch.int32 or n_cols * 4 > 48 * 1024:
        return NotImplemented
    x2 = lhs.reshape(-1, lhs.shape[-1])
    y = torch.empty((x2.shape[0], n_cols), dtype=lhs.dtype, device=lhs.device)
    rc = _csr_mm(x2.data_ptr(), _CODE[lhs.dtype], indptr.data_ptr(), indices.data_ptr(), values.data_ptr(), y.data_ptr(),
                 x2.shape[0], n_rows, n_cols, int(values.numel()), _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "dense_csr_matmul")
    _count("dense_csr_matmul")
    return y.view(*lhs.shape[:-1], n_cols)


@native("gather")
def gather_cuda(w, idx, axis, zero_OOR):
    if axis != 0 or w.dim() != 2 or not _ok(w) or idx.dtype != torch.int32 or not idx.is_contiguous():
        return NotImplemented
    out = torch.empty((*idx.shape, w.shape[1]), dtype=w.dtype, device=w.device)
    _check(_gather_rows(w.data_ptr(), _CODE[w.dtype], idx.data_ptr(), out.data_ptr(), idx.numel(), w.shape[0], w.shape[1],
                        _stream()), "gather_rows")
    _count("gather_rows")
    return out


@native("gather_grad")
def gather_grad_cuda(g, idx, axis, zero_OOR, w_shape):
    if axis != 0 or len(w_shape) != 2 or not _ok(g) or idx.dtype != torch.int32 or not idx.is_contiguous():
        return NotImplemented
    acc = torch.zeros(tuple(w_shape), dtype=torch.float32, device=g.device)
    _check(_scatter_rows(g.data_ptr(), _CODE[g.dtype], idx.data_ptr(), acc.data_ptr(), idx.numel(), w_shape[0], w_shape[1],
                         _stream()), "scatter_add_rows")
    _count("scatter_add_rows")
    return acc if g.dtype == torch.float32 else acc.to(g.dtype)


def row_sum_sumsq(x):
    """`(2, rows)` fp32: per-row sum and sum of squares of a 2-D tensor (local part of a hidden-sharded LayerNorm)."""
    stats = torch.empty((2, x.shape[0]), dtype=torch.float32, device=x.device)
    _check(_row_sum_sumsq(x.data_ptr(), _CODE[x.dtype], stats.data_ptr(), x.shape[0], x.shape[1], _stream()), "row_stats")
    _count("row_sum_sumsq")
    return stats


def ln_apply_stats(x, stats, w, b, hidden, eps):
    """LayerNorm of hidden-sharded rows given the all-reduced `(2, rows)` sums; returns `(y, mean, rstd)`."""
    rows, cols = x.shape
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(_ln_apply_stats(x.data_ptr(), _CODE[x.dtype], stats.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(),
                           mean.data_ptr(), rstd.data_ptr(), rows, cols, float(hidden), float(eps), _stream()), "ln_apply")
    _count("ln_apply_stats")
    return y, mean, rstd


def _labels_i32(labels):
    lab = labels.reshape(-1)
    return lab if lab.dtype == torch.int32 and lab.is_contiguous() else lab.to(torch.int32).contiguous()


def ce_shard_stats(x, labels, label_offset: int = 0, out=None):
    """`(3, rows)` fp32 of one vocabulary shard: row maximum, sum of exp(x - that maximum), and `x[label - offset]` where
    that column belongs to the shard (else 0). One pass over the shard."""
    rows, cols = x.shape
    stats = out if out is not None else torch.empty((3, rows), dtype=torch.float32, device=x.device)
    _check(_ce_stats(x.data_ptr(), _CODE[x.dtype], _labels_i32(labels).data_ptr(), int(label_offset), stats.data_ptr(),
                     rows, cols, _stream()), "ce_shard_stats")
    _count("ce_shard_stats")
    return stats


def ce_shard_rescale(stats, gmax):
    """`(2, rows)`: the shard's sum rescaled to the group maximum, and its picked logit: what is summed over the group."""
    rows = stats.shape[1]
    out = torch.empty((2, rows), dtype=torch.float32, device=stats.device)
    _check(_ce_rescale(stats.data_ptr(), gmax.data_ptr(), out.data_ptr(), rows, _stream()), "ce_shard_rescale")
    _count("ce_shard_rescale")
    return out


def ce_shard_combine(stats_all):
    """`(n_shards, 3, rows)` statistics of shards held by one device -> `(3, rows)` = group max, sum, picked logit."""
    n, _, rows = stats_all.shape
    out = torch.empty((3, rows), dtype=torch.float32, device=stats_all.device)
    _check(_ce_combine(stats_all.data_ptr(), out.data_ptr(), n, rows, _stream()), "ce_shard_combine")
    _count("ce_shard_combine")
    return out


def ce_shard_grad_loss(x, gmax, gsum, gpicked, labels, label_offset, row_scale, want_loss=True):
    """`dlogits = (softmax - onehot) * row_scale[row]` for this shard and, with `want_loss`, the fp32 loss per row."""
    rows, cols = x.shape
    dx = torch.empty_like(x)
    loss = torch.empty(rows, dtype=torch.float32, device=x.device) if want_loss else None
    _check(_ce_grad_loss(x.data_ptr(), _CODE[x.dtype], gmax.data_ptr(), gsum.data_ptr(), gpicked.data_ptr(),
                         _labels_i32(labels).data_ptr(), int(label_offset), row_scale.data_ptr(), dx.data_ptr(),
                         loss.data_ptr() if want_loss else None, rows, cols, _stream()), "ce_shard_grad_loss")
    _count("ce_shard_grad_loss")
    return dx, loss


def ce_shard_nls(x, gmax, gsum, gpicked, want_loss=True):
    """Negative log-softmax of this shard (dtype of x) and, with `want_loss`, the loss per row (dtype of x)."""
    rows, cols = x.shape
    nls = torch.empty_like(x)
    loss = torch.empty(rows, dtype=x.dtype, device=x.device) if want_loss else None
    _check(_ce_nls(x.data_ptr(), _CODE[x.dtype], gmax.data_ptr(), gsum.data_ptr(), gpicked.data_ptr(), nls.data_ptr(),
                   loss.data_ptr() if want_loss else None, rows, cols, _stream()), "ce_shard_nls")
    _count("ce_shard_nls")
    return nls, loss


def ce_nls_grad(nls, labels, label_offset, dloss):
    rows, cols = nls.shape
    dx = torch.empty_like(nls)
    _check(_ce_nls_grad(nls.data_ptr(), _CODE[nls.dtype], _labels_i32(labels).data_ptr(), int(label_offset),
                        dloss.data_ptr(), dx.data_ptr(), rows, cols, _stream()), "ce_nls_grad")
    _count("ce_nls_grad")
    return dx


def ce_sharded_grad_cuda(nls, idx, dloss):
    if not _ok(nls, dloss) or nls.dim() != 2 or dloss.dtype != nls.dtype or not idx.is_cuda:
        return NotImplemented
    return ce_nls_grad(nls, idx, 0, dloss)


def ce_sharded_wr_cuda(*tensors, n):
    """All shards are tensors of this device: statistics per shard (labels offset by the columns before it), one combine
    kernel, then the negative log-softmax of every shard; the loss comes with the first shard's pass."""
    logits, indices = tensors[:n], tensors[n:]
    if not _ok(*logits) or any(l.dim() != 2 or l.dtype != logits[0].dtype for l in logits):
        return NotImplemented
    rows = logits[0].shape[0]
    stats_all = torch.empty((n, 3, rows), dtype=torch.float32, device=logits[0].device)
    off = 0
    for i, (l, idx) in enumerate(zip(logits, indices)):
        ce_shard_stats(l, idx, off, out=stats_all[i])
        off += l.shape[1]
    g = ce_shard_combine(stats_all)
    outs, loss = [], None
    for i, l in enumerate(logits):
        nls, lo = ce_shard_nls(l, g[0], g[1], g[2], want_loss=(i == 0))
        outs.append(nls)
        loss = lo if i == 0 else loss
    return (loss, *outs)


def ce_sharded_wr_grad_cuda(*tensors, n):
    nls, indices, dloss = tensors[:n], tensors[n:2 * n], tensors[2 * n]
    if not _ok(*nls, dloss) or any(x.dtype != dloss.dtype for x in nls):
        return NotImplemented
    outs, off = [], 0
    for x, idx in zip(nls, indices):
        outs.append(ce_nls_grad(x, idx, off, dloss))
        off += x.shape[1]
    return tuple(outs)


def ln_shard_bwd_stats(x, w, mean, rstd, g):
    """`(2, rows)` fp32: sums over this rank's columns of `g*w` and `g*w*xhat` (hidden-sharded LayerNorm backward)."""
    rows, cols = x.shape
    stats = torch.empty((2, rows), dtype=torch.float32, device=x.device)
    _check(_ln_shard_bwd_stats(x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), g.data_ptr(),
                               stats.data_ptr(), rows, cols, _CODE[x.dtype], _stream()), "ln_shard_bwd_stats")
    _count("ln_shard_bwd_stats")
    return stats


def ln_shard_bwd_apply(x, w, mean, rstd, g, gstats, hidden):
    """`(dx, dw, db)` of a hidden-sharded LayerNorm given the group sums `gstats (2, rows)`; NotImplemented if the shard
    is wider than the kernel's register tiling."""
    rows, cols = x.shape
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    parts = _ln_shard_bwd_parts(rows)
    ws = workspace(parts * 2 * cols * 4, x.device, "ln_shard_bwd")
    rc = _ln_shard_bwd_apply(x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), g.data_ptr(),
                             gstats.data_ptr(), dx.data_ptr(), dw.data_ptr(), db.data_ptr(), ws.data_ptr(), rows, cols,
                             float(hidden), _CODE[x.dtype], _stream())
    if rc == -1:
        return NotImplemented
    _check(rc, "ln_shard_bwd_apply")
    _count("ln_shard_bwd_apply")
    return dx, dw, db


# ---- registration of ops defined outside xl.ops ------------------------------------------------------------------------
def _register_late():
    from . import grad_reduce_square_add as _g, group_quantize_decompress as _q  # noqa: F401  (define the OpDefs)

    OPS["grad_reduce_square_add"].native["cuda"] = grad_sumsq_cuda
    OPS["group_quantize_decompress"].native["cuda"] = gq_decompress_cuda
    from . import fp8_mse_scale as _m, static_sparse_ops as _s  # noqa: F401

    OPS["fp8_mse_scale"].native["cuda"] = fp8_mse_scale_cuda
    from . import cross_entropy_sharded_loss as _ce  # noqa: F401

    OPS["ce_sharded_grad"].native["cuda"] = ce_sharded_grad_cuda
    OPS["ce_sharded_wr"].native["cuda"] = ce_sharded_wr_cuda
    OPS["ce_sharded_wr_grad"].native["cuda"] = ce_sharded_wr_grad_cuda
    OPS["dense_csr_matmul"].native["cuda"] = dense_csr_matmul_cuda

    from ..layers import linear_gq as _lgq  # noqa: F401

    def linear_gq_cuda(x, packed, scale, zero, *b, dim):
        x2 = x.reshape(-1, x.shape[-1])
        if dim == 0 and x2.shape[0] <= 16 and x2.is_contiguous():
            y = gq_gemm_small_m(x2, packed, scale, zero, b[0] if b else None)
            if y is not NotImplemented:
                return y.view(*x.shape[:-1], packed.shape[0])
        if x.dtype not in (torch.bfloat16, torch.float16):
            return NotImplemented
        w = gq_decompress_cuda(packed, scale, zero, out_dtype=x.dtype)
        if w is NotImplemented:
            return NotImplemented
        wt = w if dim in (-1, 1) else w.t()
        res = gemm(x.reshape(-1, x.shape[-1]), wt, bias=b[0] if b else None)
        if res is NotImplemented:
            return res
        return res.view(*x.shape[:-1], wt.shape[-1])

    OPS["linear_gq"].native["cuda"] = linear_gq_cuda

    def linear_gq_window_cuda(x, packed, scale, zero, *b, x_col, k, act_from_col):
        xw = x[:, x_col:x_col + k]
        if xw.shape[0] > 16:
            return NotImplemented
        return gq_gemm_small_m(xw, packed, scale, zero, b[0] if b else None, act_from_col=act_from_col)

    OPS["linear_gq_window"].native["cuda"] = linear_gq_window_cuda

    def linear_gq_window_t_cuda(x, packed, sz, *b, x_col, k, act_from_col):
        xw = x[:, x_col:x_col + k]
        if xw.shape[0] > 16:
            return NotImplemented
        return gq_gemm_small_m(xw, packed, sz, None, b[0] if b else None, act_from_col=act_from_col)

    OPS["linear_gq_window_t"].native["cuda"] = linear_gq_window_t_cuda


_register_late()
