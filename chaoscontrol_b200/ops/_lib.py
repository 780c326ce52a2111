"""ctypes binding of ``libccb200.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`chaoscontrol_b200._build`.  On a machine
with a CUDA device the kernels are mandatory: :func:`lib` raises if the shared
object is missing instead of silently falling back to PyTorch ops, mirroring
the reference dispatcher that refuses silent fallback
(src/chaoscontrol/kernels/_lm_head_loss/__init__.py:1041-1145).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libccb200.so"
_lib: Optional[C.CDLL] = None

i64 = C.c_int64
f32 = C.c_float
vp = C.c_void_p


class GemmArgs(C.Structure):
    _fields_ = [
        ("A", vp), ("B", vp), ("C", vp), ("C2", vp), ("Cin", vp), ("R1", vp), ("R2", vp),
        ("rowss", vp), ("ss_out", vp),
        ("M", i64), ("N", i64), ("K", i64),
        ("batch", i64), ("splits", i64),
        ("lda", i64), ("ldb", i64), ("ldc", i64), ("ldcin", i64), ("ldr", i64),
        ("a_batch", i64), ("b_batch", i64), ("c_batch", i64), ("cin_batch", i64), ("c_split", i64),
        ("a_mn", i64), ("b_mn", i64),
        ("epi", i64), ("out_fp32", i64), ("ss_atomic", i64),
        ("alpha", f32), ("beta", f32), ("inv_dim", f32), ("eps", f32),
        ("a_fp8", i64), ("b_fp8", i64), ("dscale_a", vp), ("dscale_b", vp), ("bias", vp),
        ("targets", vp), ("lse", vp), ("rowweight", vp), ("part_out", vp), ("zt_out", vp),
    ]


(EPI_STORE, EPI_ROWSCALE, EPI_ROWSCALE_SILU, EPI_RESID_SS, EPI_DSILU, EPI_RMSBWD, EPI_LSE_PART,
 EPI_CE_GRAD) = range(8)

_SIGS = {
    "ccb_init": ([], C.c_int),
    "ccb_read_status": ([C.c_int], C.c_int),
    "ccb_num_sms": ([], C.c_int),
    "ccb_launch_count": ([], C.c_int),
    "ccb_last_error": ([], C.c_char_p),
    "ccb_status_ptr": ([], vp),
    "ccb_gemm": ([C.POINTER(GemmArgs), vp], C.c_int),
    "ccb_lse_combine": ([vp, i64, i64, vp, vp, vp, vp], C.c_int),
    "ccb_fp8_quant_rows": ([vp, i64, vp, f32, vp, vp, vp, vp, i64, i64, vp], C.c_int),
    "ccb_fp8_quant_blocks": ([vp, vp, vp, vp, i64, i64, vp], C.c_int),
    "ccb_fp8_block_gemm": ([vp, vp, vp, vp, i64, i64, vp, i64, i64, vp, i64, i64, i64, vp], C.c_int),
    "ccb_fp8_cast_amax": ([vp, vp, vp, vp, i64, i64, vp], C.c_int),
    "ccb_fp8_cast_transpose_amax": ([vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, vp], C.c_int),
    "ccb_fp8_flush_amax": ([vp, i64, vp, vp, f32, vp], C.c_int),
    "ccb_pack_write_events": ([vp, vp, vp, vp, i64, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64, i64,
                               i64, vp], C.c_int),
    "ccb_scan_poly_exp": ([C.c_int], C.c_int),
    "ccb_gemm_pdl": ([C.c_int], C.c_int),
    "ccb_gemm_pair_resident": ([C.c_int], C.c_int),
    "ccb_scan_fwd": ([vp, i64, vp, vp, vp, vp, vp, i64, i64, i64, i64, vp], C.c_int),
    "ccb_scan_bwd": ([vp, i64, vp, vp, vp, vp, vp, vp, f32, f32, vp, i64, vp, vp, i64, i64, i64, i64, vp],
                     C.c_int),
    "ccb_plain_scan_fwd": ([vp, i64, vp, i64, vp, vp, i64, i64, i64, vp], C.c_int),
    "ccb_plain_scan_bwd": ([vp, i64, vp, vp, vp, i64, vp, vp, vp, i64, i64, i64, vp], C.c_int),
    "ccb_embed_fwd": ([vp, i64, vp, vp, vp, i64, i64, i64, vp], C.c_int),
    "ccb_embed_bwd_sorted": ([vp, vp, vp, vp, vp, i64, i64, i64, vp], C.c_int),
    "ccb_embed_bwd_slots": ([i64, i64, i64], C.c_int64),
    "ccb_lmhead_epilogue_parts": ([C.c_int], C.c_int),
    "ccb_gemm_cta_group": ([C.c_int], C.c_int),
    "ccb_gemm_debug": ([C.c_int], C.c_int),
    "ccb_gemm_resident_b": ([C.c_int], C.c_int),
    "ccb_gemm_l2_prefetch": ([C.c_int], C.c_int),
    "ccb_lmhead_debug": ([C.c_int], C.c_int),
    "ccb_lmhead_deep_ring": ([C.c_int], C.c_int),
    "ccb_splitk_reduce": ([vp, i64, i64, i64, i64, vp, vp, vp, i64, vp, vp, i64, vp], C.c_int),
    "ccb_colsum": ([vp, i64, i64, vp, i64, vp], C.c_int),
    "ccb_fold_colscale": ([vp, vp, vp, i64, i64, vp], C.c_int),
    "ccb_rmsnorm_fwd": ([vp, vp, vp, vp, vp, vp, i64, i64, f32, vp], C.c_int),
    "ccb_rmsnorm_bwd_blocks": ([i64], i64),
    "ccb_rmsnorm_bwd": ([vp, vp, vp, vp, vp, vp, vp, i64, i64, vp], C.c_int),
    "ccb_muon_momentum": ([vp, vp, vp, vp, i64, i64, f32, i64, vp], C.c_int),
    "ccb_muon_normalize": ([vp, vp, i64, i64, f32, vp], C.c_int),
    "ccb_muon_apply": ([vp, vp, i64, f32, f32, vp], C.c_int),
    "ccb_adamw": ([vp, i64, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, f32, vp, vp], C.c_int),
    "ccb_clip_grad_norm": ([vp, i64, f32, vp, vp], C.c_int),
    "ccb_sgd": ([vp, vp, i64, f32, vp], C.c_int),
    "ccb_cast_f32_to_bf16": ([vp, vp, i64, f32, vp], C.c_int),
    "ccb_cast_bf16_to_f32": ([vp, vp, i64, f32, i64, vp], C.c_int),
}


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    """True when the kernel library exists and a CUDA device is visible."""
    return _LIB_PATH.exists() and torch.cuda.is_available()


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: run `python -m chaoscontrol_b200._build` "
            "(the CUDA path never falls back to PyTorch ops)")
    L = C.CDLL(str(_LIB_PATH))
    for name, (argtypes, restype) in _SIGS.items():
        try:
            fn = getattr(L, name)
        except AttributeError:
            continue
        fn.argtypes = argtypes
        fn.restype = restype
    _late_sigs(L)
    _lib = L
    # process-wide kernel switches from the environment (A/B measurements, test runs of a non-default mode)
    for var, fn in (("CCB_GEMM_PDL", "ccb_gemm_pdl"), ("CCB_SCAN_ARITH", "ccb_scan_poly_exp"),
                    ("CCB_GEMM_PAIR_RESIDENT", "ccb_gemm_pair_resident")):
        val = os.environ.get(var)
        if val is not None and hasattr(L, fn):
            getattr(L, fn)(int(val))
    return L


_EXTRA_SIGS: dict[str, tuple[list, object]] = {}


def register_sig(name: str, argtypes: list, restype=C.c_int) -> None:
    """Declare the signature of a launcher defined by another ops module."""
    _EXTRA_SIGS[name] = (argtypes, restype)
    if _lib is not None:
        _late_sigs(_lib)


def _late_sigs(L: C.CDLL) -> None:
    for name, (argtypes, restype) in _EXTRA_SIGS.items():
        try:
            fn = getattr(L, name)
        except AttributeError:
            continue
        fn.argtypes = argtypes
        fn.restype = restype


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().ccb_last_error().decode(errors="replace")
        raise RuntimeError(f"libccb200 {what} failed ({rc}): {msg}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def read_status(reset: bool = True) -> int:
    """Synchronise and return the device status word (0 == OK)."""
    return int(lib().ccb_read_status(1 if reset else 0))


def assert_ok() -> None:
    st = read_status()
    if st != 0:
        names = {1: "a bounded mbarrier wait ran out", 2: "bad shape", 3: "peer flag timeout"}
        raise RuntimeError(f"libccb200 device status {st}: {names.get(st, 'unknown')}")


def launch_count() -> int:
    return int(lib().ccb_launch_count()) if _lib is not None else 0
