"""ctypes binding of ``libvelox_b200.so`` (declarations mirror ``include/velox_b200.h``).

There is no fallback: if the shared object is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

from . import build as _build

# ---- enums (include/velox_b200.h)
FMT_ROWSCALE, FMT_BLK16_A, FMT_BLK16_B, FMT_MX32, FMT_NV16, FMT_FP8_1X128 = range(6)
FMT_BY_NAME = {
    "rowscale": FMT_ROWSCALE,
    "blk16": FMT_BLK16_A,
    "blk16_a": FMT_BLK16_A,
    "blk16_b": FMT_BLK16_B,
    "mx32": FMT_MX32,
    "nv16": FMT_NV16,
    "fp8_1x128": FMT_FP8_1X128,
}
DT_F32, DT_BF16, DT_FP4 = 0, 1, 2
ABI_VERSION = 6  # VX_ABI_VERSION of include/velox_b200.h
EPI_NONE, EPI_BIAS, EPI_BIAS_SWISH, EPI_BIAS_GLU, EPI_BIAS_RESIDUAL, EPI_BIAS_ARGMAX, EPI_BIAS_QKVPACK = range(7)
GEMM_DIRECT_STORE = 1
GEMM_STREAM_B = 2
GEMM_WIDE_TILES = 4
GEMM_NARROW_TILES = 8
GEMM_OUT_HEADS = 16

EXPORTS = (
    "vx_abi_version",
    "vx_last_error",
    "vx_device_status",
    "vx_sf_kgroups",
    "vx_sf_bytes",
    "vx_quantize_pack",
    "vx_ln_quantize_pack",
    "vx_ln2_quantize_pack",
    "vx_amax",
    "vx_sf_from_natural",
    "vx_bsgemm",
    "vx_mma_peak_probe",
    "vx_set_trace_buffer",
    "vx_blkscale_gemm_noalloc",
    "vx_glu_tile",
    "vx_argmax_ids",
    "vx_qkv_pack",
    "vx_wait_selftest",
    "vx_tmap_cache_stats",
    "vx_ctc_lse_parts",
    "vx_ctc_finish",
    "vx_ctc_topk_threshold",
    "vx_ctc_topk_finish",
    "vx_power_mel_log_supported",
    "vx_power_mel_log",
    "vx_relpos_attention",
    "vx_bsgemm_residual_ln_supported",
    "vx_bsgemm_residual_ln",
    "vx_bsgemm_residual_ln2",
)


class GemmDesc(C.Structure):
    """``vx_gemm_desc``."""

    _fields_ = [
        ("struct_size", C.c_int32),
        ("fmt", C.c_int32),
        ("M", C.c_int64),
        ("N", C.c_int64),
        ("K", C.c_int64),
        ("a_codes", C.c_void_p),
        ("lda", C.c_int64),
        ("b_codes", C.c_void_p),
        ("ldb", C.c_int64),
        ("a_scales", C.c_void_p),
        ("b_scales", C.c_void_p),
        ("a_amax", C.c_void_p),
        ("b_amax", C.c_void_p),
        ("epilogue", C.c_int32),
        ("out_dtype", C.c_int32),
        ("out", C.c_void_p),
        ("ldo", C.c_int64),
        ("bias", C.c_void_p),
        ("residual", C.c_void_p),
        ("residual_dtype", C.c_int32),
        ("out_fmt", C.c_int32),
        ("ldr", C.c_int64),
        ("alpha", C.c_float),
        ("flags", C.c_int32),
        ("out_scales_sf", C.c_void_p),
        ("out_scales", C.c_void_p),
        ("out_amax", C.c_void_p),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("pos_u", C.c_void_p),
        ("pos_v", C.c_void_p),
        ("qk_scale", C.c_float),
        ("head_col_off", C.c_int32),
        ("lse_partials", C.c_void_p),
        ("topk_threshold", C.c_void_p),
        ("topk_candidates", C.c_void_p),
        ("topk_count", C.c_void_p),
        ("topk_capacity", C.c_int32),
        ("reserved0", C.c_int32),
    ]


_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    """The shared object that gets loaded: ``VELOX_B200_LIB`` (a path to another build of the
    same ABI) if set, else the in-tree build."""
    return os.environ.get("VELOX_B200_LIB") or _build.LIB_PATH


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load (building first when the sources are newer) and type the library."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if path == _build.LIB_PATH and build_if_missing and not _build.is_current():
            try:
                _build.build()
            except Exception as e:  # no nvcc on this machine: use the shipped binary if any
                if not os.path.exists(path):
                    raise RuntimeError(f"libvelox_b200.so is missing and cannot be built: {e}") from e
        if not os.path.exists(path):
            raise RuntimeError(f"{path} not found: run `python -m velox_voice_b200.build`")
        lib = C.CDLL(path)
        i64, vp, i32, f32 = C.c_int64, C.c_void_p, C.c_int, C.c_float
        lib.vx_abi_version.restype = i32
        lib.vx_abi_version.argtypes = []
        lib.vx_last_error.restype = C.c_char_p
        lib.vx_last_error.argtypes = []
        lib.vx_device_status.restype = i32
        lib.vx_device_status.argtypes = [C.POINTER(C.c_int)]
        lib.vx_sf_kgroups.restype = i64
        lib.vx_sf_kgroups.argtypes = [i32, i64]
        lib.vx_sf_bytes.restype = i64
        lib.vx_sf_bytes.argtypes = [i32, i64, i64]
        lib.vx_quantize_pack.restype = i32
        lib.vx_quantize_pack.argtypes = [vp, i32, i64, i64, i64, i32, vp, i64, vp, vp, vp, vp]
        lib.vx_ln2_quantize_pack.restype = i32
        lib.vx_ln2_quantize_pack.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, f32, i32, vp, i64, vp, vp, vp, vp, i32, i64, vp]
        lib.vx_ln_quantize_pack.restype = i32
        lib.vx_ln_quantize_pack.argtypes = [vp, i32, i64, i64, i64, vp, vp, f32, i32, vp, i64, vp, vp, vp, vp, i32, i64, vp]
        lib.vx_amax.restype = i32
        lib.vx_amax.argtypes = [vp, i32, i64, i64, i64, vp, vp]
        lib.vx_sf_from_natural.restype = i32
        lib.vx_sf_from_natural.argtypes = [i32, vp, i64, i64, vp, vp]
        lib.vx_bsgemm.restype = i32
        lib.vx_bsgemm.argtypes = [C.POINTER(GemmDesc), vp]
        lib.vx_blkscale_gemm_noalloc.restype = i32
        lib.vx_blkscale_gemm_noalloc.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, vp]
        lib.vx_glu_tile.restype = i32
        lib.vx_glu_tile.argtypes = [i32]
        lib.vx_qkv_pack.restype = i32
        lib.vx_qkv_pack.argtypes = [vp, i64, vp, i64, vp, vp, f32, i64, i32, i32, vp, vp, vp, vp]
        lib.vx_argmax_ids.restype = i32
        lib.vx_argmax_ids.argtypes = [vp, i64, vp, vp, vp]
        lib.vx_ctc_lse_parts.restype = i64
        lib.vx_ctc_lse_parts.argtypes = [i64]
        lib.vx_ctc_finish.restype = i32
        lib.vx_ctc_finish.argtypes = [vp, vp, i64, i64, vp, vp, vp, vp, vp]
        lib.vx_power_mel_log_supported.restype = i32
        lib.vx_power_mel_log_supported.argtypes = [i64, i64]
        lib.vx_power_mel_log.restype = i32
        lib.vx_power_mel_log.argtypes = [vp, i64, i64, i64, vp, i64, i64, vp, vp, vp, i64, vp]
        lib.vx_relpos_attention.restype = i32
        lib.vx_relpos_attention.argtypes = [vp, vp, vp, i64, i32, i32, i64, vp, i64, vp]
        lib.vx_bsgemm_residual_ln_supported.restype = i32
        lib.vx_bsgemm_residual_ln_supported.argtypes = [i32, i64, i64]
        lib.vx_bsgemm_residual_ln.restype = i32
        lib.vx_bsgemm_residual_ln.argtypes = [vp, vp, vp, C.c_float, vp, i64, vp, vp]
        lib.vx_bsgemm_residual_ln2.restype = i32
        lib.vx_bsgemm_residual_ln2.argtypes = [vp, vp, vp, vp, vp, C.c_float, vp, i64, vp, vp]
        lib.vx_ctc_topk_threshold.restype = i32
        lib.vx_ctc_topk_threshold.argtypes = [vp, i64, i64, i32, vp, vp]
        lib.vx_ctc_topk_finish.restype = i32
        lib.vx_ctc_topk_finish.argtypes = [vp, vp, i32, vp, i64, i64, i32, vp, vp, vp, vp]
        lib.vx_set_trace_buffer.restype = i32
        lib.vx_set_trace_buffer.argtypes = [vp, i64]
        lib.vx_wait_selftest.restype = i32
        lib.vx_wait_selftest.argtypes = [i64, i32, vp]
        lib.vx_tmap_cache_stats.restype = i32
        lib.vx_tmap_cache_stats.argtypes = [C.POINTER(i64), C.POINTER(i64)]
        lib.vx_mma_peak_probe.restype = i32
        lib.vx_mma_peak_probe.argtypes = [i32, i32, i32, C.POINTER(C.c_float)]
        if lib.vx_abi_version() != ABI_VERSION:
            raise RuntimeError("libvelox_b200.so: ABI version mismatch")
        _lib = lib
        return lib


class VeloxError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().vx_last_error().decode(errors="replace")
        kind = "argument error" if rc < 0 else f"CUDA error {rc}"
        raise VeloxError(f"{what}: {kind}: {msg}")


def device_status() -> int:
    """Synchronise and return the device status word (0 = OK); raises on CUDA errors."""
    out = C.c_int(0)
    check(load().vx_device_status(C.byref(out)), "vx_device_status")
    return out.value
