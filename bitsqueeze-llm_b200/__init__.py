"""bitsqz_llm for B200: Python door onto the C ABI of lib/libbitsqz_llm.so.

The product is the shared library (CUDA kernels + C++ host code, csrc/); this module only
binds its `extern "C"` entry points (include/bitsqz_llm_c.h) with ctypes so that tests, the
benchmark and Python callers can reach them.  It computes nothing itself and has no fallback:
if the library is missing, importing `lib()` raises.

Device pointers are plain integers (for example `torch.Tensor.data_ptr()`); `stream` arguments
are `cudaStream_t` handles as integers (0 = legacy default stream).
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libbitsqz_llm.so")

# enum values of include/bitsqz_llm.hpp
NONE, NF4_DQ, NF4 = -1, 10, 11
INPUT_HOST, INPUT_DEVICE = 0, 1
SECTION_NONE, SECTION_FP32, SECTION_QUANT, SECTION_TOPK = 0, 1, 2, 3
FLAG_SVD, FLAG_OUTLIER, FLAG_ERROR = 1, 2, 4


class Section(C.Structure):
    _fields_ = [("offset", C.c_uint64), ("size", C.c_uint64), ("storage", C.c_uint8), ("reserved", C.c_uint8 * 7)]


class Array(C.Structure):
    """bitsqz_llm_array_t (200 bytes)."""
    _fields_ = [
        ("num_rows", C.c_uint16), ("num_columns", C.c_uint16), ("num_elements", C.c_uint32),
        ("outlier_topk_ratio", C.c_float), ("error_correction_topk_ratio", C.c_float),
        ("svd_ranks", C.c_int16), ("svd_niters", C.c_int16), ("effective_rank", C.c_int16), ("reserved0", C.c_int16),
        ("svd_uv_format", C.c_int32), ("svd_s_format", C.c_int32), ("quantization_only_format", C.c_int32),
        ("reserved1", C.c_int32), ("flags", C.c_uint32),
        ("section_u", Section), ("section_s", Section), ("section_v", Section), ("section_direct", Section),
        ("section_outlier_topk", Section), ("section_error_topk", Section),
        ("payload", C.c_void_p),
    ]


class Profile(C.Structure):
    """bitsqz_llm_compress_profile_t (seven doubles, milliseconds)."""
    _fields_ = [(n, C.c_double) for n in (
        "topk_separation_latency_ms", "svd_lowrank_cuda_latency_ms", "quantization_compress_latency_ms",
        "reconsturct_quantization_decompress_latency_ms", "reconstruct_svd_latency_ms",
        "error_extraction_latency_ms", "other_latency_ms")]


assert C.sizeof(Section) == 24 and C.sizeof(Array) == 200 and C.sizeof(Profile) == 56

_vp, _u16, _u32, _u64, _i, _f, _sz = C.c_void_p, C.c_uint16, C.c_uint32, C.c_uint64, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); exactly the declarations of include/bitsqz_llm_c.h
SIGNATURES = {
    "bsq_compress_initialize": (_i, [_u16, _u16, _f, _f, _i, _i, _i, _i, _i, _i]),
    "bsq_compress_release": (None, []),
    "bsq_decompress_initialize": (_i, [_u16, _u16, _f, _f, _i, _i, _i, _i]),
    "bsq_decompress_release": (None, []),
    "bsq_compress": (_i, [_vp, C.POINTER(_vp), _vp]),
    "bsq_decompress": (_i, [_vp, _vp, _u32]),
    "bsq_get_packed_size": (_u64, [_vp]),
    "bsq_load_from_buffer": (_vp, [_vp, _u64]),
    "bsq_free": (None, [_vp]),
    "bsq_topk_num_columns": (_i, [_u16, _f]),
    "bsq_topk_rows": (_i, [_vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp]),
    "bsq_topk_apply": (_i, [_vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp]),
    "bsq_nf4_quantize": (_i, [_vp, _u64, _vp, _vp, _vp, _vp]),
    "bsq_nf4dq_scratch_bytes": (_sz, [_u64]),
    "bsq_nf4dq_quantize": (_i, [_vp, _u64, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bsq_nf4dq_quantize_static_max_elements": (_u64, []),
    "bsq_nf4dq_quantize_static": (_i, [_vp, _u64, _vp, _vp, _vp, _vp]),
    "bsq_nf4_dequantize": (_i, [_vp, _vp, _u64, _vp, _vp]),
    "bsq_nf4dq_dequantize": (_i, [_vp, _vp, _vp, _u64, _vp, _vp]),
    "bsq_dequantize_add_topk": (_i, [_i, _vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp, _u32, _vp, _vp, _vp]),
    "bsq_frontend_supported": (_i, [_u32, _u32, _u32]),
    "bsq_frontend_scratch_bytes": (_sz, [_u32, _u32]),
    "bsq_frontend_quantize": (_i, [_i, _vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bsq_frontend_quantize_timed": (_i, [_i, _vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "bsq_residual_error": (_i, [_vp, _vp, _u64, _vp, _vp, _vp]),
    "bsq_svd_lowrank": (_i, [_vp, _i, _i, _i, _i, C.c_ulonglong, _vp, _vp, _vp, _vp]),
    "bsq_svd_lowrank_at": (_i, [_vp, _i, _i, _i, _i, C.c_ulonglong, C.c_ulonglong, _vp, _vp, _vp, _vp]),
    "bsq_reconstruct": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "bsq_gemm": (_i, [_i, _i, _vp, C.c_long, _vp, C.c_long, _vp, C.c_long, _i, _i, _i, _vp, _sz, _i, _vp, _vp]),
    "bsq_gemm_bounded": (_i, [_i, _i, _vp, C.c_long, _vp, C.c_long, _vp, C.c_long, _i, _i, _i, _vp, _sz, _vp, _vp, _vp]),
    "bsq_shard_unique_id": (_i, [_vp, _sz]),
    "bsq_shard_comm_create": (_vp, [_vp, _i, _i]),
    "bsq_shard_comm_destroy": (None, [_vp]),
    "bsq_svd_lowrank_sharded": (_i, [_vp, _vp, _i, _i, _i, _i, _i, C.c_ulonglong, _vp, _vp, _vp, _vp]),
    "bsq_shard_svd_create": (_vp, [_vp, _i, _i, _i, _i, _i]),
    "bsq_shard_svd_destroy": (None, [_vp]),
    "bsq_shard_svd_run": (_i, [_vp, _vp, C.c_ulonglong, _vp, _vp, _vp, _vp]),
    "bsq_shard_compress": (_i, [_vp, _vp, C.c_ulonglong, C.POINTER(_vp), _vp]),
    "bsq_shard_uses_peer_exchange": (_i, [_vp]),
    "bsq_shard_svd_profile": (_i, [_vp, _i]),
    "bsq_shard_svd_profile_read": (_i, [_vp, _vp, _vp, _i]),
    "bsq_lane_create": (_vp, [_u16, _u16, _f, _f, _i, _i, _i, _i, _i]),
    "bsq_lane_destroy": (None, [_vp]),
    "bsq_lane_packed_capacity": (_u64, [_vp]),
    "bsq_lane_stream": (_vp, [_vp, _i]),
    "bsq_lane_compress_begin": (_i, [_vp, _vp, _i, _vp, _u64]),
    "bsq_lane_compress_end": (_i, [_vp, C.POINTER(_vp), _vp, C.POINTER(_u64)]),
    "bsq_lane_decompress_begin": (_i, [_vp, _vp, _i, _vp, _u64]),
    "bsq_lane_decompress_end": (_i, [_vp]),
    "bsq_lane_profile": (_i, [_vp, _i]),
    "bsq_lane_profile_read": (_i, [_vp, _vp, _vp, _i]),
    "bsq_batch_create": (_vp, [_u16, _u16, _f, _f, _i, _i, _i, _i, _i, _i]),
    "bsq_batch_destroy": (None, [_vp]),
    "bsq_batch_lanes": (_i, [_vp]),
    "bsq_batch_lane": (_vp, [_vp, _i]),
    "bsq_batch_compress": (_i, [_vp, C.POINTER(_vp), _i, _i, C.POINTER(_vp), _u64, C.POINTER(_vp), _vp, C.POINTER(_u64)]),
    "bsq_batch_decompress": (_i, [_vp, C.POINTER(_vp), _i, _i, C.POINTER(_vp), _u64]),
    "bsq_test_inject_status": (None, [_i, _u32]),
    "bsq_build_info": (C.c_char_p, []),
}

# C++ symbols of include/bitsqz_llm.hpp as the reference library exports them (Itanium mangling)
CXX_SYMBOLS = [
    "_Z30bitsqz_llm_compress_initializettffii21quantization_method_tS_S_27bitsqz_llm_input_location_t",
    "_Z27bitsqz_llm_compress_releasev",
    "_Z32bitsqz_llm_decompress_initializettffi21quantization_method_tS_S_",
    "_Z29bitsqz_llm_decompress_releasev",
    "_Z19bitsqz_llm_compressPKfPP16bitsqz_llm_arrayP29bitsqz_llm_compress_profile_t",
    "_Z21bitsqz_llm_decompressPK16bitsqz_llm_arrayPfj",
    "_Z26bitsqz_llm_get_packed_sizePK16bitsqz_llm_array",
    "_Z27load_bitsqz_llm_from_bufferPKvm",
    "_Z15bitsqz_llm_freeP16bitsqz_llm_array",
    "_Z29topk_compute_num_topk_columnstf",
]

_lib = None


def lib():
    """The loaded library with argtypes set.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: run `python bitsqueeze-llm_b200/build.py` (there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def compress_to_bytes(x_ptr, profile=None):
    """bitsqz_llm_compress on a host or device pointer; returns (header copy, packed bytes) or None."""
    L = lib()
    out = _vp(None)
    prof_ref = C.byref(profile) if profile is not None else None
    if L.bsq_compress(x_ptr, C.byref(out), prof_ref) != 0:
        return None
    size = int(L.bsq_get_packed_size(out))
    packed = np.frombuffer(C.string_at(out.value, size), np.uint8).copy()
    hdr = Array.from_buffer_copy(packed[:200].tobytes())
    L.bsq_free(out)
    return hdr, packed


def load_packed(packed):
    """load_bitsqz_llm_from_buffer on packed bytes; returns an opaque handle (free with lib().bsq_free)."""
    packed = np.ascontiguousarray(packed, np.uint8)
    return lib().bsq_load_from_buffer(packed.ctypes.data, packed.size)


def decompress_packed(packed, d_dst_ptr, n):
    """Round trip through load + bitsqz_llm_decompress; returns the C return code."""
    h = load_packed(packed)
    if not h:
        return 1
    try:
        return int(lib().bsq_decompress(h, d_dst_ptr, n))
    finally:
        lib().bsq_free(h)
