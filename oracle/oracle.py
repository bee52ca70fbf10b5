"""TEST INFRASTRUCTURE ONLY: ctypes doors onto the CPU oracle and the reference builds.

`Oracle`  -- oracle/liboracle.so, the plain-C restatement (bsq_oracle.c).
`RefCpu`  -- oracle/_ref/libref_cpu.so, the reference's own CPU NF4 / NF4_DQ code
             (legacy_modules/quantization) behind ref_cpu_shim.cpp.
`RefCuda` -- oracle/_ref/libref_cuda.so, the reference's own CUDA build for sm_100 behind
             ref_cuda_shim.cu (needs a GPU; device pointers are plain integers).

Only tests, the smoke check and the bench's CPU-baseline / reference legs import this.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_CPU_SO = os.path.join(HERE, "_ref", "libref_cpu.so")
REF_CUDA_SO = os.path.join(HERE, "_ref", "libref_cuda.so")

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_u16p = C.POINTER(C.c_uint16)


def _p(a, t):
    return a.ctypes.data_as(t)


def _f32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def nblocks(n):
    return (n + 63) // 64


class Oracle:
    def __init__(self, path=ORACLE_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} missing: run `make -C oracle`")
        L = self.lib = C.CDLL(path)
        L.bsq_oracle_nf4_code.restype = C.c_uint8
        L.bsq_oracle_nf4_code.argtypes = [C.c_float]
        L.bsq_oracle_nf4_level.restype = C.c_float
        L.bsq_oracle_nf4_level.argtypes = [C.c_uint8]
        L.bsq_oracle_e4m3_encode.restype = C.c_uint8
        L.bsq_oracle_e4m3_encode.argtypes = [C.c_float]
        L.bsq_oracle_e4m3_decode.restype = C.c_float
        L.bsq_oracle_e4m3_decode.argtypes = [C.c_uint8]
        L.bsq_oracle_nf4_quantize.argtypes = [_f32p, C.c_uint64, _f32p, _u8p]
        L.bsq_oracle_nf4_dequantize.argtypes = [_f32p, _u8p, C.c_uint64, _f32p]
        L.bsq_oracle_nf4dq_quantize.argtypes = [_f32p, C.c_uint64, _f32p, _u8p, _u8p]
        L.bsq_oracle_nf4dq_dequantize.argtypes = [C.c_float, _u8p, _u8p, C.c_uint64, _f32p]
        L.bsq_oracle_topk_num_columns.restype = C.c_uint32
        L.bsq_oracle_topk_num_columns.argtypes = [C.c_uint16, C.c_float]
        L.bsq_oracle_topk_rows.argtypes = [_f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, _u16p, _f32p]
        L.bsq_oracle_topk_apply.argtypes = [_u16p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p]
        L.bsq_oracle_residual.argtypes = [_f32p, _f32p, C.c_uint64, _f32p]
        L.bsq_oracle_reconstruct.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p]
        L.bsq_oracle_quant_section_size.restype = C.c_uint64
        L.bsq_oracle_quant_section_size.argtypes = [C.c_int, C.c_uint64]
        L.bsq_oracle_pack_quant_section.argtypes = [C.c_int, _f32p, C.c_uint64, _u8p]
        L.bsq_oracle_topk_section_size.restype = C.c_uint64
        L.bsq_oracle_topk_section_size.argtypes = [C.c_uint32, C.c_uint32]
        L.bsq_oracle_compress_nosvd.restype = C.c_uint64
        L.bsq_oracle_compress_nosvd.argtypes = [_f32p, C.c_uint16, C.c_uint16, C.c_float, C.c_float, C.c_int,
                                                _u8p, C.c_uint64]
        L.bsq_oracle_decompress_nosvd.argtypes = [_u8p, C.c_uint64, _f32p]
        L.bsq_oracle_max_threads.restype = C.c_int

    def max_threads(self):
        return int(self.lib.bsq_oracle_max_threads())

    def set_threads(self, n):
        self.lib.bsq_oracle_set_threads(int(n))

    def nf4_code(self, v):
        return int(self.lib.bsq_oracle_nf4_code(C.c_float(v)))

    def e4m3_encode(self, v):
        return int(self.lib.bsq_oracle_e4m3_encode(C.c_float(v)))

    def e4m3_decode(self, c):
        return float(self.lib.bsq_oracle_e4m3_decode(C.c_uint8(c)))

    def nf4_quantize(self, x):
        x = _f32(x).ravel()
        n = x.size
        scales = np.empty(nblocks(n), np.float32)
        data = np.empty((n + 1) // 2, np.uint8)
        assert self.lib.bsq_oracle_nf4_quantize(_p(x, _f32p), n, _p(scales, _f32p), _p(data, _u8p)) == 0
        return scales, data

    def nf4_dequantize(self, scales, data, n):
        out = np.empty(n, np.float32)
        scales = _f32(scales)
        data = np.ascontiguousarray(data, np.uint8)
        assert self.lib.bsq_oracle_nf4_dequantize(_p(scales, _f32p), _p(data, _u8p), n, _p(out, _f32p)) == 0
        return out

    def nf4dq_quantize(self, x):
        x = _f32(x).ravel()
        n = x.size
        dq = C.c_float(0)
        codes = np.empty(nblocks(n), np.uint8)
        data = np.empty((n + 1) // 2, np.uint8)
        assert self.lib.bsq_oracle_nf4dq_quantize(_p(x, _f32p), n, C.byref(dq), _p(codes, _u8p), _p(data, _u8p)) == 0
        return np.float32(dq.value), codes, data

    def nf4dq_dequantize(self, dq, codes, data, n):
        out = np.empty(n, np.float32)
        codes = np.ascontiguousarray(codes, np.uint8)
        data = np.ascontiguousarray(data, np.uint8)
        assert self.lib.bsq_oracle_nf4dq_dequantize(C.c_float(dq), _p(codes, _u8p), _p(data, _u8p), n,
                                                    _p(out, _f32p)) == 0
        return out

    def topk_num_columns(self, cols, ratio):
        return int(self.lib.bsq_oracle_topk_num_columns(cols, C.c_float(ratio)))

    def topk_rows(self, x, k, zero_selected=False):
        """Returns (idx[rows,k] u16, val[rows,k] f32, matrix after optional zeroing)."""
        x = _f32(x).copy()
        rows, cols = x.shape
        idx = np.zeros((rows, k), np.uint16)
        val = np.zeros((rows, k), np.float32)
        rc = self.lib.bsq_oracle_topk_rows(_p(x, _f32p), rows, cols, k, int(zero_selected), _p(idx, _u16p),
                                           _p(val, _f32p))
        assert rc == 0
        return idx, val, x

    def topk_apply(self, idx, val, dense):
        dense = _f32(dense).copy()
        rows, cols = dense.shape
        idx = np.ascontiguousarray(idx, np.uint16)
        val = _f32(val)
        k = idx.shape[1] if idx.ndim == 2 else 0
        assert self.lib.bsq_oracle_topk_apply(_p(idx, _u16p), _p(val, _f32p), rows, cols, k, _p(dense, _f32p)) == 0
        return dense

    def reconstruct(self, U, S, V):
        U, S, V = _f32(U), _f32(S), _f32(V)
        m, k = U.shape
        n = V.shape[0]
        out = np.empty((m, n), np.float32)
        assert self.lib.bsq_oracle_reconstruct(_p(U, _f32p), _p(S, _f32p), _p(V, _f32p), m, n, k, _p(out, _f32p)) == 0
        return out

    def quant_section(self, method, x):
        x = _f32(x).ravel()
        size = int(self.lib.bsq_oracle_quant_section_size(method, x.size))
        dst = np.zeros(size, np.uint8)
        assert self.lib.bsq_oracle_pack_quant_section(method, _p(x, _f32p), x.size, _p(dst, _u8p)) == 0
        return dst

    def compress_nosvd(self, x, outlier_ratio, error_ratio, quant_method):
        """Packed bytes (200-byte header + payload) the reference produces without SVD."""
        x = _f32(x)
        rows, cols = x.shape
        cap = 200 + x.size * 4 + 64 + 2 * (8 + x.size * 6) + x.size
        dst = np.zeros(cap, np.uint8)
        size = int(self.lib.bsq_oracle_compress_nosvd(_p(x, _f32p), rows, cols, C.c_float(outlier_ratio),
                                                      C.c_float(error_ratio), quant_method, _p(dst, _u8p), cap))
        assert size >= 200
        return dst[:size].copy()

    def decompress_nosvd(self, packed, rows, cols):
        packed = np.ascontiguousarray(packed, np.uint8)
        out = np.empty((rows, cols), np.float32)
        assert self.lib.bsq_oracle_decompress_nosvd(_p(packed, _u8p), packed.size, _p(out, _f32p)) == 0
        return out


class RefCpu:
    def __init__(self, path=REF_CPU_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = self.lib = C.CDLL(path)
        L.ref_nf4_quantize.argtypes = [_f32p, C.c_ulonglong, _f32p, _u8p]
        L.ref_nf4_roundtrip.argtypes = [_f32p, C.c_ulonglong, _f32p]
        L.ref_nf4dq_quantize.argtypes = [_f32p, C.c_ulonglong, _f32p, _u8p, _u8p]
        L.ref_nf4dq_roundtrip.argtypes = [_f32p, C.c_ulonglong, _f32p]
        L.ref_nf4_dequantize.argtypes = [_f32p, _u8p, C.c_ulonglong, _f32p]
        L.ref_nf4dq_dequantize.argtypes = [C.c_float, _u8p, _u8p, C.c_ulonglong, _f32p]
        L.ref_cpu_max_threads.restype = C.c_int

    def max_threads(self):
        return int(self.lib.ref_cpu_max_threads())

    def set_threads(self, n):
        self.lib.ref_cpu_set_threads(int(n))

    def nf4_quantize(self, x):
        x = _f32(x).ravel()
        n = x.size
        scales = np.empty(nblocks(n), np.float32)
        data = np.empty((n + 1) // 2, np.uint8)
        assert self.lib.ref_nf4_quantize(_p(x, _f32p), n, _p(scales, _f32p), _p(data, _u8p)) == 0
        return scales, data

    def nf4dq_quantize(self, x):
        x = _f32(x).ravel()
        n = x.size
        dq = C.c_float(0)
        codes = np.empty(nblocks(n), np.uint8)
        data = np.empty((n + 1) // 2, np.uint8)
        assert self.lib.ref_nf4dq_quantize(_p(x, _f32p), n, C.byref(dq), _p(codes, _u8p), _p(data, _u8p)) == 0
        return np.float32(dq.value), codes, data

    def nf4_roundtrip(self, x):
        x = _f32(x).ravel()
        out = np.empty_like(x)
        assert self.lib.ref_nf4_roundtrip(_p(x, _f32p), x.size, _p(out, _f32p)) == 0
        return out

    def nf4dq_roundtrip(self, x):
        x = _f32(x).ravel()
        out = np.empty_like(x)
        assert self.lib.ref_nf4dq_roundtrip(_p(x, _f32p), x.size, _p(out, _f32p)) == 0
        return out

    def nf4_dequantize(self, scales, data, n):
        out = np.empty(n, np.float32)
        scales, data = _f32(scales), np.ascontiguousarray(data, np.uint8)
        assert self.lib.ref_nf4_dequantize(_p(scales, _f32p), _p(data, _u8p), n, _p(out, _f32p)) == 0
        return out

    def nf4dq_dequantize(self, dq, codes, data, n):
        out = np.empty(n, np.float32)
        codes, data = np.ascontiguousarray(codes, np.uint8), np.ascontiguousarray(data, np.uint8)
        assert self.lib.ref_nf4dq_dequantize(C.c_float(dq), _p(codes, _u8p), _p(data, _u8p), n, _p(out, _f32p)) == 0
        return out


class RefCuda:
    """Device pointers are passed as integers (e.g. torch.Tensor.data_ptr())."""

    def __init__(self, path=REF_CUDA_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = self.lib = C.CDLL(path)
        vp, u16, u64, i, f = C.c_void_p, C.c_uint16, C.c_uint64, C.c_int, C.c_float
        L.ref_compress_initialize.argtypes = [u16, u16, f, f, i, i, i, i, i, i]
        L.ref_decompress_initialize.argtypes = [u16, u16, f, f, i, i, i, i]
        L.ref_compress.argtypes = [vp, C.POINTER(vp), vp]
        L.ref_decompress.argtypes = [vp, vp, C.c_uint32]
        L.ref_get_packed_size.restype = u64
        L.ref_get_packed_size.argtypes = [vp]
        L.ref_load_from_buffer.restype = vp
        L.ref_load_from_buffer.argtypes = [vp, u64]
        L.ref_free.argtypes = [vp]
        L.ref_topk_num_columns.argtypes = [u16, f]
        L.ref_topk_rows.argtypes = [vp, u16, u16, u16, i, vp, vp]
        L.ref_topk_apply.argtypes = [vp, vp, u16, u16, u16, vp]
        L.ref_quant_compress.argtypes = [i, vp, u64, vp, vp, vp, vp]
        L.ref_quant_decompress.argtypes = [i, vp, vp, vp, vp, u64, vp]
        L.ref_svd_initialize.argtypes = [i, i, i, i, C.c_ulonglong]
        L.ref_svd_run.argtypes = [vp, vp, vp, vp, C.c_ulonglong]
        L.ref_reconstruct.argtypes = [vp, vp, vp, i, i, i, vp]

    def compress_bytes(self, x_ptr, profile=None):
        """bitsqz_llm_compress through the reference; returns the packed bytes."""
        out = C.c_void_p(None)
        rc = self.lib.ref_compress(x_ptr, C.byref(out), profile)
        if rc != 0:
            return None
        size = int(self.lib.ref_get_packed_size(out))
        buf = np.frombuffer(C.string_at(out.value, size), np.uint8).copy()
        self.lib.ref_free(out)
        return buf
