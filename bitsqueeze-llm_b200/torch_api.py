"""PyTorch door onto the library: compress / decompress CUDA tensors in place on the GPU, ordered after the work already
queued on PyTorch's current stream.

The reference has no Python binding; its callers are C++ programs that hand `bitsqz_llm_compress` a raw pointer and get a
host object back (include/bitsqz_llm.hpp:121-135).  A training or serving loop that wants to park activations in
compressed form needs neither the host object nor a device-wide synchronisation: this module keeps the packed object in a
`torch.uint8` CUDA tensor (same bytes and layout as the host object, see `bsq_lane_compress_begin` in
include/bitsqz_llm_c.h) and lets the work run on a stream of the library's own that first waits for PyTorch's current
stream.  It is a thin wrapper: every byte is produced by the shared library, there is no fallback.

    comp = Compressor(rows, cols, outlier=0.005, error=0.01, rank=256, niters=2, uv=NF4)
    packed = comp.compress(x)            # x: float32 CUDA tensor (rows, cols); packed.data: uint8 CUDA tensor
    y = comp.decompress(packed)          # float32 CUDA tensor (rows, cols)
    blob = packed.to_bytes()             # the serialised object, loadable by load_bitsqz_llm_from_buffer anywhere
"""
import ctypes as C

import numpy as np
import torch

from . import Array, INPUT_DEVICE, INPUT_HOST, NF4, NF4_DQ, NONE, lib  # noqa: F401  (re-exported for callers)


class PackedMatrix:
    """A compressed matrix resident on the GPU: `data` holds header + payload, `header` is a host copy of the 200-byte
    header whose payload member points into `data`."""

    def __init__(self, data, header, nbytes):
        self.data = data
        self.header = header
        self.nbytes = int(nbytes)

    def to_bytes(self):
        """The serialised object (numpy uint8), as bitsqz_llm_get_packed_size / a byte copy of a host object would give."""
        return self.data[: self.nbytes].cpu().numpy()

    @property
    def compression_ratio(self):
        return self.header.num_elements * 4 / self.nbytes


class _Pending:
    def __init__(self, owner, finish):
        self._owner, self._finish, self._result = owner, finish, None

    def wait(self):
        """Blocks the host until the call is done and returns its result."""
        if self._finish is not None:
            self._result = self._finish()
            self._finish = None
        return self._result


class Compressor:
    """One shape and one set of pipeline settings on the current CUDA device (a lane of the library: a compress and a
    decompress runtime with a stream of their own).  Not thread-safe; one call in flight at a time."""

    def __init__(self, rows, cols, outlier=0.0, error=0.0, rank=-1, niters=2, uv=NONE, s=NONE, q=NONE):
        self.rows, self.cols = int(rows), int(cols)
        self._lib = lib()
        self._device = torch.cuda.current_device()
        self._lane = self._lib.bsq_lane_create(self.rows, self.cols, outlier, error, rank, niters, uv, s, q)
        if not self._lane:
            raise RuntimeError("bsq_lane_create failed (invalid settings or out of device memory)")
        self.capacity = int(self._lib.bsq_lane_packed_capacity(self._lane))
        self._c_stream = torch.cuda.ExternalStream(self._lib.bsq_lane_stream(self._lane, 0), device=self._device)
        self._d_stream = torch.cuda.ExternalStream(self._lib.bsq_lane_stream(self._lane, 1), device=self._device)

    def close(self):
        if self._lane:
            self._lib.bsq_lane_destroy(self._lane)
            self._lane = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- compress ----
    def compress_async(self, x, out=None):
        """Queues the compression of `x` behind the work on PyTorch's current stream and returns a handle whose wait()
        gives the PackedMatrix.  `x`: float32, contiguous, (rows, cols), on this device or in (pinned) host memory."""
        if x.dtype != torch.float32 or tuple(x.shape) != (self.rows, self.cols) or not x.is_contiguous():
            raise ValueError("expected a contiguous float32 tensor of shape (%d, %d)" % (self.rows, self.cols))
        if out is None:
            out = torch.empty(self.capacity, dtype=torch.uint8, device=torch.device("cuda", self._device))
        elif out.dtype != torch.uint8 or out.numel() < self.capacity or not out.is_cuda or not out.is_contiguous():
            raise ValueError("out must be a contiguous uint8 CUDA tensor of at least %d bytes" % self.capacity)
        location = INPUT_DEVICE if x.is_cuda else INPUT_HOST
        self._c_stream.wait_stream(torch.cuda.current_stream(self._device))      # x and out may still be written there
        if self._lib.bsq_lane_compress_begin(self._lane, x.data_ptr(), location, out.data_ptr(), out.numel()) != 0:
            raise RuntimeError("bsq_lane_compress_begin failed")
        # x and out are kept alive by this closure until wait() has seen the lane's stream finish, so the caching
        # allocator cannot hand their memory to anybody else in the meantime

        def finish(x=x, out=out):
            hdr, size = Array(), C.c_uint64(0)
            if self._lib.bsq_lane_compress_end(self._lane, None, C.byref(hdr), C.byref(size)) != 0:
                raise RuntimeError("compression failed (a kernel reported an error)")
            return PackedMatrix(out, hdr, size.value)
        return _Pending(self, finish)

    def compress(self, x, out=None):
        return self.compress_async(x, out).wait()

    # ---- decompress ----
    def decompress_async(self, packed, out=None):
        """Queues the decompression of `packed` (a PackedMatrix, or serialised bytes as numpy uint8 / bytes) behind the work on
        PyTorch's current stream; wait() gives the float32 (rows, cols) CUDA tensor."""
        if out is None:
            out = torch.empty((self.rows, self.cols), dtype=torch.float32, device=torch.device("cuda", self._device))
        elif out.dtype != torch.float32 or out.numel() < self.rows * self.cols or not out.is_cuda or not out.is_contiguous():
            raise ValueError("out must be a contiguous float32 CUDA tensor of rows x cols elements")
        self._d_stream.wait_stream(torch.cuda.current_stream(self._device))
        host_obj = None
        if isinstance(packed, PackedMatrix):
            rc = self._lib.bsq_lane_decompress_begin(self._lane, C.byref(packed.header), 1, out.data_ptr(), out.numel())
        else:
            blob = np.ascontiguousarray(np.frombuffer(packed, np.uint8) if isinstance(packed, (bytes, bytearray)) else packed, np.uint8)
            host_obj = self._lib.bsq_load_from_buffer(blob.ctypes.data, blob.size)
            if not host_obj:
                raise ValueError("not a loadable packed object")
            rc = self._lib.bsq_lane_decompress_begin(self._lane, host_obj, 0, out.data_ptr(), out.numel())
        if rc != 0:
            if host_obj:
                self._lib.bsq_free(host_obj)
            raise RuntimeError("object does not fit this Compressor (shape, rank, formats or top-k capacity)")

        def finish(packed=packed, out=out):                   # (references held until the lane's stream has finished)
            rc2 = self._lib.bsq_lane_decompress_end(self._lane)
            if host_obj:
                self._lib.bsq_free(host_obj)
            if rc2 != 0:
                raise RuntimeError("decompression failed (a kernel reported an error)")
            return out
        return _Pending(self, finish)

    def decompress(self, packed, out=None):
        return self.decompress_async(packed, out).wait()
