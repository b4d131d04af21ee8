"""ctypes front end of the host quantisation codec (ti_host_* ABI v1).

Mirrors the reference's llm/host_codec.py:10-54 (`HostCodec.quantized_bytes`,
`HostCodec.dequantized_half_bytes`, ValueError on rejection) and adds numpy-array variants
used by the artifact writer, which avoid a Python-level pass over every element.
"""
import ctypes
import struct
import sys
from pathlib import Path

import numpy as np

from . import library


class HostCodec:
    def __init__(self, library_path=None):
        self.path = Path(library_path).resolve(strict=True) if library_path else library("host_codec")
        self.lib = ctypes.CDLL(str(self.path))
        self.lib.ti_host_codec_abi_version.argtypes = []
        self.lib.ti_host_codec_abi_version.restype = ctypes.c_int
        if self.lib.ti_host_codec_abi_version() != 1:
            raise ValueError("native host codec ABI v1 required")
        p, z = ctypes.c_void_p, ctypes.c_size_t
        for name in ("ti_host_quantize_f16", "ti_host_dequantize_i8"):
            fn = getattr(self.lib, name)
            fn.argtypes, fn.restype = [p, z, z, p, z, p, z], ctypes.c_int
        if sys.byteorder != "little":
            raise ValueError("exporter codec requires little endian host")

    # ---- numpy interface -------------------------------------------------------------
    def quantize_array(self, w16):
        """float16 [K, N] -> (int8 [K, N], float32 [N]); ValueError when the codec rejects it."""
        w16 = np.ascontiguousarray(w16, np.float16)
        if w16.ndim != 2 or w16.size == 0:
            raise ValueError("nonempty rectangular [K,N] FP16 reference required")
        q = np.empty(w16.shape, np.int8)
        scales = np.empty(w16.shape[1], np.float32)
        status = self.lib.ti_host_quantize_f16(w16.ctypes.data, w16.size, w16.shape[1], q.ctypes.data, q.size,
                                               scales.ctypes.data, scales.size)
        if status:
            raise ValueError(f"native quantization rejected buffers/values ({status})")
        return q, scales

    def dequantize_array(self, q, scales):
        q, scales = np.ascontiguousarray(q, np.int8), np.ascontiguousarray(scales, np.float32)
        if q.ndim != 2 or q.size == 0 or scales.shape != (q.shape[1],):
            raise ValueError("nonempty rectangular INT8 matrix with FP32 output-channel scales required")
        out = np.empty(q.shape, np.float16)
        status = self.lib.ti_host_dequantize_i8(q.ctypes.data, q.size, q.shape[1], scales.ctypes.data, scales.size,
                                                out.ctypes.data, out.size)
        if status:
            raise ValueError(f"native dequantization rejected buffers/values ({status})")
        return out

    # ---- the reference wrapper's byte interface ---------------------------------------
    def quantized_bytes(self, values, columns):
        if type(columns) is not int or columns <= 0 or not len(values) or len(values) % columns:
            raise ValueError("nonempty rectangular [K,N] FP16 reference required")
        half = np.array(struct.unpack(f"<{len(values)}e", struct.pack(f"<{len(values)}e", *values)), np.float16)
        q, scales = self.quantize_array(half.reshape(-1, columns))
        return q.tobytes(), scales.tobytes()

    def dequantized_half_bytes(self, q_bytes, scale_bytes, columns):
        if type(columns) is not int or columns <= 0 or len(scale_bytes) != columns * 4:
            raise ValueError("FP32 output-channel scales required")
        if not len(q_bytes) or len(q_bytes) % columns:
            raise ValueError("nonempty rectangular INT8 matrix required")
        q = np.frombuffer(q_bytes, np.int8).reshape(-1, columns)
        return self.dequantize_array(q, np.frombuffer(scale_bytes, np.float32)).tobytes()
