"""Device handle: the host-side mirror of `ferrum_wgpu::device::Gpu`
(ferrum_wgpu/src/device/mod.rs:L98-L176). Errors are values turned into exceptions here:
`CudaError` carries the status code and the library's message."""
from __future__ import annotations

import ctypes as C
import json
import weakref

from . import _ffi


class CudaError(RuntimeError):
    """`GpuError(String)` of the reference (device/mod.rs:L18-L27) plus the C status code."""

    def __init__(self, code: int, message: str):
        super().__init__(message or _ffi.STATUS_NAMES.get(code, f"error {code}"))
        self.code = code


class Device:
    def __init__(self, handle, ordinal: int = 0):
        self._h = handle
        self.ordinal = ordinal
        self._lib = _ffi.load()
        # weights and models opened on this device: closed before the device is, whatever order the
        # interpreter drops them in
        self._children = weakref.WeakSet()

    @classmethod
    def open(cls, ordinal: int = 0) -> "Device":
        lib = _ffi.load()
        h = C.c_void_p()
        rc = lib.fc_device_open(ordinal, C.byref(h))
        if rc != _ffi.FC_OK:
            raise CudaError(rc, lib.fc_last_error(None).decode())
        return cls(h, ordinal)

    def adopt(self, child):
        self._children.add(child)

    def close(self):
        if self._h:
            for c in list(self._children):
                c.close()
            self._lib.fc_device_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def check(self, rc: int):
        if rc != _ffi.FC_OK:
            raise CudaError(rc, self._lib.fc_last_error(self._h).decode())

    def name(self) -> str:
        buf = C.create_string_buffer(256)
        self.check(self._lib.fc_device_name(self._h, buf, 256))
        return buf.value.decode()

    def props(self):
        sm, mem = C.c_int(), C.c_uint64()
        self.check(self._lib.fc_device_props(self._h, C.byref(sm), C.byref(mem)))
        return sm.value, mem.value

    def sync(self):
        self.check(self._lib.fc_device_sync(self._h))

    def stream(self) -> int:
        return self._lib.fc_device_stream(self._h) or 0

    def launch_count(self) -> int:
        return self._lib.fc_device_launch_count(self._h)

    def profile(self, enable: bool):
        """Bracket every launch with CUDA events (per-kernel timing); off by default."""
        self.check(self._lib.fc_debug_profile(self._h, 1 if enable else 0))

    def matvec_kernel(self, choice: int):
        """Measurement hook: 0 = the library's rule, 1 = f32 FMA kernel, 2 = small-batch mma.sync kernel (1..8 rows)."""
        self.check(self._lib.fc_debug_matvec_kernel(self._h, int(choice)))

    def profile_report(self) -> dict:
        """{kernel: {"launches": n, "ms": total}} since the last report; synchronises."""
        buf = C.create_string_buffer(1 << 16)
        self.check(self._lib.fc_debug_profile_report(self._h, buf, len(buf)))
        return json.loads(buf.value.decode())

    def attention_f16(self, qkv, n_seqs: int, t: int, heads: int, kv_heads: int, variant: int = 0, iters: int = 0):
        """Causal attention over packed fp16 rows (q heads | k heads | v heads, head_dim 64).

        Returns (out fp16 [n_seqs * t, heads * 64], mean milliseconds of `iters` timed launches).
        variant 0 = the kernel the model passes pick, 1 / 2 = mma.sync with one / two row tiles per
        warp, 3 = tcgen05 with tensor-memory accumulators."""
        import numpy as np
        qkv = np.ascontiguousarray(qkv, dtype=np.float16)
        rows = n_seqs * t
        if qkv.size != rows * (heads + 2 * kv_heads) * 64:
            raise ValueError("qkv must hold n_seqs * t rows of (heads + 2 * kv_heads) * 64 values")
        out = np.empty((rows, heads * 64), dtype=np.float16)
        ms = C.c_float(0.0)
        self.check(self._lib.fc_debug_attention_f16(self._h, qkv.ctypes.data, n_seqs, t, heads, kv_heads,
                                                    out.ctypes.data, variant, iters, C.byref(ms)))
        return out, ms.value

    def topk(self, logits, k: int, repetition_penalty: float = 1.0, recent=()):
        """`fc_topk_dev` on a host row (uploaded for the call): the top-k candidates in `sampling::sample`'s order."""
        import numpy as np
        import torch
        row = np.ascontiguousarray(logits, dtype=np.float32).reshape(-1)
        d = torch.from_numpy(row).to(f"cuda:{self.ordinal}")
        torch.cuda.synchronize(self.ordinal)
        idx = np.empty(k, dtype=np.int32)
        val = np.empty(k, dtype=np.float32)
        rec = np.ascontiguousarray(np.asarray(list(recent), dtype=np.int32))
        n = C.c_uint32()
        self.check(self._lib.fc_topk_dev(self._h, d.data_ptr(), row.size, k, float(repetition_penalty),
                                         rec.ctypes.data if rec.size else None, rec.size, idx.ctypes.data,
                                         val.ctypes.data, C.byref(n)))
        return idx[:n.value], val[:n.value]

    def fail_after(self, n: int | None):
        """`Gpu::fail_after` (device/runtime.rs:L214-L256): refuse launches after `n` more; None disarms."""
        self.check(self._lib.fc_debug_fail_after(self._h, -1 if n is None else n))
