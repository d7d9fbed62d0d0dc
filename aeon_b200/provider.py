"""Python caller of the provider entry points: encoded records (bytes) -> augmented batch.

Mirrors what aeon's batch_decoder does with a provider per decode chunk
(src/batch_decoder.cpp:62-99); all work happens inside libaeon_b200.so.
"""
import ctypes as C
import json

import numpy as np

from . import _lib as L

NP_DTYPE = {L.U8: np.uint8, L.I8: np.int8, L.I16: np.int16, L.U16: np.uint16, L.I32: np.int32, L.F32: np.float32,
            L.F64: np.float64}


class Provider:
    def __init__(self, ctx, config):
        self.ctx = ctx
        self.lib = ctx.lib
        self.config = dict(config)
        h = C.c_void_p()
        L.check(self.lib.aeonb_provider_create(ctx.handle, json.dumps(self.config).encode(), C.byref(h)))
        self.handle = h
        self.batch_size = int(self.config["batch_size"])
        self.batch_major = bool(self.config.get("batch_major", True))
        self.input_count = self.lib.aeonb_provider_input_count(h)
        self.outputs = []
        for i in range(self.lib.aeonb_provider_output_count(h)):
            dims = (C.c_int64 * 8)()
            dt = C.c_int32()
            rank = self.lib.aeonb_provider_output_shape(h, i, dims, C.byref(dt))
            name = self.lib.aeonb_provider_output_name(h, i).decode()
            self.outputs.append((name, tuple(int(dims[k]) for k in range(rank)), int(dt.value),
                                 int(self.lib.aeonb_provider_output_bytes(h, i))))

    def close(self):
        if self.handle:
            self.lib.aeonb_provider_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _pack(self, records):
        n = len(records)
        k = self.input_count
        for r, rec in enumerate(records):
            if len(rec) != k:
                raise ValueError("record %d has %d elements, the configuration needs %d" % (r, len(rec), k))
        flat = [blob for rec in records for blob in rec]
        sizes = (C.c_size_t * (n * k))(*map(len, flat))
        if all(type(b) is bytes for b in flat):
            # one pass inside ctypes: each element points at the bytes object's own buffer, which the array keeps alive
            ptrs = (C.c_char_p * (n * k))(*flat)
            return C.cast(ptrs, C.POINTER(C.c_void_p)), sizes, (ptrs, flat)
        ptrs = (C.c_void_p * (n * k))()
        keep = []
        for i, blob in enumerate(flat):
            buf = np.frombuffer(blob, np.uint8)
            keep.append(buf)
            ptrs[i] = buf.ctypes.data if len(buf) else None
        return ptrs, sizes, keep

    def _shape(self, dims):
        if self.batch_major:
            return (self.batch_size,) + dims
        return (int(np.prod(dims)), self.batch_size)

    def run_host(self, records, out=None):
        """Process `records` (list of tuples of bytes); returns {name: numpy array} in host memory."""
        ptrs, sizes, keep = self._pack(records)
        if out is None:
            out = {name: np.zeros(self._shape(dims), NP_DTYPE[dt]) for name, dims, dt, _ in self.outputs}
        outs = (C.c_void_p * len(self.outputs))(*[out[name].ctypes.data for name, _, _, _ in self.outputs])
        L.check(self.lib.aeonb_provider_run(self.handle, ptrs, sizes, len(records), outs, 0))
        return out

    def submit_host(self, records, out):
        """Pipelined run_host: enqueue the batch into the caller's (pinned) arrays `out` and return a ticket
        for wait().  Records and `out` must stay alive and untouched until the ticket has been waited for."""
        ptrs, sizes, keep = self._pack(records)
        outs = (C.c_void_p * len(self.outputs))(*[out[name].ctypes.data for name, _, _, _ in self.outputs])
        ticket = C.c_int64()
        L.check(self.lib.aeonb_provider_run_async(self.handle, ptrs, sizes, len(records), outs, 0, C.byref(ticket)))
        self._inflight = getattr(self, "_inflight", {})
        self._inflight[ticket.value] = (keep, ptrs, sizes, outs)
        return ticket.value

    def submit_device(self, records, out):
        """Pipelined run_device: enqueue the batch into the caller's CUDA tensors `out` ({name: tensor}) and return a
        ticket for wait().  The host stages of the next call overlap this batch's GPU work."""
        ptrs, sizes, keep = self._pack(records)
        outs = (C.c_void_p * len(self.outputs))(*[out[name].data_ptr() for name, _, _, _ in self.outputs])
        ticket = C.c_int64()
        L.check(self.lib.aeonb_provider_run_async(self.handle, ptrs, sizes, len(records), outs, 1, C.byref(ticket)))
        self._inflight = getattr(self, "_inflight", {})
        self._inflight[ticket.value] = (keep, ptrs, sizes, outs)
        return ticket.value

    def wait(self, ticket):
        L.check(self.lib.aeonb_provider_wait(self.handle, ticket))
        getattr(self, "_inflight", {}).pop(ticket, None)

    def run_device(self, records, out=None):
        """Same, leaving the batch in device memory: returns {name: torch tensor on the context's GPU}."""
        import torch
        from .kernels import _TORCH_DTYPE
        ptrs, sizes, keep = self._pack(records)
        if out is None:
            with torch.cuda.stream(self.ctx.torch_stream):
                out = {name: torch.zeros(self._shape(dims), dtype=_TORCH_DTYPE[dt], device="cuda:%d" % self.ctx.device)
                       for name, dims, dt, _ in self.outputs}
            self.ctx.torch_stream.synchronize()
        outs = (C.c_void_p * len(self.outputs))(*[out[name].data_ptr() for name, _, _, _ in self.outputs])
        L.check(self.lib.aeonb_provider_run(self.handle, ptrs, sizes, len(records), outs, 1))
        return out

    def stats(self):
        h2d, d2h, launches = C.c_int64(), C.c_int64(), C.c_int32()
        L.check(self.lib.aeonb_provider_stats(self.handle, C.byref(h2d), C.byref(d2h), C.byref(launches)))
        return dict(h2d_bytes=h2d.value, d2h_bytes=d2h.value, launches=launches.value)
