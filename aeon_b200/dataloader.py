"""Python iterator with the surface of aeon's ``aeon.DataLoader`` (aeon src/api.cpp:104-425).

    dl = DataLoader(config={...})        # aeon's loader JSON as a dict
    for batch in dl:                     # tuple of (name, array) pairs, one per output buffer
        ...
    len(dl); dl.ndata; dl.batch_size; dl.axes_info; dl.config; dl.reset()

Arrays are numpy views of the loader's pinned host buffers (valid until the next batch, as in
aeon), or torch CUDA tensors when the config sets ``"device_output": true``.  With
``"batch_major": false`` they are 2-D ``(elements, batch)`` views, as in aeon.
"""
import ctypes as C
import json

import numpy as np

from . import _lib as L
from .provider import NP_DTYPE


def dict2json(config):
    """aeon.dict2json: the JSON text aeon builds from a python dict."""
    return json.dumps(config)


class DataLoader:
    def __init__(self, config, device=0):
        if not isinstance(config, dict):
            raise TypeError("config must be a dict")
        self.lib = L.load()
        self.config = dict(config)
        h = C.c_void_p()
        L.check(self.lib.aeonb_loader_create(dict2json(self.config).encode(), int(device), C.byref(h)))
        self.handle = h
        self.device = int(device)
        self.batch_size = self.lib.aeonb_loader_batch_size(h)
        self.ndata = self.lib.aeonb_loader_record_count(h)
        self.batch_major = bool(self.config.get("batch_major", True))
        self.device_output = bool(self.config.get("device_output", False))
        self.outputs = []
        self.axes_info = {}
        for i in range(self.lib.aeonb_loader_output_count(h)):
            dims = (C.c_int64 * 8)()
            dt = C.c_int32()
            rank = self.lib.aeonb_loader_output_shape(h, i, dims, C.byref(dt))
            name = self.lib.aeonb_loader_output_name(h, i).decode()
            shape = tuple(int(dims[k]) for k in range(rank))
            axes = self.lib.aeonb_loader_axis_names(h, i).decode()
            self.outputs.append((name, shape, int(dt.value)))
            if axes:
                self.axes_info[name] = dict(zip(axes.split(","), shape))

    def __len__(self):
        return self.ndata

    def __iter__(self):
        return self

    def _wrap(self, ptr, shape, dt):
        full = (self.batch_size,) + shape if self.batch_major else (int(np.prod(shape)), self.batch_size)
        count = int(np.prod(full))
        if self.device_output:
            import torch
            from .kernels import _TORCH_DTYPE, DTYPE_SIZE

            class _Mem:  # minimal __cuda_array_interface__ holder
                pass
            m = _Mem()
            m.__cuda_array_interface__ = {"shape": full, "typestr": np.dtype(NP_DTYPE[dt]).str, "data": (ptr, False),
                                          "version": 2}
            return torch.as_tensor(m, device="cuda:%d" % self.device)
        buf = (C.c_char * (count * np.dtype(NP_DTYPE[dt]).itemsize)).from_address(ptr)
        return np.frombuffer(buf, NP_DTYPE[dt]).reshape(full)

    def __next__(self):
        ptrs = (C.c_void_p * len(self.outputs))()
        status = L.check(self.lib.aeonb_loader_next(self.handle, ptrs))
        if status == L.END:
            raise StopIteration
        return tuple((name, self._wrap(ptrs[i], shape, dt)) for i, (name, shape, dt) in enumerate(self.outputs))

    next = __next__

    def reset(self):
        L.check(self.lib.aeonb_loader_reset(self.handle))

    @property
    def position(self):
        return self.lib.aeonb_loader_position(self.handle)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.aeonb_loader_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
