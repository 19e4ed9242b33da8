"""Device memory through the C ABI (ts2_dev_*): numpy in, numpy out."""
import ctypes as C

import numpy as np

from . import capi


def check(rc, lib=None, model=None):
    if rc != capi.TS2_OK:
        lib = lib or capi.load_library()
        msg = lib.ts2_last_error(model)
        raise capi.Ts2Error(rc, msg.decode() if msg else "")


class DeviceBuffer:
    def __init__(self, nbytes, device=0):
        self.lib = capi.load_library()
        self.device = device
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(self.lib.ts2_dev_alloc(device, self.nbytes, C.byref(p)))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, a, device=0):
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes, device)
        b.upload(a)
        return b

    def upload(self, a):
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        check(self.lib.ts2_dev_upload(self.device, self.ptr, a.ctypes.data, a.nbytes))

    def download(self, shape, dtype):
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        check(self.lib.ts2_dev_download(self.device, out.ctypes.data, self.ptr, out.nbytes))
        return out

    def zero(self):
        check(self.lib.ts2_dev_memset(self.device, self.ptr, 0, self.nbytes))

    def free(self):
        if self.ptr:
            self.lib.ts2_dev_free(self.device, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def sync(device=0):
    check(capi.load_library().ts2_dev_sync(device))
