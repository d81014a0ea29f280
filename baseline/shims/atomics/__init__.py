"""Import-time stand-in for the `atomics` cffi package: single-process integer views guarded by a lock."""
import struct
import threading

INT = "int"
UINT = "uint"
_lock = threading.Lock()


class _View:
    def __init__(self, buffer, atype=INT):
        self.buf = memoryview(buffer)
        self.fmt = {1: "b", 2: "h", 4: "i", 8: "q"}[len(self.buf)]

    def load(self):
        return struct.unpack(self.fmt, self.buf)[0]

    def store(self, v):
        struct.pack_into(self.fmt, self.buf, 0, v)

    def cmpxchg_weak(self, expected, desired):
        with _lock:
            cur = self.load()
            if cur == expected:
                self.store(desired)
                return True
            return False

    cmpxchg_strong = cmpxchg_weak

    def fetch_add(self, v):
        with _lock:
            cur = self.load()
            self.store(cur + v)
            return cur

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def atomicview(buffer, atype=INT):
    return _View(buffer, atype)
