"""Import-time stand-in for `rpyc` (only the names the engine modules import; no RPC is performed)."""


class Service:
    pass


def connect(*a, **k):
    raise RuntimeError("rpyc is not available in this environment")


class _Async:
    def __init__(self, f):
        self.f = f

    def __call__(self, *a, **k):
        return self.f(*a, **k)


def async_(f):
    return _Async(f)
