def unix_connect(*a, **k):
    raise RuntimeError("rpyc is not available in this environment")
