"""Signed pickles between machines: a body is unpickled only under a matching signature."""
import pytest

from lightllm_b200.utils.signed_msg import derive_key, seal, unseal


def test_round_trip_and_rejections(monkeypatch):
    monkeypatch.delenv("LLB_X_KEY", raising=False)
    a, b = derive_key("LLB_X_KEY", "10.0.0.1:9000"), derive_key("LLB_X_KEY", "10.0.0.2:9000")
    assert a != b and len(a) == 32 and a == derive_key("LLB_X_KEY", "10.0.0.1:9000")
    monkeypatch.setenv("LLB_X_KEY", "secret")
    assert derive_key("LLB_X_KEY", "10.0.0.1:9000") == derive_key("LLB_X_KEY", "elsewhere") != a
    frames = seal(a, ("req", 7, [1, 2, 3]))
    assert unseal(a, frames) == ("req", 7, [1, 2, 3])

    class Boom:
        def __reduce__(self):
            raise AssertionError("the body was unpickled")

    import pickle

    evil = pickle.dumps(("x",))
    for bad in ([frames[0], evil], [b"\0" * 32, frames[1]], [frames[1]], [], seal(b, "other key")):
        with pytest.raises(PermissionError):
            unseal(a, bad)
