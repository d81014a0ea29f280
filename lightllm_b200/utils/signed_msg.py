"""Signed pickles for the control sockets between machines of one deployment.

`seal(key, obj)` gives two frames (HMAC-SHA256 signature, pickled body); `unseal(key, frames)` checks the signature
before it unpickles and raises PermissionError otherwise, so that a stranger who reaches the port cannot make the
process unpickle his bytes.  `derive_key(env_name, seed)` takes the secret from the environment variable (the same
value on every machine) or, without one, from an address both sides know: that keeps other deployments out, not
someone who knows the address.
"""
from __future__ import annotations

import hashlib
import hmac
import os
import pickle
from typing import Sequence


def derive_key(env_name: str, seed: str) -> bytes:
    k = os.environ.get(env_name)
    if k:
        return hashlib.sha256(k.encode()).digest()
    return hashlib.sha256(f"{env_name}:{seed}".encode()).digest()


def seal(key: bytes, obj) -> list:
    body = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    return [hmac.new(key, body, hashlib.sha256).digest(), body]


def unseal(key: bytes, frames: Sequence[bytes]):
    if len(frames) != 2 or not hmac.compare_digest(bytes(frames[0]), hmac.new(key, frames[1], hashlib.sha256).digest()):
        raise PermissionError("message signature does not match (another deployment's key?)")
    return pickle.loads(frames[1])
