"""Image preload knobs: `--max_image_pixels` / `--disable_image_resize` and the URL cache
(`--enable_multimodal_url_cache`).  Reference: lightllm/server/multimodal_params.py:137-190,
lightllm/utils/multimodal_utils.py."""
import asyncio
import base64
import json
import os
from io import BytesIO

from lightllm_b200.server import multimodal_params as mp
from lightllm_b200.server.core.objs import start_args as sa


def _with_args(monkeypatch, **kw):
    d = sa.StartArgs.defaults().to_dict()
    d.update(kw)
    monkeypatch.setenv(sa.ENV_KEY, json.dumps(d))


def _png(w, h):
    from PIL import Image

    buf = BytesIO()
    Image.new("RGB", (w, h), (10, 200, 30)).save(buf, format="PNG")
    return buf.getvalue()


def test_resize_rule():
    assert mp.resized_dimensions(100, 50, 10000) == (100, 50)
    w, h = mp.resized_dimensions(4000, 2000, 3686400)
    assert w * h <= 3686400 and abs(w / h - 2.0) < 0.01 and w * h > 0.98 * 3686400
    assert mp.resized_dimensions(10, 10, 0) == (10, 10)


def test_large_images_are_resized_unless_disabled(monkeypatch):
    from PIL import Image

    raw = base64.b64encode(_png(400, 200)).decode()
    _with_args(monkeypatch, max_image_pixels=20000)
    it = mp.ImageItem(type="base64", data=raw)
    asyncio.run(it.preload())
    assert it.image_w * it.image_h <= 20000 and abs(it.image_w / it.image_h - 2.0) < 0.05
    with Image.open(BytesIO(it.read())) as im:
        assert im.size == (it.image_w, it.image_h)
    _with_args(monkeypatch, max_image_pixels=20000, disable_image_resize=True)
    it = mp.ImageItem(type="base64", data=raw)
    asyncio.run(it.preload())
    assert (it.image_w, it.image_h) == (400, 200)
    _with_args(monkeypatch, max_image_pixels=20000)
    it = mp.ImageItem(type="image_size", data=(400, 200))
    asyncio.run(it.preload())
    assert it.image_w * it.image_h <= 20000


def test_url_cache(monkeypatch):
    calls = []

    async def fake_download(url, timeout, proxy):
        calls.append(url)
        return url.encode() * 10

    monkeypatch.setattr(mp, "_download", fake_download)
    monkeypatch.setattr(mp, "_url_cache", mp.UrlCache(max_items=2, max_bytes=1 << 20))
    _with_args(monkeypatch, enable_multimodal_url_cache=True)
    get = lambda u: asyncio.run(mp.fetch_resource(u))  # noqa: E731
    assert get("http://a") == get("http://a") and calls == ["http://a"]
    get("http://b")
    get("http://a")            # a is the most recent now
    get("http://c")            # evicts b
    get("http://b")
    assert calls == ["http://a", "http://b", "http://c", "http://b"]
    _with_args(monkeypatch, enable_multimodal_url_cache=False)
    get("http://c")
    assert calls[-1] == "http://c" and len(calls) == 5
    c = mp.UrlCache(max_items=10, max_bytes=25)
    c.put("x", b"1" * 10)
    c.put("y", b"2" * 10)
    c.put("z", b"3" * 10)
    assert c.get("x") is None and c.get("z") is not None and c.bytes == 20
    c.put("big", b"0" * 26)
    assert c.get("big") is None
