"""Images and audio clips attached to a request.

An item arrives as `{"type": "url" | "base64" | "image_size", "data": ...}`; `preload` fetches and decodes it
in the HTTP worker; the embed cache then assigns it `uuid` (cache record id), `token_id` (first id of a run
of `token_num` virtual token ids placed in the prompt where the item's embeddings go) and
`start_index_in_embed_cache` (first row of its embeddings in the shared arena).  Only the small dict form
(`to_dict`) travels to the router and the ranks.
Reference: lightllm/server/multimodal_params.py.
"""
from __future__ import annotations

import asyncio
import base64
import hashlib
import os
from io import BytesIO
from typing import List, Optional

import numpy as np

MIN_AUDIO_LEN = 480  # samples at 16 kHz: shorter clips are zero padded


class UrlCache:
    """Downloaded bytes by URL, least recently used first out (`--enable_multimodal_url_cache`): the same picture
    asked for again (a conversation that carries its earlier turns) is not downloaded again.
    Reference: lightllm/utils/multimodal_utils.py (the URL cache around fetch_resource)."""

    def __init__(self, max_items: int = 256, max_bytes: int = 256 << 20):
        from collections import OrderedDict

        self.max_items, self.max_bytes = max_items, max_bytes
        self.items: "OrderedDict[str, bytes]" = OrderedDict()
        self.bytes = 0
        self.hits = self.misses = 0

    def get(self, url: str) -> Optional[bytes]:
        data = self.items.get(url)
        if data is None:
            self.misses += 1
            return None
        self.items.move_to_end(url)
        self.hits += 1
        return data

    def put(self, url: str, data: bytes) -> None:
        if len(data) > self.max_bytes:
            return
        old = self.items.pop(url, None)
        if old is not None:
            self.bytes -= len(old)
        self.items[url] = data
        self.bytes += len(data)
        while len(self.items) > self.max_items or self.bytes > self.max_bytes:
            _, gone = self.items.popitem(last=False)
            self.bytes -= len(gone)


_url_cache = UrlCache(int(os.getenv("LLB_MULTIMODAL_URL_CACHE_ITEMS", "256")),
                      int(os.getenv("LLB_MULTIMODAL_URL_CACHE_MB", "256")) << 20)


def _start_args():
    from .core.objs.start_args import get_env_start_args

    return get_env_start_args()


async def _download(url: str, timeout: int, proxy: Optional[str]) -> bytes:
    import aiohttp

    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=timeout)) as sess:
        async with sess.get(url, proxy=proxy) as resp:
            resp.raise_for_status()
            return await resp.read()


async def fetch_resource(url: str, request=None, timeout: int = 5, proxy: Optional[str] = None) -> bytes:
    use_cache = bool(getattr(_start_args(), "enable_multimodal_url_cache", False))
    if use_cache:
        data = _url_cache.get(url)
        if data is not None:
            return data
    data = await _download(url, timeout, proxy)
    if use_cache:
        _url_cache.put(url, data)
    return data


def resized_dimensions(w: int, h: int, max_pixels: int):
    """(w, h) scaled down, keeping the aspect ratio, so that w * h <= max_pixels (unchanged when it already is)."""
    if max_pixels is None or max_pixels <= 0 or w * h <= max_pixels:
        return w, h
    f = (max_pixels / float(w * h)) ** 0.5
    nw, nh = max(1, int(w * f)), max(1, int(h * f))
    return nw, nh


def _resize_image_bytes(raw: bytes, w: int, h: int) -> bytes:
    from PIL import Image

    with Image.open(BytesIO(raw)) as im:
        fmt = im.format if im.format in ("PNG", "JPEG", "WEBP") else "PNG"
        out = im.convert("RGB").resize((w, h), Image.BICUBIC)
    buf = BytesIO()
    out.save(buf, format=fmt)
    return buf.getvalue()


class _Item:
    kind = "item"

    def __init__(self, **kw):
        self._type = kw["type"]
        self._data = kw["data"]
        self.uuid = None
        self.token_id = None
        self.token_num = None
        self.start_index_in_embed_cache = None
        self.md5 = None
        self._preload_data: Optional[bytes] = None
        self.extra_params = {}

    async def _raw(self, request) -> bytes:
        if self._type == "url":
            return await fetch_resource(self._data, request, int(os.getenv("REQUEST_TIMEOUT", "5")),
                                        os.getenv("REQUEST_PROXY"))
        if self._type == "base64":
            return base64.b64decode(self._data)
        if self._type == "bytes":
            return self._data
        raise ValueError(f"cannot read {self.kind} of type {self._type}")

    def read(self) -> bytes:
        assert self._preload_data is not None, "preload() first"
        data, self._preload_data, self._data = self._preload_data, None, None
        return data

    def content_md5(self, salt: str = "") -> str:
        h = hashlib.md5(self._preload_data or b"")
        h.update(salt.encode())
        return h.hexdigest()

    def to_dict(self):
        return {"uuid": self.uuid, "token_id": self.token_id, "token_num": self.token_num,
                "start_index_in_embed_cache": self.start_index_in_embed_cache, "md5": self.md5,
                "extra_params": dict(self.extra_params), **self._extra_dict()}

    def _extra_dict(self):
        return {}

    def to_origin_dict(self):
        """The item as the client sent it (for forwarding the request to another node)."""
        return {"type": self._type, "data": self._data}


class ImageItem(_Item):
    kind = "image"

    def __init__(self, **kw):
        super().__init__(**kw)
        self.image_w = self.image_h = 0
        self.grid_thwd = None  # (t, h, w, merge) filled by the tokenizer for grid based vision towers

    async def preload(self, request=None):
        if self._preload_data is not None:
            return
        args = _start_args()
        max_pixels = int(getattr(args, "max_image_pixels", 0) or 0)
        if bool(getattr(args, "disable_image_resize", False)):
            max_pixels = 0
        try:
            if self._type == "image_size":  # synthetic image for benchmarks: data = (w, h)
                from PIL import Image

                w, h = resized_dimensions(int(self._data[0]), int(self._data[1]), max_pixels)
                buf = BytesIO()
                Image.new("RGB", (int(w), int(h)), (127, 127, 127)).save(buf, format="PNG")
                raw = buf.getvalue()
            else:
                raw = await self._raw(request)
            from PIL import Image

            with Image.open(BytesIO(raw)) as im:
                self.image_w, self.image_h = im.size
            w, h = resized_dimensions(self.image_w, self.image_h, max_pixels)
            if (w, h) != (self.image_w, self.image_h):      # `--max_image_pixels` unless `--disable_image_resize`
                raw = await asyncio.get_running_loop().run_in_executor(None, _resize_image_bytes, raw, w, h)
                self.image_w, self.image_h = w, h
            self._preload_data = raw
        except Exception as e:
            raise ValueError(f"Failed to read image type={self._type}, data[:100]={str(self._data)[:100]}: {e}")

    def _extra_dict(self):
        return {"image_w": self.image_w, "image_h": self.image_h, "grid_thwd": self.grid_thwd}


class AudioItem(_Item):
    kind = "audio"

    def __init__(self, **kw):
        super().__init__(**kw)
        self.audio_length = None

    @staticmethod
    def _decode_wav(raw: bytes) -> np.ndarray:
        """16 kHz mono float32 from a RIFF/WAVE payload (PCM 16-bit or float32); linear resampling."""
        import wave

        with wave.open(BytesIO(raw)) as w:
            n, ch, sw, sr = w.getnframes(), w.getnchannels(), w.getsampwidth(), w.getframerate()
            pcm = w.readframes(n)
        if sw == 2:
            x = np.frombuffer(pcm, dtype="<i2").astype(np.float32) / 32768.0
        elif sw == 4:
            x = np.frombuffer(pcm, dtype="<i4").astype(np.float32) / 2147483648.0
        else:
            x = (np.frombuffer(pcm, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
        if ch > 1:
            x = x.reshape(-1, ch).mean(axis=1)
        if sr != 16000 and x.size:
            t = np.arange(int(x.size * 16000 / sr)) * (sr / 16000.0)
            x = np.interp(t, np.arange(x.size), x).astype(np.float32)
        return x

    async def preload(self, request=None):
        if self._preload_data is not None:
            return
        try:
            raw = await self._raw(request)
            x = await asyncio.to_thread(self._decode_wav, raw)
            if x.shape[0] < MIN_AUDIO_LEN:
                x = np.pad(x, (0, MIN_AUDIO_LEN - x.shape[0]))
            self.audio_length = int(x.shape[0])
            self._preload_data = x.astype(np.float32).tobytes()
        except Exception as e:
            raise ValueError(f"Failed to read audio type={self._type}, data[:100]={str(self._data)[:100]}: {e}")

    def _extra_dict(self):
        return {"audio_length": self.audio_length}


class MultimodalParams:
    def __init__(self, images: Optional[List[dict]] = None, audios: Optional[List[dict]] = None, **_):
        self.images = [ImageItem(**i) for i in (images or [])]
        self.audios = [AudioItem(**a) for a in (audios or [])]

    async def verify_and_preload(self, request=None):
        await asyncio.gather(*[x.preload(request) for x in self.images + self.audios])

    def items(self):
        return self.images + self.audios

    def to_dict(self):
        return {"images": [i.to_dict() for i in self.images], "audios": [a.to_dict() for a in self.audios]}

    def to_origin_dict(self):
        return {"images": [i.to_origin_dict() for i in self.images], "audios": [a.to_origin_dict() for a in self.audios]}

    def __bool__(self):
        return bool(self.images or self.audios)
