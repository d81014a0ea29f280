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


async def fetch_resource(url: str, request=None, timeout: int = 5, proxy: Optional[str] = None) -> bytes:
    import aiohttp

    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=timeout)) as sess:
        async with sess.get(url, proxy=proxy) as resp:
            resp.raise_for_status()
            return await resp.read()


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
        try:
            if self._type == "image_size":  # synthetic image for benchmarks: data = (w, h)
                from PIL import Image

                w, h = self._data
                buf = BytesIO()
                Image.new("RGB", (int(w), int(h)), (127, 127, 127)).save(buf, format="PNG")
                raw = buf.getvalue()
            else:
                raw = await self._raw(request)
            from PIL import Image

            with Image.open(BytesIO(raw)) as im:
                self.image_w, self.image_h = im.size
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
