"""Multimodal plumbing on CPU: embed cache (records, eviction, arena), its zmq service, multimodal params, the
visual server's embed-and-forward step with a tiny random vision tower, and the config server's id ranges."""
import asyncio
import base64
import threading
from io import BytesIO
from types import SimpleNamespace

import numpy as np
import pytest
import torch
import zmq

from lightllm_b200.server.embed_cache.cache import EmbedArena, EmbedCache, RowAllocator


def test_row_allocator_coalesces():
    a = RowAllocator(100)
    x, y, z = a.alloc(30), a.alloc(30), a.alloc(40)
    assert (x, y, z) == (0, 30, 60) and a.alloc(1) is None
    a.release(y, 30)
    a.release(x, 30)
    assert a.free == [(0, 60)] and a.alloc(60) == 0
    a.release(0, 60)
    a.release(z, 40)
    assert a.free == [(0, 100)]


def test_embed_cache_refcount_and_eviction():
    c = EmbedCache(capacity=3, arena_rows=100)
    r = c.alloc(["a", "b", "a"], [10, 20, 10])
    assert r[0]["id"] == r[2]["id"] and r[0]["token_id"] == 100_000_000 and r[1]["token_id"] == 100_000_010
    assert c.by_md5["a"].ref == 2 and c.by_md5["b"].ref == 1
    assert c.alloc(["c", "d"], [40, 40]) is None and "c" not in c.by_md5     # capacity 3: would need to evict pinned
    assert c.by_md5["a"].ref == 2                                            # failed alloc leaves refs alone
    c.release([r[0]["id"], r[1]["id"], r[2]["id"]])
    r2 = c.alloc(["c", "a"], [40, 10])                                       # "a" is a hit and keeps its ids
    assert r2[1]["token_id"] == 100_000_000 and c.by_md5["a"].ref == 1
    c.set_items_data([r2[0]["id"]], [b"png"])
    assert c.get_items_data([r2[0]["id"], 999]) == [True, False] and c.get_payload(r2[0]["id"]) == b"png"
    c.set_items_embed([r2[0]["id"]])
    assert c.get_items_embed([r2[0]["id"]]) == [True] and c.get_payload(r2[0]["id"]) is None


def test_arena_roundtrip():
    a = EmbedArena("llb_test_arena", 64, 16, create=True)
    try:
        x = torch.randn(5, 16).bfloat16()
        a.write(7, x)
        b = EmbedArena("llb_test_arena", 64, 16, create=False)
        assert torch.equal(b.read_torch(7, 5), x)
        assert torch.equal(b.read_rows(torch.tensor([9, 7])), x[[2, 0]])
        b.close()
    finally:
        a.close()


def _png(w, h, seed=0):
    from PIL import Image

    rng = np.random.default_rng(seed)
    buf = BytesIO()
    Image.fromarray(rng.integers(0, 255, (h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def test_multimodal_params_preload():
    from lightllm_b200.server.multimodal_params import MultimodalParams

    raw = _png(90, 60)
    mm = MultimodalParams(images=[{"type": "base64", "data": base64.b64encode(raw).decode()},
                                  {"type": "image_size", "data": [64, 48]}])
    asyncio.run(mm.verify_and_preload(None))
    assert (mm.images[0].image_w, mm.images[0].image_h) == (90, 60) and mm.images[1].image_w == 64
    assert mm.images[0].content_md5() != mm.images[1].content_md5()
    assert mm.to_origin_dict()["images"][1] == {"type": "image_size", "data": [64, 48]}
    with pytest.raises(ValueError):
        bad = MultimodalParams(images=[{"type": "base64", "data": base64.b64encode(b"not an image").decode()}])
        asyncio.run(bad.verify_and_preload(None))


def test_visual_manager_embeds_and_forwards():
    from lightllm_b200.models.vit.qwen2_vl_visual import Qwen2VLVisionTower, image_token_num, preprocess_image
    from lightllm_b200.models.weights import RandomSource
    from lightllm_b200.server.core.objs.io_objs import GroupReqIndexes
    from lightllm_b200.server.embed_cache import manager as cm
    from lightllm_b200.server.visualserver.manager import VisualManager

    vcfg = dict(depth=1, embed_dim=32, hidden_size=24, num_heads=2, mlp_ratio=2, patch_size=14, spatial_merge_size=2,
                temporal_patch_size=2)
    tower = Qwen2VLVisionTower(vcfg, RandomSource(Qwen2VLVisionTower.weight_shapes(vcfg), dtype=torch.float32),
                               torch.device("cpu"), torch.float32)
    port = 23000 + (id(tower) % 2000)
    args = SimpleNamespace(cache_port=port, unique_server_name="llbmmtest", embed_cache_storage_size=0.001,
                           cache_capacity=8, config_server_host=None, config_server_port=None)
    rows = cm.arena_rows(args, 24)
    arena = EmbedArena(cm.arena_name(args), rows, 24, create=True)
    cache = EmbedCache(8, rows)
    sock = zmq.Context.instance().socket(zmq.REP)
    sock.bind(f"tcp://127.0.0.1:{port}")
    stop = threading.Event()
    th = threading.Thread(target=cm.serve, args=(cache, sock, None, stop), daemon=True)
    th.start()
    try:
        client = cm.EmbedCacheClient(args, hidden=24, open_arena=True)
        raw = _png(84, 56, seed=3)
        n, (t, gh, gw) = image_token_num(84, 56)
        assert n == 6
        rec = client.alloc(["m1"], [n])[0]
        client.set_items_data([rec["id"]], [raw])
        item = {"uuid": rec["id"], "token_id": rec["token_id"], "token_num": n,
                "start_index_in_embed_cache": rec["start_index_in_embed_cache"], "grid_thwd": (t, gh, gw, 2)}
        sent = []
        vm = VisualManager(args, tower, client, sent.append, None)
        g = GroupReqIndexes(8, {"images": [item], "audios": []}, [0], 0.0)
        vm.handle(g)
        assert sent == [g] and client.get_items_embed([rec["id"]]) == [True]
        patches, grid = preprocess_image(raw)
        want = tower.forward(patches, [grid]).bfloat16()
        got = arena.read_torch(rec["start_index_in_embed_cache"], n)
        assert torch.equal(got, want)
        vm.handle(g)  # already embedded: forwarded without another tower pass (no payload left to read)
        assert len(sent) == 2
        client.arena.close()
        client.sock.close(0)
    finally:
        stop.set()
        th.join(timeout=5)
        arena.close()
        sock.close(0)


def test_config_server_ranges():
    from fastapi.testclient import TestClient

    from lightllm_b200.server.config_server.api_http import MM_ID_RANGE, REQ_ID_RANGE, app

    c = TestClient(app)
    assert c.get("/health").status_code == 200
    a, b = c.get("/allocate_global_unique_id_range").json(), c.get("/allocate_global_unique_id_range").json()
    assert a["end_id"] - a["start_id"] == REQ_ID_RANGE and b["start_id"] == a["end_id"]
    m = c.get("/allocate_global_unique_multimodal_id_range").json()
    assert m["start_id"] >= 100_000_000 and m["end_id"] - m["start_id"] == MM_ID_RANGE
    assert c.get("/registered_objects").status_code == 200
