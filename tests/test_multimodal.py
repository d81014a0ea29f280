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
        # requests that arrived together share encoder passes and travel on in arrival order, control messages too
        raw2 = _png(56, 56, seed=5)
        n2 = image_token_num(56, 56)[0]
        rec2 = client.alloc(["m2"], [n2])[0]
        client.set_items_data([rec2["id"]], [raw2])
        t2, gh2, gw2 = image_token_num(56, 56)[1]
        item2 = {"uuid": rec2["id"], "token_id": rec2["token_id"], "token_num": n2,
                 "start_index_in_embed_cache": rec2["start_index_in_embed_cache"], "grid_thwd": (t2, gh2, gw2, 2)}
        calls = []
        real = tower.encode_images
        tower.encode_images = lambda payloads, items=None: (calls.append(len(payloads)), real(payloads, items=items))[1]
        ga = GroupReqIndexes(16, {"images": [item2], "audios": []}, [1], 0.0)
        gb = GroupReqIndexes(24, {"images": [item2, item], "audios": []}, [2], 0.0)   # the same picture again
        queue = [ga, "control", gb]
        vm2 = VisualManager(args, tower, client, sent.append, lambda: queue.pop(0),
                            try_recv=lambda: queue.pop(0) if queue else None, send_batch_size=8)
        msgs = [vm2.recv()]
        while (m := vm2.try_recv()) is not None:
            msgs.append(m)
        vm2.handle_many(msgs)
        assert sent[2:] == [ga, "control", gb] and calls == [1]          # one pass, one new picture
        assert client.get_items_embed([rec2["id"]]) == [True]
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


def test_qwen_vl_v1_tower_and_tokenizer():
    """First-generation Qwen-VL: ViT with per-head packed qkv, resampler against torch's MultiheadAttention, prompt
    formatting with picture numbers."""
    import torch
    import torch.nn.functional as F
    from types import SimpleNamespace

    from lightllm_b200.models.llama import QwenVLV1Tokenizer
    from lightllm_b200.models.registry import get_model_class, is_multimodal
    from lightllm_b200.models.vit.qwen_vl_visual import QwenVLVisionTower, resize_positions, sincos_2d
    from lightllm_b200.models.weights import RandomSource

    vcfg = dict(image_size=56, patch_size=14, width=32, layers=2, heads=4, mlp_ratio=2.0, output_dim=128, n_queries=16)
    shapes = QwenVLVisionTower.weight_shapes(vcfg)
    src = RandomSource(shapes, dtype=torch.float32, seed=0)
    tower = QwenVLVisionTower(vcfg, src, torch.device("cpu"), torch.float32)
    pixels = torch.randn(2, 3, 56, 56)
    out = tower.forward(pixels)
    assert out.shape == (2, 16, 128) and torch.isfinite(out).all()
    # resampler == nn.MultiheadAttention with the same tensors
    E, W = 128, 32
    feats = torch.randn(2, 16, W)
    mha = torch.nn.MultiheadAttention(E, tower.pool_heads)
    with torch.no_grad():
        mha.in_proj_weight.copy_(tower.pool["attn.in_proj_weight"])
        mha.in_proj_bias.copy_(tower.pool["attn.in_proj_bias"])
        mha.out_proj.weight.copy_(tower.pool["attn.out_proj.weight"])
        mha.out_proj.bias.copy_(tower.pool["attn.out_proj.bias"])
        x = F.linear(feats, tower.pool_kv_w)
        kv = F.layer_norm(x, (E,), tower.pool["ln_kv.weight"], tower.pool["ln_kv.bias"], 1e-6).permute(1, 0, 2)
        q = F.layer_norm(tower.pool["query"], (E,), tower.pool["ln_q.weight"], tower.pool["ln_q.bias"], 1e-6)
        pe = tower.pool["pos_embed"]
        want = mha(q.unsqueeze(1).repeat(1, 2, 1) + pe.unsqueeze(1), kv + resize_positions(pe, 16).unsqueeze(1), kv)[0]
        got = tower._resample(feats)
    assert (got - want.permute(1, 0, 2)).abs().max().item() < 1e-5
    pe = sincos_2d(8, 2)      # 2 x 2 grid, 8 channels: [sin, cos] of the column index, then of the row index
    assert pe.shape == (4, 8) and torch.allclose(pe[0], torch.tensor([0., 0., 1., 1., 0., 0., 1., 1.]))
    assert torch.allclose(pe[1, :4], torch.tensor([0.8415, 0.0100, 0.5403, 0.99995]), atol=1e-4)
    assert torch.allclose(pe[2, 4:], pe[1, :4]) and torch.allclose(pe[2, :4], pe[0, :4])

    cfg = {"model_type": "qwen", "visual": vcfg, "hidden_size": 128}
    assert is_multimodal(cfg) and not is_multimodal({"model_type": "qwen"})
    assert get_model_class(cfg).__name__ == "QwenVLV1LM" and get_model_class({"model_type": "qwen"}).__name__ == "QwenV1LM"

    class Tok:
        img_start_id, img_end_id = 900, 901

        def encode(self, text):
            out = []
            for w in text.replace("<img>", " <img> ").replace("</img>", " </img> ").replace("\n", " NL ").split():
                out.append({"<img>": 900, "</img>": 901, "NL": 7}.get(w, 1 if w.startswith("Picture") else 5))
            return out

    tk = QwenVLV1Tokenizer(Tok(), cfg)
    assert tk.get_image_token_length(None) == 16
    mp = SimpleNamespace(images=[SimpleNamespace(token_id=5000, token_num=16), SimpleNamespace(token_id=6000, token_num=16)])
    ids = tk.encode("look <img>a.jpg</img> and <img>b.jpg</img> ok", mp)
    assert ids == [5, 1, 5, 900] + list(range(5000, 5016)) + [901, 7, 5, 1, 5, 900] + list(range(6000, 6016)) + [901, 7, 5]


def test_encoder_replicas_share_a_batch_of_pictures():
    """`--visual_dp` / `--audio_dp`: the pictures of one pass are dealt to the replicas, which run on threads of
    their own; payload reads and arena writes stay on the manager's thread; results do not depend on the dealing."""
    import threading as th

    from lightllm_b200.server.audioserver.manager import AudioManager
    from lightllm_b200.server.core.objs.io_objs import GroupReqIndexes
    from lightllm_b200.server.visualserver.manager import VisualManager, encode_on_replicas, replica_devices

    main = th.get_ident()

    class Tower:
        def __init__(self):
            self.batches, self.threads = [], set()

        def encode_images(self, payloads, items=None):
            self.batches.append(len(payloads))
            self.threads.add(th.get_ident())
            return [torch.full((it["token_num"], 4), float(p[0])) for p, it in zip(payloads, items)]

        def encode_audios(self, clips, items=None):
            self.threads.add(th.get_ident())
            return [torch.full((it["token_num"], 4), float(c[0])) for c, it in zip(clips, items)]

    class Cache:
        def __init__(self, payloads):
            self.payloads, self.ready, self.rows, self.callers = payloads, set(), {}, set()
            self.arena = SimpleNamespace(write=lambda start, e: (self.callers.add(th.get_ident()),
                                                                 self.rows.__setitem__(start, e.clone())))

        def get_items_embed(self, ids):
            return [i in self.ready for i in ids]

        def set_items_embed(self, ids):
            self.callers.add(th.get_ident())
            self.ready.update(ids)

        def get_payload(self, uid):
            self.callers.add(th.get_ident())
            return self.payloads[uid]

    items = [{"uuid": u, "token_num": 1 + u % 3, "start_index_in_embed_cache": 10 * u} for u in range(7)]
    towers = [Tower(), Tower(), Tower()]
    cache = Cache({u: bytes([u + 1]) * 4 for u in range(7)})
    sent = []
    vm = VisualManager(SimpleNamespace(), None, cache, sent.append, None, infer_batch_size=2, towers=towers)
    g = GroupReqIndexes(8, {"images": items + [items[0]], "audios": []}, [0], 0.0)
    vm.handle_many([g])
    assert sent == [g] and cache.ready == set(range(7)) and cache.callers == {main}
    assert [sorted(t.batches, reverse=True) for t in towers] == [[2, 1], [2], [2]]     # 3 + 2 + 2 pictures
    assert all(t.threads and main not in t.threads for t in towers)
    for it in items:
        assert torch.equal(cache.rows[it["start_index_in_embed_cache"]], torch.full((it["token_num"], 4), it["uuid"] + 1.0))
    # one picture: no threads, the first replica does it
    cache.payloads[9] = bytes([42]) * 4
    vm.handle_many([GroupReqIndexes(16, {"images": [{"uuid": 9, "token_num": 2, "start_index_in_embed_cache": 99}],
                                        "audios": []}, [1], 0.0)])
    assert main in towers[0].threads and float(cache.rows[99][0, 0]) == 42.0

    clips = {u: np.full(8, u + 0.5, dtype=np.float32).tobytes() for u in range(5)}
    acache = Cache(clips)
    atowers = [Tower(), Tower()]
    am = AudioManager(SimpleNamespace(), None, acache, sent.append, None, infer_batch_size=2, towers=atowers)
    am.handle(GroupReqIndexes(24, {"images": [], "audios": [{"uuid": u, "token_num": 2, "start_index_in_embed_cache": u}
                                                           for u in range(5)]}, [2], 0.0))
    assert acache.ready == set(range(5)) and acache.callers == {main} and all(t.threads for t in atowers)
    assert float(acache.rows[3][0, 0]) == 3.5

    assert replica_devices(None, 3) == [torch.device("cpu")] * 3 or torch.cuda.is_available()
    out = encode_on_replicas([Tower(), Tower()], 5, 2, lambda t, idx: [torch.tensor(float(i)) for i in idx])
    assert [float(x) for x in out] == [0.0, 1.0, 2.0, 3.0, 4.0]
