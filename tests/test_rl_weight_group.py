"""Weight pushes from a trainer into a running engine: over a dedicated process group (gloo on CPU; the trainer is
rank 0 and hosts the store) and through a shared-memory segment on the same host."""
import socket
import threading
from multiprocessing import shared_memory
from types import SimpleNamespace

import numpy as np
import torch

from lightllm_b200.engine import rl_ops
from lightllm_b200.engine.llm import LLM
from lightllm_b200.parallel import dist as pdist
from lightllm_b200.server.core.objs.io_objs import RLCmd
from lightllm_b200.utils.rl_group import broadcast_from_trainer, join_weight_update_group

TINY = dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            head_dim=32, intermediate_size=256, vocab_size=512, rms_norm_eps=1e-6, rope_theta=1e4, eos_token_id=2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _engine():
    pdist.init_distributed(1, 0, device=torch.device("cpu"))
    llm = LLM(config=TINY, data_type="float32", max_total_token_num=2048, running_max_req_size=4,
              max_req_total_len=128, batch_max_tokens=256, random_seed=0)
    return llm, SimpleNamespace(model=llm.model, backend=llm.backend, ps=llm.ps)


def test_update_weights_from_distributed_group():
    llm, loop = _engine()
    prompt = [list(range(5, 30))]
    before = llm.generate(prompt, {"max_new_tokens": 6, "ignore_eos": True})[0]["token_ids"]
    port = _free_port()
    new_head = torch.randn(512, 128, generator=torch.Generator().manual_seed(3)) * 0.05
    new_norm = torch.full((128,), 0.5)
    box = {}

    def trainer():
        pg = join_weight_update_group("127.0.0.1", port, 0, 2, "wug", "gloo", timeout_s=60)
        box["pg"] = pg
        for t in (new_head.clone(), new_norm.clone()):
            broadcast_from_trainer(pg, t)

    th = threading.Thread(target=trainer)
    th.start()
    rl_ops.handle_rl_cmd(loop, RLCmd("init_weights_update_group", {"master_address": "127.0.0.1", "master_port": port,
                                                                   "rank_offset": 1, "world_size": 2,
                                                                   "group_name": "wug", "backend": "nccl"}))
    rl_ops.handle_rl_cmd(loop, RLCmd("update_weights_from_distributed",
                                     {"names": ["lm_head.weight", "model.norm.weight"], "dtypes": ["float32", "float32"],
                                      "shapes": [[512, 128], [128]], "group_name": "wug", "weight_version": "step-7"}))
    th.join(60)
    assert not th.is_alive()
    assert torch.equal(llm.model.lm_head_w.cpu(), new_head) and torch.equal(llm.model.final_norm_w.cpu(), new_norm)
    assert llm.model.weight_version == "step-7"
    after = llm.generate(prompt, {"max_new_tokens": 6, "ignore_eos": True})[0]
    assert after["token_ids"] != before and after["prompt_cache_len"] == 0      # new weights, prefix cache flushed
    rl_ops.handle_rl_cmd(loop, RLCmd("destroy_weights_update_group", {"group_name": "wug"}))
    try:
        rl_ops.handle_rl_cmd(loop, RLCmd("destroy_weights_update_group", {"group_name": "wug"}))
        raise AssertionError("destroying an unknown group must fail")
    except ValueError:
        pass
    pdist.destroy()


def test_update_weights_from_shared_memory():
    llm, loop = _engine()
    new_head = (torch.randn(512, 128, generator=torch.Generator().manual_seed(4)) * 0.05)
    raw = new_head.numpy().tobytes()
    shm = shared_memory.SharedMemory(create=True, size=len(raw) + 256)
    try:
        shm.buf[256:256 + len(raw)] = raw
        handle = {0: {"shm_name": shm.name, "manifest": [["lm_head.weight", "float32", [512, 128], 256]]}}
        rl_ops.handle_rl_cmd(loop, RLCmd("update_weights_from_ipc", {"ipc_handle": handle, "use_shm": True,
                                                                     "weight_version": "shm-1"}))
        assert torch.equal(llm.model.lm_head_w.cpu(), new_head) and llm.model.weight_version == "shm-1"
    finally:
        shm.close()
        shm.unlink()
    pdist.destroy()


def test_release_and_resume_weights_with_and_without_host_backup():
    llm, loop = _engine()
    prompt = [list(range(5, 30))]
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    before = llm.generate(prompt, sp)[0]["token_ids"]
    m = llm.model
    tied = m.lm_head_w is m.embed_w
    n_layer_tensors = sum(1 for lw in m.layers for t in lw.tensors().values() if isinstance(t, torch.Tensor))
    head_before = m.lm_head_w.clone()

    loop.args = SimpleNamespace(enable_weight_cpu_backup=True)
    rl_ops.release_memory_occupation(loop, tags=("kv_cache", "weights"))
    assert m.mem_manager.kv_buffer is None and m.embed_w is None and m.lm_head_w is None and m.final_norm_w is None
    assert all(not isinstance(t, torch.Tensor) for lw in m.layers for t in lw.tensors().values())
    keep, saved, slots = m._weight_backup
    assert keep and len(slots) == n_layer_tensors + 3 and all(isinstance(v, torch.Tensor) for v in saved.values())
    rl_ops.release_memory_occupation(loop, tags=("weights",))        # a second release keeps the first backup
    assert m._weight_backup[2] is slots
    rl_ops.resume_memory_occupation(loop, tags=("kv_cache", "weights"))
    assert m._weight_backup is None and (m.lm_head_w is m.embed_w) == tied
    assert llm.generate(prompt, sp)[0]["token_ids"] == before

    loop.args = SimpleNamespace(enable_weight_cpu_backup=False)
    rl_ops.release_memory_occupation(loop, tags=("weights",))
    assert all(isinstance(v, tuple) for v in m._weight_backup[1].values())          # shapes only
    rl_ops.resume_memory_occupation(loop, tags=("weights",))
    assert m.lm_head_w.shape == head_before.shape and float(m.lm_head_w.abs().sum()) == 0.0   # to be filled by a push
    assert (m.lm_head_w is m.embed_w) == tied
