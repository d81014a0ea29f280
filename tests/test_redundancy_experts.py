"""Redundant experts under data-parallel attention + expert-parallel MoE (CPU / gloo, world 2): physical id table,
hit counters, the same tokens as a single process with copies placed from a file, and a live re-placement.
Reference: lightllm/common/basemodel/layer_weights/meta_weights/fused_moe/ep_redundancy.py,
lightllm/server/router/model_infer/mode_backend/redundancy_expert_manager.py."""
import json
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from lightllm_b200.engine.redundancy import RedundancyConfig, physical_table
from lightllm_b200.ops import moe as moe_ops

CFG = dict(model_type="qwen3_moe", hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8,
           num_experts_per_tok=2, norm_topk_prob=True, vocab_size=512, rms_norm_eps=1e-6, eos_token_id=2,
           decoder_sparse_step=1, mlp_only_layers=[])


def test_physical_table_and_counter():
    # 8 experts over 2 ranks, 2 copies per rank: physical ids 0-3 + copies 4, 5 on rank 0; 6-9 + copies 10, 11 on rank 1
    t0 = physical_table(8, 2, 0, [6, 1])          # expert 1 is rank 0's own: the slot stays unused
    assert t0.tolist() == [0, 1, 2, 3, 6, 7, 4, 9]
    t1 = physical_table(8, 2, 1, [0, 3])
    assert t1.tolist() == [10, 1, 2, 11, 6, 7, 8, 9]
    ids = torch.tensor([[0, 6], [6, 7], [3, -1]], dtype=torch.int32)
    cnt = torch.zeros(8, dtype=torch.int32)
    out = moe_ops.count_remap(ids, t0, cnt)
    assert out.tolist() == [[0, 4], [4, 9], [3, -1]]
    assert cnt.tolist() == [1, 0, 0, 1, 0, 0, 2, 1]
    with pytest.raises(ValueError):
        physical_table(8, 2, 0, [8])


def test_config_file(tmp_path):
    p = tmp_path / "red.json"
    p.write_text(json.dumps({"redundancy_expert_num": 2, "0": [5, 6], "default": [0, 7]}))
    c = RedundancyConfig.load(str(p))
    assert c.num == 2 and c.ids(0) == [5, 6] and c.ids(3) == [0, 7]
    assert RedundancyConfig.load(None).ids(0) == []
    p.write_text(json.dumps({"redundancy_expert_num": 2, "default": [0]}))
    with pytest.raises(ValueError):
        RedundancyConfig.load(str(p))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompts():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(3, 512, (n,), generator=g).tolist() for n in (21, 40, 9, 33, 17)]


def _worker(rank, world, port, out_dir, red_path, auto):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    os.chdir(out_dir)
    os.environ["LLB_REDUNDANCY_EXPERT_UPDATE_INTERVAL"] = "0"
    pdist.init_distributed(world, rank, dp=world, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=CFG, data_type="float32", max_total_token_num=4096, running_max_req_size=8, max_req_total_len=128,
              batch_max_tokens=64, random_seed=0, enable_ep_moe=world > 1, ep_redundancy_expert_config_path=red_path,
              auto_update_redundancy_expert=auto)
    prompts = _prompts()
    mine = prompts if world == 1 else (prompts[:3] if rank == 0 else prompts[3:])
    outs = llm.generate(mine, {"max_new_tokens": 12, "ignore_eos": True})
    lws = [lw for lw in llm.model.layers if getattr(lw, "ep_table", None) is not None]
    torch.save({"tokens": [o["token_ids"] for o in outs], "stats": dict(llm.backend.stats),
                "shapes": [tuple(lw.w13.shape) for lw in lws], "red": [lw.ep_red_ids for lw in lws],
                "tables": [lw.ep_table.tolist() for lw in lws],
                "hits": [int(lw.ep_counter.sum()) for lw in lws]},
               os.path.join(out_dir, f"w{world}_r{rank}_a{int(auto)}.pt"))
    pdist.destroy()


@pytest.mark.timeout(900)
def test_dp2_ep2_with_redundant_experts_matches_single(tmp_path):
    red = tmp_path / "red.json"
    red.write_text(json.dumps({"redundancy_expert_num": 2, "0": [1, 6], "default": [3, 4]}))
    mp.spawn(_worker, args=(1, _free_port(), str(tmp_path), None, False), nprocs=1, join=True)
    one = torch.load(tmp_path / "w1_r0_a0.pt")
    # copies placed from the file
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), str(red), False), nprocs=2, join=True)
    r0, r1 = torch.load(tmp_path / "w2_r0_a0.pt"), torch.load(tmp_path / "w2_r1_a0.pt")
    assert r0["tokens"] == one["tokens"][:3] and r1["tokens"] == one["tokens"][3:]
    assert r0["shapes"] == [(6, 128, 128)] * 2            # 4 own experts + 2 copies, gate and up rows stacked
    assert r0["red"] == [[1, 6], [3, 4]] and r0["hits"][0] > 0
    assert r0["tables"][0] == [0, 1, 2, 3, 6, 7, 5, 9] and r1["tables"][0] == [0, 10, 2, 3, 6, 7, 8, 9]
    # live re-placement (interval 0: the first steps choose, read and commit new copies); outputs must not change
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), str(red), True), nprocs=2, join=True)
    a0, a1 = torch.load(tmp_path / "w2_r0_a1.pt"), torch.load(tmp_path / "w2_r1_a1.pt")
    assert a0["tokens"] == one["tokens"][:3] and a1["tokens"] == one["tokens"][3:]
    assert a0["stats"]["redundancy_updates"] == 1 and a1["stats"]["redundancy_updates"] == 1
    for res, own in ((a0, range(0, 4)), (a1, range(4, 8))):
        assert all(e not in own for ids in res["red"] for e in ids)      # never a copy of an own expert
    written = json.loads((tmp_path / "redundancy_expert_config.json").read_text())
    assert written["redundancy_expert_num"] == 2 and len(written["0"]) == 2 and len(written["1"]) == 2


def test_write_expert_slot_bf16_and_fp8():
    """Replacing one expert inside the stacked tensors the grouped GEMMs read (what a live re-placement commits)."""
    from lightllm_b200.engine.redundancy import write_expert_slot
    from lightllm_b200.ops import fp8

    torch.manual_seed(0)
    stacked = torch.randn(4, 64, 128)
    new = torch.randn(64, 128)
    keep = stacked.clone()
    write_expert_slot(stacked, 2, new)
    assert torch.equal(stacked[2], new) and torch.equal(stacked[[0, 1, 3]], keep[[0, 1, 3]])
    ws = [fp8.Fp8Weight.from_float(torch.randn(128, 256), 32) for _ in range(3)]
    ex = fp8.Fp8Experts(fp8.stack_experts(ws), 3)
    before = ex.dequant().clone()
    repl = fp8.Fp8Weight.from_float(torch.randn(128, 256) * 3, 32)
    write_expert_slot(ex, 1, repl)
    after = ex.dequant()
    assert torch.equal(after[1], repl.dequant()) and torch.equal(after[[0, 2]], before[[0, 2]])
