"""`--enable_dp_prefill_balance`: split sizes on hand-made cases, the exchange and its inverse over gloo, and a
data-parallel + expert-parallel run (2 replicas with very different prompt loads) that must produce the tokens of
a single process.  Reference: lightllm/common/basemodel/infer_struct.py:167-351."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from lightllm_b200.common.dp_balance import plan_balance

MOE = dict(model_type="qwen3_moe", hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8,
           num_experts_per_tok=2, norm_topk_prob=True, vocab_size=512, rms_norm_eps=1e-6, eos_token_id=2,
           decoder_sparse_step=1, mlp_only_layers=[])


def test_plan_by_hand():
    S = plan_balance([10, 2, 0, 4])                 # total 16 -> 4 each
    assert S == [[4, 2, 4, 0], [0, 2, 0, 0], [0, 0, 0, 0], [0, 0, 0, 4]]
    S = plan_balance([7, 0, 0])                     # shares 3, 2, 2
    assert S == [[3, 2, 2], [0, 0, 0], [0, 0, 0]]
    S = plan_balance([1, 9])                        # 5 each: replica 1 sheds 4
    assert S == [[1, 0], [4, 5]]
    for lens in ([5, 5, 5], [0, 0, 12, 1], [3, 100, 7, 50, 0, 0, 1, 8]):
        S = plan_balance(lens)
        n, total = len(lens), sum(lens)
        assert [sum(r) for r in S] == lens
        cols = [sum(S[s][d] for s in range(n)) for d in range(n)]
        assert max(cols) - min(cols) <= 1 and sum(cols) == total
    assert plan_balance([8, 0], multiple=4) == [[4, 4], [0, 0]]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _exchange_worker(rank, world, port, out_dir):
    from lightllm_b200.common.dp_balance import DPBalance
    from lightllm_b200.parallel import dist as pdist

    ps = pdist.init_distributed(world, rank, dp=world, host="127.0.0.1", port=port, backend="gloo",
                                device=torch.device("cpu"))
    lens = [11, 1, 0 + 2][: world]
    n = lens[rank]
    bal = DPBalance.prepare(ps, n)
    x = torch.arange(n * 3, dtype=torch.float32).view(n, 3) + 1000 * rank
    y = bal.to_balanced(x)
    back = bal.to_origin(y * 2)
    ok = torch.equal(back, x * 2)
    none = DPBalance.prepare(ps, 10 + rank) is None          # 10 / 11 / 12 tokens: balanced enough
    torch.save({"rows": y.shape[0], "ok": ok, "none": none, "first": y[:, 0].tolist()},
               os.path.join(out_dir, f"x{rank}.pt"))
    pdist.destroy()


@pytest.mark.timeout(300)
def test_exchange_and_inverse(tmp_path):
    mp.spawn(_exchange_worker, args=(3, _free_port(), str(tmp_path)), nprocs=3, join=True)
    rs = [torch.load(tmp_path / f"x{r}.pt") for r in range(3)]
    assert [r["rows"] for r in rs] == [5, 5, 4] and all(r["ok"] and r["none"] for r in rs)
    # replica 0 keeps its first 5 rows; rows 5..8 go to replica 1 (behind... in source-rank order: its own row last)
    assert rs[0]["first"] == [0.0, 3.0, 6.0, 9.0, 12.0]
    assert rs[1]["first"] == [15.0, 18.0, 21.0, 24.0, 1000.0]
    assert rs[2]["first"] == [27.0, 30.0, 2000.0, 2003.0]


def _prompts():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(3, 512, (n,), generator=g).tolist() for n in (60, 40, 33, 5)]


def _worker(rank, world, port, out_dir, balance):
    from lightllm_b200.common import dp_balance
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, dp=world, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=MOE, data_type="float32", max_total_token_num=4096, running_max_req_size=8, max_req_total_len=128,
              batch_max_tokens=256, random_seed=0, enable_ep_moe=world > 1, enable_dp_prefill_balance=balance)
    made = []
    real = dp_balance.DPBalance.prepare.__func__

    def spy(cls, ps, n, min_gain=0.1):
        b = real(cls, ps, n, min_gain)
        made.append((n, None if b is None else b.handle_len))
        return b

    dp_balance.DPBalance.prepare = classmethod(spy)
    prompts = _prompts()
    mine = prompts if world == 1 else (prompts[:3] if rank == 0 else prompts[3:])     # 133 tokens against 5
    outs = llm.generate(mine, {"max_new_tokens": 8, "ignore_eos": True})
    torch.save({"tokens": [o["token_ids"] for o in outs], "made": made},
               os.path.join(out_dir, f"w{world}_r{rank}_b{int(balance)}.pt"))
    pdist.destroy()


@pytest.mark.timeout(600)
def test_dp2_ep2_balanced_prefill_matches_single(tmp_path):
    mp.spawn(_worker, args=(1, _free_port(), str(tmp_path), False), nprocs=1, join=True)
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), True), nprocs=2, join=True)
    one = torch.load(tmp_path / "w1_r0_b0.pt")
    r0, r1 = torch.load(tmp_path / "w2_r0_b1.pt"), torch.load(tmp_path / "w2_r1_b1.pt")
    assert r0["tokens"] == one["tokens"][:3] and r1["tokens"] == one["tokens"][3:]
    # the prompt pass ran balanced: 133 + 5 tokens -> 69 each
    assert (133, 69) in r0["made"] and (5, 69) in r1["made"]
