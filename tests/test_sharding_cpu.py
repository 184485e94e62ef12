"""Head sharding over ranks, exercised as two gloo processes on CPU: shard planning with KV
co-location / replication, output reassembly and CSR merging.  The attention itself is replaced by
the CPU oracle, which is head-independent exactly like the kernels."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def test_plan_head_shard():
    from risaattention_b200.sharding import plan_head_shard

    s = plan_head_shard(16, 4, 3, 8)   # 8 ranks, 4 kv heads: two ranks share one kv head
    assert (s.q_start, s.q_stop, s.kv_start, s.kv_stop) == (6, 8, 1, 2)
    s = plan_head_shard(16, 4, 1, 2)
    assert (s.q_start, s.q_stop, s.kv_start, s.kv_stop) == (8, 16, 2, 4)
    s = plan_head_shard(40, 40, 7, 8)
    assert (s.q_start, s.q_stop, s.kv_start, s.kv_stop) == (35, 40, 35, 40)
    with pytest.raises(ValueError):
        plan_head_shard(16, 4, 0, 3)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import risa_oracle as O
    from risaattention_b200.sharding import (gather_heads, merge_patterns, plan_head_shard,
                                             shard_inputs)

    torch.manual_seed(0)
    b, hq, hkv, lq, lk, d = 2, 4, 2, 130, 200, 64
    q, k, v = torch.randn(b, hq, lq, d), torch.randn(b, hkv, lk, d), torch.randn(b, hkv, lk, d)
    shard = plan_head_shard(hq, hkv, rank, world)
    ql, kl, vl, _ = shard_inputs(q, k, v, shard)
    local = O.int8_attention(ql, kl, vl)
    full = gather_heads(local)
    want = O.int8_attention(q, k, v)
    assert torch.equal(full, want), "head-sharded result must equal the single-device result"

    # CSR merge: rows [batch, head, q-block]; build a per-rank pattern and compare with the global one
    n_q, n_k = 2, 4
    g = torch.Generator().manual_seed(5)
    masses = torch.rand(b * hq * n_q, n_k, generator=g)
    ro, bi, _ = O.select_retained_mass(masses, 0.6)
    view = masses.view(b, hq, n_q, n_k)[:, shard.q_start:shard.q_stop].reshape(-1, n_k)
    lro, lbi, _ = O.select_retained_mass(view, 0.6)
    mro, mbi = merge_patterns(lro, lbi, b)
    assert torch.equal(mro, ro) and torch.equal(mbi, bi)
    dist.destroy_process_group()
    Path(tmp, f"ok{rank}").write_text("ok")


def test_two_rank_head_sharding(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
