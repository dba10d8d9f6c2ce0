"""Batch partition across ranks, exercised with two (and three) gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from trimkv_b200.parallel import gather_rows, generate_partitioned, partition_bounds


def test_partition_bounds_cover_every_request_once():
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = partition_bounds(n, world, r)
                assert 0 <= lo <= hi <= n
                seen += list(range(lo, hi))
            assert seen == list(range(n))
            sizes = [partition_bounds(n, world, r)[1] - partition_bounds(n, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        partition_bounds(4, 2, 2)


def _fake_generate(ids):
    # stands in for model.generate on this rank's requests: a pure function of each request's own tokens
    new = (ids.sum(dim=1, keepdim=True) * torch.arange(1, 4)) % 1000
    return torch.cat([ids, new], dim=1)


def _worker(rank, world, port, n_requests, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        ids = torch.randint(0, 100, (n_requests, 6))
        out = generate_partitioned(_fake_generate, ids)
        lo, hi = partition_bounds(n_requests, world, rank)
        block = gather_rows(torch.full((hi - lo, 2), rank, dtype=torch.int64), n_requests)
        q.put((rank, out, block))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,n_requests", [(2, 8), (2, 5), (3, 2)])
def test_partitioned_generation_equals_single_rank(world, n_requests):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_requests, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    torch.manual_seed(0)
    ids = torch.randint(0, 100, (n_requests, 6))
    want = _fake_generate(ids)
    for rank, out, block in results:
        assert torch.equal(out, want), rank          # same rows, same order, on every rank
        owners = torch.cat([torch.full((partition_bounds(n_requests, world, r)[1] - partition_bounds(n_requests, world, r)[0],),
                                       r) for r in range(world)])
        assert torch.equal(block[:, 0], owners)


# ---- KV-head sharding: how the projections are cut and how the gathered attention output is ordered (CPU, gloo)
def _shard_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import types
        import torch.nn.functional as F
        from trimkv_b200 import TrimKVQwen3Config, TrimKVQwen3ForCausalLM
        from trimkv_b200.decoder import HeadShardedDecodeStep
        cfg = TrimKVQwen3Config(vocab_size=64, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                num_attention_heads=8, num_key_value_heads=4, head_dim=128,
                                retention_gate_intermediate_size=16, retention_gate_bias_init=3.0)
        torch.manual_seed(0)
        model = TrimKVQwen3ForCausalLM(cfg).eval()
        hkv_l, hq_l, d = cfg.num_key_value_heads // world, cfg.num_attention_heads // world, 128
        class _CacheStub:                      # what the step reads of a cache at construction (it holds it weakly)
            _hkv = hkv_l
        stub = _CacheStub()
        step = HeadShardedDecodeStep(model, stub, group=None)
        h = torch.randn(3, cfg.hidden_size)
        ok = True
        for l, (layer, w, bias, _, _) in enumerate(step.layers):
            w_l, b_l, g2_l, gb_l = step.local[l]
            full = F.linear(h, w, bias)
            mine = F.linear(h, w_l, b_l)
            hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
            q_cols = slice(rank * hq_l * d, (rank + 1) * hq_l * d)
            k_cols = slice(hq * d + rank * hkv_l * d, hq * d + (rank + 1) * hkv_l * d)
            v_cols = slice((hq + hkv) * d + rank * hkv_l * d, (hq + hkv) * d + (rank + 1) * hkv_l * d)
            want = torch.cat([full[:, q_cols], full[:, k_cols], full[:, v_cols], full[:, (hq + 2 * hkv) * d:]], 1)
            ok &= torch.equal(mine, want)
            g = layer.self_attn.retention_gate
            ok &= torch.equal(g2_l, g.linear2.weight[rank * hkv_l:(rank + 1) * hkv_l])
            ok &= torch.equal(gb_l, g.bias[rank * hkv_l:(rank + 1) * hkv_l])
        # the per-layer exchange: every rank contributes [B, hq_l * D]; rank-major blocks are the head order
        o_full = torch.arange(3 * cfg.num_attention_heads * d, dtype=torch.float32).view(3, -1)
        o_mine = o_full[:, rank * hq_l * d:(rank + 1) * hq_l * d].contiguous()
        parts = [torch.empty(3, hq_l * d) for _ in range(world)]
        dist.all_gather(parts, o_mine)
        gathered = torch.stack(parts)                                   # what all_gather_into_tensor fills on the GPU path
        ok &= torch.equal(gathered.permute(1, 0, 2).reshape(3, -1), o_full)
        q.put((rank, bool(ok)))
    except Exception:
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_head_sharded_projection_slices_and_gather_order(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_shard_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert got == {r: True for r in range(world)}
