"""KV-head-sharded decode on two B200s (NCCL): every rank's logits equal the unsharded step's."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from trimkv_b200 import TrimKVCache, TrimKVQwen3Config, TrimKVQwen3ForCausalLM
        from trimkv_b200.decoder import GreedyDecoder
        cfg = TrimKVQwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                num_attention_heads=8, num_key_value_heads=4, head_dim=128,
                                retention_gate_intermediate_size=32, retention_gate_bias_init=3.0, memory_size=48,
                                buffer_size=8, initializer_range=0.02)
        torch.manual_seed(0)
        model = TrimKVQwen3ForCausalLM(cfg).to(torch.bfloat16).eval().to(dev)
        gen = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, cfg.vocab_size, (3, 70), generator=gen).to(dev)
        forced = torch.randint(0, cfg.vocab_size, (24, 3, 1), generator=gen).to(dev)
        results = {}
        with torch.inference_mode():
            for mode in ("full", "sharded", "sharded_graph"):
                cache = TrimKVCache(device=dev)
                out = model(input_ids=prompt, past_key_values=cache, logits_to_keep=1)   # replicated prompt pass
                if mode == "full":
                    dec = GreedyDecoder(model, cache, use_graph=False, fused=True)
                else:
                    local = cache.head_shard(rank, world)
                    dec = GreedyDecoder(model, local, use_graph=(mode == "sharded_graph"), head_shard_group=dist.group.WORLD)
                    cache = local
                logits = []
                for t in range(24):
                    dec.step(forced[t], eager=(t < 2))
                    logits.append(dec.logits.float().clone())
                cache.check_status()
                n = cache.get_cache_length(0)
                results[mode] = (torch.stack(logits).cpu().numpy(), cache.kv_positions[0][:, :, :n].cpu().numpy(), n)  # by value
        q.put((rank, results))
        q.close()
        q.join_thread()          # results are on their way before anything else can go wrong
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        # Leave without NCCL / CUDA-graph teardown: destroying a communicator whose collectives were captured in a
        # still-live CUDA graph did not return here, and the test is about the numbers, which are already sent.
        os._exit(0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_decode_equals_unsharded():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q, port, world = ctx.Queue(), _free_port(), 2
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = dict(q.get(timeout=240) for _ in range(world))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    for rank in range(world):
        full_logits, full_pos, n_full = got[rank]["full"]
        for mode in ("sharded", "sharded_graph"):
            logits, pos, n = got[rank][mode]
            assert n == n_full
            assert float(np.abs(logits - full_logits).max()) <= 2e-2, (rank, mode)
            hl = full_pos.shape[1] // world
            assert np.array_equal(pos, full_pos[:, rank * hl:(rank + 1) * hl]), (rank, mode)  # same survivors per head
    # both ranks hold the same logits (replicated tail of the layer)
    assert np.array_equal(got[0]["sharded"][0], got[1]["sharded"][0])
