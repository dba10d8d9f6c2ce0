"""KV-head-sharded decode on two B200s: every rank's logits equal the unsharded step's, with the all-gather done
by NCCL and with the attention merge pushing its block into the peers' buffers itself."""
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


MODES = ("full", "sharded", "sharded_graph", "pushed", "pushed_graph")


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from trimkv_b200 import TrimKVCache, TrimKVQwen3Config, TrimKVQwen3ForCausalLM
        from trimkv_b200.decoder import GreedyDecoder
        results = {}
        # (memory_size, buffer_size, prompt length, layers): a cache of one chunk per segment, and one of several
        # chunks (merge of partials) with an odd number of layers (buffer rotation across steps)
        for tag, (M, Bf, P, L) in {"short": (48, 8, 70, 2), "long": (600, 40, 700, 3)}.items():
            cfg = TrimKVQwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=L,
                                    num_attention_heads=8, num_key_value_heads=4, head_dim=128,
                                    retention_gate_intermediate_size=32, retention_gate_bias_init=3.0, memory_size=M,
                                    buffer_size=Bf, initializer_range=0.02)
            torch.manual_seed(0)
            model = TrimKVQwen3ForCausalLM(cfg).to(torch.bfloat16).eval().to(dev)
            gen = torch.Generator().manual_seed(3)
            prompt = torch.randint(0, cfg.vocab_size, (3, P), generator=gen).to(dev)
            forced = torch.randint(0, cfg.vocab_size, (24, 3, 1), generator=gen).to(dev)
            with torch.inference_mode():
                for mode in MODES:
                    cache = TrimKVCache(device=dev)
                    out = model(input_ids=prompt, past_key_values=cache, logits_to_keep=1)   # replicated prompt pass
                    if mode == "full":
                        dec = GreedyDecoder(model, cache, use_graph=False, fused=True)
                    else:
                        local = cache.head_shard(rank, world)
                        dec = GreedyDecoder(model, local, use_graph=mode.endswith("_graph"), head_shard_group=dist.group.WORLD,
                                            fused_gather=mode.startswith("pushed"))
                        cache = local
                    logits = []
                    for t in range(24):
                        dec.step(forced[t], eager=(t < 2))
                        logits.append(dec.logits.float().clone())
                    cache.check_status()
                    n = cache.get_cache_length(0)
                    results[tag + "/" + mode] = (torch.stack(logits).cpu().numpy(),
                                                 cache.kv_positions[0][:, :, :n].cpu().numpy(), n)  # by value
                    # The captured step holds the communicator's collectives; the communicator can only be
                    # destroyed once no such graph is left.
                    dec.close()
                    del dec
                    torch.cuda.synchronize()
                    dist.barrier()
        q.put((rank, results))
        q.close()
        q.join_thread()          # results are on their way before anything else can go wrong
    except Exception:            # the parent must see the failure instead of waiting for a result that never comes
        import traceback
        q.put((rank, {"error": traceback.format_exc()}))
        q.close()
        q.join_thread()
        os._exit(1)
    # Orderly teardown, bounded: a destroy that does not return ends the process with code 3, which the parent checks.
    import threading
    torch.cuda.synchronize()
    dist.barrier()
    watchdog = threading.Timer(60.0, lambda: os._exit(3))
    watchdog.daemon = True
    watchdog.start()
    dist.destroy_process_group()
    watchdog.cancel()


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
            p.join(timeout=90)
            if p.is_alive():
                p.terminate()
    for rank in range(world):
        assert "error" not in got[rank], got[rank]["error"]
    assert [p.exitcode for p in procs] == [0] * world, "communicator teardown did not complete"
    for tag in ("short", "long"):
        for rank in range(world):
            full_logits, full_pos, n_full = got[rank][tag + "/full"]
            for mode in MODES[1:]:
                logits, pos, n = got[rank][tag + "/" + mode]
                assert n == n_full
                assert float(np.abs(logits - full_logits).max()) <= 2e-2, (tag, rank, mode)
                hl = full_pos.shape[1] // world
                assert np.array_equal(pos, full_pos[:, rank * hl:(rank + 1) * hl]), (tag, rank, mode)  # same survivors per head
            # the pushed exchange moves the same bf16 values as the all-gather
            assert np.array_equal(got[rank][tag + "/pushed"][0], got[rank][tag + "/sharded"][0]), (tag, rank)
            assert np.array_equal(got[rank][tag + "/pushed_graph"][0], got[rank][tag + "/sharded_graph"][0]), (tag, rank)
        # both ranks hold the same logits (replicated tail of the layer)
        assert np.array_equal(got[0][tag + "/sharded"][0], got[1][tag + "/sharded"][0])
        assert np.array_equal(got[0][tag + "/pushed"][0], got[1][tag + "/pushed"][0])
