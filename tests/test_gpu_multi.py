"""Neuron-sharded training on several GPUs (one process per GPU; the per-shard BMU records are exchanged by
peer-memory stores or by an NCCL all-gather)
against the single-process CPU oracle.  Needs at least two GPUs; skipped otherwise."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, mode, exchange, q):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    options = {"nccl": {"exchange": 1}, "peer": {"rotation_sharing": 0}, "shared": {},
               "two-kernel": {"step_kernel": 1}, "contiguous": {"sharding": 1}}[exchange]
    import torch
    import torch.distributed as dist
    from pink_b200 import capi, engine
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    lay, s0, s1, idim, nd, ed, R, flip, n_img = 0, 5, 4, 32, 22, 15, 40, True, 37      # three batches, the last one ragged
    N = s0 * s1
    rng = np.random.default_rng(77)
    som = rng.random((N, 1, nd, nd), dtype=np.float32)
    som[13] = som[4]                                   # identical neurons in different shards: BMU ties
    imgs = rng.random((n_img, 1, idim, idim), dtype=np.float32)
    F = engine.update_factors(lay, s0, s1, capi.FUNC_GAUSSIAN, 1.1, 0.2)
    eng = engine.Engine(N, 1, idim, nd, ed, R, flip, mode, device=rank, rank=rank, world_size=world, options=options)
    uid = [engine.Engine.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, 0)
    eng.comm_init(uid[0])
    kind = eng.exchange_kind()
    eng.set_som(som)
    eng.set_update_factors(F)
    eng.train(imgs)
    eng.synchronize()
    part = eng.get_som(np.zeros_like(som))
    counts = eng.update_counts()
    out = [None] * world
    dist.all_gather_object(out, (eng.neurons, part[eng.neurons], counts))
    if rank == 0:
        whole = np.zeros_like(som)
        seen = np.zeros(N, int)
        for neurons, rows, _ in out:
            whole[neurons] = rows
            seen[neurons] += 1
        assert (seen == 1).all()                       # the shards partition the map
        q.put((whole, sum(p[2] for p in out), som, imgs, F, kind))
    eng.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["shared", "peer", "nccl", "two-kernel", "contiguous"])
@pytest.mark.parametrize("mode", [2, 1, 0])
def test_two_gpu_sharded_training_bit_exact(cuda, mode, exchange):
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import oracle as O
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + 5 * mode + ["shared", "peer", "nccl", "two-kernel", "contiguous"].index(exchange) + (os.getpid() % 100)
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, exchange, q)) for r in range(world)]
    for p in procs:
        p.start()
    whole, counts, som, imgs, F, kind = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert kind == {"shared": 3, "peer": 2, "nccl": 1, "two-kernel": 3, "contiguous": 3}[exchange]      # the intended exchange really ran
    want = som.copy()
    bmus = [O.train_step(want, im, F, 15, 40, True, mode)[2] for im in imgs]
    if mode == 0:        # float32 distances: same best matching units (no near-ties in this seed), same arithmetic
        np.testing.assert_allclose(whole, want, rtol=1e-5, atol=1e-7)
    else:
        assert np.array_equal(whole.view(np.uint32), want.view(np.uint32))
    assert counts.sum() == len(imgs) and all(counts[b] > 0 for b in bmus)


def _silent_worker(rank, world, port, q):
    """Rank 1 stops delivering records after two images; rank 0 trains a third and must get a time-out status
    (not a hang) from its update kernel's bounded wait.  Rank 1 keeps its context until rank 0 is done, so that
    rank 0's stores into rank 1's record ring stay valid."""
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import time
    import torch
    import torch.distributed as dist
    from pink_b200 import capi, engine
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    N, idim, nd, ed, R = 12, 24, 16, 11, 8
    rng = np.random.default_rng(3)
    som = rng.random((N, 1, nd, nd), dtype=np.float32)
    imgs = rng.random((3, 1, idim, idim), dtype=np.float32)
    F = engine.update_factors(0, 4, 3, capi.FUNC_GAUSSIAN, 1.1, 0.2)
    eng = engine.Engine(N, 1, idim, nd, ed, R, True, capi.UINT8, device=rank, rank=rank, world_size=world)
    uid = [engine.Engine.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, 0)
    eng.comm_init(uid[0])
    eng.set_som(som)
    eng.set_update_factors(F)
    eng.train(imgs[:2])
    eng.synchronize()
    dist.barrier()
    outcome = None
    if rank == 0:
        t0 = time.time()
        try:
            eng.train(imgs[2:])
            eng.synchronize()
            outcome = "no error"
        except capi.PinkError as ex:
            outcome = (ex.code if hasattr(ex, "code") else None, str(ex), time.time() - t0)
    dist.barrier()                       # rank 1 leaves only now, between steps, with nothing in flight
    if rank == 0:
        q.put((eng.exchange_kind(), outcome))
    eng.close()
    dist.destroy_process_group()


def test_missing_rank_gives_a_timeout_status(cuda):
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29850 + (os.getpid() % 100)
    procs = [ctx.Process(target=_silent_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    kind, outcome = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert kind == 3                                         # peer-memory exchange with shared rotation work
    assert outcome != "no error"
    import re
    assert re.search(r"bounded device-side wait expired \(code 1[34]\)", outcome[1])     # record or rotation-share wait
    assert outcome[2] < 30                                   # seconds: a bounded wait, not a hang
