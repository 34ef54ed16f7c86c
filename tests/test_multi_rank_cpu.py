"""The multi-GPU algorithm on CPU ranks (gloo, world_size 2 and 3): neurons sharded with the library's own
shard_range, per-shard distances and first-minimum records from the oracle, one all-gather of the
(code, neuron) records, lexicographic global minimum, shard-local update -- with the rotation sets either computed
by every rank or in shares (each rank rotates a contiguous part of the images, the parts are gathered), as the
GPU library does.  The concatenated result must equal the single-process oracle bit for bit, including the tie rule
(lowest neuron index wins across shards)."""
import os
import sys

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, mode, share, ret):
    sys.path.insert(0, ROOT)
    import torch
    import oracle as O
    from pink_b200 import engine
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lay, s0, s1, idim, nd, ed, R, flip, n_img = 0, 3, 3, 16, 12, 7, 16, True, 4
    N = s0 * s1
    rng = np.random.default_rng(11)
    som = rng.random((N, 1, nd, nd), dtype=np.float32)
    som[5] = som[2]                      # two identical neurons in different shards: an exact BMU tie
    imgs = rng.random((n_img, idim, idim), dtype=np.float32)
    F = O.update_factors(lay, s0, s1, O.FUNC_GAUSSIAN, 1.1, 0.2)
    first, count = engine.shard_range(N, world, rank)
    mine = som[first:first + count].copy()
    T = R * 2
    bmus = []
    shared_rot = None
    if share:
        # the library's split of a batch: ceil(n / world) consecutive images per rank, the last ranks possibly none
        per = (n_img + world - 1) // world
        lo, hi = min(rank * per, n_img), min(rank * per + per, n_img)
        parts = [None] * world
        dist.all_gather_object(parts, [O.rotation_set(imgs[k], nd, R, flip) for k in range(lo, hi)])
        shared_rot = [r for part in parts for r in part]
        assert len(shared_rot) == n_img
    for k, img in enumerate(imgs):
        rot = shared_rot[k] if share else O.rotation_set(img, nd, R, flip)
        if mode == O.MODE_F32:
            d, best = O.distance_f32(mine, rot, ed)
            code = d.view(np.uint32).astype(np.uint64)               # non-negative floats order like their bits
        else:
            S = O.distance_int(O.crop_quantize(mine, ed, mode), O.crop_quantize(rot, ed, mode), mode)
            code, best = O.min_over_transforms_int(S)
        loc = int(np.lexsort((np.arange(count), code))[0])
        rec = torch.tensor([int(code[loc]), first + loc], dtype=torch.int64)
        recs = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(recs, rec)
        bmu = min((int(r[0]), int(r[1])) for r in recs)[1]
        bmus.append(bmu)
        O.update(mine.reshape(count, -1), rot.reshape(T, -1), best, bmu, np.ascontiguousarray(F[:, first:first + count]))
    # the shard-local update used F[bmu, first + n]: pko_update indexes factors[bmu * n_cols + n]
    parts = [None] * world
    dist.all_gather_object(parts, (first, mine, bmus))
    if rank == 0:
        whole = np.concatenate([p[1] for p in sorted(parts, key=lambda p: p[0])])
        ret.put((whole, bmus, som, imgs, F))
    dist.destroy_process_group()


@pytest.mark.parametrize("share", [False, True])
@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("mode", [2, 0])
def test_sharded_training_equals_single_process(world, mode, share):
    import oracle as O
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + world * 20 + mode * 2 + int(share) + (os.getpid() % 200)
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, share, q)) for r in range(world)]
    for p in procs:
        p.start()
    whole, bmus, som, imgs, F = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = som.copy()
    want_bmu = [O.train_step(want, im, F, 7, 16, True, mode)[2] for im in imgs]
    assert bmus == want_bmu
    assert np.array_equal(whole.view(np.uint32), want.view(np.uint32))
