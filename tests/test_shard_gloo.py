"""The multi-rank logic on CPU: two gloo ranks shard one batch, evaluate their rows (with the oracle,
since the engine itself has no CPU path), and agree on the dataset mean and on the max-over-ranks time."""
import os

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

from spnb.shard import shard_rows


def test_shard_rows_cover_the_batch_exactly():
    for n in (0, 1, 1023, 1024, 1025, 10_000_000, 2_000_001):
        for world in (1, 2, 3, 4, 8):
            rows = [shard_rows(n, world, r) for r in range(world)]
            assert rows[0][0] == 0 and rows[-1][1] == n
            for (a0, a1), (b0, b1) in zip(rows, rows[1:]):
                assert a1 == b0 and a0 <= a1 and b0 <= b1
            assert all(r0 % 1024 == 0 for r0, r1 in rows if r1 > r0)


def _rank_main(rank, world, port, query, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle
    from spnb import synth
    from spnb.shard import dataset_mean, max_over_ranks
    x = synth.config2_inputs(5000, 123)
    r0, r1 = shard_rows(len(x), world, rank)
    ll = oracle.evaluate(oracle.load_model(query), x[r0:r1], "log_f32_gpu")
    mean = dataset_mean(ll.astype(np.float64).sum(), len(ll))
    slowest = max_over_ranks(10.0 + rank)
    np.save(os.path.join(out_dir, "ll%d.npy" % rank), ll)
    np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([mean, slowest, r0, r1]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_agree(tmp_path):
    from oracle import oracle
    from spnb import synth
    from tests.util_models import write_query
    world = 2
    query = write_query(synth.config2(target_nodes=300), True, directory=str(tmp_path))
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(world, port, query, str(tmp_path)), nprocs=world, join=True)
    x = synth.config2_inputs(5000, 123)
    whole = oracle.evaluate(oracle.load_model(query), x, "log_f32_gpu")
    parts = [np.load(tmp_path / ("ll%d.npy" % r)) for r in range(world)]
    assert np.array_equal(np.concatenate(parts), whole)
    metas = [np.load(tmp_path / ("meta%d.npy" % r)) for r in range(world)]
    for m in metas:
        assert abs(m[0] - whole.astype(np.float64).mean()) < 1e-9
        assert m[1] == 10.0 + world - 1
