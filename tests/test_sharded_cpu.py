"""CPU tests of the multi-GPU host logic: the row partition, and the in-place all-gather of C run
as real torch.distributed ranks over gloo (world sizes 2 and 3).  The slab of each rank is filled
by the CPU oracle standing in for the GEMM launch, so the assembled C can be checked exactly."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_partition_rows_covers_every_row_once():
    from cudaintro_b200.sharded import partition_rows

    for M in (1, 7, 8, 1000, 8192):
        for world in (1, 2, 3, 4, 8):
            parts = [partition_rows(M, world, r) for r in range(world)]
            covered = []
            for p in parts:
                assert p.slot_rows == -(-M // world) and p.padded_rows >= M
                assert p.row0 == min(M, p.rank * p.slot_rows)
                covered.extend(range(p.row0, p.row0 + p.rows))
            assert covered == list(range(M))
    with pytest.raises(ValueError):
        partition_rows(8, 2, 2)
    with pytest.raises(ValueError):
        partition_rows(0, 2, 0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, N, K, fail_rank, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import oracle as O
    from cudaintro_b200.sharded import ShardedGemm

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)  # every rank draws the same full problem, then keeps its rows
        a = rng.integers(-127, 128, (M, K)).astype(np.int8)
        b = rng.integers(-127, 128, (K, N)).astype(np.int8)
        sg = ShardedGemm(M, N, torch.int32, "cpu")
        p = sg.part

        def compute(c_slab):
            rows = np.arange(p.row0, p.row0 + p.rows, dtype=np.int64)
            c_slab.copy_(torch.from_numpy(O.gemm_i8_i32(a, b, M, N, K, O.ROW_MAJOR, rows)))

        if rank == fail_rank:
            raise RuntimeError("injected failure before the step")
        sg.step(compute)
        want = a.astype(np.int64) @ b.astype(np.int64)
        ok = np.array_equal(sg.result().numpy(), want)
        open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,M", [(2, 64), (2, 37), (3, 10)])
def test_all_gather_assembles_c_on_every_rank(tmp_path, world, M):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(world, port, M, 24, 40, -1, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def test_a_failing_rank_surfaces_as_an_error(tmp_path):
    """A rank that raises before its step must fail the job (the others must not hang for ever):
    the spawn context reports the exception of the failing rank."""
    import torch.multiprocessing as mp

    port = _free_port()
    with pytest.raises(Exception):
        # whichever rank's error arrives first is reported: the injected one, or the surviving
        # rank's broken connection inside the all-gather
        mp.spawn(_worker, args=(2, port, 16, 8, 8, 1, str(tmp_path)), nprocs=2, join=True)
    assert not (tmp_path / "rank1.txt").exists()
