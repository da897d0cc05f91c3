"""N > 1 path of the benchmark protocol on CPU: two gloo ranks, barrier + max over ranks."""
import os
import socket

import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world_size, port, out):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world_size),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from dyninfer_b200 import replicas
    assert replicas.world() == (rank, rank, world_size)
    replicas.init("gloo")
    replicas.barrier()
    ms = [10.0, 40.0][rank]                       # rank 1 is the slow one
    e2e = [7.0, 3.0][rank]
    got = replicas.max_over_ranks([ms, e2e])
    rate = replicas.whole_job_rate(256, got[0], world_size)
    out.put((rank, got, rate))
    replicas.shutdown()


def test_two_gloo_ranks_agree_on_the_slowest_time():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, got, rate in results:
        assert got == [40.0, 7.0]                 # element-wise maximum, identical on every rank
        assert abs(rate - 2 * 256 / 0.040) < 1e-9


def test_single_process_is_identity():
    from dyninfer_b200 import replicas
    assert replicas.max_over_ranks([1.5, 2.5]) == [1.5, 2.5]
    assert replicas.whole_job_rate(100, 50.0, 1) == 2000.0
    replicas.barrier()


def test_bench_lays_its_timed_steps_out_as_generations():
    """The bench times K steps as decode phases of the named configuration (32 greedy steps after the
    16-token prompt), the way the reference's perf runner repeats its iterations."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import bench
    assert bench.GEN_STEPS == 32 and bench.PROMPT_LEN == 16
    assert bench.phases(256) == [32] * 8
    assert bench.phases(2) == [2] and bench.phases(32) == [32]
    assert bench.phases(40) == [32, 8] and bench.phases(0) == []
    for k in (1, 5, 31, 33, 100, 257):
        p = bench.phases(k)
        assert sum(p) == k and all(0 < n <= 32 for n in p)
