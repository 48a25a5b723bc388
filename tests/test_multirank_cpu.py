"""World-size-2 `gloo` test of the head-sharded path's host logic on CPU: each rank generates only its own
head slice, computes it (with the oracle standing in for the GPU kernel), the slices are all-gathered in
rank-major order and laid out with the same contract dt_permute_gathered implements; the result must equal
the unsharded oracle.  Also: a rank that never joins makes the collective time out on the others instead
of hanging."""
import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "draw-things-community_b200"))
    from dtattn import sharding
    from oracle import sdpa_oracle as so
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = so.CONFIGS["flux_joint"].shrink(Sq=96, Sk=96, Hq=8, Hkv=4, D=32, dtype="f32", rope_hw=(8, 8, 32))
        q0, q1, kv0, kv1 = sharding.head_range(rank, world, cfg.Hq, cfg.Hkv)
        ql, kl, vl = so.make_inputs(cfg, heads=(q0, q1))
        assert ql.shape[2] == q1 - q0 and kl.shape[2] == kv1 - kv0
        out_chunks = []
        for r0, r1 in sharding.chunk_rows(cfg.Sq, 2, sms=1, tile=32):
            out_chunks.append(so.sdpa_explicit(ql[:, r0:r1], kl, vl, cfg.scale))
        ol = torch.cat(out_chunks, 1).contiguous()
        bufs = [torch.empty_like(ol) for _ in range(world)]
        dist.all_gather(bufs, ol)
        full = sharding.gathered_to_bshd(torch.stack(bufs, 0), world)
        # unsharded reference from the same per-head seeds
        qf, kf, vf = so.make_inputs(cfg, heads=(0, cfg.Hq))
        ref = so.sdpa_explicit(qf, kf, vf, cfg.scale)
        err = float((full - ref).abs().max())
        # output projection over the head slices: every rank multiplies its heads by its K-slice of the weight,
        # the partial products are summed and each rank keeps its block of rows (reduce-scatter)
        C = 24
        w_full = so.seeded_normal((C, cfg.Hq * cfg.D), 5)
        M = cfg.B * cfg.Sq
        rpr, owned = sharding.projection_rows(M, world, tile=32)
        partial = ol.reshape(M, -1) @ sharding.weight_slice(w_full, rank, world, cfg.Hq, cfg.D).t()
        padded = torch.zeros(world * rpr, C)
        padded[:M] = partial
        # gloo has no reduce_scatter: all-reduce and keep the owned block (same arithmetic)
        dist.all_reduce(padded)
        r0, r1 = owned[rank]
        want = ref.reshape(M, -1) @ w_full.t()
        err = max(err, float((padded[r0:r1] - want[r0:r1]).abs().max())) if r1 > r0 else err
        assert sum(b - a for a, b in owned) == M and rpr % 32 == 0
        q.put((rank, err))
    finally:
        dist.destroy_process_group()


def test_head_sharded_host_logic_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert [r for r, _ in res] == [0, 1]
    assert all(err < 5e-5 for _, err in res), res


def _lonely_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        q.put("joined")
    except Exception as e:  # the missing rank makes rendezvous give up
        q.put("timeout:" + type(e).__name__)


def test_missing_rank_times_out_instead_of_hanging():
    """Failure injected on the host: rank 1 of 2 never starts; rank 0's set-up ends with an error."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(0, 2, _free_port(), q))
    p.start()
    msg = q.get(timeout=90)
    p.join(30)
    assert msg.startswith("timeout:"), msg


def test_head_range_rules():
    sys.path.insert(0, os.path.join(ROOT, "draw-things-community_b200"))
    from dtattn import sharding
    assert sharding.head_range(3, 8, 40, 40) == (15, 20, 15, 20)         # Wan: 5 heads per GPU
    assert sharding.head_range(1, 2, 24, 24) == (12, 24, 12, 24)         # Flux on 2 GPUs
    assert sharding.head_range(1, 4, 32, 8) == (8, 16, 2, 4)             # GQA: whole groups per rank
    assert sharding.head_range(3, 8, 32, 4) == (12, 16, 1, 2)            # two ranks share one KV head
    with pytest.raises(ValueError):
        sharding.head_range(0, 7, 24, 24)
    assert sharding.chunk_rows(75600, 4, items_per_row_block=10) == [(0, 18944), (18944, 37888), (37888, 56832), (56832, 75600)]
    assert sharding.chunk_rows(75600, 4, items_per_row_block=5) == [(0, 37888), (37888, 75600)]   # Wan on 8 GPUs
    assert sharding.chunk_rows(100, 1) == [(0, 100)]


def _steps_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the ranks measured slightly different times for the same five steps: their own clocks would give 21 and 22
        # extra steps (1200 / 54.6 and 1200 / 54.4), i.e. one rank would enter a collective step the other never joins
        own_ms = 5 * (54.6 if rank == 0 else 54.4)
        own_count = int(min(400, 1200 / (own_ms / 5)))
        agreed_ms, n = bench.agreed_extra_steps(dist, torch.device("cpu"), own_ms, 5)
        q.put((rank, own_count, agreed_ms, n, bench.agreed_extra_steps(dist, torch.device("cpu"), 5000.0 + rank, 5)[1]))
    finally:
        dist.destroy_process_group()


def test_every_rank_runs_the_same_number_of_extra_steps():
    """bench.py keeps the GPUs loaded for the clock sampler with extra steps, and every step is a collective: the
    count comes from the all-reduced maximum so that all ranks agree on it."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_steps_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert res[0][1] != res[1][1], "the scenario must be one where the ranks' own clocks disagree"
    assert res[0][2] == res[1][2] == pytest.approx(5 * 54.6)
    assert res[0][3] == res[1][3] == 21
    assert res[0][4] == res[1][4] == 0  # long enough already: no extra steps
