"""Head-sharded attention on 2 GPUs (skipped on a single-GPU box): each rank computes its heads, the output
is exchanged with NCCL and laid out as [B,Sq,H,D]; every rank must hold the same full result as the oracle."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "draw-things-community_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import dtattn
    from dtattn import sharding
    from oracle import sdpa_oracle as so
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        def bcast(b):
            obj = [b]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        comm = dtattn.HeadShardedComm(rank, world, bcast, timeout_ms=60000)
        errs = []
        keep = []
        for (B, S, H, D, chunks) in [(1, 1000, 8, 128, 3), (2, 300, 4, 64, 1)]:
            cfg = so.AttnConfig("t", B, S, S, H, H, D, "bf16", 7)
            q0, q1, kv0, kv1 = sharding.head_range(rank, world, H, H)
            ql, kl, vl = so.make_inputs(cfg, heads=(q0, q1))
            o_full = torch.zeros((B, S, H, D), dtype=torch.bfloat16, device=dev)
            comm.forward(ql.to(dev), kl.to(dev), vl.to(dev), cfg.scale, o_full, chunks=chunks)
            torch.cuda.synchronize()
            qf, kf, vf = so.make_inputs(cfg, heads=(0, H))
            ref = so.sdpa_explicit(qf, kf, vf, cfg.scale)
            errs.append(so.error_stats(o_full.float().cpu(), ref))
            # fused mode: the same call on a registered buffer stores tiles straight into both ranks' buffers
            o_fused = torch.zeros((B, S, H, D), dtype=torch.bfloat16, device=dev)
            comm.register_output(o_fused)
            for _ in range(2):
                comm.forward(ql.to(dev), kl.to(dev), vl.to(dev), cfg.scale, o_fused, chunks=chunks)
            torch.cuda.synchronize()
            dist.barrier()
            errs.append(so.error_stats(o_fused.float().cpu(), ref))
            assert torch.equal(o_fused, o_full), "fused and gathered results must be bitwise equal"
            keep.append(o_fused)
            # attention + output projection, row-parallel over the head slices, reduce-scattered over the rows
            C = 512 if D == 128 else 200
            w_full = (so.seeded_normal((C, H * D), 77) * (H * D) ** -0.5 * 2.0).to(torch.bfloat16)
            bias = so.seeded_normal((C,), 78).to(torch.bfloat16)
            w_local = w_full[:, q0 * D:q1 * D].contiguous().to(dev)
            _, recv_bytes, rpr = comm.projected_sizes(ql.to(dev), kl.to(dev), vl.to(dev), cfg.scale, C)
            recv = torch.zeros(recv_bytes // 4, dtype=torch.float32, device=dev)
            comm.register_output(recv)
            rows = torch.full((rpr, C), float("nan"), dtype=torch.bfloat16, device=dev)
            for _ in range(3):  # both halves of the receive buffer, and the first one again
                comm.forward_projected(ql.to(dev), kl.to(dev), vl.to(dev), cfg.scale, w_local, bias.to(dev), recv, rows)
            torch.cuda.synchronize()
            dist.barrier()
            attn = ref.to(torch.bfloat16).reshape(B * S, H * D).double()
            want = (attn @ w_full.double().t() + bias.double()).float()[rank * rpr:(rank + 1) * rpr]
            got = rows[:want.shape[0]].float().cpu()
            assert torch.isfinite(got).all()
            mx, mean = so.error_stats(got, want)
            # stated tolerance plus the bf16 rounding of an output of this magnitude (bias makes |out| ~ 1..4)
            assert mx <= 2e-3 + 2 * 2.0 ** -8 * float(want.abs().max()), ("projected max-abs", rank, mx)
            assert mean <= 2e-4 + 2.0 ** -8 * float(want.abs().mean()), ("projected mean-abs", rank, mean)
            keep.append(recv)
        # the same registered buffer in consecutive calls with DIFFERENT inputs, one rank reading its result late:
        # a rank that runs ahead must not store the next call's tiles into the slow rank's buffer before that rank's
        # stream has read the previous result (the library puts a rendezvous in front of such a call)
        B, S, H, D = 1, 1024, 8, 128
        q0, q1, kv0, kv1 = sharding.head_range(rank, world, H, H)
        o_same = torch.zeros((B, S, H, D), dtype=torch.bfloat16, device=dev)
        comm.register_output(o_same)
        steps, snaps, wants = 4, [], []
        step_inputs = []
        for st in range(steps):
            cfg = so.AttnConfig("t", B, S, S, H, H, D, "bf16", 100 + st)
            step_inputs.append((cfg, [t.to(dev) for t in so.make_inputs(cfg, heads=(q0, q1))]))
        for st in range(steps):  # expected results through the all-gather path into separate buffers
            cfg, (ql, kl, vl) = step_inputs[st]
            want = torch.zeros_like(o_same)
            comm.forward(ql, kl, vl, cfg.scale, want, chunks=1)
            wants.append(want)
        torch.cuda.synchronize()
        dist.barrier()
        for st in range(steps):
            cfg, (ql, kl, vl) = step_inputs[st]
            comm.forward(ql, kl, vl, cfg.scale, o_same, chunks=1)
            if rank == 1:
                torch.cuda._sleep(int(3e6))  # a slow consumer in front of the read, in stream order (about 2 ms)
            snaps.append(o_same.clone())
        torch.cuda.synchronize()
        dist.barrier()
        for st in range(steps):
            assert torch.equal(snaps[st], wants[st]), f"step {st}: the late reader saw another step's tiles"
        # buffers of different sizes on the two ranks are refused on every rank
        odd = torch.zeros(4096 * (rank + 1), dtype=torch.uint8, device=dev)
        try:
            comm.register_output(odd)
            mismatch = "accepted"
        except dtattn.DtError as e:
            mismatch = e.status
        assert mismatch == dtattn.DT_BAD_ARG, mismatch
        comm.close()
        q.put((rank, errs, dtattn.device_status()))
    finally:
        dist.destroy_process_group()


def test_head_sharded_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
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
    for rank, errs, status in res:
        assert status == 0
        for mx, mean in errs:
            assert mx <= 2e-3 + 2 ** -8 and mean <= 4e-4, (rank, errs)
