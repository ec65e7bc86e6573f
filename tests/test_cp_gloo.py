"""Context-parallel plumbing among CPU ranks (gloo, world_size 2 and 3).

The local arithmetic comes from the CPU oracle; what is under test is the
exchange: record layout, rank order of the gather, the combine across ranks and
the gradient reductions giving the unsharded result.
"""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from oracle import flare_oracle as O  # noqa: E402

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import __graft_entry__
        __graft_entry__.build()
        from flare_b200.parallel import RecordExchange, shard_bounds
        from oracle import flare_oracle as O

        B, H, N, M, D, scale = 2, 2, 203, 12, 8, 0.8
        q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=torch.float64, seed=3)
        n0, n1 = shard_bounds(N, world, rank, multiple=8)
        ex = RecordExchange()
        # forward: local record -> gather -> combine
        m, l, acc = O.gather_partials(q, k, v, scale, [(n0, n1)])
        rec = torch.cat([acc[0], m[0][..., None], l[0][..., None]], dim=-1)      # [B,H,M,D+2]
        allrec = ex.gather_records(rec)
        assert allrec.shape == (world, B, H, M, D + 2)
        assert torch.equal(allrec[rank], rec)
        z, L = O.lse_combine(allrec[..., D], allrec[..., D + 1], allrec[..., :D])
        z_ref, L_ref = O.gather(q, k, v, scale)
        assert O.rel_l2(z, z_ref) < 1e-12 and O.rel_l2(L, L_ref) < 1e-12
        y_loc, C_loc = O.scatter(q, k[:, :, n0:n1], z, scale)
        y_ref = O.mixer_explicit(q, k, v, scale)
        assert O.rel_l2(y_loc, y_ref[:, :, n0:n1]) < 1e-12
        # backward: dZ partial summed over ranks, then local token grads and summed dQ
        A_loc = torch.exp(scale * (q[None] @ k[:, :, n0:n1].transpose(-2, -1)) - C_loc[..., None, :])
        dz = ex.sum_(A_loc @ dy[:, :, n0:n1])
        dq_ref, dk_ref, dv_ref = O.mixer_bwd_closed_form(q, k, v, dy, scale)
        kk, vv, gg = k[:, :, n0:n1], v[:, :, n0:n1], dy[:, :, n0:n1]
        S = scale * (q[None] @ kk.transpose(-2, -1))
        P = torch.exp(S - L[..., None])
        dS = P * (dz @ vv.transpose(-2, -1) - (dz * z).sum(-1)[..., None]) \
            + A_loc * (z @ gg.transpose(-2, -1) - (gg * y_loc).sum(-1)[..., None, :])
        dq = ex.sum_((scale * (dS @ kk)).sum(0))
        assert O.rel_l2(dq, dq_ref) < 1e-12
        assert O.rel_l2(scale * dS.transpose(-2, -1) @ q[None], dk_ref[:, :, n0:n1]) < 1e-12
        assert O.rel_l2(P.transpose(-2, -1) @ dz, dv_ref[:, :, n0:n1]) < 1e-12
        q_out.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q_out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_record_exchange_among_cpu_ranks(world):
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def test_shard_bounds_cover_all_tokens():
    from flare_b200.parallel import shard_bounds
    for n, w, mult in [(1000, 8, 128), (1 << 20, 8, 128), (7, 4, 1), (203, 3, 8)]:
        spans = [shard_bounds(n, w, r, mult) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a0 <= a1


def _leaver(rank, world, port, q_out):
    """Rank 1 leaves between two steps; rank 0 must learn of it from its next exchange (an error after the
    short group timeout), not wait forever."""
    import datetime
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        import __graft_entry__
        __graft_entry__.build()
        from flare_b200.parallel import RecordExchange
        ex = RecordExchange()
        rec = torch.full((1, 1, 2, 4), float(rank))
        allrec = ex.gather_records(rec)                      # step 1: everybody is there
        assert allrec.shape[0] == world and allrec[1].eq(1.0).all()
        if rank == 1:
            q_out.put((rank, "left"))
            q_out.close()
            q_out.join_thread()                              # the message is on its way before the process goes
            os._exit(0)                                      # between steps, nothing in flight
        try:
            ex.gather_records(rec)                           # step 2: the peer is gone
            q_out.put((rank, "no error"))
        except Exception as e:
            q_out.put((rank, "detected"))
    except Exception as e:  # pragma: no cover
        q_out.put((rank, repr(e)))


def test_a_rank_that_leaves_between_steps_is_detected():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = dict(q_out.get(timeout=120) for _ in procs)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    assert results == {1: "left", 0: "detected"}, results


def _glue_worker(rank, world, port, q_out):
    """The training glue without the mixer: sharded synthetic data, the global-mean loss and the group-wide
    gradient sum give, on a pointwise model with replicated weights, the gradient of the unsharded loss."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import __graft_entry__
        __graft_entry__.build()
        from flare_b200.cp_train import ContextParallel, ShardedPointCloud
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(5, 8), torch.nn.Tanh(), torch.nn.Linear(8, 2)).double()
        cp = ContextParallel(bucket_bytes=256)                       # several buckets even for this tiny model
        N = 1000
        shards = [ShardedPointCloud(N, 2, 2, r, world, seed=3, device="cpu", dtype=torch.float64, multiple=8) for r in range(world)]
        assert shards[0].n0 == 0 and shards[-1].n1 == N and all(a.n1 == b.n0 for a, b in zip(shards, shards[1:]))
        x, t = shards[rank].sample(0)
        n_global = cp.global_count(t.numel(), "cpu")
        assert n_global == N * 2
        loss_local = (model(x) - t).square().sum() / n_global
        loss_local.backward()
        cp.reduce_gradients(model)
        # the unsharded problem, rebuilt from every rank's shard
        xs, ts = zip(*(sh.sample(0) for sh in shards))
        ref = torch.nn.Sequential(torch.nn.Linear(5, 8), torch.nn.Tanh(), torch.nn.Linear(8, 2)).double()
        ref.load_state_dict(model.state_dict())
        torch.nn.functional.mse_loss(ref(torch.cat(xs, 1)), torch.cat(ts, 1)).backward()
        for a, b in zip(model.parameters(), ref.parameters()):
            assert O.rel_l2(a.grad, b.grad) < 1e-12
        q_out.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q_out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_training_glue_among_cpu_ranks():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_glue_worker, args=(r, 3, port, q_out)) for r in range(3)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results
