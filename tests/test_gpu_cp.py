"""Context-parallel mixer on GPUs: equals the unsharded mixer and the CPU oracle.

With one GPU the group has a single rank (the collectives are trivial but the whole record ->
merge -> gather -> combine -> scatter chain and its backward run on the device); with two or more
GPUs the token axis is really sharded over NCCL ranks.
"""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_out, exchange="nccl"):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import flare_b200 as fb
        from flare_b200.parallel import PeerExchange, RecordExchange, flare_mixer_context_parallel, shard_bounds
        from oracle import flare_oracle as O
        ex = PeerExchange() if exchange == "peer" else RecordExchange()
        # every rank runs both rounds whatever the first one finds (the ranks must make the same sequence
        # of exchanges); the findings are reported together afterwards
        problems = []
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            B, H, N, M, D, scale = 2, 4, 1500, 64, 32, 0.9
            q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=dtype, seed=7)
            n0, n1 = shard_bounds(N, world, rank, multiple=128)
            qd = q.to(dev).requires_grad_(True)
            kd = k[:, :, n0:n1].contiguous().to(dev).requires_grad_(True)
            vd = v[:, :, n0:n1].contiguous().to(dev).requires_grad_(True)
            y = flare_mixer_context_parallel(qd, kd, vd, scale, exchange=ex)
            y.backward(dy[:, :, n0:n1].contiguous().to(dev))
            torch.cuda.synchronize()
            qf, kf, vf, dyf = (t.float() for t in (q, k, v, dy))
            y_ref = O.mixer_sdpa(qf, kf, vf, scale)
            dq_ref, dk_ref, dv_ref = O.mixer_bwd_closed_form(qf, kf, vf, dyf, scale)
            errs = dict(y=O.rel_l2(y.float().cpu(), y_ref[:, :, n0:n1]), dq=O.rel_l2(qd.grad.float().cpu(), dq_ref),
                        dk=O.rel_l2(kd.grad.float().cpu(), dk_ref[:, :, n0:n1]),
                        dv=O.rel_l2(vd.grad.float().cpu(), dv_ref[:, :, n0:n1]))
            bad = {n: e for n, e in errs.items() if not e <= tol}
            if bad:
                problems.append((str(dtype), bad))
        status = fb.device_status()
        if status:
            problems.append(("device status", status))
        assert not problems, problems
        q_out.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q_out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def _run(world, exchange="nccl"):
    import __graft_entry__
    __graft_entry__.build()
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q_out, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = [q_out.get(timeout=300) for _ in procs]
    finally:
        for p in procs:
            p.join(timeout=60)
        for p in procs:                        # a rank that is still alive is waiting for one that is gone
            if p.is_alive():
                p.terminate()
    assert all(msg == "ok" for _, msg in results), results


def test_single_rank_group(cuda_dev):
    _run(1)


def test_two_ranks_shard_the_tokens(cuda_dev):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2)


def test_two_ranks_peer_memory_exchange(cuda_dev):
    """The exchanges fused into the combine / reduce kernels over symmetric memory (plain peer loads)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, "peer")


def _graph_worker(rank, world, port, q_out, exchange):
    """The step recorded in a CUDA graph (two steps per graph) and replayed gives, bit for bit, what eager
    launches give, replay after replay, also with eager steps in between."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import flare_b200 as fb
        from flare_b200.parallel import GraphedStep, PeerExchange, flare_mixer_context_parallel, shard_bounds
        from oracle import flare_oracle as O
        B, H, N, M, D = 1, 4, 4096, 128, 32
        q, k, v, dy = O.make_inputs(B, H, N, M, D, dtype=torch.bfloat16, seed=11)
        n0, n1 = shard_bounds(N, world, rank, multiple=128)
        qd = q.to(dev).requires_grad_(True)
        kd = k[:, :, n0:n1].contiguous().to(dev).requires_grad_(True)
        vd = v[:, :, n0:n1].contiguous().to(dev).requires_grad_(True)
        dyd = dy[:, :, n0:n1].contiguous().to(dev)
        ex_eager, ex_graph = PeerExchange(), PeerExchange()
        ex_graph.prepare_mixer(B, H, M, D, dev)

        def step(ex):
            qd.grad = kd.grad = vd.grad = None
            y = flare_mixer_context_parallel(qd, kd, vd, 1.0, exchange=ex)
            y.backward(dyd)
            return y

        # (nothing of the eager step's autograd graph may stay alive into the recording: its gradient
        # accumulators belong to the stream they were made on)
        y0 = step(ex_eager).detach()
        want = [t.clone() for t in (y0, qd.grad, kd.grad, vd.grad)]
        gs = GraphedStep(lambda: step(ex_graph))
        problems = []
        for it in range(3):
            y = gs.replay()
            torch.cuda.synchronize()
            got = (y.detach(), qd.grad, kd.grad, vd.grad)
            for name, a, b_ in zip(("y", "dq", "dk", "dv"), got, want):
                if not torch.equal(a, b_):
                    problems.append((it, name, O.rel_l2(a.float().cpu(), b_.float().cpu())))
            if it == 0:
                step(ex_eager).detach_()                    # eager steps between replays use their own buffers
        if fb.device_status():
            problems.append("device status")
        assert not problems, problems
        q_out.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q_out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_step_replayed_from_a_cuda_graph(cuda_dev):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import __graft_entry__
    __graft_entry__.build()
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_graph_worker, args=(r, 2, port, q_out, "peer")) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = [q_out.get(timeout=300) for _ in procs]
    finally:
        for p in procs:
            p.join(timeout=60)
        for p in procs:
            if p.is_alive():
                p.terminate()
    assert all(msg == "ok" for _, msg in results), results


def test_peer_barrier_gives_up_when_the_peer_never_arrives(cuda_dev):
    """One rank alone in a group described as two: the flag of the absent peer never changes, the barrier
    kernel runs out of its bounded wait, records bit 1 in the status word and returns; the context stays
    usable.  (Host-made failure: no kernel traps, nothing waits without a limit.)"""
    import ctypes as C
    import __graft_entry__
    __graft_entry__.build()
    import flare_b200 as fb
    from flare_b200 import _cabi
    dev = cuda_dev
    fb.device_status()                                     # clear
    flags = torch.zeros(2, 3, dtype=torch.int32, device=dev)       # "rank 0" and a peer whose array nobody writes (world + 1 slots each)
    buf = torch.zeros(16, device=dev)
    flag_ptrs = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64, device=dev)
    buf_ptrs = torch.tensor([buf.data_ptr(), buf.data_ptr()], dtype=torch.int64, device=dev)
    g = _cabi.FlarePeers()
    g.rank, g.world, g.epoch = 0, 2, 1
    g.bufs, g.mine, g.flags = buf_ptrs.data_ptr(), buf.data_ptr(), flag_ptrs.data_ptr()
    _cabi.check(_cabi.lib.flare_peer_barrier(C.byref(g), None), "flare_peer_barrier")
    torch.cuda.synchronize()
    assert fb.device_status() & 2
    assert flags[1, 0].item() == 1                         # the signal to the peer was sent
    assert fb.device_status() == 0                         # cleared, and the device still answers
    assert torch.ones(4, device=dev).sum().item() == 4.0


def _model_worker(rank, world, port, q_out, exchange):
    """A FLAREModel whose points are sharded over the ranks, trained one step with the context-parallel glue,
    against the same model on one GPU with all the points (built from the ranks' shards)."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import flare_b200 as fb
        from oracle import flare_oracle as O
        torch.manual_seed(0)
        kw = dict(in_dim=5, out_dim=2, channel_dim=64, num_blocks=2, num_heads=2, num_latents=64)
        model = fb.FLAREModel(**kw).to(dev)
        ref = fb.FLAREModel(**kw).to(dev)
        ref.load_state_dict(model.state_dict())
        cp = fb.ContextParallel(exchange=exchange)
        fb.enable_context_parallel(model, cp, checkpoint_blocks=True)
        N = 3000
        shards = [fb.ShardedPointCloud(N, 2, 2, r, world, seed=11, device=dev, multiple=128) for r in range(world)]
        x, t = shards[rank].sample(0)
        opt = torch.optim.SGD(model.parameters(), lr=0.0)             # keeps the weights: gradients are compared
        model.train()
        n_global = cp.global_count(t.numel(), dev)
        loss_local = (model(x) - t).square().sum() / n_global
        loss_local.backward()
        cp.reduce_gradients(model)
        xs, ts = zip(*(sh.sample(0) for sh in shards))                # every rank rebuilds the unsharded sample
        loss_ref = torch.nn.functional.mse_loss(ref(torch.cat(xs, 1)), torch.cat(ts, 1))
        loss_ref.backward()
        loss = loss_local.detach().clone()
        dist.all_reduce(loss)
        problems = []
        if abs(loss.item() - loss_ref.item()) > 1e-5 * abs(loss_ref.item()):
            problems.append(("loss", loss.item(), loss_ref.item()))
        for (n, a), b in zip(model.named_parameters(), ref.parameters()):
            e = O.rel_l2(a.grad.cpu(), b.grad.cpu())
            if e > 2e-4:
                problems.append((n, e))
        # and the step function end to end under bf16 autocast
        opt2 = torch.optim.SGD(model.parameters(), lr=1e-3)
        l2 = fb.cp_train_step(model, opt2, x, t, cp, autocast_dtype=torch.bfloat16, clip_grad_norm=1.0)
        if not torch.isfinite(l2) or abs(l2.item() - loss_ref.item()) > 5e-2 * abs(loss_ref.item()):
            problems.append(("autocast step loss", l2.item(), loss_ref.item()))
        if fb.device_status():
            problems.append("device status")
        assert not problems, problems
        q_out.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        q_out.put((rank, repr(e) + traceback.format_exc()[-600:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["collective", "peer"])
def test_sharded_model_step_equals_the_unsharded_one(cuda_dev, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import __graft_entry__
    __graft_entry__.build()
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_model_worker, args=(r, 2, port, q_out, exchange)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = [q_out.get(timeout=300) for _ in procs]
    finally:
        for p in procs:
            p.join(timeout=60)
        for p in procs:
            if p.is_alive():
                p.terminate()
    assert all(msg == "ok" for _, msg in results), results
