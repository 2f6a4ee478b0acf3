"""Multi-GPU test of the distributed step (needs >= 2 GPUs; skipped otherwise): after `Muon.step`
every rank holds every updated parameter, bit-identical to what `SingleDeviceMuon` produces on one
GPU with the same kernels, for the three exchange transports (stores from the update kernel,
copy-engine pushes, NCCL all_gather)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")]

SHAPES = [(512, 1024)] * 6 + [(1024, 512)] * 4 + [(256, 256)] * 5 + [(64, 32, 3, 3)] * 3


def _problem(steps=2):
    g = torch.Generator().manual_seed(5)
    p0 = [torch.randn(s, generator=g) * 0.02 for s in SHAPES]
    grads = [[torch.randn(s, generator=g) for s in SHAPES] for _ in range(steps)]
    return p0, grads


def _worker(rank, world, tmpdir, exchange, dtype, policy="round_robin"):
    import datetime
    os.environ["MUON_B200_EXCHANGE"] = exchange
    os.environ["MUON_B200_OWNERSHIP"] = policy
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{tmpdir}/pg_{exchange}", rank=rank,
                            world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        import muon_b200 as mb
        dev = torch.device("cuda", rank)
        p0, grads = _problem()
        params = [torch.nn.Parameter(p.to(dtype).to(dev)) for p in p0]
        opt = mb.Muon(list(params), lr=0.02, weight_decay=0.01)
        for step_grads in grads:
            for p, gr in zip(params, step_grads):
                p.grad = gr.to(dtype).to(dev)
            opt.step()
        torch.cuda.synchronize()
        used_ce = any(v is not None for v in opt.__dict__.get("_muon_b200_exchange", {}).values())
        owned = [i for i, p in enumerate(opt.param_groups[0]["params"]) if len(opt.state[p]) > 0]
        torch.save(dict(params=[p.detach().cpu() for p in params], used_ce=used_ce, owned=owned,
                        status=mb.device_status()), f"{tmpdir}/out_{exchange}_{rank}.pt")
    finally:
        dist.destroy_process_group()


def _worker_overlap(rank, world, tmpdir, exchange):
    """Three steps of `MuonWithAuxAdam` driven by StepInBackward: updates and pushes start inside
    the backward pass, one parameter gets no gradient in the second step."""
    import datetime
    os.environ["MUON_B200_EXCHANGE"] = exchange
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{tmpdir}/pg_ov_{exchange}", rank=rank,
                            world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        import muon_b200 as mb
        dev = torch.device("cuda", rank)
        p0, _ = _problem()
        g = torch.Generator().manual_seed(6)
        weights = [[torch.randn(s, generator=g) for s in SHAPES] for _ in range(3)]
        params = [torch.nn.Parameter(p.to(dev)) for p in p0]
        gain = torch.nn.Parameter(torch.ones(64, device=dev))
        opt = mb.MuonWithAuxAdam([dict(params=list(params), use_muon=True, lr=0.02, weight_decay=0.01),
                                  dict(params=[gain], use_muon=False, lr=1e-3)])
        overlap = mb.StepInBackward(opt)
        for step, w in enumerate(weights):
            skip = 2 if step == 1 else -1
            for q in params + [gain]:
                q.grad = None
            loss = sum((p * wi.to(dev)).sum() for i, (p, wi) in enumerate(zip(params, w)) if i != skip) * gain.sum()
            loss.backward()
            overlap.step()
        torch.cuda.synchronize()
        overlap.remove()
        torch.save(dict(params=[p.detach().cpu() for p in params], gain=gain.detach().cpu(),
                        status=mb.device_status()), f"{tmpdir}/ov_{exchange}_{rank}.pt")
    finally:
        dist.destroy_process_group()


def _worker_sharded(rank, world, tmpdir, dtype):
    import datetime
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{tmpdir}/pg_sharded", rank=rank,
                            world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        import muon_b200 as mb
        from muon_b200.sharded import shard_rows
        dev = torch.device("cuda", rank)
        p0, grads = _problem()

        def piece(t):
            chunk, mine = shard_rows(t.shape[0], world, rank)
            return t[rank * chunk: rank * chunk + mine].to(dtype).to(dev).contiguous()

        params = [torch.nn.Parameter(piece(p)) for p in p0]
        opt = mb.ShardedMuon(list(params), lr=0.02, weight_decay=0.01, full_shapes=SHAPES)
        for step_grads in grads:
            for p, gr in zip(params, step_grads):
                p.grad = piece(gr)
            opt.step()
        torch.cuda.synchronize()
        torch.save(dict(local=[p.detach().cpu() for p in params], status=mb.device_status()),
                   f"{tmpdir}/sharded_{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_sharded_muon_matches_single_device(tmp_path, dtype):
    """Row-sharded parameters on 2 to 4 GPUs: every rank's rows equal those of SingleDeviceMuon on
    the full parameters, bit for bit (SHAPES includes row counts the world size does not divide)."""
    from muon_b200.sharded import shard_rows
    world = min(torch.cuda.device_count(), 3)
    mp.spawn(_worker_sharded, args=(world, str(tmp_path), dtype), nprocs=world, join=True)
    outs = [torch.load(f"{tmp_path}/sharded_{r}.pt", weights_only=False) for r in range(world)]

    import muon_b200 as mb
    p0, grads = _problem()
    ref = [torch.nn.Parameter(p.to(dtype).cuda()) for p in p0]
    opt = mb.SingleDeviceMuon(ref, lr=0.02, weight_decay=0.01)
    for step_grads in grads:
        for p, gr in zip(ref, step_grads):
            p.grad = gr.to(dtype).cuda()
        opt.step()
    for r, o in enumerate(outs):
        assert o["status"] == 0
        for i, (piece, full) in enumerate(zip(o["local"], ref)):
            chunk, mine = shard_rows(full.shape[0], world, r)
            assert torch.equal(piece, full.detach().cpu()[r * chunk: r * chunk + mine]), f"rank {r}, parameter {i}"


@pytest.mark.parametrize("exchange", ["st", "ce"])
def test_step_in_backward_on_a_distributed_optimizer(tmp_path, exchange):
    """Every rank ends with the parameters a single GPU gets from the plain optimizer step."""
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_worker_overlap, args=(world, str(tmp_path), exchange), nprocs=world, join=True)
    outs = [torch.load(f"{tmp_path}/ov_{exchange}_{r}.pt", weights_only=False) for r in range(world)]

    import muon_b200 as mb
    p0, _ = _problem()
    g = torch.Generator().manual_seed(6)
    weights = [[torch.randn(s, generator=g) for s in SHAPES] for _ in range(3)]
    params = [torch.nn.Parameter(p.cuda()) for p in p0]
    gain = torch.nn.Parameter(torch.ones(64, device="cuda"))
    opt = mb.SingleDeviceMuonWithAuxAdam([dict(params=list(params), use_muon=True, lr=0.02, weight_decay=0.01),
                                          dict(params=[gain], use_muon=False, lr=1e-3)])
    for step, w in enumerate(weights):
        skip = 2 if step == 1 else -1
        for q in params + [gain]:
            q.grad = None
        loss = sum((p * wi.cuda()).sum() for i, (p, wi) in enumerate(zip(params, w)) if i != skip) * gain.sum()
        loss.backward()
        opt.step()
    for r, o in enumerate(outs):
        assert o["status"] == 0
        assert torch.equal(o["gain"], gain.detach().cpu())
        for i, (p, q) in enumerate(zip(o["params"], params)):
            assert torch.equal(p, q.detach().cpu()), f"rank {r}, parameter {i} ({exchange})"


@pytest.mark.parametrize("exchange,policy", [("st", "round_robin"), ("ce", "round_robin"), ("nccl", "round_robin"),
                                             ("ce", "balanced"), ("nccl", "balanced")])
@pytest.mark.parametrize("dtype", [torch.bfloat16])
def test_distributed_step_matches_single_device(tmp_path, exchange, policy, dtype):
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_worker, args=(world, str(tmp_path), exchange, dtype, policy), nprocs=world, join=True)
    outs = [torch.load(f"{tmp_path}/out_{exchange}_{r}.pt", weights_only=False) for r in range(world)]

    import muon_b200 as mb
    p0, grads = _problem()
    ref = [torch.nn.Parameter(p.to(dtype).cuda()) for p in p0]
    opt = mb.SingleDeviceMuon(ref, lr=0.02, weight_decay=0.01)
    for step_grads in grads:
        for p, gr in zip(ref, step_grads):
            p.grad = gr.to(dtype).cuda()
        opt.step()
    ref = [p.detach().cpu() for p in ref]

    for r, o in enumerate(outs):
        assert o["status"] == 0
        assert o["used_ce"] == (exchange in ("ce", "st"))
        if policy == "round_robin":
            assert o["owned"] == list(range(r, len(SHAPES), world))  # muon.py:56-58
        else:
            from muon_b200 import ownership
            assert o["owned"] == ownership.owned_indices([torch.empty(s) for s in sorted(SHAPES, reverse=True)],
                                                         world, r, "balanced")
        for i, (p, q) in enumerate(zip(o["params"], ref)):
            assert torch.equal(p, q), f"rank {r}, parameter {i} {tuple(q.shape)} ({exchange})"
