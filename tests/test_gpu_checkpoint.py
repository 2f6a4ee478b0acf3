"""Consolidated optimizer checkpoints with CUDA tensors: state saved from a distributed
``MuonWithAuxAdam`` on an NCCL process group (one rank is enough: the format does not depend on
the world size), loaded into a fresh optimizer over fresh parameter tensors, must continue
bit for bit like the optimizer it was taken from. The world-size change itself (2 -> 3 ranks)
is covered on gloo CPU ranks in test_host_logic.py."""
import copy

import pytest
import torch
import torch.distributed as dist

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_consolidated_checkpoint_round_trip_on_cuda(tmp_path):
    import muon_b200 as mb
    from muon_b200 import checkpoint as ck
    dist.init_process_group("nccl", init_method=f"file://{tmp_path}/pg", rank=0, world_size=1)
    try:
        g = torch.Generator().manual_seed(91)
        shapes = [(256, 512)] * 3 + [(512, 256)] * 2 + [(64, 32, 3, 3)]
        p0 = [torch.randn(s, generator=g) * 0.02 for s in shapes]
        gains0 = [torch.ones(256), torch.zeros(512)]
        grads = [[torch.randn(s, generator=g) for s in shapes] for _ in range(3)]
        gain_grads = [[torch.randn(p.shape, generator=g) * 0.1 for p in gains0] for _ in range(3)]

        def make(values, gains):
            ps = [torch.nn.Parameter(p.clone().to(DEV)) for p in values]
            gs = [torch.nn.Parameter(p.clone().to(DEV)) for p in gains]
            opt = mb.MuonWithAuxAdam([dict(params=ps, use_muon=True, lr=0.02, weight_decay=0.01),
                                      dict(params=gs, use_muon=False, lr=1e-3)])
            return ps, gs, opt

        def step(ps, gs, opt, k):
            for p, gr in zip(ps, grads[k]):
                p.grad = gr.clone().to(DEV)
            for p, gr in zip(gs, gain_grads[k]):
                p.grad = gr.clone().to(DEV)
            opt.step()

        ps, gs, opt = make(p0, gains0)
        step(ps, gs, opt, 0)
        step(ps, gs, opt, 1)
        state = copy.deepcopy(ck.consolidated_state_dict(opt))
        assert state["format"] == ck.FORMAT and state["saved_world_size"] == 1
        assert all(not t.is_cuda for t in state["groups"][0]["momentum"].values())  # portable: on CPU
        mid = [p.detach().cpu().clone() for p in ps], [p.detach().cpu().clone() for p in gs]
        step(ps, gs, opt, 2)

        qs, hs, opt2 = make(*mid)
        ck.load_consolidated_state_dict(opt2, state)
        for p in qs:
            assert opt2.state[p]["momentum_buffer"].is_cuda
        step(qs, hs, opt2, 2)
        torch.cuda.synchronize()
        for a, b in zip(ps + gs, qs + hs):
            assert torch.equal(a.detach(), b.detach())
        assert opt2.state[hs[0]]["step"] == 3
        assert mb.device_status() == 0
    finally:
        dist.destroy_process_group()
