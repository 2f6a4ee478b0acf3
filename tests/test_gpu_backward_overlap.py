"""StepInBackward on a GPU: updates enqueued from the backward pass on a side stream (hooks
running on the autograd thread, gradients kept alive with record_stream) must leave the parameters
bit-identical to optimizer.step() after the backward pass. The bookkeeping alone is covered on CPU
in test_host_logic.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_step_in_backward_matches_plain_step_on_gpu():
    import muon_b200 as mb
    shapes = [(512, 1024)] * 6 + [(1024, 256)] * 4 + [(256, 256)] * 3
    g = torch.Generator().manual_seed(13)
    p0 = [torch.randn(s, generator=g) * 0.02 for s in shapes]
    weights = [[torch.randn(s, generator=g).to(DEV) for s in shapes] for _ in range(3)]

    def make():
        ps = [torch.nn.Parameter(p.clone().to(DEV)) for p in p0]
        gain = torch.nn.Parameter(torch.ones(64, device=DEV))
        opt = mb.SingleDeviceMuonWithAuxAdam([dict(params=ps, use_muon=True, lr=0.02, weight_decay=0.01),
                                              dict(params=[gain], use_muon=False, lr=1e-3)])
        return ps, gain, opt

    def loss_of(ps, gain, w, skip):
        return sum((p * wi).sum() for i, (p, wi) in enumerate(zip(ps, w)) if i != skip) * gain.sum()

    ps_a, gain_a, opt_a = make()
    ps_b, gain_b, opt_b = make()
    overlap = mb.StepInBackward(opt_b)
    for step, w in enumerate(weights):
        skip = 1 if step == 1 else -1
        for q in ps_a + [gain_a] + ps_b + [gain_b]:
            q.grad = None
        loss_of(ps_a, gain_a, w, skip).backward()
        opt_a.step()
        loss_of(ps_b, gain_b, w, skip).backward()
        overlap.step()
        torch.cuda.synchronize()
        for x, y in zip(ps_a + [gain_a], ps_b + [gain_b]):
            assert torch.equal(x, y)
    overlap.remove()
    assert mb.device_status() == 0
