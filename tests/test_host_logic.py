"""CPU tests of the host side: the C-ABI library's symbol table, the drop-in API surface
(constructor behaviour recorded from the real reference in tests/golden/api.pt), the engine's
grouping helpers, and the distributed ownership/windowing logic on gloo CPU ranks with a
stand-in backend (the CUDA kernels need a GPU; the stand-in is test-only and uses the oracle)."""
import os
import re

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import muon_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ------------------------------------------------------------------ library / header
def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "muon_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(muon_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import muon_b200._lib as L
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(L.lib, n), f"{n} declared in include/muon_b200.h but not exported"
    assert set(names) == set(L.PROTOTYPES), "ctypes prototypes and header disagree"
    assert L.lib.muon_b200_version() >= 100
    assert L.lib.muon_b200_last_error() is not None


def test_public_header_is_plain_c(tmp_path):
    """include/muon_b200.h is the drop-in boundary: it must compile as C99 and as C++ on its own
    (plain pointers and sizes, no torch or CUDA types), and a C program that only includes it and
    takes the address of an entry point must link against the library."""
    import shutil
    import subprocess
    header = os.path.join(ROOT, "include", "muon_b200.h")
    gcc, gxx = shutil.which("gcc"), shutil.which("g++")
    if not gcc or not gxx:
        pytest.skip("no host compiler")
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c", header], check=True)
    subprocess.run([gxx, "-std=c++11", "-fsyntax-only", "-x", "c++", header], check=True)
    src = tmp_path / "use.c"
    src.write_text('#include "muon_b200.h"\n#include <stdio.h>\n'
                   'int main(void) { muon_b200_ns_layout l; int rc = muon_b200_ns_workspace_layout(2, 64, 96, &l);\n'
                   '  printf("%d %lld %d\\n", rc, (long long)l.total_bytes, muon_b200_version()); return rc; }\n')
    exe = tmp_path / "use"
    libdir = os.path.join(ROOT, "muon_b200")
    subprocess.run([gcc, "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-lmuon_b200", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out[0] == "0" and int(out[1]) > 0 and int(out[2]) >= 100


def test_workspace_layout_is_host_only_and_consistent():
    import muon_b200._lib as L
    lay = L.ns_layout(3, 200, 330)
    assert lay.ldn == 336 and lay.ldm == 200 and lay.x_bs == 200 * 336 and lay.a_bs == 200 * 200
    offs = [lay.x_offset_bytes, lay.c_offset_bytes, lay.a_offset_bytes, lay.b_offset_bytes,
            lay.partials_offset_bytes, lay.total_bytes]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs)
    assert lay.c_offset_bytes - lay.x_offset_bytes >= 3 * lay.x_bs * 2
    with pytest.raises(L.MuonB200Error):
        L.ns_layout(1, 300, 200)  # m must be the short side
    with pytest.raises(L.MuonB200Error):
        L.ns_layout(0, 8, 8)


def test_argument_errors_are_reported_without_a_gpu():
    import ctypes
    import muon_b200._lib as L
    rc = L.lib.muon_b200_ns_run(None, 1, 8, 8, 0, 0, None, 1e-7, None, None)
    assert rc == -1 and b"workspace" in L.lib.muon_b200_last_error()
    rc = L.lib.muon_b200_ns_run(ctypes.c_void_p(256 * 10), 1, 8, 8, 7, 0, None, 1e-7, None, None)
    assert rc == -1 and b"mode" in L.lib.muon_b200_last_error()
    rc = L.lib.muon_b200_ns_run(ctypes.c_void_p(8), 1, 8, 8, 0, 0, None, 1e-7, None, None)
    assert rc == -2
    one = L.ptr_array([16])
    rc = L.lib.muon_b200_prologue(one, one, 1, 8, 8, 5, 0.95, 1, ctypes.c_void_p(256), 8, 64, 0, None)
    assert rc == -1 and b"dtype" in L.lib.muon_b200_last_error()


def test_split_along_k_is_sized_without_a_gpu():
    """Scratch of the functional line 1 / Newton-Schulz for a Gram product that is split along K: a
    function of the sizes alone (no device needed). One or a few small matrices with a long K are
    split; launches that fill the GPU, and short contractions, are not."""
    import muon_b200._lib as L
    tile_bytes = 256 * 256 * 4
    one = L.lib.muon_b200_ns_line1_scratch_bytes(1, 768, 3072)
    assert one > 0 and one % (6 * tile_bytes) == 0          # 6 lower-triangle tiles x slices
    assert 3 <= one // (6 * tile_bytes) <= 16
    assert L.lib.muon_b200_ns_line1_scratch_bytes(1, 1024, 8192) > 0
    assert L.lib.muon_b200_ns_line1_scratch_bytes(12, 768, 3072) == 0    # 72 tiles: one wave of CTA pairs
    assert L.lib.muon_b200_ns_line1_scratch_bytes(1, 4096, 14336) == 0
    assert L.lib.muon_b200_ns_line1_scratch_bytes(1, 768, 512) == 0      # too few k-blocks per slice
    assert L.lib.muon_b200_ns_line1_scratch_bytes(1, 100, 2050) > 0      # one single-CTA tile
    # the functional Newton-Schulz includes that room, the optimizer's workspace does not
    assert L.lib.muon_b200_zeropower_scratch_bytes(1, 768, 3072, L.NS_AOL4) >= one
    lay = L.ns_layout(1, 768, 3072, L.NS_AOL4)
    assert lay.total_bytes < L.lib.muon_b200_zeropower_scratch_bytes(1, 768, 3072, L.NS_AOL4) + 768 * 3072 * 2


def test_ramped_launch_groups():
    """Slowly growing groups at the start of a set whose gradients are still arriving (a group may
    hold one more than a quarter of everything before it); every parameter stays in exactly one
    group and the largest planned group is never exceeded."""
    from muon_b200.engine import ramped_sizes
    assert ramped_sizes([13, 13, 13, 13, 12]) == [1, 1, 1, 1, 2, 2, 3, 3, 4, 5, 6, 8, 10, 12, 5]
    assert ramped_sizes([1]) == [1] and ramped_sizes([8]) == [1, 1, 1, 1, 2, 2]
    for planned in ([5], [2, 2], [7, 6], [40, 40, 3], [13] * 5):
        got = ramped_sizes(planned)
        assert sum(got) == sum(planned) and max(got) <= max(planned) and got[0] == 1
        for i in range(1, len(got)):
            assert got[i] <= 1 + sum(got[:i]) // 4 or got[i] <= max(planned)


def test_no_cpu_fallback():
    import muon_b200
    p = torch.nn.Parameter(torch.randn(8, 16))
    p.grad = torch.randn(8, 16)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        muon_b200.SingleDeviceMuon([p]).step()
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        muon_b200.zeropower_via_newtonschulz5(torch.randn(8, 16))
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        muon_b200.adam_update(torch.randn(4), torch.zeros(4), torch.zeros(4), 1, (0.9, 0.95), 1e-10)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        muon_b200.mark_grad_ready(p)  # readiness marks are CUDA events: CPU gradients have none
    with pytest.raises(ValueError, match="no gradient"):
        muon_b200.mark_grad_ready(torch.nn.Parameter(torch.randn(4, 4)))  # nothing would consume the mark
    from muon_b200 import engine
    assert not engine._grad_ready


# ------------------------------------------------------------------------ API surface
def test_constructors_behave_like_the_reference(golden):
    import muon_b200 as mb
    api = golden("api")
    shapes = [(32, 64), (64, 32), (64, 64), (16, 64), (64, 32)]
    ps = [torch.nn.Parameter(torch.zeros(s)) for s in shapes]
    m = mb.Muon(list(ps))
    assert [tuple(p.shape) for p in m.param_groups[0]["params"]] == api["muon_sorted_shapes"]
    assert {k: m.param_groups[0][k] for k in ("lr", "momentum", "weight_decay")} == api["muon_defaults"]
    assert set(api["muon_group_keys"]) <= set(m.param_groups[0].keys())
    with pytest.raises(AssertionError):
        mb.Muon([dict(params=ps)])
    assert api["muon_rejects_group_dicts"]
    s = mb.SingleDeviceMuon([dict(params=ps)])
    assert [tuple(p.shape) for p in s.param_groups[0]["params"]] == api["single_order_kept"]
    aux = mb.MuonWithAuxAdam([dict(params=list(ps), use_muon=True),
                              dict(params=[torch.nn.Parameter(torch.zeros(5))], use_muon=False)])
    assert {k: v for k, v in aux.param_groups[0].items() if k != "params"} == api["aux_muon_group"]
    assert {k: v for k, v in aux.param_groups[1].items() if k != "params"} == api["aux_adam_group"]
    assert [tuple(p.shape) for p in aux.param_groups[0]["params"]] == api["aux_sorted_shapes"]
    saux = mb.SingleDeviceMuonWithAuxAdam([dict(params=list(ps), use_muon=True)])
    assert [tuple(p.shape) for p in saux.param_groups[0]["params"]] == api["single_aux_order_kept"]
    for bad in ("nesterov", "ns_steps"):
        assert api[f"aux_rejects_{bad}"]
        with pytest.raises(AssertionError):
            mb.MuonWithAuxAdam([dict(params=list(ps), use_muon=True, **{bad: 1})])
    with pytest.raises(AssertionError):
        mb.MuonWithAuxAdam([dict(params=list(ps))])
    assert issubclass(mb.Muon, torch.optim.Optimizer)


def test_muon_module_alias_exports_reference_names():
    import muon
    for name in ("Muon", "SingleDeviceMuon", "MuonWithAuxAdam", "SingleDeviceMuonWithAuxAdam",
                 "muon_update", "adam_update", "zeropower_via_newtonschulz5",
                 "ns_line_1", "ns_line_2", "ns_line_3"):
        assert callable(getattr(muon, name))


def test_engine_helpers():
    from muon_b200 import engine as E
    assert E.view_2d((256, 256, 3, 3)) == (256, 2304) and E.view_2d((5, 7)) == (5, 7)
    with pytest.raises(ValueError):
        E.view_2d((5,))
    assert E.aspect_scale((3072, 768)) == 2.0 and E.aspect_scale((768, 3072)) == 1
    assert E.aspect_scale((256, 256, 3, 3)) == 1 and E.aspect_scale((32, 16, 4, 2)) == 2 ** 0.5
    assert E.tri_tiles(128) == 1 and E.tri_tiles(256) == 1 and E.tri_tiles(768) == 6
    assert E.tri_tiles(4096) == 136
    assert E.batch_size_for(128, 1152, 64, 4 << 30) == 64
    assert E.batch_size_for(4096, 14336, 64, 4 << 30) == 7
    assert E.batch_size_for(4096, 14336, 64, 4 << 30) >= 1
    assert E.batch_size_for(4096, 14336, 64, 1 << 20) == 1
    E.set_ns_mode("classic5", 3)
    assert E.get_ns_mode() == ("classic5", 3)
    E.set_ns_mode("aol4")
    with pytest.raises(ValueError):
        E.set_ns_mode("cubic")


def test_launch_planner():
    from muon_b200 import engine as E
    cap = 4 << 30
    for m, n, count in [(4096, 14336, 64), (4096, 14336, 32), (4096, 4096, 64), (1024, 4096, 64),
                        (4096, 14336, 8), (768, 3072, 12), (128, 1152, 64), (4096, 14336, 1), (40, 72, 3)]:
        sizes = E.plan_launches(m, n, count, cap)
        assert sum(sizes) == count and min(sizes) >= 1 and max(sizes) - min(sizes) <= 1
        per_matrix = 2 * (2 * m * n + 2 * m * m)
        assert max(sizes) * per_matrix <= cap
        # never worse (in partial waves) than one matrix per launch
        waves = lambda b: -(-(E.tri_tiles(m) * b) // 74)
        assert sum(waves(b) for b in sizes) <= count * waves(1)
    assert E.plan_launches(4096, 14336, 0, cap) == []
    assert E.plan_launches(4096, 14336, 64, 1 << 20) == [1] * 64  # workspace cap of one matrix


# -------------------------------------------------- distributed logic on gloo CPU ranks
class OracleBackend:
    """Test-only stand-in for the CUDA backend: same interface, oracle arithmetic."""

    name = "oracle-test-double"
    workspace_cap_bytes = 4 << 30

    def __init__(self):
        self.muon_calls = []

    def muon_step(self, params, grads, moms, lr, weight_decay, beta, nesterov=True):
        self.muon_calls.append([tuple(p.shape) for p in params])
        for p, g, m in zip(params, grads, moms):
            orc.muon_param_step(p, g, m, lr, weight_decay, beta)

    def adam_step(self, params, grads, exp_avgs, exp_avg_sqs, steps, lr, weight_decay, betas, eps):
        for p, g, m, v, s in zip(params, grads, exp_avgs, exp_avg_sqs, steps):
            orc.adam_param_step(p, g, m, v, s, lr, weight_decay, betas, eps)

    def muon_orthogonalize(self, grads, moms, shape, beta, nesterov, out):
        rows, cols = shape[0], int(torch.tensor(shape[1:]).prod())
        for k, (g, m) in enumerate(zip(grads, moms)):
            u = orc.muon_update(g.view(shape), m.view(shape), beta=beta, nesterov=nesterov)
            out[k, :rows, :cols] = u.reshape(rows, cols)

    def apply_update(self, shards, u, rows, cols, lr, weight_decay):
        for k, p in enumerate(shards):
            p.mul_(1 - lr * weight_decay)
            p.add_(u[k, :rows, :cols].reshape(p.shape).to(p.dtype), alpha=-lr)


def _make_problem(shapes, seed=0, steps=2):
    g = torch.Generator().manual_seed(seed)
    p0 = [torch.randn(s, generator=g) * 0.02 for s in shapes]
    grads = [[torch.randn(s, generator=g) for s in shapes] for _ in range(steps)]
    return p0, grads


def _rank_main(rank, world, shapes, tmpdir, with_adam, policy="round_robin"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    dist.init_process_group("gloo", init_method=f"file://{tmpdir}/pg", rank=rank, world_size=world)
    try:
        import muon_b200 as mb
        from muon_b200 import engine as E
        from muon_b200 import ownership
        mb.set_ownership(policy)
        backend = OracleBackend()
        E._set_backend_for_testing(backend)
        p0, grads = _make_problem(shapes)
        params = [torch.nn.Parameter(p.clone()) for p in p0]
        gains = [torch.nn.Parameter(torch.ones(8)) for _ in range(3)]
        if with_adam:
            opt = mb.MuonWithAuxAdam([dict(params=list(params), use_muon=True, lr=0.02, weight_decay=0.01),
                                      dict(params=gains, use_muon=False)])
        else:
            opt = mb.Muon(list(params), lr=0.02, weight_decay=0.01)
        skip_grad_for = 1  # this parameter never gets a gradient: it must be treated as zeros
        for step_grads in grads:
            for i, (p, gr) in enumerate(zip(params, step_grads)):
                p.grad = None if i == skip_grad_for else gr.clone()
            for gp in gains:
                gp.grad = torch.full((8,), 0.5)
            opt.step()
        sorted_params = opt.param_groups[0]["params"]
        owned = ownership.owned_indices(sorted_params, world, rank)
        if policy == "round_robin":
            assert owned == [i for i in range(len(sorted_params)) if i % world == rank]  # muon.py:56-58
        has_state = [i for i, p in enumerate(sorted_params) if len(opt.state[p]) > 0]
        torch.save(dict(params=[p.detach().clone() for p in params], owned=owned, has_state=has_state,
                        calls=backend.muon_calls, gains=[g.detach().clone() for g in gains]),
                   f"{tmpdir}/out{rank}.pt")
    finally:
        dist.destroy_process_group()


def _single_device_oracle(shapes, skip_grad_for=1, steps=2):
    p0, grads = _make_problem(shapes, steps=steps)
    params = [p.clone() for p in p0]
    moms = [torch.zeros_like(p) for p in p0]
    for step_grads in grads:
        for i, (p, gr, m) in enumerate(zip(params, step_grads, moms)):
            g = torch.zeros_like(p) if i == skip_grad_for else gr.clone()
            orc.muon_param_step(p, g, m, 0.02, 0.01, 0.95)
    return params


@pytest.mark.parametrize("world,with_adam", [(2, False), (2, True), (3, False)])
def test_distributed_muon_on_gloo_ranks(tmp_path, world, with_adam):
    # counts per shape are multiples of the world size so that windows are shape-homogeneous
    # (gloo, like the reference on gloo, rejects unequal sizes inside one all_gather) except for
    # the tail window, which is shorter than the world and exercises the padding rule.
    shapes = [(24, 48)] * (2 * world) + [(48, 24)] * world + [(16, 16)] * (world - 1)
    mp.spawn(_rank_main, args=(world, shapes, str(tmp_path), with_adam), nprocs=world, join=True)
    outs = [torch.load(f"{tmp_path}/out{r}.pt", weights_only=False) for r in range(world)]
    ref = _single_device_oracle(shapes)
    for r, o in enumerate(outs):
        for p, q in zip(o["params"], ref):
            assert torch.equal(p, q), f"rank {r} disagrees with the single-device result"
        assert o["has_state"] == o["owned"], "momentum state must exist on the owning rank only"
        # same-shape parameters owned by a rank are handed to the backend together
        assert all(len(set(c)) == 1 for c in o["calls"])
        assert max(len(c) for c in o["calls"]) > 1
    if with_adam:
        g0 = outs[0]["gains"]
        for o in outs[1:]:
            for a, b in zip(o["gains"], g0):
                assert torch.equal(a, b)
        assert not torch.equal(g0[0], torch.ones(8))


@pytest.mark.parametrize("world,shapes", [
    (2, [(48, 24)] * 3 + [(24, 48)] * 3 + [(16, 16)]),          # a middle window mixes two shapes
    (3, [(48, 24)] * 3 + [(24, 48)] + [(16, 16)]),              # the tail window mixes shapes and pads
])
def test_distributed_muon_with_mixed_shape_windows(tmp_path, world, shapes):
    """Windows whose parameters differ in shape cannot go through one all_gather (the reference
    raises there); they are exchanged by per-parameter broadcasts and give the single-device result."""
    mp.spawn(_rank_main, args=(world, shapes, str(tmp_path), False), nprocs=world, join=True)
    outs = [torch.load(f"{tmp_path}/out{r}.pt", weights_only=False) for r in range(world)]
    ref = _single_device_oracle(shapes)
    for r, o in enumerate(outs):
        for p, q in zip(o["params"], ref):
            assert torch.equal(p, q), f"rank {r} disagrees with the single-device result"
        assert o["has_state"] == o["owned"]


@pytest.mark.parametrize("world", [2, 3])
def test_distributed_muon_with_cost_balanced_ownership(tmp_path, world):
    """`balanced` ownership: parameters go to the rank with the least Newton-Schulz work so far
    instead of round-robin. The parameters after two steps are those of the single-device run bit
    for bit (who updates a parameter does not enter its update), the momentum lives on the owner
    only, and the work is spread more evenly than round-robin spreads this mix."""
    from muon_b200 import ownership
    shapes = [(64, 96)] * (world + 1) + [(96, 32)] * 2 + [(16, 16)] * 5 + [(8, 4, 3, 3)] * 3
    mp.spawn(_rank_main, args=(world, shapes, str(tmp_path), False, "balanced"), nprocs=world, join=True)
    outs = [torch.load(f"{tmp_path}/out{r}.pt", weights_only=False) for r in range(world)]
    ref = _single_device_oracle(shapes)
    for r, o in enumerate(outs):
        for p, q in zip(o["params"], ref):
            assert torch.equal(p, q), f"rank {r} disagrees with the single-device result"
        assert o["has_state"] == o["owned"], "momentum state must exist on the owning rank only"
    assert sorted(i for o in outs for i in o["owned"]) == list(range(len(shapes)))
    sorted_shapes = sorted(shapes, reverse=True)

    def spread(policy):
        who = ownership.owners(sorted_shapes, world, policy)
        load = [sum(ownership.ns_cost(s) for s, w in zip(sorted_shapes, who) if w == r) for r in range(world)]
        return max(load) - min(load)
    assert spread("balanced") < spread("round_robin")
    assert spread("balanced") <= max(ownership.ns_cost(s) for s in shapes)


def _sharded_rank(rank, world, shapes, tmpdir, as_dtensor):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = "29871"
    dist.init_process_group("gloo", init_method=f"file://{tmpdir}/pg", rank=rank, world_size=world)
    try:
        import muon_b200 as mb
        from muon_b200 import engine as E
        from muon_b200.sharded import shard_rows
        E._set_backend_for_testing(OracleBackend())
        p0, grads = _make_problem(shapes)

        def piece(t):
            chunk, mine = shard_rows(t.shape[0], world, rank)
            return t[rank * chunk: rank * chunk + mine].clone()

        if as_dtensor:
            from torch.distributed.tensor import Shard, distribute_tensor, init_device_mesh
            mesh = init_device_mesh("cpu", (world,))
            params = [torch.nn.Parameter(distribute_tensor(p.clone(), mesh, [Shard(0)])) for p in p0]
            opt = mb.ShardedMuon(list(params), lr=0.02, weight_decay=0.01)
        else:
            params = [torch.nn.Parameter(piece(p)) for p in p0]
            opt = mb.ShardedMuon(list(params), lr=0.02, weight_decay=0.01, full_shapes=shapes)
        skip_grad_for = 1
        for step_grads in grads:
            for i, (p, gr) in enumerate(zip(params, step_grads)):
                if i == skip_grad_for:
                    p.grad = None
                elif as_dtensor:
                    p.grad = distribute_tensor(gr.clone(), mesh, [Shard(0)])
                else:
                    p.grad = piece(gr)
            opt.step()
        local = [(p.to_local() if as_dtensor else p).detach().clone() for p in params]
        has_state = [i for i, p in enumerate(params) if len(opt.state[p]) > 0]
        torch.save(dict(local=local, has_state=has_state), f"{tmpdir}/out{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,as_dtensor", [(2, False), (3, False), (2, True)])
def test_sharded_muon_on_gloo_ranks(tmp_path, world, as_dtensor):
    """Row-sharded parameters (plain shards with full shapes, or DTensor Shard(0)): gradients go to
    the owners, updates come back in bf16, every rank updates its rows. The shards must be the
    rows of the single-device result bit for bit, also where the rows do not divide evenly (one
    rank short, one rank empty) and for a parameter that never gets a gradient."""
    from muon_b200.sharded import shard_rows
    shapes = [(24, 48)] * 3 + [(50, 24)] * 2 + [(4, 16)] * 2 + [(8, 4, 3, 3)]
    mp.spawn(_sharded_rank, args=(world, shapes, str(tmp_path), as_dtensor), nprocs=world, join=True)
    outs = [torch.load(f"{tmp_path}/out{r}.pt", weights_only=False) for r in range(world)]
    ref = _single_device_oracle(shapes)
    owners_state = set()
    for r, o in enumerate(outs):
        for i, (piece, full) in enumerate(zip(o["local"], ref)):
            chunk, mine = shard_rows(full.shape[0], world, r)
            assert torch.equal(piece, full[r * chunk: r * chunk + mine]), f"rank {r}, parameter {i}"
        assert not owners_state & set(o["has_state"]), "a momentum buffer lives on exactly one rank"
        owners_state |= set(o["has_state"])
    assert owners_state == set(range(len(shapes)))


def _fixture_rank(rank, world, tmpdir, fixture_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    dist.init_process_group("gloo", init_method=f"file://{tmpdir}/pg", rank=rank, world_size=world)
    try:
        import muon_b200 as mb
        from muon_b200 import engine as E
        E._set_backend_for_testing(OracleBackend())
        fx = torch.load(fixture_path, weights_only=False)
        params = [torch.nn.Parameter(p.clone()) for p in fx["p0"]]
        opt = mb.Muon(list(params), **fx["hyper"])
        for step_grads in fx["grads"]:
            for i, (p, gr) in enumerate(zip(params, step_grads)):
                p.grad = None if i == fx["no_grad_index"] else gr.clone()
            opt.step()
        sorted_params = opt.param_groups[0]["params"]
        out = dict(params=[p.detach().clone() for p in params],
                   sorted_shapes=[tuple(p.shape) for p in sorted_params],
                   has_state=[i for i, p in enumerate(sorted_params) if len(opt.state[p]) > 0])
        params = [torch.nn.Parameter(p.clone()) for p in fx["p0"]]
        gains = [torch.nn.Parameter(g.clone()) for g in fx["gains0"]]
        aux = mb.MuonWithAuxAdam([dict(params=list(params), use_muon=True, lr=0.02, weight_decay=0.01),
                                  dict(params=gains, use_muon=False, lr=3e-3, weight_decay=0.01)])
        for step_grads, gain_grads in zip(fx["grads"], fx["gain_grads"]):
            for i, (p, gr) in enumerate(zip(params, step_grads)):
                p.grad = None if i == fx["no_grad_index"] else gr.clone()
            for q, gr in zip(gains, gain_grads):
                q.grad = gr.clone()
            aux.step()
        sorted_params = aux.param_groups[0]["params"]
        out["aux"] = dict(params=[p.detach().clone() for p in params], gains=[q.detach().clone() for q in gains],
                          has_state=[i for i, p in enumerate(sorted_params) if len(aux.state[p]) > 0],
                          adam_steps=[aux.state[q]["step"] for q in gains])
        torch.save(out, f"{tmpdir}/out{rank}.pt")
    finally:
        dist.destroy_process_group()


def test_distributed_muon_matches_the_real_reference_class(tmp_path):
    """Fixture `distributed`: the reference's own `Muon` and `MuonWithAuxAdam` run on two gloo ranks. Same parameters,
    same gradients, same world size here: every rank must end with the same parameters bit for
    bit, the same sort order and momentum state on the same (owned) parameters only."""
    path = os.path.join(os.path.dirname(__file__), "golden", "distributed.pt")
    fx = torch.load(path, weights_only=False)
    world = fx["world"]
    mp.spawn(_fixture_rank, args=(world, str(tmp_path), path), nprocs=world, join=True)
    for r in range(world):
        mine = torch.load(f"{tmp_path}/out{r}.pt", weights_only=False)
        theirs = fx["ranks"][r]
        assert mine["sorted_shapes"] == theirs["sorted_shapes"]
        assert mine["has_state"] == theirs["has_state"]
        for p, q in zip(mine["params"], theirs["params"]):
            assert torch.equal(p, q)
        # the same problem through MuonWithAuxAdam, with an Adam group of 1-D parameters
        assert mine["aux"]["has_state"] == theirs["aux"]["has_state"]
        assert mine["aux"]["adam_steps"] == theirs["aux"]["adam_steps"]
        for p, q in zip(mine["aux"]["params"] + mine["aux"]["gains"], theirs["aux"]["params"] + theirs["aux"]["gains"]):
            assert torch.equal(p, q)


# ------------------------------------------- consolidated checkpoints across world sizes
CKPT_SHAPES = [(24, 48)] * 6 + [(48, 24)] * 6


def _ckpt_rank(rank, world, tmpdir, phase):
    dist.init_process_group("gloo", init_method=f"file://{tmpdir}/pg{phase}", rank=rank, world_size=world)
    try:
        import muon_b200 as mb
        from muon_b200 import checkpoint as ck
        from muon_b200 import engine as E
        E._set_backend_for_testing(OracleBackend())
        p0, grads = _make_problem(CKPT_SHAPES, seed=7, steps=3)
        if phase == 1:
            params = [torch.nn.Parameter(p.clone()) for p in p0]
            opt = mb.Muon(list(params), lr=0.02, weight_decay=0.01)
            for step_grads in grads[:2]:
                for p, gr in zip(params, step_grads):
                    p.grad = gr.clone()
                opt.step()
            state = ck.consolidated_state_dict(opt)
            if rank == 0:
                assert sorted(state["groups"][0]["momentum"]) == list(range(len(CKPT_SHAPES)))
                torch.save(dict(opt=state, params=[p.detach().clone() for p in params]), f"{tmpdir}/ckpt.pt")
            else:
                assert state is None
        else:
            saved = torch.load(f"{tmpdir}/ckpt.pt", weights_only=False)
            params = [torch.nn.Parameter(p.clone()) for p in saved["params"]]
            opt = mb.Muon(list(params), lr=0.5, weight_decay=0.5)  # overwritten by the checkpoint
            ck.load_consolidated_state_dict(opt, saved["opt"])
            sorted_params = opt.param_groups[0]["params"]
            assert [i for i, p in enumerate(sorted_params) if len(opt.state[p])] == \
                list(range(rank, len(sorted_params), world))
            for p, gr in zip(params, grads[2]):
                p.grad = gr.clone()
            opt.step()
            torch.save([p.detach().clone() for p in params], f"{tmpdir}/final{rank}.pt")
    finally:
        dist.destroy_process_group()


def test_consolidated_checkpoint_survives_a_world_size_change(tmp_path):
    mp.spawn(_ckpt_rank, args=(2, str(tmp_path), 1), nprocs=2, join=True)
    mp.spawn(_ckpt_rank, args=(3, str(tmp_path), 2), nprocs=3, join=True)
    p0, grads = _make_problem(CKPT_SHAPES, seed=7, steps=3)
    ref = [p.clone() for p in p0]
    moms = [torch.zeros_like(p) for p in p0]
    for step_grads in grads:
        for p, gr, m in zip(ref, step_grads, moms):
            orc.muon_param_step(p, gr.clone(), m, 0.02, 0.01, 0.95)
    for r in range(3):
        got = torch.load(f"{tmp_path}/final{r}.pt", weights_only=False)
        for p, q in zip(got, ref):
            assert torch.equal(p, q), f"rank {r} after resume differs from the uninterrupted run"


# --------------------------------------------------- updates started from the backward pass
def test_step_in_backward_gives_the_result_of_a_plain_step():
    """StepInBackward starts the update of a same-shape set when the backward pass has delivered
    its last gradient; parameters without gradient and Adam groups are finished in step(). The
    result equals optimizer.step() after the backward pass, bit for bit, over three steps."""
    import muon_b200 as mb
    from muon_b200 import engine as E
    prev = E._set_backend_for_testing(OracleBackend())
    try:
        shapes = [(24, 48)] * 3 + [(48, 24)] * 2 + [(16, 16)]
        g = torch.Generator().manual_seed(3)
        p0 = [torch.randn(s, generator=g) * 0.02 for s in shapes]
        weights = [[torch.randn(s, generator=g) for s in shapes] for _ in range(3)]

        def make():
            ps = [torch.nn.Parameter(p.clone()) for p in p0]
            gain = torch.nn.Parameter(torch.ones(8))
            opt = mb.SingleDeviceMuonWithAuxAdam([dict(params=ps, use_muon=True, lr=0.02, weight_decay=0.01),
                                                  dict(params=[gain], use_muon=False, lr=1e-3)])
            return ps, gain, opt

        def loss_of(ps, gain, w, skip):
            # gradient of parameter i is w[i] * (sum of gain); parameter `skip` takes no part
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
            if skip < 0:  # every set was updated inside backward(): nothing is waiting
                assert all(e["done"] for e in overlap._sets)
            overlap.step()
            for x, y in zip(ps_a + [gain_a], ps_b + [gain_b]):
                assert torch.equal(x, y)
        assert not torch.equal(ps_a[0], p0[0])
        with pytest.raises(TypeError):
            mb.StepInBackward(torch.optim.SGD([torch.nn.Parameter(torch.zeros(2))], lr=0.1))
        overlap.remove()
    finally:
        E._set_backend_for_testing(prev)
