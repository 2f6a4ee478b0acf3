"""Property tests (hypothesis) of host-side rules: the launch planner, the ownership rule of the
distributed optimizer, and the mirror rules of the restated symmetric products."""
import math

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import muon_oracle as orc

dims = st.integers(min_value=1, max_value=20000)


@settings(max_examples=150, deadline=None)
@given(m=dims, n=dims, count=st.integers(0, 300), cap_mib=st.integers(1, 8192))
def test_launch_planner_always_covers_every_matrix(m, n, count, cap_mib):
    from muon_b200 import engine as E
    m, n = min(m, n), max(m, n)
    cap = cap_mib << 20
    sizes = E.plan_launches(m, n, count, cap)
    assert sum(sizes) == count
    if count == 0:
        assert sizes == []
        return
    assert min(sizes) >= 1 and max(sizes) - min(sizes) <= 1
    per_matrix = 2 * (2 * m * ((n + 7) // 8 * 8) + 2 * m * ((m + 7) // 8 * 8)) + 2048
    # the cap is respected whenever a single matrix fits it at all
    assert max(sizes) == 1 or max(sizes) * per_matrix <= cap
    # one launch never takes more than the default batch size doubled
    assert max(sizes) <= max(1, 2 * E.batch_size_for(m, n, count, cap))


@settings(max_examples=100, deadline=None)
@given(m=st.integers(1, 40000))
def test_triangular_tile_count(m):
    from muon_b200 import engine as E
    t = E.tri_tiles(m)
    if m <= 128:
        assert t == 1
    else:
        rows = math.ceil(m / 256)
        # row tile i of 256 rows owns the column tiles j with 256 * j <= 256 * i + 255
        assert t == sum(min(rows, (256 * i + 255) // 256 + 1) for i in range(rows))


shape2d = st.tuples(st.integers(1, 6), st.integers(1, 6))


@settings(max_examples=100, deadline=None)
@given(shapes=st.lists(shape2d, min_size=1, max_size=24), world=st.integers(1, 9))
def test_ownership_rule(shapes, world):
    order = orc.sorted_param_order(shapes)
    # the reference sorts torch.Size objects descending; Python compares them as tuples and keeps ties in order
    params = [torch.empty(s) for s in shapes]
    ref_sorted = sorted(params, key=lambda x: x.size(), reverse=True)
    assert [id(params[i]) for i in order] == [id(p) for p in ref_sorted]
    n = len(shapes)
    padded = orc.padded_length(n, world)
    assert padded % world == 0 and 0 < padded - n <= world
    owners = [orc.owner_of(i, world) for i in range(n)]
    for r in range(world):
        assert [i for i, o in enumerate(owners) if o == r] == list(range(r, n, world))


@settings(max_examples=100, deadline=None)
@given(shapes=st.lists(st.tuples(st.integers(1, 40), st.integers(1, 40)), min_size=1, max_size=30),
       world=st.integers(1, 9))
def test_balanced_ownership(shapes, world):
    """Every parameter has exactly one owner; the assignment is a function of the shape list alone;
    greedy assignment in order of decreasing cost keeps the heaviest rank within one parameter of
    the lightest: max load - min load <= the largest single cost (and <= the cost of the parameter
    that was placed last on the heaviest rank)."""
    from muon_b200 import ownership
    shapes = sorted(shapes, reverse=True)
    who = ownership.owners(shapes, world, "balanced")
    assert len(who) == len(shapes) and all(0 <= r < world for r in who)
    assert who == ownership.owners(list(shapes), world, "balanced")
    cost = [ownership.ns_cost(s) for s in shapes]
    load = [sum(c for c, w in zip(cost, who) if w == r) for r in range(world)]
    assert max(load) - min(load) <= max(cost)
    assert ownership.owners(shapes, world, "round_robin") == [i % world for i in range(len(shapes))]
    m, n = min(shapes[0]), max(shapes[0])
    assert ownership.ns_cost(shapes[0]) == m * (m + 1) * n + m * m * (m + 1) + 2 * m * m * n


@settings(max_examples=200, deadline=None)
@given(rows=st.integers(1, 5000), world=st.integers(1, 64))
def test_row_shards_partition_the_rows(rows, world):
    """The row split of ShardedMuon is torch.chunk's (= DTensor Shard(0)): chunks of ceil(rows/W),
    consecutive, covering every row once; the last ranks may be short or empty."""
    from muon_b200.sharded import shard_rows
    pieces = [shard_rows(rows, world, r) for r in range(world)]
    chunk = pieces[0][0]
    assert all(c == chunk for c, _ in pieces) and chunk == -(-rows // world)
    assert sum(n for _, n in pieces) == rows
    assert [n for _, n in pieces] == [len(t) for t in torch.arange(rows).chunk(world)] + \
        [0] * (world - len(torch.arange(rows).chunk(world)))


@settings(max_examples=40, deadline=None)
@given(m=st.integers(1, 70), seed=st.integers(0, 2 ** 16), tile=st.sampled_from([8, 16, 64]))
def test_mirror_rules(m, seed, tile):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(m, m, generator=g)              # not symmetric
    X = torch.randn(m, m + 3, generator=g)
    G1 = orc.ns_line_1(X, mirror="lower")
    assert torch.equal(G1, G1.mT)
    alpha, beta = 1.7, -0.6
    B = orc.ns_line_2(A, alpha, beta, mirror="product")
    # product rule: B - beta * A is the mirrored product, hence symmetric, and equals the formula below the diagonal
    P = B - beta * A
    assert torch.allclose(P, P.mT, atol=1e-5)
    full = alpha * (A @ A.mT) + beta * A
    low = torch.tril(torch.ones(m, m, dtype=torch.bool))
    assert torch.allclose(B[low], full[low], atol=1e-5)
    # store-order rule of square tiles: off-diagonal tiles lower-authoritative, diagonal tiles transposed
    R = orc.ns_line_2(A, alpha, beta, mirror="ref_square_tiles", tile=tile)
    for s in range(0, m, tile):
        e = min(s + tile, m)
        assert torch.allclose(R[s:e, s:e], full[s:e, s:e].mT, atol=1e-5)
        assert torch.allclose(R[e:, s:e], full[e:, s:e], atol=1e-5)
        assert torch.allclose(R[s:e, e:], full[e:, s:e].mT, atol=1e-5)
    # for a symmetric A all rules agree
    S = A + A.mT
    outs = [orc.ns_line_2(S, alpha, beta, mirror=p, tile=tile) for p in ("product", "lower", "ref_square_tiles", "none")]
    for o in outs[1:]:
        assert torch.allclose(o, outs[0], atol=1e-4)
