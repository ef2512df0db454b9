"""clusten_nbhd_build against the gather formulation of models/aff_transformer.py:476-487: members of the
nearest clusters, their mask bits and the position-table rows of their offsets; integer work, bit-exact."""
import pytest
import torch

from oracle import formula

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(b, n, cs, nnc, seed, on_grid=True, with_mask=None):
    g = torch.Generator(device=DEV).manual_seed(seed)
    k = (n + cs - 1) // cs
    if on_grid:
        side = int(n ** 0.5) + 1
        perm = torch.stack([torch.randperm(side * side, generator=g, device=DEV)[:n] for _ in range(b)])
        pos = torch.stack([perm % side, perm // side], 2).float()
        width = side - 1
    else:
        pos = torch.rand(b, n, 2, generator=g, device=DEV) * 40
        width = 41
    member = torch.arange(k * cs, device=DEV)
    member = torch.where(member < n, member, torch.zeros_like(member)).reshape(1, k, cs).expand(b, -1, -1).contiguous()
    mask = None
    if with_mask if with_mask is not None else k * cs != n:
        mask = (torch.arange(k * cs, device=DEV) < n).long().reshape(1, k, cs).expand(b, -1, -1).contiguous()
    nearest = torch.randint(k, (b, n, nnc), generator=g, device=DEV)
    return pos, member, mask, nearest, width, 2 * width + 1


@pytest.mark.parametrize("b,n,cs,nnc", [(2, 3136, 8, 6), (3, 784, 8, 6), (2, 73, 8, 6), (1, 368, 8, 4),
                                        (2, 100, 4, 3), (1, 50, 5, 2), (4, 196, 8, 1)])
def test_tables_match_the_gather_formulation(lib, b, n, cs, nnc):
    from clusten import ops
    pos, member, mask, nearest, width, table = _case(b, n, cs, nnc, seed=n + cs)
    got = ops.nbhd_build(pos, member, mask, nearest, width, table)
    want = formula.nbhd_tables(pos, member, mask, nearest, width, table)
    assert got[0].dtype == torch.int64 and got[0].shape == (b, n, nnc * cs)
    assert torch.equal(got[0], want[0])
    assert (got[1] is None) == (want[1] is None)
    if want[1] is not None:
        assert torch.equal(got[1], want[1])
    assert torch.equal(got[2], want[2])
    assert int(got[2].min()) >= 0 and int(got[2].max()) < table * table      # rows of the table


def test_positions_off_the_grid_and_shuffled_members(lib):
    """Non-integer positions (the fp32 arithmetic must round like the formulation's) and an arbitrary member table."""
    from clusten import ops
    b, n, cs, nnc = 2, 500, 8, 6
    pos, member, _, nearest, width, table = _case(b, n, cs, nnc, seed=3, on_grid=False)
    g = torch.Generator(device=DEV).manual_seed(9)
    member = torch.randint(n, member.shape, generator=g, device=DEV)
    mask = torch.randint(2, member.shape, generator=g, device=DEV)
    got = ops.nbhd_build(pos, member, mask, nearest, width, table)
    want = formula.nbhd_tables(pos, member, mask, nearest, width, table)
    for a, w in zip(got, want):
        assert torch.equal(a, w)


def test_ids_out_of_range_name_nobody(lib):
    from clusten import ops
    b, n, cs, nnc = 1, 64, 8, 3
    pos, member, _, nearest, width, table = _case(b, n, cs, nnc, seed=1)
    mask = torch.ones_like(member)
    nearest[0, 5, 1] = 8           # k = 8 clusters: one past the end
    nearest[0, 6, 0] = -1
    member[0, 2, 3] = n + 7        # a member that is no token
    idx, msk, pe = ops.nbhd_build(pos, member, mask, nearest, width, table)
    assert bool((idx[0, 5, 8:16] == -1).all()) and bool((msk[0, 5, 8:16] == 0).all()) and bool((pe[0, 5, 8:16] == 0).all())
    assert bool((idx[0, 6, 0:8] == -1).all())
    hit = (nearest[0] == 2).nonzero()
    i, r = int(hit[0, 0]), int(hit[0, 1])
    assert int(idx[0, i, r * cs + 3]) == n + 7 and int(pe[0, i, r * cs + 3]) == 0
    ok = nearest.clone()
    ok[0, 5, 1] = 0
    ok[0, 6, 0] = 0
    rest = torch.ones(n, nnc, dtype=torch.bool, device=DEV)
    rest[5, 1] = rest[6, 0] = False
    rest &= nearest[0] != 2
    want = formula.nbhd_tables(pos, member.clamp(max=n - 1), mask, ok, width, table)
    sel = rest.repeat_interleave(cs, dim=1)
    assert torch.equal(idx[0][sel], want[0][0][sel]) and torch.equal(pe[0][sel], want[2][0][sel])


def test_argument_checks(lib):
    p = 256
    args = lambda **kw: [kw.get("pos", p), p, kw.get("cmask"), p, p, kw.get("omask"), p,
                         kw.get("b", 1), 8, 2, 4, 2, 3, 7, None]
    assert lib.clusten_nbhd_build(*args(b=0)) == -2
    assert lib.clusten_nbhd_build(*args(pos=None)) == -3
    assert lib.clusten_nbhd_build(*args(cmask=p)) == -3          # a mask in, nowhere to put it
