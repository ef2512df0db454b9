"""clusten_knn2d against torch.cdist + sort: the k nearest database points of every query, ascending,
ties towards the lower index (the search the reference runs with pykeops, models/point_utils.py:27-58)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference(q, d, k):
    dist = torch.cdist(q.double(), d.double())
    # stable sort: among equal distances the lower index comes first
    order = torch.sort(dist, dim=2, stable=True)
    return order.indices[:, :, :k], order.values[:, :, :k]


@pytest.mark.parametrize("b,nq,n,k", [(3, 700, 90, 6), (2, 333, 333, 2), (1, 50, 5000, 8), (4, 9, 12, 1), (2, 3136, 392, 6)])
def test_random_positions(lib, b, nq, n, k):
    from clusten import ops
    g = torch.Generator(device=DEV).manual_seed(5)
    q = torch.rand(b, nq, 2, generator=g, device=DEV) * 56
    d = torch.rand(b, n, 2, generator=g, device=DEV) * 56
    idx, dist = ops.knn2d(q, d, k, return_dist=True)
    want_idx, want_dist = _reference(q, d, k)
    assert idx.dtype == torch.int64 and idx.shape == (b, nq, k)
    assert torch.allclose(dist.double(), want_dist, rtol=1e-6, atol=1e-5)
    # the same neighbours, up to the order of candidates whose distances differ by less than fp32 resolves
    true_dist = torch.cdist(q.double(), d.double()).gather(2, idx)
    assert torch.allclose(true_dist, want_dist, rtol=0, atol=1e-5)
    assert (idx == want_idx).float().mean() > 0.9999
    assert bool((idx.sort(dim=2).values.diff(dim=2) != 0).all()) if k > 1 else True     # k distinct points
    assert torch.equal(ops.knn2d(q, d, k), idx)


def test_grid_positions_with_ties(lib):
    """Tokens on the integer grid (stage 1 of the model): many exactly equal distances."""
    from clusten import ops
    ys, xs = torch.meshgrid(torch.arange(14.), torch.arange(14.), indexing="ij")
    pos = torch.stack([xs, ys], 2).reshape(1, -1, 2).to(DEV).repeat(2, 1, 1)
    idx, dist = ops.knn2d(pos, pos, 5, return_dist=True)
    want_idx, want_dist = _reference(pos, pos, 5)
    assert torch.equal(dist, want_dist.float())           # squared distances are small integers: exact
    assert torch.equal(idx, want_idx)
    assert bool((idx[:, :, 0] == torch.arange(196, device=DEV)).all()) and bool((dist[:, :, 0] == 0).all())


def test_argument_checks(lib):
    p = 256
    assert lib.clusten_knn2d(p, p, 1, 4, 4, 9, p, None, None) == -6      # k above 8
    assert lib.clusten_knn2d(p, p, 1, 4, 3, 4, p, None, None) == -6      # k above n
    assert lib.clusten_knn2d(p, p, 0, 4, 4, 2, p, None, None) == -2
    assert lib.clusten_knn2d(None, p, 1, 4, 4, 2, p, None, None) == -3
