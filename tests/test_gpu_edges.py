"""GPU parity tests of the radius-graph edge builder against the CPU oracle (bit-exact edge sets after canonical sort)."""
import numpy as np
import pytest

from deepscalemd_b200 import capi
from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu


def to_dev(a, dtype=None):
    import torch
    return torch.tensor(np.ascontiguousarray(a), dtype=dtype, device="cuda")


def canon(rows):
    rows = np.asarray(rows)
    return rows[:, np.lexsort(rows[::-1])]


def test_edges_match_oracle_plain_and_bounded(cuda_device):
    rng = np.random.default_rng(10)
    n, L, cutoff = 5000, 40.0, 5.0
    pos = rng.uniform(0, L, (n, 3))
    x, y, z = (to_dev(pos[:, k]) for k in range(3))
    eb = capi.EdgeBuilder()
    want, _ = co.edges(pos[:, 0], pos[:, 1], pos[:, 2], cutoff)
    for lo, hi in ((None, None), (np.zeros(3), np.full(3, L))):
        idx, sh = eb.build(x, y, z, cutoff, lo=lo, hi=hi)
        assert sh is None
        got = idx.cpu().numpy()
        assert got.dtype == np.int64 and got.shape == want.shape
        assert np.array_equal(canon(got), canon(want))
        # grouped by centre: row 0 changes value n_centres - 1 times at most
        assert (np.diff(got[0]) != 0).sum() <= n - 1
    eb.close()


def test_edges_with_images_and_pruning(cuda_device):
    rng = np.random.default_rng(11)
    n, L, cutoff = 3000, 30.0, 5.0
    pos = rng.uniform(0, L, (n, 3))
    box = np.full(3, L)
    im = co.images(pos[:, 0], pos[:, 1], pos[:, 2], box, np.zeros(3), -np.full(3, cutoff + 1e-8), box + cutoff + 1e-8,
                   np.ones(3, dtype=np.int32))
    total = len(im["x"])
    ok = (rng.uniform(size=n) < 0.6).astype(np.uint8)
    x, y, z = to_dev(im["x"]), to_dev(im["y"]), to_dev(im["z"])
    owner = to_dev(im["owner"])
    shift = tuple(to_dev(im["shift"][:, k]) for k in range(3))
    eb = capi.EdgeBuilder()
    for row, mask in ((1, None), (0, ok), (1, ok)):
        want_idx, want_sh = co.edges(im["x"], im["y"], im["z"], cutoff, n_centers=n, owner=im["owner"],
                                     shift=im["shift"], receiver_ok=mask, row=row)
        idx, sh = eb.build(x, y, z, cutoff, n_centers=n, owner=owner, shift=shift,
                           receiver_ok=None if mask is None else to_dev(mask), row=row)
        got = np.concatenate([idx.cpu().numpy().astype(np.float64), sh.cpu().numpy().T])
        want = np.concatenate([want_idx.astype(np.float64), want_sh.T])
        assert got.shape == want.shape
        assert np.array_equal(canon(got), canon(want))
    assert total > n
    eb.close()


def test_edges_errors(cuda_device):
    rng = np.random.default_rng(12)
    pos = rng.uniform(0, 10.0, (100, 3))
    x, y, z = (to_dev(pos[:, k]) for k in range(3))
    eb = capi.EdgeBuilder()
    with pytest.raises(capi.DsmdError) as err:
        eb.build(x, y, z, 2.0, lo=np.zeros(3), hi=np.full(3, 5.0))      # atoms outside the given box
    assert err.value.code == capi.ERR_OUT_OF_DOMAIN
    with pytest.raises(capi.DsmdError) as err:
        eb.build(x, y, z, -1.0)
    assert err.value.code == capi.ERR_INVALID
    bad = pos.copy()
    bad[3, 0] = np.nan
    with pytest.raises(capi.DsmdError):
        eb.build(to_dev(bad[:, 0]), y, z, 2.0, lo=np.zeros(3), hi=np.full(3, 10.0))
    idx, _ = eb.build(x[:1], y[:1], z[:1], 2.0)                          # a single atom has no edges
    assert idx.shape[1] == 0
    eb.close()


def test_compact_periodic_graph(cuda_device):
    s = syn.disordered_solid(20000, seed=5)
    L = s.box[0]
    x, y, z = (to_dev(s.pos[:, k]) for k in range(3))
    eb = capi.EdgeBuilder()
    src, dst, sh, vec = eb.build_periodic(x, y, z, s.box, s.cutoff)
    src, dst, sh, vec = src.cpu().numpy(), dst.cpu().numpy(), sh.cpu().numpy(), vec.cpu().numpy()
    # oracle: explicit images, then edges with shifts
    im = co.images(s.pos[:, 0], s.pos[:, 1], s.pos[:, 2], s.box, np.zeros(3), -np.full(3, s.cutoff + 1e-8),
                   s.box + s.cutoff + 1e-8, np.ones(3, dtype=np.int32))
    want_idx, want_sh = co.edges(im["x"], im["y"], im["z"], s.cutoff, n_centers=s.n, owner=im["owner"], shift=im["shift"])
    want = np.stack([want_idx[0], want_idx[1], *(np.rint(want_sh[:, k] / L).astype(np.int64) for k in range(3))])
    got = np.stack([src.astype(np.int64), dst.astype(np.int64), *(sh[:, k].astype(np.int64) for k in range(3))])
    assert np.array_equal(canon(got), canon(want))
    # already sorted by (src, dst, shift)
    assert np.array_equal(got, canon(got))
    d = s.pos[dst] + sh * s.box - s.pos[src]
    assert np.abs(vec - d).max() < 1e-5
    assert abs(len(src) / s.n - 4.18879 * 125 * 0.05) < 1.0      # 26.2 neighbours per atom
    eb.close()
