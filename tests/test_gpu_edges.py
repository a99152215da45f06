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
    # grouped by centre: row 0 changes value n - 1 times at most
    assert (np.diff(src) != 0).sum() <= s.n - 1
    d = s.pos[dst] + sh * s.box - s.pos[src]
    assert np.abs(vec - d).max() < 1e-5
    assert 24.0 < len(src) / s.n < 26.2      # 26.2 neighbours per atom at this density, less what the minimum distance excludes
    # positions given some box lengths away from the box: the same edges in the same order, the same displacements, and
    # lattice shifts that refer to the coordinates as given
    moved = s.pos + np.random.default_rng(3).integers(-3, 4, s.pos.shape) * s.box
    src2, dst2, sh2, vec2 = eb.build_periodic(*(to_dev(moved[:, k]) for k in range(3)), s.box, s.cutoff)
    src2, dst2, sh2, vec2 = src2.cpu().numpy(), dst2.cpu().numpy(), sh2.cpu().numpy(), vec2.cpu().numpy()
    assert np.array_equal(src2, src) and np.array_equal(dst2, dst)
    assert np.abs(vec2 - vec).max() < 1e-5
    assert np.abs(moved[dst2] + sh2 * s.box - moved[src2] - vec2).max() < 1e-5
    assert np.abs(sh2).max() > 1
    eb.close()


def test_image_atoms_receivers_and_the_whole_mlip_preparation(cuda_device):
    """The device versions of MLIPStep's image atoms and receiver mask equal the oracle's bit for bit, and feeding them
    to the edge builder (images as shifts + receiver pruning) gives the oracle's edge list: the whole preparation of one
    model call for a periodic box on one rank, unwrapped input positions included."""
    import torch
    rng = np.random.default_rng(21)
    n, L, cutoff = 4000, 32.0, 5.0
    box = np.full(3, L)
    pos = rng.uniform(0, L, (n, 3)) + rng.integers(-2, 3, (n, 3)) * L      # not wrapped
    types = rng.integers(0, 3, n).astype(np.int32)
    reach = cutoff + 1e-8
    lo, hi = -np.full(3, reach), box + reach
    want = co.images(pos[:, 0], pos[:, 1], pos[:, 2], box, np.zeros(3), lo, hi, np.ones(3, dtype=np.int32))
    eb = capi.EdgeBuilder()
    x, y, z = (to_dev(pos[:, k]) for k in range(3))
    got = eb.images(x, y, z, to_dev(types), box, np.zeros(3), lo, hi, (1, 1, 1))
    assert got["n_all"] == len(want["x"]) > n
    for k in "xyz":
        assert np.array_equal(got[k].cpu().numpy(), want[k])
    assert np.array_equal(got["owner"].cpu().numpy(), want["owner"])
    assert np.array_equal(got["type"].cpu().numpy(), types[want["owner"]])
    assert np.array_equal(torch.stack(got["shift"], dim=1).cpu().numpy(), want["shift"])
    # receivers: the atoms within 2 A of an inner box
    inner_lo, inner_hi = np.full(3, 8.0), np.full(3, 20.0)
    ok_want = co.mark_receivers(want["x"][:n], want["y"][:n], want["z"][:n], inner_lo, inner_hi, 2.0)
    ok = eb.mark_receivers(got["x"][:n].clone(), got["y"][:n].clone(), got["z"][:n].clone(), inner_lo, inner_hi, 2.0)
    assert np.array_equal(ok.cpu().numpy(), ok_want) and 0 < ok_want.sum() < n
    # edges over wrapped atoms + images, centred on real atoms, pruned to edges received by marked atoms
    gx, gy, gz = got["x"].clone(), got["y"].clone(), got["z"].clone()
    owner, shift = got["owner"].clone(), tuple(t.clone() for t in got["shift"])
    idx, sh = eb.build(gx, gy, gz, cutoff, n_centers=n, owner=owner, shift=shift, receiver_ok=ok, row=1)
    want_idx, want_sh = co.edges(want["x"], want["y"], want["z"], cutoff, n_centers=n, owner=want["owner"],
                                 shift=want["shift"], receiver_ok=ok_want, row=1)
    a = np.concatenate([idx.cpu().numpy().astype(np.float64), sh.cpu().numpy().T])
    b = np.concatenate([want_idx.astype(np.float64), want_sh.T])
    assert a.shape == b.shape and np.array_equal(canon(a), canon(b))
    eb.close()


def test_image_forces_fold_back_and_virial(cuda_device):
    """Forces a model returns for atoms + image atoms are folded back onto the atoms (images summed in slot order) exactly
    as the oracle does it, with and without the image part and for a prefix of the atoms; the r.F sums agree with the
    oracle's extended-precision sums to rounding."""
    import torch
    rng = np.random.default_rng(5)
    n, L = 3000, 24.0
    box = np.full(3, L)
    pos = rng.uniform(0, L, (n, 3))
    reach = 4.0
    lo, hi = -np.full(3, reach), box + reach
    eb = capi.EdgeBuilder()
    x, y, z = (to_dev(pos[:, k]) for k in range(3))
    img = eb.images(x, y, z, None, box, np.zeros(3), lo, hi, (1, 1, 0))       # two image axes, one without
    n_all = img["n_all"]
    owner = img["owner"].cpu().numpy()
    assert n_all > n and np.all(img["shift"][2].cpu().numpy() == 0.0)
    f = rng.normal(size=(n_all, 3))
    before = rng.normal(size=(n, 3))
    fdev = [to_dev(f[:, k]) for k in range(3)]
    for n_out, with_images in ((-1, True), (n // 3, True), (-1, False)):
        t = [to_dev(before[:, k]) for k in range(3)]
        eb.fold_image_forces(*fdev, *t, n_out=n_out, with_images=with_images)
        got = np.stack([v.cpu().numpy() for v in t], axis=1)
        want = co.fold_image_forces(f, n, owner, before, n_out=None if n_out < 0 else n_out, with_images=with_images)
        assert np.array_equal(got, want)
    # momentum: what went in on images comes out on atoms
    t = [torch.zeros(n, dtype=torch.float64, device="cuda") for _ in range(3)]
    eb.fold_image_forces(*fdev, *t)
    assert np.allclose(np.stack([v.cpu().numpy() for v in t], axis=1).sum(0), f.sum(0), rtol=0, atol=1e-9)
    all_pos = np.stack([img[k].cpu().numpy() for k in "xyz"], axis=1)
    got = eb.virial_from_forces(img["x"].clone(), img["y"].clone(), img["z"].clone(), *fdev)
    want = co.virial_from_forces(all_pos, f)
    scale = np.abs(all_pos * f).sum()
    assert np.abs(got - want).max() <= 1e-13 * scale
    eb.close()



@pytest.mark.parametrize("halo_extra", [0.0, 1.3])
def test_edges_under_an_eight_way_decomposition_equal_the_periodic_graph(cuda_device, halo_extra):
    """The radius graph of a periodic solid built brick by brick, as the model runner of one rank is fed: 2 x 2 x 2 bricks,
    each with its owned atoms and the ghost atoms of a halo as wide as the cutoff (second case: the reference's halo,
    cutoff + skin + 1 A, here + 1.3 A) as explicit, image-shifted atoms, no periodic images (every axis is decomposed).
    The edges centred on owned atoms, translated to global ids and lattice shifts, are over all bricks exactly the
    periodic graph of the undivided box."""
    import torch
    s = syn.disordered_solid_lattice(28, seed=7)              # 21,952 atoms, box 76 A, cutoff 5 A
    cutoff = s.cutoff
    halo = cutoff + halo_extra
    eb = capi.EdgeBuilder()
    x, y, z = (to_dev(s.pos[:, k]) for k in range(3))
    src, dst, shift, _ = eb.build_periodic(x, y, z, s.box, cutoff)
    whole = np.concatenate([np.stack([src.cpu().numpy(), dst.cpu().numpy()], axis=0).astype(np.int64),
                            shift.cpu().numpy().T.astype(np.int64)])
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    parts = []
    for brick in syn.brick_decompose(s.pos, s.box, (2, 2, 2), halo):
        own, gsrc, gimg = brick["owned"], brick["ghost_src"], brick["ghost_image"]
        pos = np.concatenate([wrapped[own], wrapped[gsrc] + gimg * s.box])
        gid = np.concatenate([own, gsrc])
        image = np.concatenate([np.zeros((len(own), 3), dtype=np.int64), gimg.astype(np.int64)])
        cols = [to_dev(pos[:, k]) for k in range(3)]
        idx, _ = eb.build(*cols, cutoff, lo=brick["lo"] - halo - 1e-9, hi=brick["hi"] + halo + 1e-9)
        e = idx.cpu().numpy()
        e = e[:, e[0] < len(own)]                             # the edges an owned atom is the centre of
        assert len(gsrc) > 0 and e.shape[1] > 0
        parts.append(np.concatenate([gid[e], image[e[1]].T]))
    got = np.concatenate(parts, axis=1)
    assert got.shape == whole.shape
    assert np.array_equal(canon(got.astype(np.float64)), canon(whole.astype(np.float64)))
    eb.close()


def test_full_size_disordered_solid_whole_and_in_eight_bricks(cuda_device):
    """The 1,000,000-atom disordered solid (uniform random placement with a 1.8 A minimum distance, cutoff 5 A) at full
    size: the periodic radius graph has the edge count and the order-independent checksum of the (centre, neighbour,
    lattice shift) set that the CPU oracle gave (tests/golden/make_edge_checksums.py); built brick by brick under a
    2 x 2 x 2 decomposition with a cutoff-wide halo of explicit ghost atoms, the edges centred on owned atoms, translated
    to global ids, add up to the same count and checksum, with the fixture's owned and ghost counts per brick."""
    import json
    import os
    import sys
    import torch
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, here)
    from pair_checksum import MASK, checksum_torch
    with open(os.path.join(here, "full_size_edge_checksums.json")) as f:
        want = json.load(f)
    s = syn.disordered_solid(want["atoms"])
    cutoff = want["cutoff"]
    eb = capi.EdgeBuilder()
    x, y, z = (to_dev(s.pos[:, k]) for k in range(3))
    src, dst, shift, vec = eb.build_periodic(x, y, z, s.box, cutoff)
    sh = shift.to(torch.int64)
    code = dst.to(torch.int64) * 27 + (sh[:, 0] + 1) * 9 + (sh[:, 1] + 1) * 3 + (sh[:, 2] + 1)
    got = checksum_torch(src.to(torch.int64), code)
    assert got == (want["edges"], int(want["sum1"]), int(want["sum2"]))
    assert float((vec * vec).sum(1).max()) < cutoff * cutoff * (1 + 1e-6)
    del src, dst, shift, vec, sh, code
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    count = s1 = s2 = 0
    for brick, numbers in zip(syn.brick_decompose(s.pos, s.box, (2, 2, 2), cutoff), want["bricks"]):
        own, gsrc, gimg = brick["owned"], brick["ghost_src"], brick["ghost_image"]
        assert (len(own), len(gsrc)) == (numbers["owned"], numbers["ghosts"])
        pos = np.concatenate([wrapped[own], wrapped[gsrc] + gimg * s.box])
        gid = to_dev(np.concatenate([own, gsrc]), dtype=torch.int64)
        image = to_dev(np.concatenate([np.zeros((len(own), 3), dtype=np.int64), gimg.astype(np.int64)]), dtype=torch.int64)
        cols = [to_dev(pos[:, k]) for k in range(3)]
        idx, _ = eb.build(*cols, cutoff, lo=brick["lo"] - cutoff - 1e-9, hi=brick["hi"] + cutoff + 1e-9)
        centred = idx[0] < len(own)
        i, j = idx[0][centred], idx[1][centred]
        im = image[j]
        c, a, b = checksum_torch(gid[i], gid[j] * 27 + (im[:, 0] + 1) * 9 + (im[:, 1] + 1) * 3 + (im[:, 2] + 1))
        count, s1, s2 = count + c, (s1 + a) & MASK, (s2 + b) & MASK
    assert (count, s1, s2) == (want["edges"], int(want["sum1"]), int(want["sum2"]))
    eb.close()
