"""CPU tests of the multi-rank path: two ranks over gloo run the domain logic (migration, ghost plan, positions-only
refresh, rebuild vote) against a numpy stand-in for the device context; results must equal the undivided system's."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepscalemd_b200 import domain
from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


_PORT = {}


def free_port_once():
    """One port per test invocation, shared by both ranks."""
    key = os.environ.get("PYTEST_CURRENT_TEST", "")
    if key not in _PORT:
        _PORT[key] = free_port()
    return _PORT[key]


def reference_md(s, steps, dt):
    pos = [np.ascontiguousarray(s.pos[:, k]) for k in range(3)]
    vel = [np.ascontiguousarray(s.vel[:, k]) for k in range(3)]
    c6, c12 = co.lj_tables(s.eps, s.sig)

    def force():
        p = co.pairs(*pos, s.n, s.box, search=s.cutoff)
        f, sc = co.forces(*pos, s.n, s.box, p, c6, c12, s.cutoff)
        return [np.ascontiguousarray(f[:, k]) for k in range(3)], sc

    frc, sc0 = force()
    f0 = np.stack(frc, axis=1)
    for _ in range(steps):
        co.vv_half(True, dt, 1.0, pos, vel, frc, s.mass)
        frc, sc = force()
        co.vv_half(False, dt, 1.0, pos, vel, frc, s.mass)
    return f0, sc0, np.stack(pos, axis=1), sc


def worker(rank, world, port, dims, steps, dt, out_path):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from fake_context import FakeContext
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    s = syn.fcc_lj(8, seed=33)
    dec = domain.Decomposition(s.box, world, rank, dims=dims)
    mine = np.nonzero(dec.owner_of(s.pos) == rank)[0]
    ctx = FakeContext(s.n, s.box, s.eps, s.sig, s.cutoff, s.skin)
    ctx.set_split(dec.split)
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    ctx.upload(wrapped[mine], s.vel[mine], s.mass[mine], mine.astype(np.int32))
    run = domain.DomainRunner(ctx, dec, s.cutoff + s.skin, "cpu")
    run.rebuild()
    ctx.compute_forces(0, True)
    first = run.global_scalars()
    n_owned, n_total = ctx.counts()
    f_first = np.stack([ctx.a[k][:n_owned].copy() for k in ("fx", "fy", "fz")], axis=1)
    gid_first = ctx.gid[:n_owned].copy()
    ghosts_first = n_total - n_owned
    for _ in range(steps):
        run.step(dt, 1.0, s.skin, 0.5, lagged=False, overlap=True, want_energy=True)
    last = run.global_scalars()
    n_owned, _ = ctx.counts()
    result = dict(gid_first=gid_first, f_first=f_first, first=first, ghosts_first=ghosts_first,
                  gid=ctx.gid[:n_owned].copy(), pos=np.stack([ctx.a[k][:n_owned] for k in "xyz"], axis=1), last=last,
                  rebuilds=run.rebuilds)
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        torch.save(gathered, out_path)
    dist.destroy_process_group()


@pytest.mark.parametrize("dims", [(2, 1, 1), (1, 2, 1), (2, 2, 2)])
def test_ranks_equal_the_undivided_system(tmp_path, dims):
    """Two ranks (one split axis) and eight ranks (2 x 2 x 2: every axis split, 26 directions towards 7 peers, several
    messages per peer)."""
    steps, dt = 25, 0.005
    world = dims[0] * dims[1] * dims[2]
    out = str(tmp_path / "out.pt")
    procs = [mp.get_context("spawn").Process(target=worker, args=(rank, world, free_port_once(), dims, steps, dt, out))
             for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    assert not hung and all(p.exitcode == 0 for p in procs)
    parts = torch.load(out, weights_only=False)
    s = syn.fcc_lj(8, seed=33)
    f0, sc0, pos_end, sc_end = reference_md(s, steps, dt)
    # first evaluation: every atom owned exactly once, forces and energy equal the undivided system's
    gid = np.concatenate([p["gid_first"] for p in parts])
    assert np.array_equal(np.sort(gid), np.arange(s.n))
    f = np.empty_like(f0)
    for p in parts:
        f[p["gid_first"]] = p["f_first"]
    assert np.abs(f - f0).max() < 1e-9
    assert abs(parts[0]["first"]["pe"] - sc0["pe"]) < 1e-9 * abs(sc0["pe"])
    assert abs(parts[0]["first"]["virial"] - sc0["virial"]) < 1e-9 * abs(sc0["virial"])
    assert all(p["ghosts_first"] > 0 for p in parts)
    # after MD with migration, refresh and rebuilds: same trajectory (positions modulo the box) and energy
    gid = np.concatenate([p["gid"] for p in parts])
    assert np.array_equal(np.sort(gid), np.arange(s.n))
    pos = np.empty_like(pos_end)
    for p in parts:
        pos[p["gid"]] = p["pos"]
    d = pos - pos_end
    d -= s.box * np.round(d / s.box)
    assert np.abs(d).max() < 1e-9
    assert abs(parts[0]["last"]["pe"] - sc_end["pe"]) < 1e-9 * abs(sc_end["pe"])
    assert parts[0]["rebuilds"] >= 3 and all(p["rebuilds"] == parts[0]["rebuilds"] for p in parts)


def test_brick_grids_and_directions():
    box = np.array([10.0, 10.0, 10.0])
    assert domain.grid_dims(1, box) == (1, 1, 1)
    assert domain.grid_dims(2, box) == (2, 1, 1)
    assert domain.grid_dims(4, box) == (2, 2, 1)
    assert domain.grid_dims(8, box) == (2, 2, 2)
    assert domain.grid_dims(4, np.array([40.0, 10.0, 10.0])) == (4, 1, 1)
    for world, n_dirs in ((2, 2), (4, 8), (8, 26)):
        decs = [domain.Decomposition(box, world, r) for r in range(world)]
        for d in decs:
            assert len(d.directions) == n_dirs
            for dr in d.directions:
                # what I send along e arrives at dest along e, and dest names me as the source of that direction
                other = decs[dr.dest].directions[dr.index]
                assert other.src == d.rank and other.e == dr.e
        # owners tile the box
        pos = np.random.default_rng(0).uniform(-5, 15, (2000, 3))
        owner = decs[0].owner_of(pos)
        w = pos - box * np.floor(pos / box)
        for d in decs:
            inside = np.all((w >= d.lo) & (w < d.hi), axis=1)
            assert np.array_equal(inside, owner == d.rank)


def field_worker(rank, world, port, dims, out_path):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from fake_context import FakeContext
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    s = syn.fcc_lj(8, seed=33)
    dec = domain.Decomposition(s.box, world, rank, dims=dims)
    mine = np.nonzero(dec.owner_of(s.pos) == rank)[0]
    ctx = FakeContext(s.n, s.box, s.eps, s.sig, s.cutoff, s.skin)
    ctx.set_split(dec.split)
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    ctx.upload(wrapped[mine], s.vel[mine], s.mass[mine], mine.astype(np.int32))
    run = domain.DomainRunner(ctx, dec, s.cutoff + s.skin, "cpu")
    run.rebuild()
    n_owned, n_total = ctx.counts()
    gid = torch.from_numpy(ctx.gid[:n_total].astype(np.int64))
    # forward: every ghost row becomes its owner's row
    field = torch.zeros((n_total, 3), dtype=torch.float64)
    field[:n_owned, 0] = gid[:n_owned].double()
    field[:n_owned, 1] = 2.0 * gid[:n_owned].double() + 1.0
    field[:n_owned, 2] = float(rank)
    run.exchange_field(field)
    forward_ok = bool(torch.equal(field[:, 0], gid.double()) and torch.equal(field[:, 1], 2.0 * gid.double() + 1.0))
    owner_rank = torch.from_numpy(dec.owner_of(s.pos)[ctx.gid[:n_total]].astype(np.float64))
    forward_ok = forward_ok and bool(torch.equal(field[:, 2], owner_rank))
    # reverse: every ghost row is added to its owner's row (float32 this time)
    back = torch.zeros((n_total, 2), dtype=torch.float32)
    back[n_owned:, 0] = 1.0
    back[n_owned:, 1] = gid[n_owned:].float()
    back[:n_owned, 0] = 100.0
    run.exchange_field(back, reverse=True)
    result = dict(forward_ok=forward_ok, gid=ctx.gid[:n_owned].copy(), copies=back[:n_owned, 0].numpy() - 100.0,
                  gid_sum=back[:n_owned, 1].numpy(), ghosts=n_total - n_owned)
    try:
        run.exchange_field(torch.zeros((n_total + 1, 2), dtype=torch.float64))
        result["refused"] = False
    except ValueError:
        result["refused"] = True
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        torch.save(gathered, out_path)
    dist.destroy_process_group()


@pytest.mark.parametrize("dims", [(2, 1, 1), (2, 2, 2)])
def test_feature_field_exchange_along_the_ghost_plan(tmp_path, dims):
    """Forward copies owner rows into every ghost copy; reverse adds every ghost copy's row to its owner (the adjoint):
    how often an atom is a ghost somewhere follows from the geometry alone (built here independently)."""
    world = dims[0] * dims[1] * dims[2]
    out = str(tmp_path / "out.pt")
    procs = [mp.get_context("spawn").Process(target=field_worker, args=(rank, world, free_port_once(), dims, out))
             for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    assert not hung and all(p.exitcode == 0 for p in procs)
    parts = torch.load(out, weights_only=False)
    assert all(p["forward_ok"] and p["refused"] for p in parts)
    s = syn.fcc_lj(8, seed=33)
    want = np.zeros(s.n)
    for brick in syn.brick_decompose(s.pos, s.box, dims, s.cutoff + s.skin):
        want += np.bincount(brick["ghost_src"], minlength=s.n)
    got = np.zeros(s.n)
    gid_sum = np.zeros(s.n)
    for p in parts:
        got[p["gid"]] = p["copies"]
        gid_sum[p["gid"]] = p["gid_sum"]
    assert np.array_equal(got, want) and want.sum() == sum(p["ghosts"] for p in parts) and want.max() >= (1 if world == 2 else 3)
    assert np.array_equal(gid_sum, want * np.arange(s.n))
