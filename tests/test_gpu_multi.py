"""Multi-GPU parity test (needs two CUDA devices; skipped otherwise): two ranks over NCCL run the real contexts through
migration, ghost plan, positions-only refresh and list rebuilds; forces, energy and the trajectory must match the
undivided system computed by the CPU oracle."""
import os
import socket

import numpy as np
import pytest
import torch

from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(worker_fn, args, world, limit_s=240):
    """Runs worker_fn(rank, *args) in `world` child processes; a rank that has not finished within the limit is terminated
    (by its own pid) and the test fails, so that a communication hang cannot hold the GPUs."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=worker_fn, args=(rank, *args)) for rank in range(world)]
    for p in procs:
        p.start()
    import time
    deadline = time.time() + limit_s
    for p in procs:
        p.join(max(0.0, deadline - time.time()))
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    for p in hung:
        p.join(10)
        if p.is_alive():
            p.kill()
    assert not hung, f"{len(hung)} rank(s) did not finish within {limit_s} s"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def worker(rank, world, port, steps, dt, out_path):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    from deepscalemd_b200 import capi, domain
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=device)
    s = syn.fcc_lj(10, seed=44)
    dec = domain.Decomposition(s.box, world, rank)
    mine = np.nonzero(dec.owner_of(s.pos) == rank)[0]
    halo = s.cutoff + s.skin
    ctx = capi.Context(s.n * 2, device=rank)
    lo = [dec.lo[a] if dec.split[a] else 0.0 for a in range(3)]
    hi = [dec.hi[a] if dec.split[a] else 0.0 for a in range(3)]
    ctx.set_box(s.box, (1, 1, 1), lo, hi, halo + 2 * s.skin)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    ctx.upload(wrapped[mine], vel=s.vel[mine], mass=s.mass[mine], types=s.types[mine], gid=mine.astype(np.int32))
    run = domain.DomainRunner(ctx, dec, halo, device)
    run.rebuild()
    ctx.compute_forces(capi.PHASE_FULL, True)
    first = run.global_scalars()
    n_owned, n_total = ctx.counts()
    gid_first = ctx.download("global_id", n_owned)
    f_first = np.stack([ctx.download(k, n_owned) for k in ("fx", "fy", "fz")], axis=1)
    for _ in range(steps):
        run.step(dt, 1.0, s.skin, 0.5, lagged=True, overlap=True)
    torch.cuda.synchronize()
    n_owned, _ = ctx.counts()
    result = dict(gid_first=gid_first, f_first=f_first, first=first, ghosts=n_total - n_owned,
                  gid=ctx.download("global_id", n_owned),
                  pos=np.stack([ctx.download(k, n_owned) for k in "xyz"], axis=1), rebuilds=run.rebuilds,
                  worst=run.worst_disp_sq)
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        torch.save(gathered, out_path)
    ctx.close()
    dist.destroy_process_group()


def worker_native(rank, world, port, steps, dt, out_path):
    """The same run through the native domain code (dsmd_domain_*: its own NCCL communicator; gloo only carries the
    unique id and the result gathering)."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    from deepscalemd_b200 import capi, domain
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    s = syn.fcc_lj(10, seed=44)
    dec = domain.Decomposition(s.box, world, rank)
    mine = np.nonzero(dec.owner_of(s.pos) == rank)[0]
    halo = s.cutoff + s.skin
    ctx = capi.Context(s.n * 2, device=rank)
    lo = [dec.lo[a] if dec.split[a] else 0.0 for a in range(3)]
    hi = [dec.hi[a] if dec.split[a] else 0.0 for a in range(3)]
    ctx.set_box(s.box, (1, 1, 1), lo, hi, halo + 2 * s.skin)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    ctx.upload(wrapped[mine], vel=s.vel[mine], mass=s.mass[mine], types=s.types[mine], gid=mine.astype(np.int32))
    uid = [capi.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    dom = capi.Domain(ctx, rank, world, dec.dims, s.box, halo, s.skin, uid[0])
    dom.rebuild()
    ctx.compute_forces(capi.PHASE_FULL, True)
    sc = ctx.read_scalars()
    first = torch.tensor([sc["pe"], sc["virial"]], dtype=torch.float64)
    dist.all_reduce(first)
    n_owned, n_total = ctx.counts()
    gid_first = ctx.download("global_id", n_owned)
    f_first = np.stack([ctx.download(k, n_owned) for k in ("fx", "fy", "fz")], axis=1)
    dom.run(steps, dt, 1.0, 0.5)
    torch.cuda.synchronize()
    n_owned, n_total_now = ctx.counts()
    st = dom.stats()
    # the host-buffer call: the owned atoms' positions in, forces out; equal to the device-resident evaluation
    ctx.compute_forces(capi.PHASE_FULL)
    f_device = np.stack([ctx.download(k, n_owned) for k in ("fx", "fy", "fz")], axis=1)
    host_in = [torch.from_numpy(ctx.download(k, n_owned)).pin_memory() for k in "xyz"]
    host_out = [torch.zeros(n_owned, dtype=torch.float64).pin_memory() for _ in range(3)]
    dom.forces_host(*[t.data_ptr() for t in host_in], *[t.data_ptr() for t in host_out], n_owned, rebuild=False)
    f_host = np.stack([t.numpy().copy() for t in host_out], axis=1)
    host_call_ok = bool(np.abs(f_host - f_device).max() <= 1e-5 * np.abs(f_device).max())   # two passes against one: fp32 partial sums differ in the last bits
    too_short = False
    try:
        dom.forces_host(*[t.data_ptr() for t in host_in], *[t.data_ptr() for t in host_out], n_owned - 1, rebuild=False)
    except capi.DsmdError as err:
        too_short = err.code == capi.ERR_CAPACITY
    result = dict(gid_first=gid_first, f_first=f_first, first=dict(pe=float(first[0]), virial=float(first[1])),
                  ghosts=n_total - n_owned, gid=ctx.download("global_id", n_owned),
                  pos=np.stack([ctx.download(k, n_owned) for k in "xyz"], axis=1), rebuilds=st["rebuilds"],
                  worst=st["worst_disp_sq"], peers=dom.peers(), host_call_ok=host_call_ok, too_short=too_short)
    # -- the exchanges of the MLIP path along the same ghost plan ---------------------------------------------------------
    device = torch.device("cuda", rank)
    gid_all = torch.tensor(ctx.download("global_id", n_total_now), device=device, dtype=torch.float64)
    is_ghost = torch.arange(n_total_now, device=device) >= n_owned
    # forward: a ghost row becomes a copy of its owner's row (rows carry the global id, so it can be checked locally)
    for dtype in (torch.float32, torch.float64):
        field = torch.stack([gid_all + 0.25 * w for w in range(5)], dim=1).to(dtype)
        want = field.clone()
        field[is_ghost] = -1.0
        dom.exchange_field(field, reverse=False)
        torch.cuda.synchronize()
        result[f"forward_ok_{field.element_size()}"] = bool(torch.equal(field, want))
    # reverse: every ghost row holds (1, 2, 3); owners end up with (number of ghost copies elsewhere) x (1, 2, 3)
    grad = torch.zeros(n_total_now, 3, device=device, dtype=torch.float64)
    grad[is_ghost] = torch.tensor([1.0, 2.0, 3.0], device=device, dtype=torch.float64)
    dom.exchange_field(grad, reverse=True)
    # the force version of the same thing, on the context's own force arrays
    f = [capi._tensor_from_ptr(ctx.device_pointer(k), (n_total_now,), torch.float64, device) for k in ("fx", "fy", "fz")]
    for k in range(3):
        f[k].zero_()
        f[k][is_ghost] = float(k + 1)
    dom.reverse_forces()
    torch.cuda.synchronize()
    result["reverse_field"] = grad[:n_owned].cpu().numpy()
    result["reverse_force"] = np.stack([f[k][:n_owned].cpu().numpy() for k in range(3)], axis=1)
    result["ghost_gid"] = ctx.download("global_id", n_total_now)[n_owned:]
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        torch.save(gathered, out_path)
    dom.close()
    ctx.close()
    dist.destroy_process_group()


def chain_system():
    return syn.chain_fluid(4, 8, spacing=14.0, seed=14)      # 64 flexible chains, box 56 A


def chain_setup(ctx, s, n_global):
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    ctx.set_coulomb(True)
    ctx.set_exclusions(n_global, s.exclusions)
    ctx.set_bonded(n_global, s.bonded)


def worker_chains(rank, world, port, steps, dt, out_path):
    """Flexible chains over two bricks: pair and bonded forces of the first evaluation, then `steps` steps of the native loop."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    from deepscalemd_b200 import capi, domain
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    s = chain_system()
    dec = domain.Decomposition(s.box, world, rank)
    mine = np.nonzero(dec.owner_of(s.pos) == rank)[0]
    halo = s.cutoff + s.skin
    ctx = capi.Context(s.n * 2, device=rank)
    lo = [dec.lo[a] if dec.split[a] else 0.0 for a in range(3)]
    hi = [dec.hi[a] if dec.split[a] else 0.0 for a in range(3)]
    ctx.set_box(s.box, (1, 1, 1), lo, hi, halo + 2 * s.skin)
    chain_setup(ctx, s, s.n)
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    ctx.upload(wrapped[mine], vel=s.vel[mine], mass=s.mass[mine], types=s.types[mine], charge=s.charge[mine],
               gid=mine.astype(np.int32))
    uid = [capi.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    dom = capi.Domain(ctx, rank, world, dec.dims, s.box, halo, s.skin, uid[0])
    dom.rebuild()

    def energies():
        ctx.compute_forces(capi.PHASE_FULL, True)
        ctx.compute_bonded()
        v = torch.tensor([ctx.read_scalars()["pe"], ctx.read_bonded_scalars()["pe"], ctx.kinetic_energy() / s.force_to_accel],
                         dtype=torch.float64)
        dist.all_reduce(v)
        return v.tolist()

    first = energies()
    n_owned, _ = ctx.counts()
    result = dict(first=first, gid_first=ctx.download("global_id", n_owned),
                  f_first=np.stack([ctx.download(k, n_owned) for k in ("fx", "fy", "fz")], axis=1))
    dom.run(steps, dt, s.force_to_accel, 0.5)
    torch.cuda.synchronize()
    result["last"] = energies()
    result["rebuilds"] = dom.stats()["rebuilds"]
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        torch.save(gathered, out_path)
    dom.close()
    ctx.close()
    dist.destroy_process_group()


def test_bonded_terms_on_two_gpus_equal_one_gpu(tmp_path):
    """Flexible chains cut by a brick boundary: the first evaluation's forces (pair + bonded) and energies equal the
    one-GPU values, and after 100 steps of the native loop the two runs' energies still agree (terms that cross the
    boundary are evaluated on both ranks, each keeping the forces of its own atoms)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    from deepscalemd_b200 import capi
    steps, dt = 100, 0.5
    out = str(tmp_path / "chains.pt")
    run_ranks(worker_chains, (2, free_port(), steps, dt, out), 2)
    parts = torch.load(out, weights_only=False)
    s = chain_system()
    ctx = capi.Context(s.n)
    ctx.set_box(s.box)
    chain_setup(ctx, s, s.n)
    ctx.upload(s.pos, vel=s.vel, mass=s.mass, types=s.types, charge=s.charge)
    ctx.build_neighbor_list()

    def energies():
        ctx.compute_forces(capi.PHASE_FULL, True)
        ctx.compute_bonded()
        return [ctx.read_scalars()["pe"], ctx.read_bonded_scalars()["pe"], ctx.kinetic_energy() / s.force_to_accel]

    want = energies()
    gid = ctx.download("global_id", s.n)
    f_want = np.empty((s.n, 3))
    f_want[gid] = np.stack([ctx.download(k, s.n) for k in ("fx", "fy", "fz")], axis=1)
    f_got = np.empty_like(f_want)
    for p in parts:
        f_got[p["gid_first"]] = p["f_first"]
    rms = lambda a: np.sqrt((a * a).sum(1).mean())
    assert rms(f_got - f_want) <= 1e-5 * rms(f_want)
    got = parts[0]["first"]
    assert abs(got[0] - want[0]) <= 1e-5 * abs(want[1]) and abs(got[1] - want[1]) <= 1e-10 * abs(want[1])
    assert abs(got[2] - want[2]) <= 1e-10 * want[2]
    ctx.run_nve(steps, dt, s.force_to_accel, 0.5, 0, True)
    after = energies()
    last = parts[0]["last"]
    total0 = sum(want)
    assert abs(sum(last) - total0) < 0.02 * want[2] and abs(sum(after) - total0) < 0.02 * want[2]
    assert abs(last[1] - after[1]) < 0.05 * want[2]          # the same physics: bonded energy after 100 steps agrees closely
    assert abs(after[1] - want[1]) > 0.05 * want[2]
    ctx.close()


@pytest.mark.parametrize("which", ["torch_distributed", "native"])
def test_two_gpus_equal_the_undivided_system(tmp_path, which):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    steps, dt = 40, 0.005
    out = str(tmp_path / "out.pt")
    run_ranks(worker if which == "torch_distributed" else worker_native, (2, free_port(), steps, dt, out), 2)
    parts = torch.load(out, weights_only=False)
    s = syn.fcc_lj(10, seed=44)
    pos = [np.ascontiguousarray(s.pos[:, k]) for k in range(3)]
    vel = [np.ascontiguousarray(s.vel[:, k]) for k in range(3)]
    c6, c12 = co.lj_tables(s.eps, s.sig)

    def force():
        p = co.pairs(*pos, s.n, s.box, search=s.cutoff)
        f, sc = co.forces(*pos, s.n, s.box, p, c6, c12, s.cutoff)
        return [np.ascontiguousarray(f[:, k]) for k in range(3)], sc

    frc, sc0 = force()
    f0 = np.stack(frc, axis=1)
    gid = np.concatenate([p["gid_first"] for p in parts])
    assert np.array_equal(np.sort(gid), np.arange(s.n))
    f = np.empty_like(f0)
    for p in parts:
        f[p["gid_first"]] = p["f_first"]
    rms = lambda a: np.sqrt((a * a).sum(1).mean())
    assert rms(f - f0) <= 1e-5 * rms(f0)
    assert abs(parts[0]["first"]["pe"] - sc0["pe"]) <= 1e-6 * abs(sc0["pe"])
    assert abs(parts[0]["first"]["virial"] - sc0["virial"]) <= 1e-6 * abs(sc0["virial"])
    assert all(p["ghosts"] > 0 for p in parts)
    for _ in range(steps):
        co.vv_half(True, dt, 1.0, pos, vel, frc, s.mass)
        frc, _ = force()
        co.vv_half(False, dt, 1.0, pos, vel, frc, s.mass)
    gid = np.concatenate([p["gid"] for p in parts])
    assert np.array_equal(np.sort(gid), np.arange(s.n))
    got = np.empty((s.n, 3))
    for p in parts:
        got[p["gid"]] = p["pos"]
    d = got - np.stack(pos, axis=1)
    d -= s.box * np.round(d / s.box)
    assert np.abs(d).max() < 1e-4      # fp32 pair forces: round-off grows along the (chaotic) trajectory
    assert parts[0]["rebuilds"] >= 4
    assert parts[0]["worst"] <= (0.5 * s.skin) ** 2 * 1.2
    if which == "native":
        # two bricks are each other's only neighbour rank: one message each way per exchange
        assert all(p["peers"]["ranks"] == [1 - r] and p["peers"]["messages_per_exchange"] == 2 for r, p in enumerate(parts))
        assert all(p["forward_ok_4"] and p["forward_ok_8"] for p in parts)
        assert all(p["host_call_ok"] and p["too_short"] for p in parts)
        copies = np.zeros(s.n)
        for p in parts:
            np.add.at(copies, p["ghost_gid"], 1.0)             # how often each atom is a ghost somewhere
        assert copies.max() >= 1
        for p in parts:
            want = copies[p["gid"]][:, None] * np.array([1.0, 2.0, 3.0])
            assert np.array_equal(p["reverse_field"], want)
            assert np.array_equal(p["reverse_force"], want)
