"""Multi-GPU leg of bench.py: strong scaling of the 4,000,000-atom LJ system over the GPUs of one node, one process per
GPU (torchrun), bricks of a spatial decomposition, ghost exchange over NCCL point-to-point."""
from __future__ import annotations

import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist


def run(args):
    import bench   # the driver script: shared constants and helpers
    from deepscalemd_b200 import capi, domain

    os.environ.setdefault("NCCL_DEBUG", "WARN")   # keep NCCL's banner off stdout: rank 0 prints exactly one JSON line
    # point-to-point messages and an 8-byte all-reduce gain nothing from NVLink multicast objects: do not set them up
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # Watchdog: a communication hang must end this process (and free its GPU) instead of running into the caller's
    # limit; the limit is generous for the work below (set-up 15 s, MD a few seconds, timing sections a few seconds).
    import threading

    def give_up():
        if rank == 0:
            print(json.dumps({"metric": "atom-steps/s", "value": None, "n_gpus": world,
                              "error": "multi-GPU benchmark did not finish within its time limit"}), flush=True)
        os._exit(3)

    watchdog = threading.Timer(float(os.environ.get("DSMD_BENCH_LIMIT_S", "240")), give_up)
    watchdog.daemon = True
    watchdog.start()
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if not dist.is_initialized():
        # control plane only (unique id, timing reductions): the data plane is the library's own NCCL communicator
        dist.init_process_group("gloo")
    stream = torch.cuda.current_stream()
    hbm_peak, peak_kind = bench.measured_peaks()

    s = bench.fcc_for(args.workload)
    dec = domain.Decomposition(s.box, world, rank)
    owner = dec.owner_of(s.pos)
    mine = np.nonzero(owner == rank)[0]
    halo = s.cutoff + s.skin
    capacity = int(len(mine) * 2.2) + 200_000
    ctx = capi.Context(capacity, device=local)
    lo = [dec.lo[a] if dec.split[a] else 0.0 for a in range(3)]
    hi = [dec.hi[a] if dec.split[a] else 0.0 for a in range(3)]
    ctx.set_box(s.box, (1, 1, 1), lo, hi, halo + 2.0 * s.skin)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    wrapped = s.pos - s.box * np.floor(s.pos / s.box)
    ctx.upload(wrapped[mine], vel=s.vel[mine], mass=s.mass[mine], types=s.types[mine], gid=mine.astype(np.int32))
    uid = [capi.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    dom = capi.Domain(ctx, rank, world, dec.dims, s.box, halo, s.skin, uid[0])
    dom.rebuild(stream)

    def total_energy():
        ctx.compute_forces(capi.PHASE_FULL, True, stream)
        v = torch.tensor([ctx.read_scalars(stream)["pe"] + ctx.kinetic_energy(stream)], dtype=torch.float64)
        dist.all_reduce(v)
        return float(v.item())

    e0 = total_energy()

    def md(n):
        dom.run(n, bench.DT, 1.0, 0.5, stream)

    md(bench.SETTLE_STEPS)      # set-up: through the first in-loop rebuild with atoms that really migrate
    md(args.warmup)
    sampler = bench.ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0, rebuilds0 = ctx.launch_count() + dom.stats()["launches"], dom.stats()["rebuilds"]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    start.record(stream)
    md(args.steps)
    stop.record(stream)
    torch.cuda.synchronize()
    elapsed = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64)
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    dist.barrier()
    elapsed_ms = float(elapsed.item())
    st = dom.stats()
    launches = ctx.launch_count() + st["launches"] - launches0
    rebuilds = st["rebuilds"] - rebuilds0
    clocks = sampler.stop() if sampler else None
    n_owned, n_total = ctx.counts()

    e1 = total_energy()
    # phase breakdown of a short profiled run (synchronises every step: not part of the timed region)
    dom.profile(True)
    md(min(args.steps, 60))
    phases = dom.profile(False)

    # per-kernel time of the pair kernel on this rank's share (roofline of the dominant kernel)
    stats = ctx.list_stats()
    t_pair = bench.time_calls(lambda: ctx.compute_forces(capi.PHASE_FULL, False, stream), 20, stream)
    p_list_local = stats["directed_entries"] / 2.0
    pair_bytes = 16.0 * n_total + 4.0 * p_list_local + 24.0 * n_owned
    flops = ctx.fma_probe(1, stream)
    t_probe = bench.time_calls(lambda: ctx.fma_probe(20000, stream), 3, stream)
    fp32_peak = flops * 20000 / (t_probe * 1e-3) / 1e12
    # pairs inside the cutoff seen from this rank: owned-owned once, owned-ghost half (the other half is the neighbour's)
    ctx.compute_forces(capi.PHASE_FULL, True, stream)
    p_cut_local = ctx.read_scalars(stream)["pairs_in_cutoff"]
    pair_flops = 8.0 * p_list_local + 19.0 * p_cut_local

    # end to end: host positions in, forces out, ghost refresh in between (every rank its own atoms)
    # A failure of this part (a status from the library, a rank that stopped answering: the waits give up after 20 s) must
    # not cost the line its device-timed numbers: every rank falls through to the same reductions below, and the entry
    # then carries the error instead of a value. No host-side barrier sits inside the part that may fail (ranks that have
    # left it and ranks still inside it would otherwise meet in different collectives); the calls themselves keep the
    # ranks in step through their exchanges.
    e2e_steps = max(4, min(args.steps, 40))
    cadence = max(1, round(args.steps / max(rebuilds, 1)))
    e2e_error, e2e_seconds = None, float("nan")
    dist.barrier()
    try:
        dom.set_wait_limit(20.0)
        # The host keeps handing over the same positions. They are taken right after a rebuild, so that every atom lies in
        # its owner's brick: the rebuilds inside the loop then move no atom and the owned set and its order stay as they
        # are (a rebuild after a drift would hand atoms to other ranks, and positions indexed by the old order would be wrong).
        dom.rebuild(stream)
        n_owned, n_total = ctx.counts()
        room = n_owned + 4096
        host = [torch.zeros(room, dtype=torch.float64).pin_memory() for _ in range(3)]
        for k, name in enumerate(("x", "y", "z")):
            host[k][:n_owned] = torch.from_numpy(ctx.download(name, n_owned))
        hf = [torch.empty(room, dtype=torch.float64).pin_memory() for _ in range(3)]
        calls = {"k": 0}

        def e2e_call():
            # what the single-GPU end-to-end call does, per rank, in one native call: positions in, rebuild (migration,
            # ghost plan, list) at the MD run's cadence or else pack + ghost refresh beside the interior pass, forces out
            dom.forces_host(host[0].data_ptr(), host[1].data_ptr(), host[2].data_ptr(), hf[0].data_ptr(), hf[1].data_ptr(),
                            hf[2].data_ptr(), room, rebuild=(calls["k"] % cadence == 0), stream=stream)
            calls["k"] += 1

        for _ in range(3):
            e2e_call()
        calls["k"] = 0
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_call()
        e2e_seconds = time.perf_counter() - t0
    except Exception as err:   # noqa: BLE001 - whatever went wrong, the line is still printed
        e2e_error = f"{type(err).__name__}: {err}"
    failed = torch.tensor([1.0 if e2e_error else 0.0], dtype=torch.float64)
    dist.all_reduce(failed, op=dist.ReduceOp.MAX)
    e2e_t = torch.tensor([e2e_seconds if not e2e_error else 0.0], dtype=torch.float64)
    dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    if failed.item() > 0 and not e2e_error:
        e2e_error = "the host-buffer call failed on another rank"

    counts = torch.tensor([n_owned, n_total - n_owned, 24 * st["positions_sent_per_step"]], dtype=torch.float64)
    gathered = [torch.zeros_like(counts) for _ in range(world)]
    dist.all_gather(gathered, counts)

    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        value = s.n * args.steps / (elapsed_ms * 1e-3)
        per_rank = [[int(v) for v in g.tolist()] for g in gathered]
        line = {
            "metric": "atom-steps/s", "value": value, "unit": "atom-steps/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": bench.WORKLOAD_NAME if args.workload == "lj_4m" else args.workload,
                "atoms": s.n, "decomposition": "x".join(str(d) for d in dec.dims) + " bricks",
                "halo_width": halo, "ns_per_day": bench.ns_per_day(ms_per_step), "rebuilds": rebuilds,
                "owned_ghost_sentbytes_per_rank": per_rank,
                "worst_displacement_over_half_skin": float(np.sqrt(st["worst_disp_sq"]) / (0.5 * s.skin)),
                "l2": "inputs larger than L2 on every rank (list %.2f GB on rank 0)" % (4.0 * stats["directed_entries"] / 1e9),
                "energy_per_atom_before": e0 / s.n, "energy_per_atom_after": e1 / s.n,
                "phase_ms_per_step_rank0": phases,
                "neighbour_ranks": dom.peers(),
                "exchange": "native loop (dsmd_domain_run): positions-only refresh (24 B/ghost), one ncclSend/ncclRecv per "
                            "neighbour rank, on a side stream, overlapped with the interior force pass; 8-byte MAX all-reduce "
                            "for the rebuild vote on its own communicator and stream; gloo only for set-up and timing reductions",
            },
            "clocks": clocks,
            "roofline": {
                "kernel": "k_pair (LJ, full list, forces only), rank 0's brick", "bound": "hbm",
                "achieved": pair_bytes / (t_pair * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                "frac": pair_bytes / (t_pair * 1e-3) / 1e9 / hbm_peak, "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)",
                "traffic": None, "algorithmic_bytes_per_launch": pair_bytes, "algorithmic_flops_per_launch": pair_flops,
                "ms": t_pair,
                "fp32": {"achieved_tflops": pair_flops / (t_pair * 1e-3) / 1e12, "peak_tflops": fp32_peak,
                         "frac": pair_flops / (t_pair * 1e-3) / 1e12 / fp32_peak,
                         "peak_source": "measured in this run (independent FMA chains on every SM)"},
            },
            "cpu_baseline": None,
            "e2e": {"value": None if e2e_error else s.n * e2e_steps / float(e2e_t.item()), "unit": "atom-steps/s",
                    **({"error": e2e_error} if e2e_error else {}),
                    "h2d_bytes_per_step": 24 * s.n, "d2h_bytes_per_step": 24 * s.n, "steps": e2e_steps,
                    "rebuild_every": cadence,
                    "call": "dsmd_domain_forces_host on every rank: pinned host positions of the owned atoms in, rebuild "
                            "(migration, ghost plan, list) at the MD run's cadence or pack + ghost refresh beside the interior "
                            "pass, forces out; bytes are the sum over the ranks"},
            "gpu_launches": int(launches),
        }
        print(json.dumps(line))
    watchdog.cancel()
    dom.close()
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()
