#!/usr/bin/env python
"""Benchmark of the short-range nonbonded MD step (neighbour list + pair forces) on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...   # the reference's own CPU code on the host cores

One JSON line on stdout (rank 0). A "step" is one MD step of the hot path on the LJ NVE system of 4,000,000 atoms
(FCC start, density 0.8442, T* = 1.44, cutoff 2.5, skin 0.3, dt = 0.005): first velocity-Verlet half + conversion of the
positions to the kernels' layout + displacement check, neighbour-list rebuild when the displacement exceeds skin / 2,
pair forces, second velocity-Verlet half. Inputs are synthetic (seeded); the metric is atom-steps/s over all GPUs.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DT = 0.005
ARGON_TAU_FS = 2156.0          # sigma sqrt(m / epsilon) of argon in fs: maps dt = 0.005 tau to 10.78 fs for ns/day
L2_BYTES = 126e6
WORKLOAD_NAME = "LJ NVE 4,000,000 atoms (FCC 100^3, rho*=0.8442, T*=1.44, rc=2.5, skin=0.3, dt=0.005)"
SETTLE_STEPS = 12              # untimed MD steps of the set-up: they take the run through its first list rebuild (and, on several
                               # GPUs, the first migration), so that no first-use cost lands in the timed steps
NCU_PAIR_TRAFFIC_BYTES_PER_ATOM = 171.4e6 / 500_000   # measured DRAM bytes per launch / atoms (full list + positions)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML polled every 2 ms from a thread (the timed
    call runs in native code with the interpreter lock released), or, where the NVML binding is missing, nvidia-smi at its
    fastest rate. Reading only: no setting of the GPU is touched."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    # bits of the clocks-event (throttle) reasons word
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []
        self.nvml = None
        self.samples = []        # (sm MHz, reasons word)
        self.sm_max = None
        self.running = False

    def _visible_index(self):
        """The NVML index of the CUDA device (CUDA_VISIBLE_DEVICES may renumber)."""
        visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        ids = [v for v in visible.split(",") if v.strip()]
        if ids and self.device_index < len(ids) and ids[self.device_index].strip().isdigit():
            return int(ids[self.device_index])
        return self.device_index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._visible_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        reasons_of = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while self.running:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                word = int(reasons_of(self.handle)) if reasons_of else 0
                self.samples.append((mhz, word))
            except Exception:
                pass
            time.sleep(0.002)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=1.0)
            sm = [m for m, _ in self.samples]
            word = 0
            for _, w in self.samples:
                word |= w
            reasons = sorted(name for name, bit in self.REASON_BITS.items() if word & bit)
            try:
                self.nvml.nvmlShutdown()
            except Exception:
                pass
            return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": self.sm_max, "samples": len(sm),
                    "reasons": reasons, "source": "NVML, every 2 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for k, name in enumerate(names):
                if f[5 + k].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi -lms 100"}


def clocks_max_ghz(device_index: int) -> float:
    """clocks.max.sm of the device in GHz (for the nominal fp32 peak: SMs x 128 lanes x 2 flops x clock)."""
    try:
        out = subprocess.run(["nvidia-smi", f"--id={device_index}", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=10).stdout.strip()
        return float(out.splitlines()[0]) * 1e-3 if out else 1.965
    except (OSError, ValueError, subprocess.SubprocessError):
        return 1.965


def fcc_for(workload: str):
    from deepscalemd_b200 import synthetic as syn
    cells = {"lj_4m": 100, "lj_500k": 50, "lj_256k": 40, "lj_108k": 30, "lj_32k": 20}[workload]
    return syn.fcc_lj(cells, seed=12345)


# ---------------------------------------------------------------------------------------------------------------------
# CPU baseline: the reference's own CPU code (oracle/_ref), or the oracle restatement when that is not present
# ---------------------------------------------------------------------------------------------------------------------

class CpuMd:
    """Velocity-Verlet on the host around the reference's SpatialVerletList + ForceCalculatorCPU."""

    def __init__(self, workload):
        from oracle import cpu_oracle as co
        self.co = co
        self.s = fcc_for(workload)
        s = self.s
        self.pos = [np.ascontiguousarray(s.pos[:, k]) for k in range(3)]
        self.vel = [np.ascontiguousarray(s.vel[:, k]) for k in range(3)]
        self.kind = "reference" if co.ref_available() else "port"
        self.rebuilds = 0
        if self.kind == "reference":
            self.ref = co.RefCase(*self.pos, s.n, s.box, s.cutoff, s.skin, eps=s.eps, sig=s.sig)
            self.cores = self.ref.threads()
            self.simd = self.ref.simd_width()
            self.ref.build_list()
            self.frc = self._force()
        else:
            self.cores = 1
            self.simd = 1
            self.c6, self.c12 = co.lj_tables(s.eps, s.sig)
            self.ref_pos = [p.copy() for p in self.pos]
            self.pairs = co.pairs(*self.pos, s.n, s.box, search=s.cutoff + s.skin)
            self.frc = self._force()

    def _force(self):
        if self.kind == "reference":
            f, _ = self.ref.compute(tensor=False)
        else:
            f, _ = self.co.forces(*self.pos, self.s.n, self.s.box, self.pairs, self.c6, self.c12, self.s.cutoff)
        return [np.ascontiguousarray(f[:, k]) for k in range(3)]

    def step(self):
        s = self.s
        self.co.vv_half(True, DT, 1.0, self.pos, self.vel, self.frc, s.mass)
        if self.kind == "reference":
            self.ref.update_positions(*self.pos)
            if self.ref.needs_rebuild():
                # the reference wraps atoms into the box on rebuild steps only (at migration); its CPU list builder bins
                # by clamping, so it needs wrapped positions, and between rebuilds the list's periodic shifts need
                # positions that run on
                for k in range(3):
                    self.pos[k] -= s.box[k] * np.floor(self.pos[k] / s.box[k])
                self.ref.update_positions(*self.pos)
                self.ref.build_list()
                self.rebuilds += 1
        else:
            d = [p - r for p, r in zip(self.pos, self.ref_pos)]
            d2 = sum((dk - s.box[k] * np.round(dk / s.box[k])) ** 2 for k, dk in enumerate(d)).max()
            if d2 > (0.5 * s.skin) ** 2:
                self.pairs = self.co.pairs(*self.pos, s.n, s.box, search=s.cutoff + s.skin)
                self.ref_pos = [p.copy() for p in self.pos]
                self.rebuilds += 1
        self.frc = self._force()
        self.co.vv_half(False, DT, 1.0, self.pos, self.vel, self.frc, s.mass)


CPU_WORKLOADS = [("lj_32k", 32_000), ("lj_108k", 108_000), ("lj_256k", 256_000), ("lj_500k", 500_000), ("lj_4m", 4_000_000)]


def pick_cpu_workload(steps_total: int, budget_s: float):
    """The benchmark's own system (4,000,000 atoms) when the run fits the time budget, else the largest sample that does.
    The cost per atom-step is measured on two steps of a small system (the CPU code's time grows linearly with the atom
    count) and the largest candidate whose predicted run fits is built."""
    probe = CpuMd("lj_108k")
    t0 = time.perf_counter()
    probe.step()
    probe.step()
    per_atom_step = (time.perf_counter() - t0) / 2 / probe.s.n
    chosen = CPU_WORKLOADS[0][0]
    for name, atoms in CPU_WORKLOADS:
        set_up = 12.0 * atoms / 4e6 + 2.5 * per_atom_step * atoms      # generator + first list build and force call
        if set_up + 1.15 * per_atom_step * atoms * steps_total < budget_s:
            chosen = name
    return chosen, (probe if chosen == "lj_108k" else CpuMd(chosen))


def run_cpu_baseline(steps: int, warmup: int, budget_s: float):
    workload, md = pick_cpu_workload(steps + warmup, budget_s)
    for _ in range(warmup):
        md.step()
    r0 = md.rebuilds
    t0 = time.perf_counter()
    for _ in range(steps):
        md.step()
    elapsed = time.perf_counter() - t0
    value = md.s.n * steps / elapsed
    return {
        "value": value, "unit": "atom-steps/s", "cores": md.cores, "kind": md.kind,
        "sample": (f"{md.s.n}-atom FCC LJ box with the benchmark's density, cutoff, skin and dt ({workload}); {steps} "
                   f"MD steps, {md.rebuilds - r0} list rebuilds (displacement > skin/2); "
                   + ("reference SpatialVerletList + ForceCalculatorCPU fp64 tile kernels, "
                      f"SIMD width {md.simd} doubles, OpenMP" if md.kind == "reference"
                      else "oracle restatement, scalar fp64, 1 thread")),
        "ms_per_step": 1e3 * elapsed / steps, "atoms": md.s.n,
    }


def use_all_host_cores():
    """The launcher of multi-process runs pins OMP_NUM_THREADS to 1; the CPU arm runs on one rank and may use every
    core this process is allowed on. Must run before the OpenMP runtime starts (before the reference library loads)."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(max(1, cores))
    return cores


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_all_host_cores()
    base = run_cpu_baseline(args.steps, args.warmup, budget_s=args.cpu_budget_s)
    full = base["atoms"] == 4_000_000
    config = {"workload": WORKLOAD_NAME, "ns_per_day": ns_per_day(base["ms_per_step"] * (1.0 if full else 4e6 / base["atoms"]))}
    if not full:
        config["measured_on"] = base["sample"]
        config["scaling_assumption"] = ("atom-steps/s of the CPU code does not depend on the atom count (its time per step "
                                        "is linear in it); the full system did not fit this run's time budget")
    line = {
        "impl": "reference", "metric": "atom-steps/s", "value": base["value"], "unit": "atom-steps/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": config,
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "atom-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def ns_per_day(ms_per_step: float) -> float:
    return DT * ARGON_TAU_FS * 1e-6 * 86400.0 / (ms_per_step * 1e-3)


# ---------------------------------------------------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------------------------------------------------

def time_calls(fn, repeats, stream):
    """Average device time of fn() in ms, with CUDA events on `stream` and a synchronise on both sides."""
    import torch
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(repeats):
        fn()
    stop.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / repeats


def single_gpu(args):
    import torch
    from deepscalemd_b200 import capi
    hbm_peak, peak_kind = measured_peaks()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream()
    s = fcc_for(args.workload)
    ctx = capi.Context(s.n)
    ctx.set_box(s.box)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    ctx.upload(s.pos, vel=s.vel, mass=s.mass, types=s.types)
    ctx.build_neighbor_list(stream)
    ctx.compute_forces(capi.PHASE_FULL, True, stream)
    sc0 = ctx.read_scalars(stream)
    e0 = sc0["pe"] + ctx.kinetic_energy(stream)

    # -- the timed region: K MD steps, device resident ----------------------------------------------------------------
    ctx.run_nve(SETTLE_STEPS, DT, 1.0, 0.5, 0, True, stream)
    ctx.run_nve(args.warmup, DT, 1.0, 0.5, 0, True, stream)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = ctx.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    out = ctx.run_nve(args.steps, DT, 1.0, 0.5, 0, True, stream)
    stop.record(stream)
    torch.cuda.synchronize()
    elapsed_ms = start.elapsed_time(stop)
    launches = ctx.launch_count() - launches0
    clocks = sampler.stop()
    ms_per_step = elapsed_ms / args.steps
    value = s.n * args.steps / (elapsed_ms * 1e-3)

    ctx.compute_forces(capi.PHASE_FULL, True, stream)
    sc1 = ctx.read_scalars(stream)
    e1 = sc1["pe"] + ctx.kinetic_energy(stream)

    # -- per-kernel times for the roofline (inputs are far larger than L2, so no flush is needed) -----------------------
    ctx.build_neighbor_list(stream)
    stats = ctx.list_stats()
    ctx.compute_forces(capi.PHASE_FULL, True, stream)
    p_cut = ctx.read_scalars(stream)["pairs_in_cutoff"]
    p_list = stats["directed_entries"] / 2
    t_pair = time_calls(lambda: ctx.compute_forces(capi.PHASE_FULL, False, stream), 100, stream)
    t_pack = time_calls(lambda: ctx.pack_positions(0, None, stream), 100, stream)
    t_build = time_calls(lambda: ctx.build_neighbor_list(stream), 20, stream)
    flops = ctx.fma_probe(1, stream)
    iters = 20000
    t_probe = time_calls(lambda: ctx.fma_probe(iters, stream), 3, stream)
    fp32_peak_tflops = flops * iters / (t_probe * 1e-3) / 1e12
    pair_flops = 8.0 * p_list + 19.0 * p_cut
    pair_bytes = 16.0 * s.n + 4.0 * p_list + 24.0 * s.n
    build_bytes = 16.0 * s.n + 4.0 * p_list + 8.0 * s.n / 32
    pack_bytes = (24.0 + 4.0 + 16.0) * s.n
    kernels = {
        "pair_forces": {"ms": t_pair, "tflops": pair_flops / (t_pair * 1e-3) / 1e12,
                        "frac_fp32": pair_flops / (t_pair * 1e-3) / 1e12 / fp32_peak_tflops,
                        "gbs": pair_bytes / (t_pair * 1e-3) / 1e9, "frac_hbm": pair_bytes / (t_pair * 1e-3) / 1e9 / hbm_peak},
        "list_build_total": {"ms": t_build, "gbs": build_bytes / (t_build * 1e-3) / 1e9,
                             "frac_hbm": build_bytes / (t_build * 1e-3) / 1e9 / hbm_peak},
        "pack_positions": {"ms": t_pack, "gbs": pack_bytes / (t_pack * 1e-3) / 1e9,
                           "frac_hbm": pack_bytes / (t_pack * 1e-3) / 1e9 / hbm_peak},
    }
    # radius-graph edge build on the 1,000,000-atom disordered solid (cutoff 5 A): compact periodic form, and the
    # reference's interface form (int64 [2, E] + double [E, 3]) over explicit image atoms
    if args.workload == "lj_4m" or args.edges:
        from deepscalemd_b200 import synthetic as syn
        solid = syn.disordered_solid(1_000_000)
        sx, sy, sz = (torch.tensor(np.ascontiguousarray(solid.pos[:, k]), device="cuda") for k in range(3))
        eb = capi.EdgeBuilder()
        eb.build_periodic(sx, sy, sz, solid.box, solid.cutoff, stream)
        t_compact = time_calls(lambda: eb.build_periodic(sx, sy, sz, solid.box, solid.cutoff, stream), 20, stream)
        n_edges = int(eb.build_periodic(sx, sy, sz, solid.box, solid.cutoff, stream)[0].numel())
        reach = solid.cutoff + 1e-8
        img = eb.images(sx, sy, sz, None, solid.box, np.zeros(3), -np.full(3, reach), solid.box + reach, (1, 1, 1), stream)
        ix, iy, iz = img["x"].clone(), img["y"].clone(), img["z"].clone()
        owner, shift = img["owner"].clone(), tuple(t.clone() for t in img["shift"])
        lo_b, hi_b = -np.full(3, reach), solid.box + reach

        def interface_build():
            return eb.build(ix, iy, iz, solid.cutoff, lo=lo_b, hi=hi_b, n_centers=solid.n, owner=owner, shift=shift,
                            stream=stream)

        interface_build()
        t_interface = time_calls(interface_build, 20, stream)
        e_interface = int(interface_build()[0].shape[1])
        compact_bytes = 24.0 * solid.n + 23.0 * n_edges
        interface_bytes = 24.0 * img["n_all"] + 40.0 * e_interface
        placement = "uniform random placement with a 1.8 A minimum distance (seeded dart throwing), 0.05 atoms/A^3"
        kernels["edge_build_compact_1m"] = {"ms": t_compact, "edges": n_edges, "positions": placement, "gbs": compact_bytes / (t_compact * 1e-3) / 1e9,
                                            "frac_hbm": compact_bytes / (t_compact * 1e-3) / 1e9 / hbm_peak}
        kernels["edge_build_interface_1m"] = {"ms": t_interface, "edges": e_interface, "positions": placement, "atoms_with_images": img["n_all"],
                                              "gbs": interface_bytes / (t_interface * 1e-3) / 1e9,
                                              "frac_hbm": interface_bytes / (t_interface * 1e-3) / 1e9 / hbm_peak}
        eb.close()
        del sx, sy, sz, ix, iy, iz, owner, shift, img
    # the other named shapes, kernels only (list build and pair kernel at full size): the 1,048,576-atom binary mixture
    # (two types, explicit pair table) and the 648,000-atom rigid-water geometry box (LJ + real-space Ewald, exclusions)
    if args.workload == "lj_4m":
        from deepscalemd_b200 import synthetic as syn
        for name, system, coulomb in (("kob_andersen_1m", syn.kob_andersen(1_048_576, seed=5), False),
                                      ("water_648k", syn.water_box(60, seed=3), True)):
            c2 = capi.Context(system.n)
            c2.set_box(system.box)
            c2.set_pair_params(system.eps, system.sig, system.cutoff, system.skin)
            if coulomb:
                c2.set_coulomb(True)
            if system.exclusions is not None:
                c2.set_exclusions(system.n, system.exclusions)
            c2.upload(system.pos, mass=system.mass, types=system.types, charge=system.charge)
            c2.build_neighbor_list(stream)
            st2 = c2.list_stats()
            c2.compute_forces(capi.PHASE_FULL, True, stream)
            cut2 = c2.read_scalars(stream)["pairs_in_cutoff"]
            list2 = st2["directed_entries"] / 2
            tp = time_calls(lambda: c2.compute_forces(capi.PHASE_FULL, False, stream), 50, stream)
            tb = time_calls(lambda: c2.build_neighbor_list(stream), 10, stream)
            fl = 8.0 * list2 + (19.0 + (9.0 if coulomb else 0.0)) * cut2
            by = 16.0 * system.n + 4.0 * list2 + 24.0 * system.n + (4.0 * system.n if coulomb else 0.0)
            bb = 16.0 * system.n + 4.0 * list2 + 8.0 * system.n / 32
            kernels[name] = {
                "atoms": system.n, "pairs_listed": list2, "pairs_in_cutoff": cut2,
                "pair_forces": {"ms": tp, "tflops": fl / (tp * 1e-3) / 1e12, "frac_fp32": fl / (tp * 1e-3) / 1e12 / fp32_peak_tflops,
                                "gbs": by / (tp * 1e-3) / 1e9, "frac_hbm": by / (tp * 1e-3) / 1e9 / hbm_peak},
                "list_build_total": {"ms": tb, "gbs": bb / (tb * 1e-3) / 1e9, "frac_hbm": bb / (tb * 1e-3) / 1e9 / hbm_peak},
            }
            if coulomb:
                # the charges of this system are a function of the atom type (O, H): the table form of the kernel
                by_type = [float(system.charge[system.types == t][0]) for t in range(int(system.types.max()) + 1)]
                c2.set_type_charges(by_type)
                tq = time_calls(lambda: c2.compute_forces(capi.PHASE_FULL, False, stream), 50, stream)
                kernels[name]["pair_forces_charges_by_type"] = {
                    "ms": tq, "tflops": fl / (tq * 1e-3) / 1e12, "frac_fp32": fl / (tq * 1e-3) / 1e12 / fp32_peak_tflops,
                    "note": "dsmd_set_type_charges: partner charges from a table in shared memory instead of a gather"}
            c2.close()
    pk = kernels["pair_forces"]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    roofline = {
        "kernel": "k_pair (LJ, full list, forces only)", "bound": "fp32", "achieved": pk["tflops"], "peak": fp32_peak_tflops,
        "unit": "TFLOP/s", "frac": pk["frac_fp32"],
        "peak_source": "measured in this run (independent FMA chains on every SM); no fp32 CUDA-core figure in MEASURED_PEAKS.json",
        "peak_nominal": sms * 128 * 2 * clocks_max_ghz(0) * 1e-3,   # TFLOP/s: SMs x 128 fp32 lanes x 2 flops x max SM clock
        # dram__bytes_read + dram__bytes_write of one k_pair launch, from the ncu capture of the 500,000-atom case
        # (profiles/k_pair_k_build_list_lj_500k_ncu_full.md: 171.4 MB) scaled by the atom count
        "traffic": NCU_PAIR_TRAFFIC_BYTES_PER_ATOM * s.n,
        "algorithmic_bytes_per_launch": pair_bytes, "algorithmic_flops_per_launch": pair_flops,
        "hbm": {"achieved": pk["gbs"], "peak": hbm_peak, "unit": "GB/s", "frac": pk["frac_hbm"],
                "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)"},
        "list_build": {"kernel": "bin + sort + reorder + k_build_list", "bound": "hbm", "ms": t_build,
                       "achieved": kernels["list_build_total"]["gbs"], "peak": hbm_peak, "unit": "GB/s",
                       "frac": kernels["list_build_total"]["frac_hbm"], "algorithmic_bytes_per_launch": build_bytes},
    }

    # -- end to end: the host-buffer force call (upload positions, pack or rebuild, forces, download forces) --------------
    order = ctx.download("global_id")
    host = [torch.from_numpy(ctx.download(k)).pin_memory() for k in ("x", "y", "z")]
    hf = [torch.empty(s.n, dtype=torch.float64).pin_memory() for _ in range(3)]
    cadence = max(1, round(args.steps / max(out["rebuilds"], 1)))
    e2e_steps = max(4, min(args.steps, 40))
    calls = {"k": 0}

    def one_call():
        ctx.forces_host(host[0].data_ptr(), host[1].data_ptr(), host[2].data_ptr(), hf[0].data_ptr(), hf[1].data_ptr(),
                        hf[2].data_ptr(), rebuild=(calls["k"] % cadence == 0), scalars=None, stream=stream)
        calls["k"] += 1

    for _ in range(3):
        one_call()
    calls["k"] = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        one_call()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_value = s.n * e2e_steps / e2e_s

    cpu = None
    if not args.no_cpu_baseline:
        use_all_host_cores()
        cpu = run_cpu_baseline(steps=30, warmup=3, budget_s=25.0)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}

    line = {
        "metric": "atom-steps/s", "value": value, "unit": "atom-steps/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": WORKLOAD_NAME if args.workload == "lj_4m" else args.workload,
            "atoms": s.n, "ns_per_day": ns_per_day(ms_per_step), "rebuilds": out["rebuilds"],
            "steps_per_rebuild": args.steps / max(out["rebuilds"], 1),
            "worst_displacement_over_half_skin": float(np.sqrt(out["worst_disp_sq"]) / (0.5 * s.skin)),
            "l2": "inputs larger than L2 (list %.2f GB, positions %.0f MB)" % (4.0 * stats["directed_entries"] / 1e9,
                                                                               16.0 * s.n / 1e6),
            "list": stats, "pairs_in_cutoff": p_cut,
            "energy_per_atom_before": e0 / s.n, "energy_per_atom_after": e1 / s.n,
            "precision": "fp32 pair math on 32-bit fixed-point coordinates, fp64 positions/velocities/forces/energy sums",
        },
        "clocks": clocks,
        "roofline": roofline,
        "kernels": kernels,
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "atom-steps/s", "h2d_bytes_per_step": 24 * s.n, "d2h_bytes_per_step": 24 * s.n,
                "steps": e2e_steps, "rebuild_every": cadence,
                "call": "dsmd_forces_host: pinned host positions in, forces out, list rebuilt at the MD run's cadence"},
        "gpu_launches": int(launches),
    }
    print(json.dumps(line))
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=100)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="lj_4m")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--edges", action="store_true",
                    help="time the radius-graph build of the 1,000,000-atom solid with a smaller --workload too (it always runs with lj_4m)")
    ap.add_argument("--cpu-budget-s", type=float, default=170.0,
                    help="time the reference arm may take: it runs the 4,000,000-atom system when that fits, else a smaller sample")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        reference_arm(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 or world > 1:
        from deepscalemd_b200 import domain_bench
        domain_bench.run(args)
        return
    single_gpu(args)


if __name__ == "__main__":
    main()
