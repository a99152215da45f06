"""GPU test of dsmd_kinetic_energy_noalloc, the entry point for callers that must not allocate device memory (a plugin
inside an engine's step loop: the engine's pools own the device memory, and a cudaMalloc would stall the step's streams).
It is called through the C ABI on the arrays of a live context and must give what dsmd_kinetic_energy gives, twice in a
row (the second call reuses the library's built-in scratch array with the first call's contents still in it), and after
a call on a different, smaller system. Collected last on purpose."""
import numpy as np
import pytest

from deepscalemd_b200 import capi
from deepscalemd_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def context_for(s):
    ctx = capi.Context(s.n)
    ctx.set_box(s.box)
    ctx.set_pair_params(s.eps, s.sig, s.cutoff, s.skin)
    ctx.upload(s.pos, vel=s.vel, mass=s.mass, types=s.types)
    return ctx


def noalloc_sum(ctx, n, out):
    ptr = {k: ctx.device_pointer(k) for k in ("vx", "vy", "vz", "mass")}
    capi.kinetic_energy_noalloc(ptr["vx"], ptr["vy"], ptr["vz"], ptr["mass"], n, out.data_ptr())
    import torch
    torch.cuda.synchronize()
    return float(out.item())


def test_matches_the_allocating_entry_point_on_two_calls_in_a_row(cuda_device):
    import torch
    big = syn.fcc_lj(12, seed=6)       # 6912 atoms: 27 partial sums
    small = syn.fcc_lj(6, seed=7)      # 864 atoms: 4 partial sums, leaves the big system's other 23 in the array
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    ctx_big, ctx_small = context_for(big), context_for(small)
    want_big, want_small = ctx_big.kinetic_energy(), ctx_small.kinetic_energy()
    assert abs(want_big - 0.5 * (big.mass[:, None] * big.vel ** 2).sum()) <= 1e-12 * want_big
    first = noalloc_sum(ctx_big, big.n, out)
    second = noalloc_sum(ctx_big, big.n, out)
    assert abs(first - want_big) <= 1e-12 * abs(want_big)      # same tree of fp64 sums: equal to round-off
    assert second == first
    assert abs(noalloc_sum(ctx_small, small.n, out) - want_small) <= 1e-12 * abs(want_small)
    assert noalloc_sum(ctx_big, big.n, out) == first
    assert noalloc_sum(ctx_big, 0, out) == 0.0                  # no atoms: nothing read from the scratch array
    ctx_big.close()
    ctx_small.close()


def test_sizes_beyond_the_built_in_scratch_are_refused(cuda_device):
    import torch
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    v = torch.zeros(8, dtype=torch.float64, device="cuda")
    with pytest.raises(capi.DsmdError) as err:
        capi.kinetic_energy_noalloc(v.data_ptr(), v.data_ptr(), v.data_ptr(), v.data_ptr(), capi.NOALLOC_MAX_ATOMS + 1,
                                    out.data_ptr())
    assert err.value.code == capi.ERR_CAPACITY and "DSMD_NOALLOC_MAX_ATOMS" in str(err.value)
    with pytest.raises(capi.DsmdError) as err:
        capi.kinetic_energy_noalloc(0, v.data_ptr(), v.data_ptr(), v.data_ptr(), 8, out.data_ptr())
    assert err.value.code == capi.ERR_INVALID
