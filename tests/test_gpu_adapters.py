"""GPU tests of the C++ adapters that carry the reference's class shapes (include/dsmd/): a harness compiled against the
reference's own interface headers (oracle/ref_build/adapter_harness.cpp -> oracle/_ref/libdsmd_adapter_check.so) fills an
MDSystem as the reference's driver would and calls ForceCalculator::compute_forces, NeighborList::needs_rebuild,
the lagged displacement query, the storage provider, HaloBackend::try_gpu_direct_halo and the CommBackend reductions
(over the native domain code, one rank) and EdgeBuilder::build; results are compared with the CPU oracle. Skipped where the harness was not built (it needs the
reference headers at build time)."""
import ctypes
import os

import numpy as np
import pytest

from deepscalemd_b200 import synthetic as syn
from oracle import cpu_oracle as co

pytestmark = pytest.mark.gpu

HARNESS = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                       "libdsmd_adapter_check.so")


@pytest.fixture(scope="module")
def harness(cuda_device):
    if not os.path.exists(HARNESS):
        pytest.skip("adapter harness not built (needs the reference headers): make -C oracle ref")
    lib = ctypes.CDLL(HARNESS)
    lib.dsmd_adapter_edges.restype = ctypes.c_long
    return lib


def ptr(a, t):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(t))


def rms(a):
    return float(np.sqrt((np.asarray(a) ** 2).sum(-1).mean()))


@pytest.mark.parametrize("case", ["lj", "water"])
def test_force_calculator_adapter_matches_oracle(harness, case):
    s = syn.fcc_lj(6, seed=1) if case == "lj" else syn.water_box(11, seed=3)
    cols = [np.ascontiguousarray(s.pos[:, k]) for k in range(3)]
    vcols = [np.ascontiguousarray(s.vel[:, k]) for k in range(3)]
    eps, sig = np.ascontiguousarray(s.eps), np.ascontiguousarray(s.sig)
    excl = s.exclusions if s.exclusions is not None else np.zeros((0, 2), dtype=np.int32)
    ea, eb = np.ascontiguousarray(excl[:, 0], dtype=np.int32), np.ascontiguousarray(excl[:, 1], dtype=np.int32)
    out_f = np.zeros((s.n, 3))
    out_sc = np.zeros(10)
    err = ctypes.create_string_buffer(512)
    box = np.ascontiguousarray(s.box)
    rc = harness.dsmd_adapter_forces(
        ctypes.c_long(s.n), *(ptr(c, ctypes.c_double) for c in cols), *(ptr(c, ctypes.c_double) for c in vcols),
        ptr(s.mass, ctypes.c_double), ptr(np.ascontiguousarray(s.charge), ctypes.c_double), ptr(s.types, ctypes.c_int),
        ptr(box, ctypes.c_double), ctypes.c_int(eps.shape[0]), ptr(eps, ctypes.c_double), ptr(sig, ctypes.c_double),
        ctypes.c_double(s.cutoff), ctypes.c_double(s.skin), ctypes.c_int(int(s.coulomb)), ctypes.c_long(len(ea)),
        ptr(ea, ctypes.c_int), ptr(eb, ctypes.c_int), ptr(out_f, ctypes.c_double), ptr(out_sc, ctypes.c_double), err,
        ctypes.c_int(512))
    assert rc == 0, err.value.decode()
    pairs = co.pairs(*cols, s.n, s.box, search=s.cutoff + s.skin)
    c6, c12 = co.lj_tables(s.eps, s.sig)
    alpha = co.ewald_alpha(s.cutoff) if s.coulomb else 0.0
    f_o, sc_o = co.forces(*cols, s.n, s.box, pairs, c6, c12, s.cutoff, charge=s.charge, types=s.types,
                          do_coulomb=s.coulomb, alpha=alpha, ewald_mode=1, exclusions=s.exclusions)
    assert rms(out_f - f_o) <= 1e-5 * rms(f_o)
    assert abs(out_sc[0] - sc_o["pe"]) <= 1e-6 * abs(sc_o["pe"])
    assert abs(out_sc[1] - sc_o["virial"]) <= 1e-6 * abs(sc_o["virial"])
    assert np.allclose(out_sc[2:5], sc_o["virial_diag"], rtol=5e-6)
    ke = 0.5 * (s.mass[:, None] * s.vel ** 2).sum()
    assert abs(out_sc[5] - ke) <= 1e-12 * ke
    assert out_sc[6] == 2.0          # no rebuild right after a build, rebuild once an atom moved 0.6 skin
    # lagged displacement: nothing on the first call, then what the call before measured (the atom 0.6 skin away)
    assert out_sc[7] < 0.0 and out_sc[8] == pytest.approx((0.6 * s.skin) ** 2, rel=1e-9)
    # a rebuild step through HaloBackendB200 / CommBackendB200 over a one-rank domain leaves the physics alone
    assert abs(out_sc[9] - sc_o["pe"]) <= 1e-6 * abs(sc_o["pe"])


def test_edge_builder_adapter_matches_oracle(harness):
    rng = np.random.default_rng(5)
    n, cutoff = 3000, 4.0
    pos = rng.uniform(0, 30.0, (n, 3))
    cols = [np.ascontiguousarray(pos[:, k]) for k in range(3)]
    want, _ = co.edges(*cols, cutoff)
    E = want.shape[1]
    out = np.zeros(2 * E, dtype=np.int64)
    err = ctypes.create_string_buffer(512)
    got_e = harness.dsmd_adapter_edges(ctypes.c_long(n), *(ptr(c, ctypes.c_double) for c in cols), ctypes.c_double(cutoff),
                                       ptr(out, ctypes.c_longlong), ctypes.c_long(2 * E), err, ctypes.c_int(512))
    assert got_e == E, err.value.decode()
    got = out.reshape(2, E)
    order = lambda e: e[:, np.lexsort((e[1], e[0]))]
    assert np.array_equal(order(got), order(want))
