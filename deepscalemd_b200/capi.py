"""ctypes binding of the C ABI in ``include/dsmd_b200.h`` (``libdsmd_b200.so``).

There is no fallback: if the library is missing or fails to load, importing the symbols raises. Device buffers handed
to the library are torch CUDA tensors (``data_ptr()``); streams are ``torch.cuda.Stream.cuda_stream`` integers.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(_HERE, "libdsmd_b200.so")

OK = 0
ERR_INVALID, ERR_CUDA, ERR_BOX_TOO_SMALL, ERR_OUT_OF_DOMAIN, ERR_CAPACITY, ERR_STATE, ERR_TIMEOUT = range(1, 8)
PHASE_FULL, PHASE_INTERIOR, PHASE_BOUNDARY = 0, 1, 2
FIELDS = ["x", "y", "z", "vx", "vy", "vz", "fx", "fy", "fz", "mass", "charge", "type", "global_id"]
FIELD_ID = {name: k for k, name in enumerate(FIELDS)}

# every symbol include/dsmd_b200.h declares
SYMBOLS = [
    "dsmd_create", "dsmd_destroy", "dsmd_last_error", "dsmd_set_box", "dsmd_set_pair_params", "dsmd_set_coulomb",
    "dsmd_get_ewald_alpha", "dsmd_set_exclusions", "dsmd_set_constraints", "dsmd_constraint_failures", "dsmd_rattle",
    "dsmd_set_bonded", "dsmd_compute_bonded", "dsmd_read_bonded_scalars", "dsmd_set_type_charges", "dsmd_upload", "dsmd_upload_positions", "dsmd_download",
    "dsmd_device_pointer", "dsmd_counts", "dsmd_set_counts", "dsmd_build_neighbor_list", "dsmd_sort_owned", "dsmd_sort_owned_in_brick",
    "dsmd_ghost_slots", "dsmd_list_stats", "dsmd_list_export", "dsmd_pack_positions", "dsmd_max_displacement_sq", "dsmd_max_displacement_sq_lagged",
    "dsmd_displacement_word", "dsmd_compute_forces", "dsmd_read_scalars", "dsmd_integrate", "dsmd_kinetic_energy", "dsmd_scale_velocities",
    "dsmd_run_nve",
    "dsmd_forces_host", "dsmd_launch_count", "dsmd_fma_probe", "dsmd_halo_pack", "dsmd_halo_unpack", "dsmd_halo_select",
    "dsmd_halo_pack_records", "dsmd_halo_append_records", "dsmd_halo_append_packed", "dsmd_capacity", "dsmd_edges_create", "dsmd_edges_destroy",
    "dsmd_edges_last_error", "dsmd_edges_build", "dsmd_edges_result", "dsmd_edges_build_periodic",
    "dsmd_edges_result_compact", "dsmd_images_build", "dsmd_images_result", "dsmd_images_fold_forces",
    "dsmd_virial_from_forces", "dsmd_mark_receivers",
    "dsmd_kinetic_energy_noalloc", "dsmd_nccl_unique_id", "dsmd_domain_create",
    "dsmd_domain_destroy", "dsmd_domain_last_error", "dsmd_domain_rebuild", "dsmd_domain_refresh", "dsmd_domain_forces_host", "dsmd_domain_run",
    "dsmd_domain_stats", "dsmd_domain_profile", "dsmd_domain_set_wait_limit", "dsmd_domain_abort",
    "dsmd_domain_reverse_forces", "dsmd_domain_exchange_field", "dsmd_domain_peers", "dsmd_domain_reduce",
]

_lib = None

c_void_p, c_int, c_int64, c_double = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_double
_pd = ctypes.POINTER(ctypes.c_double)


class DsmdError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"dsmd status {code}: {message}")
        self.code = code


def load():
    """Loads libdsmd_b200.so (raises if it has not been built: there is no other compute path)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIBRARY):
        raise ImportError(f"{LIBRARY} is missing: build it with `python -m deepscalemd_b200.build` (needs nvcc)")
    lib = ctypes.CDLL(LIBRARY)
    lib.dsmd_last_error.restype = ctypes.c_char_p
    lib.dsmd_last_error.argtypes = [c_void_p]
    lib.dsmd_edges_last_error.restype = ctypes.c_char_p
    lib.dsmd_edges_last_error.argtypes = [c_void_p]
    lib.dsmd_launch_count.restype = c_int64
    lib.dsmd_launch_count.argtypes = [c_void_p]
    lib.dsmd_destroy.restype = None
    lib.dsmd_destroy.argtypes = [c_void_p]
    lib.dsmd_edges_destroy.restype = None
    lib.dsmd_edges_destroy.argtypes = [c_void_p]
    _lib = lib
    return lib


def _arr(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def _p(a):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _stream_handle(stream):
    if stream is None:
        return c_void_p(0)
    if hasattr(stream, "cuda_stream"):
        return c_void_p(stream.cuda_stream)
    return c_void_p(int(stream))


class Context:
    """One ``dsmd_ctx``: the device-resident particle arrays, neighbour list and kernels of one GPU."""

    def __init__(self, capacity: int, device: int = 0):
        self.lib = load()
        self.h = c_void_p()
        rc = self.lib.dsmd_create(c_int(device), c_int64(capacity), ctypes.byref(self.h))
        if rc != OK:
            msg = self.lib.dsmd_last_error(self.h).decode() if self.h else "dsmd_create failed"
            raise DsmdError(rc, msg)
        self.capacity = capacity
        self.device = device
        self._keep = []

    def _check(self, rc):
        if rc != OK:
            raise DsmdError(rc, self.lib.dsmd_last_error(self.h).decode())

    def close(self):
        if self.h:
            self.lib.dsmd_destroy(self.h)
            self.h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- set-up -----------------------------------------------------------------------------------------------------
    def set_box(self, box, periodic=(1, 1, 1), lo=(0, 0, 0), hi=(0, 0, 0), halo=0.0):
        b, p, l, h = _arr(box, np.float64), _arr(periodic, np.int32), _arr(lo, np.float64), _arr(hi, np.float64)
        self._check(self.lib.dsmd_set_box(self.h, _p(b), _p(p), _p(l), _p(h), c_double(halo)))

    def set_pair_params(self, eps, sig, cutoff, skin, switch=-1.0):
        e = _arr(np.atleast_2d(eps), np.float64)
        s = _arr(np.atleast_2d(sig), np.float64)
        self._check(self.lib.dsmd_set_pair_params(self.h, c_int(e.shape[0]), _p(e), _p(s), c_double(cutoff),
                                                  c_double(skin), c_double(switch)))

    def set_coulomb(self, enabled=True, alpha=0.0):
        self._check(self.lib.dsmd_set_coulomb(self.h, c_int(int(enabled)), c_double(alpha)))

    def ewald_alpha(self):
        a = c_double(0.0)
        self._check(self.lib.dsmd_get_ewald_alpha(self.h, ctypes.byref(a)))
        return a.value

    def set_exclusions(self, n_global, pairs):
        if pairs is None or len(pairs) == 0:
            self._check(self.lib.dsmd_set_exclusions(self.h, c_int64(n_global), c_int64(0), None, None))
            return
        pairs = np.asarray(pairs)
        a, b = _arr(pairs[:, 0], np.int32), _arr(pairs[:, 1], np.int32)
        self._check(self.lib.dsmd_set_exclusions(self.h, c_int64(n_global), c_int64(len(a)), _p(a), _p(b)))

    def set_constraints(self, n_global, constraints, tolerance=0.0, max_iterations=0):
        """constraints: rows (atom i, atom j, distance) by global id."""
        if constraints is None or len(constraints) == 0:
            self._check(self.lib.dsmd_set_constraints(self.h, c_int64(n_global), c_int64(0), None, None, None, c_double(0.0), c_int(0)))
            return
        rows = np.asarray(constraints, dtype=np.float64)
        a, b, d = _arr(rows[:, 0], np.int32), _arr(rows[:, 1], np.int32), _arr(rows[:, 2], np.float64)
        self._check(self.lib.dsmd_set_constraints(self.h, c_int64(n_global), c_int64(len(a)), _p(a), _p(b), _p(d),
                                                  c_double(tolerance), c_int(max_iterations)))

    def set_type_charges(self, charge_of_type):
        """Every atom's charge is the charge of its type: the pair kernel reads a table instead of the per-atom array.
        None switches back to per-atom charges."""
        if charge_of_type is None:
            self._check(self.lib.dsmd_set_type_charges(self.h, c_int(0), None))
            return
        q = _arr(charge_of_type, np.float64)
        self._check(self.lib.dsmd_set_type_charges(self.h, c_int(len(q)), _p(q)))

    def set_bonded(self, n_global, terms):
        """terms: a mapping (or object) with bonds [nb, 2], bond_k, bond_r0, angles [na, 3], angle_k, angle_theta0 (radians),
        torsions [nt, 4], torsion_k, torsion_phi0 (radians), torsion_n, specials [ns, 2], special_sigma, special_epsilon,
        special_lj_scale, special_coulomb_scale; atoms by global id; what is absent counts as empty. None clears."""
        def get(name):
            if terms is None:
                return None
            return terms.get(name) if isinstance(terms, dict) else getattr(terms, name, None)

        def table(name, width):
            a = get(name)
            return np.zeros((0, width), dtype=np.int32) if a is None else _arr(np.asarray(a).reshape(-1, width), np.int32)

        def column(name, n, dtype=np.float64):
            a = get(name)
            a = np.zeros(n, dtype=dtype) if a is None else _arr(a, dtype)
            if len(a) != n:
                raise ValueError(f"{name}: {len(a)} values for {n} terms")
            return a
        b, a, t, sp = table("bonds", 2), table("angles", 3), table("torsions", 4), table("specials", 2)
        cols = [column("bond_k", len(b)), column("bond_r0", len(b)), column("angle_k", len(a)), column("angle_theta0", len(a)),
                column("torsion_k", len(t)), column("torsion_phi0", len(t)), column("torsion_n", len(t), np.int32),
                column("special_sigma", len(sp)), column("special_epsilon", len(sp)), column("special_lj_scale", len(sp)),
                column("special_coulomb_scale", len(sp))]
        self._check(self.lib.dsmd_set_bonded(self.h, c_int64(n_global), c_int64(len(b)), _p(b), _p(cols[0]), _p(cols[1]),
                                             c_int64(len(a)), _p(a), _p(cols[2]), _p(cols[3]), c_int64(len(t)), _p(t),
                                             _p(cols[4]), _p(cols[5]), _p(cols[6]), c_int64(len(sp)), _p(sp), _p(cols[7]),
                                             _p(cols[8]), _p(cols[9]), _p(cols[10])))

    def compute_bonded(self, stream=None):
        self._check(self.lib.dsmd_compute_bonded(self.h, _stream_handle(stream)))

    def read_bonded_scalars(self, stream=None):
        out = (c_double * 5)()
        self._check(self.lib.dsmd_read_bonded_scalars(self.h, out, _stream_handle(stream)))
        return dict(pe=out[0], virial=out[1], virial_diag=np.array([out[2], out[3], out[4]]))

    def constraint_failures(self, stream=None):
        n = c_int64(0)
        self._check(self.lib.dsmd_constraint_failures(self.h, ctypes.byref(n), _stream_handle(stream)))
        return n.value

    # -- particles ----------------------------------------------------------------------------------------------------
    def upload(self, pos, n_owned=None, vel=None, mass=None, charge=None, types=None, gid=None, stream=None):
        pos = np.asarray(pos, dtype=np.float64)
        n = len(pos)
        n_owned = n if n_owned is None else n_owned
        cols = [_arr(pos[:, k], np.float64) for k in range(3)]
        vcols = [None] * 3 if vel is None else [_arr(np.asarray(vel)[:, k], np.float64) for k in range(3)]
        m, q = _arr(mass, np.float64), _arr(charge, np.float64)
        t, g = _arr(types, np.int32), _arr(gid, np.int32)
        self._check(self.lib.dsmd_upload(self.h, c_int64(n_owned), c_int64(n), _p(cols[0]), _p(cols[1]), _p(cols[2]),
                                         _p(vcols[0]), _p(vcols[1]), _p(vcols[2]), _p(m), _p(q), _p(t), _p(g),
                                         _stream_handle(stream)))
        import torch
        torch.cuda.synchronize()

    def upload_positions_ptr(self, x_ptr, y_ptr, z_ptr, stream=None):
        self._check(self.lib.dsmd_upload_positions(self.h, c_void_p(x_ptr), c_void_p(y_ptr), c_void_p(z_ptr),
                                                   _stream_handle(stream)))

    def counts(self):
        a, b = c_int64(0), c_int64(0)
        self._check(self.lib.dsmd_counts(self.h, ctypes.byref(a), ctypes.byref(b)))
        return a.value, b.value

    def set_counts(self, n_owned, n_total):
        self._check(self.lib.dsmd_set_counts(self.h, c_int64(n_owned), c_int64(n_total)))

    def download(self, field, n=None, stream=None):
        n_owned, n_total = self.counts()
        n = n_total if n is None else n
        fid = FIELD_ID[field]
        out = np.zeros(n, dtype=np.int32 if fid >= 11 else np.float64)
        self._check(self.lib.dsmd_download(self.h, c_int(fid), c_int64(n), _p(out), _stream_handle(stream)))
        return out

    def device_pointer(self, field):
        p = c_void_p()
        self._check(self.lib.dsmd_device_pointer(self.h, c_int(FIELD_ID[field]), ctypes.byref(p)))
        return p.value

    def forces_by_gid(self, n_global=None):
        """[n_global, 3] forces of the owned atoms scattered by global id (NaN where this context owns no atom)."""
        n_owned, _ = self.counts()
        gid = self.download("global_id", n_owned)
        n_global = int(gid.max()) + 1 if n_global is None else n_global
        out = np.full((n_global, 3), np.nan)
        for k, name in enumerate(("fx", "fy", "fz")):
            out[gid, k] = self.download(name, n_owned)
        return out

    def field_by_gid(self, names, n_global=None):
        n_owned, _ = self.counts()
        gid = self.download("global_id", n_owned)
        n_global = int(gid.max()) + 1 if n_global is None else n_global
        out = np.full((n_global, len(names)), np.nan)
        for k, name in enumerate(names):
            out[gid, k] = self.download(name, n_owned)
        return out

    # -- list -----------------------------------------------------------------------------------------------------------
    def build_neighbor_list(self, stream=None):
        self._check(self.lib.dsmd_build_neighbor_list(self.h, _stream_handle(stream)))

    def sort_owned(self, stream=None):
        self._check(self.lib.dsmd_sort_owned(self.h, _stream_handle(stream)))

    def ghost_slots_ptr(self):
        p = c_void_p()
        self._check(self.lib.dsmd_ghost_slots(self.h, ctypes.byref(p)))
        return p.value

    def ghost_slots(self, n_ghost):
        """The slot of every ghost atom, in the order the ghosts arrived (int32 device tensor of n_ghost entries)."""
        import torch
        return _tensor_from_ptr(self.ghost_slots_ptr(), (int(n_ghost),), torch.int32, torch.device("cuda", self.device))

    def list_stats(self):
        e, i = c_int64(0), c_int64(0)
        s, c, r = c_int(0), c_int(0), c_int(0)
        self._check(self.lib.dsmd_list_stats(self.h, ctypes.byref(e), ctypes.byref(i), ctypes.byref(s), ctypes.byref(c),
                                             ctypes.byref(r)))
        return dict(directed_entries=e.value, interior_entries=i.value, row_stride=s.value, cells=c.value,
                    rechecked_fp64=r.value)

    def list_pairs(self, stream=None):
        """Directed list entries as numpy arrays (i slot, j slot, excluded flag)."""
        ti, tj, tf = self.list_pairs_device(stream)
        return ti.cpu().numpy(), tj.cpu().numpy(), tf.cpu().numpy()

    def list_pairs_device(self, stream=None):
        """Directed list entries as device tensors (i slot int32, j slot int32, excluded flag uint8)."""
        import torch
        n = c_int64(0)
        self._check(self.lib.dsmd_list_export(self.h, None, None, None, c_int64(0), ctypes.byref(n),
                                              _stream_handle(stream)))
        dev = torch.device("cuda", self.device)
        ti = torch.empty(max(n.value, 1), dtype=torch.int32, device=dev)
        tj = torch.empty(max(n.value, 1), dtype=torch.int32, device=dev)
        tf = torch.empty(max(n.value, 1), dtype=torch.uint8, device=dev)
        self._check(self.lib.dsmd_list_export(self.h, c_void_p(ti.data_ptr()), c_void_p(tj.data_ptr()),
                                              c_void_p(tf.data_ptr()), c_int64(n.value), ctypes.byref(n),
                                              _stream_handle(stream)))
        k = n.value
        return ti[:k], tj[:k], tf[:k]

    # -- per step -------------------------------------------------------------------------------------------------------
    def pack_positions(self, first=0, count=None, stream=None):
        _, n_total = self.counts()
        count = n_total - first if count is None else count
        self._check(self.lib.dsmd_pack_positions(self.h, c_int64(first), c_int64(count), _stream_handle(stream)))

    def max_displacement_sq(self, stream=None):
        v = c_double(0.0)
        self._check(self.lib.dsmd_max_displacement_sq(self.h, ctypes.byref(v), _stream_handle(stream)))
        return v.value

    def compute_forces(self, phase=PHASE_FULL, want_energy=False, stream=None):
        self._check(self.lib.dsmd_compute_forces(self.h, c_int(phase), c_int(int(want_energy)), _stream_handle(stream)))

    def read_scalars(self, stream=None):
        out = (c_double * 6)()
        self._check(self.lib.dsmd_read_scalars(self.h, out, _stream_handle(stream)))
        v = np.array(list(out))
        return dict(pe=v[0], virial=v[1], virial_diag=v[2:5].copy(), pairs_in_cutoff=v[5])

    def integrate(self, half, dt, force_to_accel=1.0, stream=None):
        self._check(self.lib.dsmd_integrate(self.h, c_int(half), c_double(dt), c_double(force_to_accel),
                                            _stream_handle(stream)))

    def scale_velocities(self, factor, stream=None):
        self._check(self.lib.dsmd_scale_velocities(self.h, c_double(factor), _stream_handle(stream)))

    def kinetic_energy(self, stream=None):
        v = c_double(0.0)
        self._check(self.lib.dsmd_kinetic_energy(self.h, ctypes.byref(v), _stream_handle(stream)))
        return v.value

    def run_nve(self, n_steps, dt, force_to_accel=1.0, hi_frac=0.5, every=0, lagged=True, stream=None):
        nr, worst = c_int64(0), c_double(0.0)
        self._check(self.lib.dsmd_run_nve(self.h, c_int64(n_steps), c_double(dt), c_double(force_to_accel),
                                          c_double(hi_frac), c_int(every), c_int(int(lagged)), ctypes.byref(nr),
                                          ctypes.byref(worst), _stream_handle(stream)))
        return dict(rebuilds=nr.value, worst_disp_sq=worst.value)

    def forces_host(self, x, y, z, fx, fy, fz, rebuild=False, scalars=None, stream=None):
        """Host-buffer force call; all arguments are numpy arrays or raw host addresses (ints) in context order."""
        def addr(a):
            return c_void_p(a) if isinstance(a, int) else _p(a)
        sc = None if scalars is None else _p(scalars)
        self._check(self.lib.dsmd_forces_host(self.h, addr(x), addr(y), addr(z), c_int(int(rebuild)), addr(fx), addr(fy),
                                              addr(fz), sc, _stream_handle(stream)))

    def launch_count(self):
        return self.lib.dsmd_launch_count(self.h)

    def fma_probe(self, iters, stream=None):
        """Queues the fp32 FMA throughput probe; returns the flops it performs."""
        f = c_double(0.0)
        self._check(self.lib.dsmd_fma_probe(self.h, c_int(iters), ctypes.byref(f), _stream_handle(stream)))
        return f.value

    # -- halo -------------------------------------------------------------------------------------------------------------
    def halo_select(self, lo, hi, index_tensor, stream=None):
        l, h = _arr(lo, np.float64), _arr(hi, np.float64)
        n = c_int64(0)
        self._check(self.lib.dsmd_halo_select(self.h, _p(l), _p(h), c_void_p(index_tensor.data_ptr()),
                                              c_int64(index_tensor.numel()), ctypes.byref(n), _stream_handle(stream)))
        return n.value

    def halo_pack(self, index_tensor, image_tensor, count, out_tensor, stream=None):
        img = None if image_tensor is None else c_void_p(image_tensor.data_ptr())
        self._check(self.lib.dsmd_halo_pack(self.h, c_void_p(index_tensor.data_ptr()), img, c_int64(count),
                                            c_void_p(out_tensor.data_ptr()), _stream_handle(stream)))

    def displacement_word(self):
        """The device word holding max displacement^2 (bits of a double) as a one-element int64 torch tensor."""
        import torch
        p = c_void_p()
        self._check(self.lib.dsmd_displacement_word(self.h, ctypes.byref(p)))
        return _tensor_from_ptr(p.value, (1,), torch.int64, torch.device("cuda", self.device))

    def halo_unpack(self, in_tensor, first_ghost, count, stream=None):
        self._check(self.lib.dsmd_halo_unpack(self.h, c_void_p(in_tensor.data_ptr()), c_int64(first_ghost),
                                              c_int64(count), _stream_handle(stream)))

    def halo_pack_records(self, index_tensor, count, shift, real_out, int_out, stream=None):
        s = _arr(shift, np.float64)
        self._check(self.lib.dsmd_halo_pack_records(self.h, c_void_p(index_tensor.data_ptr()), c_int64(count), _p(s),
                                                    c_void_p(real_out.data_ptr()), c_void_p(int_out.data_ptr()),
                                                    _stream_handle(stream)))

    def halo_append_records(self, real_in, int_in, count, stream=None):
        self._check(self.lib.dsmd_halo_append_records(self.h, c_void_p(real_in.data_ptr()), c_void_p(int_in.data_ptr()),
                                                      c_int64(count), _stream_handle(stream)))


def nccl_library_path():
    """The NCCL library that ships with torch (newer than a system one), or None to let the loader search."""
    try:
        import nvidia.nccl
        for base in nvidia.nccl.__path__:
            path = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(path):
                return path
    except ImportError:
        pass
    return None


def nccl_unique_id() -> bytes:
    lib = load()
    buf = ctypes.create_string_buffer(128)
    path = nccl_library_path()
    rc = lib.dsmd_nccl_unique_id(path.encode() if path else None, buf)
    if rc != OK:
        raise DsmdError(rc, "cannot create an NCCL unique id (is libnccl.so.2 loadable?)")
    return buf.raw


class Domain:
    """``dsmd_domain``: one rank's brick of a spatial decomposition - migration, ghost plan, refresh and the MD loop,
    native, over NCCL point-to-point."""

    def __init__(self, ctx: Context, rank, world, dims, box, halo_width, skin, unique_id: bytes | None):
        self.lib, self.ctx = ctx.lib, ctx
        self.lib.dsmd_domain_last_error.restype = ctypes.c_char_p
        self.lib.dsmd_domain_last_error.argtypes = [c_void_p]
        self.lib.dsmd_domain_destroy.restype = None
        self.lib.dsmd_domain_destroy.argtypes = [c_void_p]
        self.h = c_void_p()
        d, b = _arr(dims, np.int32), _arr(box, np.float64)
        path = nccl_library_path()
        rc = self.lib.dsmd_domain_create(ctx.h, c_int(rank), c_int(world), _p(d), _p(b), c_double(halo_width),
                                         c_double(skin), path.encode() if path else None, unique_id, ctypes.byref(self.h))
        self._check(rc)

    def _check(self, rc):
        if rc != OK:
            raise DsmdError(rc, self.lib.dsmd_domain_last_error(self.h).decode() if self.h else "dsmd_domain_create failed")

    def rebuild(self, stream=None):
        self._check(self.lib.dsmd_domain_rebuild(self.h, _stream_handle(stream)))

    def refresh(self, stream=None):
        self._check(self.lib.dsmd_domain_refresh(self.h, _stream_handle(stream)))

    def forces_host(self, x, y, z, fx, fy, fz, buffer_atoms, rebuild=False, stream=None):
        """Host-buffer force call on several ranks: raw host addresses (ints) or numpy arrays of this rank's owned atoms,
        each buffer with room for buffer_atoms atoms."""
        def addr(a):
            return c_void_p(a) if isinstance(a, int) else _p(a)
        self._check(self.lib.dsmd_domain_forces_host(self.h, addr(x), addr(y), addr(z), c_int(int(rebuild)), addr(fx), addr(fy),
                                                     addr(fz), c_int64(int(buffer_atoms)), _stream_handle(stream)))

    def run(self, n_steps, dt, force_to_accel=1.0, hi_frac=0.5, stream=None):
        self._check(self.lib.dsmd_domain_run(self.h, c_int64(n_steps), c_double(dt), c_double(force_to_accel),
                                             c_double(hi_frac), _stream_handle(stream)))

    def reverse_forces(self, stream=None):
        """Forces held on ghost atoms go back to, and are added to, their owners."""
        self._check(self.lib.dsmd_domain_reverse_forces(self.h, _stream_handle(stream)))

    def exchange_field(self, tensor, reverse=False, stream=None):
        """A [rows, width] float32 / float64 device tensor over owned + ghost atoms: forward copies owners' rows into
        their ghosts, reverse adds the ghosts' rows to their owners'."""
        rows, width = tensor.shape
        self._check(self.lib.dsmd_domain_exchange_field(self.h, c_void_p(tensor.data_ptr()), c_int64(rows), c_int64(width),
                                                        c_int(tensor.element_size()), c_int(1 if reverse else 0),
                                                        _stream_handle(stream)))

    def set_wait_limit(self, seconds):
        self._check(self.lib.dsmd_domain_set_wait_limit(self.h, c_double(seconds)))

    def abort(self):
        self.lib.dsmd_domain_abort(self.h)

    def peers(self):
        n = ctypes.c_int32(0)
        ranks = (ctypes.c_int32 * 26)()
        msgs = (ctypes.c_int32 * 1)()
        self._check(self.lib.dsmd_domain_peers(self.h, ctypes.byref(n), ranks, msgs))
        return dict(ranks=[ranks[k] for k in range(n.value)], messages_per_exchange=msgs[0])

    def profile(self, enable=True):
        """Switches per-phase timing on or off; returns the accumulated per-step averages (ms) so far."""
        ms = (c_double * 10)()
        n = c_int64(0)
        self._check(self.lib.dsmd_domain_profile(self.h, c_int(int(enable)), ms, ctypes.byref(n)))
        names = ["integrate1_pack", "vote", "refresh_issue_interior", "boundary_or_full", "integrate2", "rebuild",
                 "rebuild_migrate", "rebuild_sort_owned", "rebuild_ghost_plan", "rebuild_list"]
        steps = max(n.value, 1)
        return {k: ms[i] / steps for i, k in enumerate(names)} | {"steps": n.value}

    def stats(self):
        v = [c_int64(0) for _ in range(4)]
        w, l = c_double(0.0), c_int64(0)
        self._check(self.lib.dsmd_domain_stats(self.h, ctypes.byref(v[0]), ctypes.byref(v[1]), ctypes.byref(v[2]),
                                               ctypes.byref(v[3]), ctypes.byref(w), ctypes.byref(l)))
        return dict(rebuilds=v[0].value, migrated=v[1].value, ghosts=v[2].value, positions_sent_per_step=v[3].value,
                    worst_disp_sq=w.value, launches=l.value)

    def close(self):
        if self.h:
            self.lib.dsmd_domain_destroy(self.h)
            self.h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


NOALLOC_MAX_ATOMS = 16777216


def kinetic_energy_noalloc(vx_ptr, vy_ptr, vz_ptr, mass_ptr, n, out_ptr, stream=None):
    """``dsmd_kinetic_energy_noalloc``: device pointers in, the sum into the device double at out_ptr; the variant of the
    kinetic-energy sum for callers that must not allocate device memory (its scratch is a fixed array inside the
    library). Raises DsmdError with the library's message when n exceeds NOALLOC_MAX_ATOMS."""
    lib = load()
    msg = ctypes.c_char_p()
    rc = lib.dsmd_kinetic_energy_noalloc(c_void_p(vx_ptr), c_void_p(vy_ptr), c_void_p(vz_ptr), c_void_p(mass_ptr),
                                         c_int64(n), c_void_p(out_ptr), _stream_handle(stream), ctypes.byref(msg))
    if rc != OK:
        raise DsmdError(rc, (msg.value or b"").decode())


class EdgeBuilder:
    """``dsmd_edges``: the radius-graph builder (the reference's EdgeBuilder, include/EdgeBuilder.cuh)."""

    def __init__(self, device: int = 0):
        self.lib = load()
        self.h = c_void_p()
        rc = self.lib.dsmd_edges_create(c_int(device), ctypes.byref(self.h))
        if rc != OK:
            raise DsmdError(rc, "dsmd_edges_create failed")
        self.device = device

    def _check(self, rc):
        if rc != OK:
            raise DsmdError(rc, self.lib.dsmd_edges_last_error(self.h).decode())

    def close(self):
        if self.h:
            self.lib.dsmd_edges_destroy(self.h)
            self.h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def build(self, x, y, z, cutoff, lo=None, hi=None, n_centers=None, owner=None, shift=None, receiver_ok=None,
              row=1, stream=None):
        """x, y, z: torch CUDA float64 tensors. Returns (edge_index [2, E] int64, edge_shift [E, 3] float64 or None)
        as torch tensors that view the builder's buffers (valid until the next build)."""
        import torch
        n = x.numel()
        l, h = _arr(lo, np.float64), _arr(hi, np.float64)
        nc = n if n_centers is None else n_centers
        ne = c_int64(0)
        sx = sy = sz = None
        if shift is not None:
            sx, sy, sz = shift
        self._check(self.lib.dsmd_edges_build(
            self.h, c_void_p(x.data_ptr()), c_void_p(y.data_ptr()), c_void_p(z.data_ptr()), c_int64(n), c_double(cutoff),
            _p(l), _p(h), c_int64(nc), c_void_p(owner.data_ptr()) if owner is not None else None,
            c_void_p(sx.data_ptr()) if sx is not None else None, c_void_p(sy.data_ptr()) if sy is not None else None,
            c_void_p(sz.data_ptr()) if sz is not None else None,
            c_void_p(receiver_ok.data_ptr()) if receiver_ok is not None else None, c_int(row), ctypes.byref(ne),
            _stream_handle(stream)))
        return self.result(with_shift=owner is not None)

    def result(self, with_shift=False):
        import torch
        pi, ps, ne = c_void_p(), c_void_p(), c_int64(0)
        self._check(self.lib.dsmd_edges_result(self.h, ctypes.byref(pi), ctypes.byref(ps), ctypes.byref(ne)))
        E = ne.value
        dev = torch.device("cuda", self.device)
        if E == 0:
            return torch.zeros((2, 0), dtype=torch.int64, device=dev), None
        idx = _tensor_from_ptr(pi.value, (2, E), torch.int64, dev)
        sh = _tensor_from_ptr(ps.value, (E, 3), torch.float64, dev) if with_shift and ps.value else None
        return idx, sh

    def images(self, x, y, z, types, box, origin, region_lo, region_hi, shells, stream=None):
        """Wrapped atoms + periodic images (MLIPStep's image atoms): dict of torch views x, y, z, type, owner, shift."""
        import torch
        n = x.numel()
        args = [_arr(v, np.float64) for v in (box, origin, region_lo, region_hi)]
        sh = _arr(shells, np.int32)
        n_all = c_int64(0)
        self._check(self.lib.dsmd_images_build(
            self.h, c_void_p(x.data_ptr()), c_void_p(y.data_ptr()), c_void_p(z.data_ptr()),
            c_void_p(types.data_ptr()) if types is not None else None, c_int64(n), *[_p(a) for a in args], _p(sh),
            ctypes.byref(n_all), _stream_handle(stream)))
        ptrs = [c_void_p() for _ in range(8)]
        self._check(self.lib.dsmd_images_result(self.h, *[ctypes.byref(p) for p in ptrs], ctypes.byref(n_all)))
        N = n_all.value
        dev = torch.device("cuda", self.device)
        f64 = lambda p: _tensor_from_ptr(p.value, (N,), torch.float64, dev)
        i32 = lambda p: _tensor_from_ptr(p.value, (N,), torch.int32, dev)
        return dict(x=f64(ptrs[0]), y=f64(ptrs[1]), z=f64(ptrs[2]), type=i32(ptrs[3]), owner=i32(ptrs[4]),
                    shift=(f64(ptrs[5]), f64(ptrs[6]), f64(ptrs[7])), n_all=N)

    def fold_image_forces(self, fx, fy, fz, tx, ty, tz, n_out=-1, with_images=True, stream=None):
        """target += model forces of the atoms and of their images (the images of the last images() call)."""
        self._check(self.lib.dsmd_images_fold_forces(
            self.h, c_void_p(fx.data_ptr()), c_void_p(fy.data_ptr()), c_void_p(fz.data_ptr()), c_int64(n_out),
            c_int(1 if with_images else 0), c_void_p(tx.data_ptr()), c_void_p(ty.data_ptr()), c_void_p(tz.data_ptr()),
            _stream_handle(stream)))

    def virial_from_forces(self, x, y, z, fx, fy, fz, stream=None):
        out = (c_double * 4)()
        self._check(self.lib.dsmd_virial_from_forces(
            self.h, *[c_void_p(t.data_ptr()) for t in (x, y, z, fx, fy, fz)], c_int64(x.numel()), out,
            _stream_handle(stream)))
        return np.array(list(out))

    def mark_receivers(self, x, y, z, lo, hi, reach, stream=None):
        import torch
        n = x.numel()
        ok = torch.empty(n, dtype=torch.uint8, device=x.device)
        l, h = _arr(lo, np.float64), _arr(hi, np.float64)
        self._check(self.lib.dsmd_mark_receivers(self.h, c_void_p(x.data_ptr()), c_void_p(y.data_ptr()),
                                                 c_void_p(z.data_ptr()), c_int64(n), _p(l), _p(h), c_double(reach),
                                                 c_void_p(ok.data_ptr()), _stream_handle(stream)))
        return ok

    def build_periodic(self, x, y, z, box, cutoff, stream=None):
        import torch
        n = x.numel()
        b = _arr(box, np.float64)
        ne = c_int64(0)
        self._check(self.lib.dsmd_edges_build_periodic(self.h, c_void_p(x.data_ptr()), c_void_p(y.data_ptr()),
                                                       c_void_p(z.data_ptr()), c_int64(n), _p(b), c_double(cutoff),
                                                       ctypes.byref(ne), _stream_handle(stream)))
        ps, pd_, psh, pv = c_void_p(), c_void_p(), c_void_p(), c_void_p()
        self._check(self.lib.dsmd_edges_result_compact(self.h, ctypes.byref(ps), ctypes.byref(pd_), ctypes.byref(psh),
                                                       ctypes.byref(pv), ctypes.byref(ne)))
        E = ne.value
        dev = torch.device("cuda", self.device)
        if E == 0:
            z32 = torch.zeros(0, dtype=torch.int32, device=dev)
            return z32, z32, torch.zeros((0, 3), dtype=torch.int8, device=dev), torch.zeros((0, 3), device=dev)
        return (_tensor_from_ptr(ps.value, (E,), torch.int32, dev), _tensor_from_ptr(pd_.value, (E,), torch.int32, dev),
                _tensor_from_ptr(psh.value, (E, 3), torch.int8, dev),
                _tensor_from_ptr(pv.value, (E, 3), torch.float32, dev))


def _tensor_from_ptr(ptr, shape, dtype, device):
    """A torch tensor viewing device memory owned by the library (no copy), through __cuda_array_interface__."""
    import torch
    typestr = {torch.int64: "<i8", torch.int32: "<i4", torch.float64: "<f8", torch.float32: "<f4", torch.int8: "|i1",
               torch.uint8: "|u1"}[dtype]

    class _Holder:
        pass

    holder = _Holder()
    holder.__cuda_array_interface__ = dict(shape=tuple(shape), typestr=typestr, data=(int(ptr), False), version=2)
    return torch.as_tensor(holder, device=device)
