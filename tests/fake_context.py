"""A CPU stand-in for deepscalemd_b200.capi.Context used by the world_size-2 gloo tests of the domain logic: the same
methods on numpy arrays / CPU torch tensors, with forces from the CPU oracle. Test infrastructure only."""
import numpy as np
import torch

from oracle import cpu_oracle as co

REAL = ["x", "y", "z", "vx", "vy", "vz", "fx", "fy", "fz", "mass", "charge"]


class FakeContext:
    def __init__(self, capacity, box, eps, sig, cutoff, skin):
        self.cap = capacity
        self.a = {k: np.zeros(capacity) for k in REAL}
        self.type = np.zeros(capacity, dtype=np.int32)
        self.gid = np.zeros(capacity, dtype=np.int32)
        self.n_owned = self.n_total = 0
        self.box = np.asarray(box, dtype=np.float64)
        self.c6, self.c12 = co.lj_tables(eps, sig)
        self.cutoff, self.skin = cutoff, skin
        self.split = (0, 0, 0)
        self.pairs = None
        self.ref = None
        self.word = torch.zeros(1, dtype=torch.int64)
        self.scalars = None

    def set_split(self, split):
        self.split = tuple(int(s) for s in split)

    def upload(self, pos, vel, mass, gid):
        n = len(pos)
        for k, name in enumerate("xyz"):
            self.a[name][:n] = pos[:, k]
            self.a["v" + name][:n] = vel[:, k]
        self.a["mass"][:n] = mass
        self.gid[:n] = gid
        self.n_owned = self.n_total = n

    def counts(self):
        return self.n_owned, self.n_total

    def set_counts(self, a, b):
        self.n_owned, self.n_total = a, b

    def halo_select(self, lo, hi, index_tensor, stream=None):
        n = self.n_owned
        m = np.ones(n, dtype=bool)
        for k, name in enumerate("xyz"):
            m &= (self.a[name][:n] >= lo[k]) & (self.a[name][:n] < hi[k])
        idx = np.nonzero(m)[0].astype(np.int32)
        index_tensor[:len(idx)] = torch.from_numpy(idx)
        return len(idx)

    def halo_pack_records(self, index, count, shift, real_out, int_out, stream=None):
        ix = index[:count].numpy()
        r = real_out.numpy().reshape(-1, 8)
        for k, name in enumerate(("x", "y", "z")):
            r[:count, k] = self.a[name][ix] + shift[k]
        for k, name in enumerate(("vx", "vy", "vz", "mass", "charge")):
            r[:count, 3 + k] = self.a[name][ix]
        i = int_out.numpy().reshape(-1, 2)
        i[:count, 0] = self.type[ix]
        i[:count, 1] = self.gid[ix]

    def halo_append_records(self, real_in, int_in, count, stream=None):
        r = real_in.numpy().reshape(-1, 8)[:count]
        i = int_in.numpy().reshape(-1, 2)[:count]
        s = slice(self.n_total, self.n_total + count)
        for k, name in enumerate(("x", "y", "z", "vx", "vy", "vz", "mass", "charge")):
            self.a[name][s] = r[:, k]
        for name in ("fx", "fy", "fz"):
            self.a[name][s] = 0.0
        self.type[s] = i[:, 0]
        self.gid[s] = i[:, 1]
        self.n_total += count

    def sort_owned(self, stream=None):
        self.n_total = self.n_owned

    def build_neighbor_list(self, stream=None):
        n = self.n_total
        self.pairs = co.pairs(self.a["x"][:n], self.a["y"][:n], self.a["z"][:n], self.n_owned, self.box, split=self.split,
                              search=self.cutoff + self.skin)
        self.ref = np.stack([self.a[k][:self.n_owned].copy() for k in "xyz"], axis=1)
        self.word[0] = 0

    def halo_pack(self, index, image, count, out, stream=None):
        ix = index[:count].numpy()
        o = out.numpy().reshape(-1, 3)
        img = image.numpy().reshape(-1, 3)[:count]
        for k, name in enumerate("xyz"):
            o[:count, k] = self.a[name][ix] + img[:, k] * self.box[k]

    def halo_unpack(self, buf, first_ghost, count, stream=None):
        b = buf.numpy().reshape(-1, 3)[:count]
        s = slice(self.n_owned + first_ghost, self.n_owned + first_ghost + count)
        for k, name in enumerate("xyz"):
            self.a[name][s] = b[:, k]

    def ghost_slots(self, n_ghost):
        return torch.arange(self.n_owned, self.n_owned + n_ghost, dtype=torch.int32)   # ghosts stay in arrival order here

    def displacement_word(self):
        return self.word

    def integrate(self, half, dt, f2a, stream=None):
        n = self.n_owned
        pos = [self.a[k][:n] for k in "xyz"]
        vel = [self.a["v" + k][:n] for k in "xyz"]
        frc = [self.a["f" + k][:n] for k in "xyz"]
        co.vv_half(half == 1, dt, f2a, pos, vel, frc, np.ascontiguousarray(self.a["mass"][:n]))
        if half == 1 and self.ref is not None:
            d2 = sum((p - self.ref[:, k]) ** 2 for k, p in enumerate(pos)).max()
            bits = np.array([max(d2, float(np.array(self.word.numpy()[0]).view(np.float64)))]).view(np.int64)[0]
            self.word[0] = int(bits)

    def compute_forces(self, phase=0, want_energy=False, stream=None):
        n = self.n_total
        p = self.pairs
        if phase == 1:
            p = p[p[:, 1] < self.n_owned]
        elif phase == 2:
            p = p[p[:, 1] >= self.n_owned]
        f, sc = co.forces(self.a["x"][:n], self.a["y"][:n], self.a["z"][:n], self.n_owned, self.box, p, self.c6, self.c12,
                          self.cutoff, gid=self.gid[:n], split=self.split)
        for k, name in enumerate(("fx", "fy", "fz")):
            if phase == 2:
                self.a[name][:self.n_owned] += f[:, k]
            else:
                self.a[name][:self.n_owned] = f[:, k]
        if phase == 2 and self.scalars is not None:
            for key in ("pe", "virial", "pairs_in_cutoff"):
                sc[key] += self.scalars[key]
            sc["virial_diag"] = sc["virial_diag"] + self.scalars["virial_diag"]
        self.scalars = sc

    def read_scalars(self, stream=None):
        return self.scalars
