"""Spatial domain decomposition over the GPUs of one node: brick grid, atom migration, ghost-atom (halo) plan and the
per-step positions-only refresh, with `torch.distributed` (NCCL over NVLink; gloo in the CPU tests) as the transport and
the C ABI's pack / select / append / unpack kernels as the data plane.

Behaviour follows what the reference obtains from its external decomposition library through
MDSystem::migrate_particles_on_device, exchange_halo_on_device(rebuild) and the split-phase
begin/end_halo_exchange_on_device (src/md_system.cpp:1448-1509): owned atoms first, ghosts behind them; a ghost is every
periodic image of a neighbour's atom that lies within the halo width of this rank's brick on the split axes (edges and
corners included) and arrives already image-shifted; an axis with a single brick gets no ghosts (the kernels' wrapping
coordinates resolve its periodicity); the refresh between list builds moves positions only (24 bytes per ghost) and is
overlapped with the interior part of the force evaluation.

The exchange has one real communication step per MD step and no collective on the data path: every rank sends to and
receives from its (at most 26) neighbour directions with grouped point-to-point operations. The only collectives are an
all-gather of the per-direction counts at a list rebuild and a one-word MAX all-reduce for the rebuild vote.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

INF = float("inf")


def grid_dims(world_size: int, box) -> tuple[int, int, int]:
    """Brick grid for `world_size` ranks that minimises the ghost volume (surface of a brick); on NVSwitch every peer is
    equally near, so nothing but geometry enters. 1 -> 1x1x1, 2 -> 2x1x1, 4 -> 2x2x1, 8 -> 2x2x2 for a cubic box."""
    best, best_cost = (world_size, 1, 1), None
    for px in range(1, world_size + 1):
        if world_size % px:
            continue
        for py in range(1, world_size // px + 1):
            if (world_size // px) % py:
                continue
            pz = world_size // (px * py)
            w = [box[0] / px, box[1] / py, box[2] / pz]
            cost = sum((2.0 * w[(a + 1) % 3] * w[(a + 2) % 3]) for a, p in enumerate((px, py, pz)) if p > 1)
            key = (round(cost, 9), -min(w), -px, -py)   # ties: the thicker brick (room for the halo), then x before y
            if best_cost is None or key < best_cost:
                best, best_cost = (px, py, pz), key
    return best


@dataclass
class Direction:
    e: tuple            # the way the data travels, each component in {-1, 0, 1}
    dest: int           # rank that receives what this rank sends along e
    src: int            # rank whose data arrives here along e
    image: tuple        # box lengths added to the sender's positions so that the receiver sees the right periodic image
    index: int          # position in the direction list (same list on every rank)


class Decomposition:
    """Brick grid over a periodic orthorhombic box, rank <-> brick coordinates, and this rank's neighbour directions."""

    def __init__(self, box, world_size: int, rank: int, periodic=(1, 1, 1), dims=None):
        self.box = np.asarray(box, dtype=np.float64)
        self.periodic = tuple(int(p) for p in periodic)
        self.dims = tuple(dims) if dims is not None else grid_dims(world_size, self.box)
        assert self.dims[0] * self.dims[1] * self.dims[2] == world_size
        self.world_size, self.rank = world_size, rank
        self.coords = self.coords_of(rank)
        self.lo = self.box * np.array(self.coords) / np.array(self.dims)
        self.hi = self.box * (np.array(self.coords) + 1) / np.array(self.dims)
        self.split = tuple(d > 1 for d in self.dims)
        # every rank enumerates the same directions in the same order (what keeps sends and receives between one pair of
        # ranks matched when both +1 and -1 along an axis lead to the same peer, as with two bricks on a periodic axis)
        all_e = [e for e in itertools.product((-1, 0, 1), repeat=3)
                 if any(e) and all(e[a] == 0 or self.split[a] for a in range(3))]
        self.directions = []
        for k, e in enumerate(all_e):
            dest, image = self._neighbour(self.coords, e)
            src, _ = self._neighbour(self.coords, tuple(-c for c in e))
            if dest is None or src is None:
                dest = src = -1     # open boundary on a non-periodic axis: nothing travels
            self.directions.append(Direction(e, dest, src, image, k))

    def coords_of(self, rank):
        px, py, pz = self.dims
        return (rank // (py * pz), (rank // pz) % py, rank % pz)

    def rank_of(self, coords):
        return (coords[0] * self.dims[1] + coords[1]) * self.dims[2] + coords[2]

    def _neighbour(self, coords, e):
        c, image = [], []
        for a in range(3):
            v = coords[a] + e[a]
            im = 0
            if v < 0 or v >= self.dims[a]:
                if not self.periodic[a]:
                    return None, (0, 0, 0)
                im = 1 if v < 0 else -1
                v %= self.dims[a]
            c.append(v)
            image.append(im)
        return self.rank_of(c), tuple(image)

    def owner_of(self, pos):
        """Rank that owns each position (positions wrapped into the box first)."""
        pos = np.asarray(pos, dtype=np.float64)
        w = pos - self.box * np.floor(pos / self.box)
        c = np.minimum((w / self.box * np.array(self.dims)).astype(np.int64), np.array(self.dims) - 1)
        return (c[:, 0] * self.dims[1] + c[:, 1]) * self.dims[2] + c[:, 2]

    def send_region(self, e, width):
        """Owned atoms within `width` of the neighbour brick along e: half-spaces on the axes where e is non-zero."""
        lo, hi = [-INF] * 3, [INF] * 3
        for a in range(3):
            if e[a] > 0:
                lo[a] = self.hi[a] - width
            elif e[a] < 0:
                hi[a] = self.lo[a] + width
        return lo, hi

    def leave_region(self, e):
        """Atoms that left the brick along e (on split axes; e = 0 there means 'still inside')."""
        lo, hi = [-INF] * 3, [INF] * 3
        for a in range(3):
            if not self.split[a]:
                continue
            if e[a] > 0:
                lo[a] = self.hi[a]
            elif e[a] < 0:
                hi[a] = self.lo[a]
            else:
                lo[a], hi[a] = self.lo[a], self.hi[a]
        return lo, hi

    def stay_region(self):
        return self.leave_region((0, 0, 0))


class DomainRunner:
    """Drives one rank's context through MD steps with ghost exchange. `ctx` is a capi.Context (or, in the CPU tests, an
    object with the same methods working on CPU tensors); `group` a torch.distributed process group."""

    def __init__(self, ctx, decomp: Decomposition, halo_width: float, device, group=None, streams=True):
        self.ctx, self.d, self.h = ctx, decomp, float(halo_width)
        self.device = torch.device(device)
        self.group = group
        self.cuda = self.device.type == "cuda"
        self.main = torch.cuda.current_stream(self.device) if self.cuda else None
        self.side = torch.cuda.Stream(self.device, priority=-1) if (self.cuda and streams) else self.main
        self.n_dirs = len(decomp.directions)
        self.send_counts = [0] * self.n_dirs
        self.recv_counts = [0] * self.n_dirs
        self.send_index = self.send_image = self.send_buf = self.recv_buf = None
        self.n_ghost = 0
        self.rebuilds = 0
        self.vote = None            # (pinned copy of the global displacement word, event): read one step late
        self.vote_history = (0.0, 0.0)
        self.worst_disp_sq = 0.0    # largest displacement under which forces were evaluated without a rebuild
        self._pinned = [torch.empty(1, dtype=torch.int64).pin_memory() for _ in range(2)] if self.cuda else None
        self._pinned_at = 0
        self.bytes_sent_per_step = 0

    # -- plumbing ---------------------------------------------------------------------------------------------------------
    def _sh(self, stream):
        return stream if self.cuda else None

    def _exchange_counts(self, mine):
        """All ranks learn every rank's per-direction send counts; returns what arrives here per direction."""
        t = torch.tensor(mine, dtype=torch.int64, device=self.device)
        out = torch.empty(self.d.world_size * self.n_dirs, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(out, t, group=self.group)
        table = out.cpu().numpy().reshape(self.d.world_size, self.n_dirs)
        return [int(table[dr.src, dr.index]) if dr.src >= 0 else 0 for dr in self.d.directions]

    def _exchange(self, send_chunks, recv_chunks, backwards=False):
        """One grouped point-to-point round: chunk k travels along direction k (backwards: against it, from the rank that
        received along k to the rank that sent)."""
        ops = []
        for dr, s, r in zip(self.d.directions, send_chunks, recv_chunks):
            if dr.dest < 0:
                continue
            to, frm = (dr.src, dr.dest) if backwards else (dr.dest, dr.src)
            if r is not None and r.numel():
                ops.append(dist.P2POp(dist.irecv, r, frm, group=self.group))
            if s is not None and s.numel():
                ops.append(dist.P2POp(dist.isend, s, to, group=self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def _select(self, lo, hi, scratch):
        n = self.ctx.halo_select(lo, hi, scratch, stream=self._sh(self.main))
        return scratch[:n].clone(), n

    def _move_records(self, index_lists, images, append_as_owned: bool):
        """Packs full records of the listed atoms per direction, exchanges them and appends what arrives."""
        ctx = self.ctx
        counts = [len(ix) for ix in index_lists]
        incoming = self._exchange_counts(counts)
        send_real, send_int, recv_real, recv_int = [], [], [], []
        for dr, ix, n_in in zip(self.d.directions, index_lists, incoming):
            n = len(ix)
            sr = torch.empty(8 * n, dtype=torch.float64, device=self.device)
            si = torch.empty(2 * n, dtype=torch.int32, device=self.device)
            if n:
                shift = np.array(images[dr.index], dtype=np.float64) * self.d.box
                ctx.halo_pack_records(ix, n, shift, sr, si, stream=self._sh(self.main))
            send_real.append(sr)
            send_int.append(si)
            recv_real.append(torch.empty(8 * n_in, dtype=torch.float64, device=self.device))
            recv_int.append(torch.empty(2 * n_in, dtype=torch.int32, device=self.device))
        self._exchange(send_real, recv_real)
        self._exchange(send_int, recv_int)
        return incoming, recv_real, recv_int

    # -- list rebuild step ----------------------------------------------------------------------------------------------------
    def migrate(self):
        """Atoms that left the brick go to the neighbour that now owns them (with the image shift that puts them inside
        it); ghosts are dropped. Collective."""
        ctx, d = self.ctx, self.d
        n_owned, _ = ctx.counts()
        scratch = torch.empty(max(n_owned, 1), dtype=torch.int32, device=self.device)
        lo, hi = d.stay_region()
        stay, n_stay = self._select(lo, hi, scratch)
        leave = []
        for dr in d.directions:
            if dr.dest < 0:
                leave.append(scratch[:0].clone())
                continue
            lo, hi = d.leave_region(dr.e)
            ix, _ = self._select(lo, hi, scratch)
            leave.append(ix)
        n_leave = sum(len(ix) for ix in leave)
        if n_stay + n_leave != n_owned:
            raise RuntimeError(f"rank {d.rank}: {n_owned - n_stay - n_leave} atoms are neither inside the brick nor in a "
                               "neighbouring one (moved more than one brick, or non-finite)")
        sr = torch.empty(8 * max(n_stay, 1), dtype=torch.float64, device=self.device)
        si = torch.empty(2 * max(n_stay, 1), dtype=torch.int32, device=self.device)
        if n_stay:
            ctx.halo_pack_records(stay, n_stay, np.zeros(3), sr, si, stream=self._sh(self.main))
        incoming, recv_real, recv_int = self._move_records(leave, [dr.image for dr in d.directions], True)
        ctx.set_counts(0, 0)
        if n_stay:
            ctx.halo_append_records(sr, si, n_stay, stream=self._sh(self.main))
        for n_in, rr, ri in zip(incoming, recv_real, recv_int):
            if n_in:
                ctx.halo_append_records(rr, ri, n_in, stream=self._sh(self.main))
        total = n_stay + sum(incoming)
        ctx.set_counts(total, total)
        return n_leave, sum(incoming)

    def build_halo(self):
        """Ghost plan: which owned atoms each neighbour direction needs (they stay in place until the next rebuild), the
        full records of the ghosts, and the buffers of the per-step refresh. Collective."""
        ctx, d = self.ctx, self.d
        n_owned, _ = ctx.counts()
        scratch = torch.empty(max(n_owned, 1), dtype=torch.int32, device=self.device)
        lists = []
        for dr in d.directions:
            if dr.dest < 0:
                lists.append(scratch[:0].clone())
                continue
            lo, hi = d.send_region(dr.e, self.h)
            ix, _ = self._select(lo, hi, scratch)
            lists.append(ix)
        incoming, recv_real, recv_int = self._move_records(lists, [dr.image for dr in d.directions], False)
        for n_in, rr, ri in zip(incoming, recv_real, recv_int):
            if n_in:
                ctx.halo_append_records(rr, ri, n_in, stream=self._sh(self.main))
        self.send_counts = [len(ix) for ix in lists]
        self.recv_counts = incoming
        self.n_ghost = sum(incoming)
        n_send = sum(self.send_counts)
        self.send_index = torch.cat(lists) if n_send else torch.empty(0, dtype=torch.int32, device=self.device)
        image = np.concatenate([np.tile(np.array(dr.image, dtype=np.int8), (n, 1))
                                for dr, n in zip(d.directions, self.send_counts)]) if n_send else np.zeros((0, 3), np.int8)
        self.send_image = torch.from_numpy(np.ascontiguousarray(image)).to(self.device)
        self.send_buf = torch.empty(3 * n_send, dtype=torch.float64, device=self.device)
        self.recv_buf = torch.empty(3 * self.n_ghost, dtype=torch.float64, device=self.device)
        self.bytes_sent_per_step = 24 * n_send

    def rebuild(self):
        """Migration, cell sort of the owned atoms, ghost plan, list build. Collective."""
        self.migrate()
        self.ctx.sort_owned(stream=self._sh(self.main))
        self.build_halo()
        self.ctx.build_neighbor_list(stream=self._sh(self.main))
        self.rebuilds += 1
        self.vote = None
        self.vote_history = (0.0, 0.0)

    # -- per-step refresh ---------------------------------------------------------------------------------------------------------
    def _chunks(self, buf, counts):
        out, at = [], 0
        for n in counts:
            out.append(buf[3 * at:3 * (at + n)])
            at += n
        return out

    def refresh_begin(self):
        """Packs the current positions of the plan's atoms and posts the exchange on the side stream."""
        if self.cuda and self.side is not self.main:
            self.side.wait_stream(self.main)
        ctx = self.ctx
        with (torch.cuda.stream(self.side) if self.cuda else _null()):
            n_send = sum(self.send_counts)
            if n_send:
                ctx.halo_pack(self.send_index, self.send_image, n_send, self.send_buf, stream=self._sh(self.side))
            self._exchange(self._chunks(self.send_buf, self.send_counts), self._chunks(self.recv_buf, self.recv_counts))
            if self.n_ghost:
                ctx.halo_unpack(self.recv_buf, 0, self.n_ghost, stream=self._sh(self.side))

    def refresh_end(self):
        """Orders the main stream behind the unpack (ForceCalculatorCUDA::make_force_stream_wait_for_halo)."""
        if self.cuda and self.side is not self.main:
            self.main.wait_stream(self.side)

    # -- per-atom feature fields along the ghost plan ------------------------------------------------------------------------
    @staticmethod
    def _row_chunks(rows, counts):
        out, at = [], 0
        for n in counts:
            out.append(rows[at:at + n])
            at += n
        return out

    def exchange_field(self, field, reverse=False):
        """Moves a per-atom field (a contiguous [n_owned + n_ghost, width] float32 / float64 tensor in the context's slot
        order) along the ghost plan of the last rebuild, as MDSystem::exchange_field_on_device does for the node features
        of a message-passing model (src/md_system.cpp:1520-1545; contract include/MLIPHaloTransport.h:16-37).
        forward: the ghost rows are overwritten with the rows of their owners. reverse (its adjoint): the ghost rows are
        added to the rows of their owners; the ghost rows are not defined afterwards. Collective."""
        n_owned, n_total = self.ctx.counts()
        if field.dim() != 2 or not field.is_contiguous() or field.shape[0] != n_total:
            raise ValueError(f"the field must be a contiguous [{n_total}, width] tensor ({n_owned} owned + "
                             f"{n_total - n_owned} ghost atoms)")
        if field.dtype not in (torch.float32, torch.float64):
            raise ValueError("the field must be float32 or float64")
        n_send = sum(self.send_counts)
        plan = self.send_index[:n_send].long()
        slots = self.ctx.ghost_slots(self.n_ghost).long()
        width = field.shape[1]
        if not reverse:
            out = field.index_select(0, plan)
            arrived = torch.empty((self.n_ghost, width), dtype=field.dtype, device=field.device)
            self._exchange(self._row_chunks(out, self.send_counts), self._row_chunks(arrived, self.recv_counts))
            field.index_copy_(0, slots, arrived)
        else:
            back = field.index_select(0, slots)
            arrived = torch.empty((n_send, width), dtype=field.dtype, device=field.device)
            self._exchange(self._row_chunks(back, self.recv_counts), self._row_chunks(arrived, self.send_counts), backwards=True)
            field.index_add_(0, plan, arrived)
        return field

    # -- rebuild vote -----------------------------------------------------------------------------------------------------------
    def vote_rebuild(self, skin, hi_frac=0.5, lagged=True):
        """True when any rank saw an owned atom move further than hi_frac * skin since the last build. lagged: the
        decision uses the all-reduced word of the previous step (read back without stalling this one), extrapolated by
        its last growth, as the reference does on several ranks (src/md_simulation.cpp:1232-1245)."""
        word = self.ctx.displacement_word()
        if self.d.world_size > 1:
            dist.all_reduce(word, op=dist.ReduceOp.MAX, group=self.group)
        limit2 = (hi_frac * skin) ** 2
        if not lagged or not self.cuda:
            d2 = float(word.cpu().view(torch.float64)[0])
            self.worst_disp_sq = max(self.worst_disp_sq, d2 if d2 <= limit2 else 0.0)
            return d2 > limit2
        if self.vote is not None:                      # what the previous step saw
            pinned, event = self.vote
            event.synchronize()
            d_seen = float(np.sqrt(pinned.view(torch.float64)[0].item()))
            self.vote_history = (self.vote_history[1], d_seen)
            self.worst_disp_sq = max(self.worst_disp_sq, d_seen * d_seen)   # its forces ran under this displacement
        slot = self._pinned[self._pinned_at]
        self._pinned_at ^= 1
        slot.copy_(word, non_blocking=True)
        event = torch.cuda.Event()
        event.record(self.main)
        self.vote = (slot, event)
        d_before, d_now = self.vote_history
        predicted = d_now + 1.5 * max(d_now - d_before, 0.0)
        return predicted * predicted > limit2

    # -- MD ------------------------------------------------------------------------------------------------------------------------
    def step(self, dt, force_to_accel, skin, hi_frac=0.5, lagged=True, overlap=True, want_energy=False):
        """One velocity-Verlet step of the hot path (MDSimulation::single_step, src/md_simulation.cpp:899-941)."""
        ctx, s = self.ctx, self._sh(self.main)
        ctx.integrate(1, dt, force_to_accel, stream=s)           # v += dt/2 a; x += dt v; pack owned; displacement
        if self.vote_rebuild(skin, hi_frac, lagged):
            self.rebuild()
            ctx.compute_forces(0, want_energy, stream=s)
        elif self.d.world_size == 1:
            ctx.compute_forces(0, want_energy, stream=s)
        elif overlap:
            self.refresh_begin()
            ctx.compute_forces(1, want_energy, stream=s)          # interior: owned partners only
            self.refresh_end()
            ctx.compute_forces(2, want_energy, stream=s)          # boundary: ghost partners
        else:
            self.refresh_begin()
            self.refresh_end()
            ctx.compute_forces(0, want_energy, stream=s)
        ctx.integrate(2, dt, force_to_accel, stream=s)

    def global_scalars(self):
        """Potential energy, virial (+diagonal) and pair count summed over the ranks (CommBackend::sum_reduce)."""
        sc = self.ctx.read_scalars(stream=self._sh(self.main))
        v = torch.tensor([sc["pe"], sc["virial"], *sc["virial_diag"], sc["pairs_in_cutoff"]], dtype=torch.float64,
                         device=self.device)
        if self.d.world_size > 1:
            dist.all_reduce(v, group=self.group)
        v = v.cpu().numpy()
        return dict(pe=v[0], virial=v[1], virial_diag=v[2:5], pairs_in_cutoff=v[5])


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
