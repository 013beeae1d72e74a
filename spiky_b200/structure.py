"""Construction-time structure of LUT layers, derived with plain torch ops.

The reference grows its connectivity with a 3-D spatial "synapse growth" engine
(src/spiky/util/synapse_growth.py) and stores it in a byte arena.  The geometry it produces for
the LUT layers is simple and is restated here directly:

* sliding windows: a detector (or output block) at window (wy, wx) sees the grid points
  y in [wy*sh, wy*sh + rh), x in [wx*sw, wx*sw + rw)            (Conv2DSynapseGrowthHelper, :364-449)
* random / grid rectangles around a centre c: integer grid points p with |p - c| <= (r-1)/2 + 1e-4
  (RandomRectanglesSynapseGrowthHelper, :531-643)
* projection rectangles around a centre c in output coordinates: |p - c| <= r/2 + 1e-4, both ends
  inclusive (GivenRectanglesSynapseGrowthHelper, :646-703)
* anchor pairs: uniformly random ordered pairs of two distinct members of the detector's input pool,
  drawn independently per pair (prepare_detectors_compact_logic,
  spiky_cuda/lut/lut_compile_time_kernels_logic.proto:70-125)
"""
from dataclasses import dataclass
from enum import Enum

import torch


class PointSamplingType(Enum):
    """How the centres of detector groups are placed (reference: synapse_growth.py:498-502)."""
    RandomUniform = 0
    RandomNormal = 1
    Grid = 2


@dataclass(frozen=True)
class PointSamplingPolicy:
    """Same fields as the reference's policy object (synapse_growth.py:505-528)."""
    type: PointSamplingType
    mu: float = None
    sigma: float = None
    pad_h: float = 0.0
    pad_w: float = 0.0
    grid_h: int = None
    grid_w: int = None
    stride_h: int = None
    stride_w: int = None

    def __post_init__(self):
        if self.sigma is not None:
            assert self.sigma > 0.0
        assert self.pad_h >= 0.0 and self.pad_w >= 0.0


def sample_centers(policy, n_points, h, w, seed=None):
    """float32 [n_points, 2] (x, y) centres inside the (h, w) grid according to `policy`
    (reference: sample_random_points / sample_grid_points, synapse_growth.py:452-495)."""
    if policy.type == PointSamplingType.Grid:
        assert policy.grid_h is not None and policy.grid_w is not None
        assert policy.grid_h * policy.grid_w == n_points
        xs = policy.pad_w + policy.stride_w * torch.arange(policy.grid_w, dtype=torch.float32)
        ys = policy.pad_h + policy.stride_h * torch.arange(policy.grid_h, dtype=torch.float32)
        yy, xx = torch.meshgrid(ys, xs, indexing="ij")
        return torch.stack([xx.reshape(-1), yy.reshape(-1)], dim=1)
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(int(seed))
    if policy.type == PointSamplingType.RandomNormal:
        mu = policy.mu if policy.mu is not None else (w / 2.0, h / 2.0)
        sigma = policy.sigma if policy.sigma is not None else (w / 6.0, h / 6.0)
        mu = mu if isinstance(mu, (tuple, list)) else (mu, mu)
        sigma = sigma if isinstance(sigma, (tuple, list)) else (sigma, sigma)
        x = torch.randn(n_points, generator=gen) * sigma[0] + mu[0]
        y = torch.randn(n_points, generator=gen) * sigma[1] + mu[1]
    else:
        x = torch.rand(n_points, generator=gen) * float(w)
        y = torch.rand(n_points, generator=gen) * float(h)
    return torch.stack([x.clamp(policy.pad_w, w - policy.pad_w), y.clamp(policy.pad_h, h - policy.pad_h)], dim=1)


class SlidingWindows:
    """grid (h, w) scanned by windows (rh, rw) with stride (sh, sw); every window owns a block of
    (kh, kw) consumers laid out as a (num_win_h*kh, num_win_w*kw) grid."""

    def __init__(self, grid_shape, window_shape, stride_shape, block_shape):
        self.h, self.w = grid_shape
        self.rh, self.rw = window_shape
        self.sh, self.sw = stride_shape
        self.kh, self.kw = block_shape
        self.num_win_h = (self.h - self.rh) // self.sh + 1
        self.num_win_w = (self.w - self.rw) // self.sw + 1
        assert self.num_win_h > 0 and self.num_win_w > 0, "window larger than the grid"
        self.out_shape = (self.num_win_h * self.kh, self.num_win_w * self.kw)

    def _window_members(self):
        """int64 [n_windows, rh*rw] grid ids (row-major) of each window."""
        wy = torch.arange(self.num_win_h).view(-1, 1, 1, 1) * self.sh
        wx = torch.arange(self.num_win_w).view(1, -1, 1, 1) * self.sw
        dy = torch.arange(self.rh).view(1, 1, -1, 1)
        dx = torch.arange(self.rw).view(1, 1, 1, -1)
        ids = (wy + dy) * self.w + (wx + dx)
        return ids.reshape(self.num_win_h * self.num_win_w, self.rh * self.rw)

    def _consumer_window(self):
        """int64 [out_h*out_w] window id of each consumer, consumers in row-major order of the out grid."""
        oy = torch.arange(self.out_shape[0]).view(-1, 1) // self.kh
        ox = torch.arange(self.out_shape[1]).view(1, -1) // self.kw
        return (oy * self.num_win_w + ox).reshape(-1)

    def input_pools(self):
        """Per consumer (detector): the grid ids it may pick anchors from.  Returns (pools [n, P], counts [n])."""
        pools = self._window_members()[self._consumer_window()]
        counts = torch.full((pools.shape[0],), pools.shape[1], dtype=torch.int64)
        return pools, counts

    def output_targets(self):
        """Per grid point (detector position): the consumers (outputs) of every window containing it.
        Returns (targets [h*w, Pmax] padded with -1, counts [h*w]); targets are sorted ascending."""
        members = self._window_members()                      # [n_win, rh*rw] grid ids
        n_win = members.shape[0]
        block = self.kh * self.kw
        # consumers of window (wy, wx): out rows wy*kh .. wy*kh+kh-1, cols wx*kw ..
        wy = (torch.arange(n_win) // self.num_win_w).view(-1, 1, 1)
        wx = (torch.arange(n_win) % self.num_win_w).view(-1, 1, 1)
        by = torch.arange(self.kh).view(1, -1, 1)
        bx = torch.arange(self.kw).view(1, 1, -1)
        consumers = ((wy * self.kh + by) * self.out_shape[1] + wx * self.kw + bx).reshape(n_win, block)
        src = members.unsqueeze(2).expand(-1, -1, block).reshape(-1)
        dst = consumers.unsqueeze(1).expand(-1, members.shape[1], -1).reshape(-1)
        return _group_pairs(src, dst, self.h * self.w)


def _group_pairs(src, dst, n_src):
    """(src, dst) edge list -> per-src sorted dst lists, padded with -1."""
    order = torch.argsort(src * (int(dst.max().item()) + 1 if dst.numel() else 1) + dst)
    src, dst = src[order], dst[order]
    counts = torch.bincount(src, minlength=n_src)
    pmax = int(counts.max().item()) if counts.numel() else 0
    starts = torch.cumsum(counts, 0) - counts
    pos = torch.arange(src.numel()) - starts[src]
    out = torch.full((n_src, max(pmax, 1)), -1, dtype=torch.int64)
    out[src, pos] = dst
    return out, counts


def sample_anchor_pairs(pools, counts, n_anchors, seed=None):
    """int32 [n_detectors * n_anchors * 2]: per detector `n_anchors` ordered pairs of distinct pool members.

    A pair code c in [0, n(n-1)) decodes as a1 = c // (n-1), a2 = c % (n-1), a2 += (a2 >= a1), the
    decoding the reference uses; the codes themselves come from torch's generator.
    """
    n_det = pools.shape[0]
    gen = None
    if seed is not None:
        gen = torch.Generator(device="cpu")
        gen.manual_seed(int(seed))
    n = counts.view(-1, 1).to(torch.int64)
    assert int(n.min().item()) >= 2, "a detector needs at least two inputs to form an anchor pair"
    u = torch.rand((n_det, n_anchors), generator=gen, dtype=torch.float64)
    codes = torch.minimum((u * (n * (n - 1)).to(torch.float64)).to(torch.int64), n * (n - 1) - 1)
    a1 = codes // (n - 1)
    a2 = codes % (n - 1)
    a2 = a2 + (a2 >= a1).to(torch.int64)
    first = torch.gather(pools, 1, a1)
    second = torch.gather(pools, 1, a2)
    return torch.stack([first, second], dim=-1).to(torch.int32).reshape(-1)


def rectangle_members(centers, half_h, half_w, grid_h, grid_w, mask=None):
    """Grid points (row-major ids) inside the axis-aligned box |x - cx| <= half_w, |y - cy| <= half_h around
    each centre (cx, cy).  Returns (members [n, Pmax] padded with -1, counts [n]), members ascending."""
    cx = centers[:, 0].to(torch.float64).view(-1, 1, 1)
    cy = centers[:, 1].to(torch.float64).view(-1, 1, 1)
    ys = torch.arange(grid_h, dtype=torch.float64).view(1, -1, 1)
    xs = torch.arange(grid_w, dtype=torch.float64).view(1, 1, -1)
    inside = ((ys - cy).abs() <= half_h) & ((xs - cx).abs() <= half_w)
    if mask is not None:
        inside &= torch.as_tensor(mask, dtype=torch.bool).view(1, grid_h, grid_w)
    inside = inside.view(centers.shape[0], -1)
    counts = inside.sum(dim=1)
    pmax = max(int(counts.max().item()), 1)
    ids = torch.arange(grid_h * grid_w).view(1, -1).expand_as(inside)
    key = torch.where(inside, ids, torch.full_like(ids, grid_h * grid_w))
    members = torch.sort(key, dim=1).values[:, :pmax]
    members = torch.where(members >= grid_h * grid_w, torch.full_like(members, -1), members)
    return members, counts


class SparseIndex:
    """Compact lookup -> output connectivity of a sparse LUT layer.

    All lookup neurons (table rows) of one detector share one target list.  The flat weight array
    keeps the reference's layout so that weights trained with the reference load verbatim: neurons in
    id order, synapse p of a row at ``row_base + p + 2 * (p // G)`` (every group of G synapses is
    preceded by a two-slot hole where the reference's arena has its group header,
    spiky_cuda/connections_manager/connections_manager.h:39-66), rows ``stride`` slots apart.

    Per detector t:   det_wbase[t]  weight index of (row 0, synapse 0)
                      det_stride[t] slots between consecutive rows
                      det_count[t]  synapses per row (P)
                      det_sstart[t] prefix sum of det_count: position of the detector in the flat lists
    Per (detector, synapse), flattened in detector order:
                      syn_det[s], syn_target[s] (output index)
    """

    def __init__(self, det_wbase, det_stride, det_count, syn_target, group_size, n_weights, n_outputs,
                 rows_per_detector):
        self.det_wbase = det_wbase.to(torch.int64).contiguous()
        self.det_stride = det_stride.to(torch.int32).contiguous()
        self.det_count = det_count.to(torch.int32).contiguous()
        self.syn_target = syn_target.to(torch.int32).contiguous()
        counts64 = self.det_count.to(torch.int64)
        self.det_sstart = (torch.cumsum(counts64, 0) - counts64).to(torch.int32).contiguous()
        self.syn_det = torch.repeat_interleave(torch.arange(counts64.numel(), dtype=torch.int32), counts64).contiguous()
        self.group_size = int(group_size)
        self.n_weights = int(n_weights)
        self.n_outputs = int(n_outputs)
        self.rows_per_detector = int(rows_per_detector)
        self.n_syn_per_sample = int(counts64.sum().item())
        self.n_synapses = self.n_syn_per_sample * self.rows_per_detector
        self.max_count = int(counts64.max().item()) if counts64.numel() else 0
        self.max_groups_per_neuron = (self.max_count + self.group_size - 1) // self.group_size
        assert self.syn_target.numel() == self.n_syn_per_sample
        if self.syn_target.numel():
            assert int(self.syn_target.min()) >= 0 and int(self.syn_target.max()) < n_outputs
        self.chunk_info = self._build_chunks()
        self.n_chunks = self.chunk_info.shape[0]
        # what the staged kernels need to know on the host: the largest detector table, and whether every table can
        # be bulk-copied with 16-byte granularity (start and size multiples of 4 slots)
        if self.n_chunks:
            ci = self.chunk_info.to(torch.int64)
            wbase0 = (ci[:, 6] & 0xFFFFFFFF) | (ci[:, 7] << 32)
            self.max_table_slots = int(ci[:, 5].max().item())
            self.tables_aligned16 = int(bool(((wbase0 % 4 == 0) & (ci[:, 5] % 4 == 0)).all().item()))
        else:
            self.max_table_slots, self.tables_aligned16 = 0, 0

    CHUNK = 32  # detectors per chunk = lanes of a warp

    def _build_chunks(self):
        """int32 [n_chunks, 8] = (first detector, detector count <= 32, offset of the shared target list in
        syn_target, synapses per row, row stride, slots per detector table, wbase0 low word, wbase0 high word).
        A chunk is a run of consecutive detectors with identical target lists (the detectors of one group)
        whose tables lie back to back in the weight array; the kernels give one warp to each (sample, chunk)."""
        counts = self.det_count.to(torch.int64).cpu()
        starts = self.det_sstart.to(torch.int64).cpu()
        tgt = self.syn_target.cpu()
        n = counts.numel()
        same = torch.zeros(n, dtype=torch.bool)  # same[t]: detector t continues the chunk of detector t-1
        if n > 1:
            pmax = int(counts.max().item())
            lists = torch.full((n, max(pmax, 1)), -1, dtype=torch.int32)
            det = torch.repeat_interleave(torch.arange(n), counts)
            pos = torch.arange(tgt.numel()) - starts[det]
            lists[det, pos] = tgt
            wbase = self.det_wbase.cpu()
            stride = self.det_stride.to(torch.int64).cpu()
            contiguous = wbase[1:] == wbase[:-1] + stride[:-1] * self.rows_per_detector
            same[1:] = (lists[1:] == lists[:-1]).all(dim=1) & (counts[1:] > 0) & contiguous
        chunks = []
        t = 0
        same_l = same.tolist()
        counts_l = counts.tolist()
        starts_l = starts.tolist()
        wbase_l = self.det_wbase.cpu().tolist()
        stride_l = self.det_stride.cpu().tolist()
        while t < n:
            end = t + 1
            while end < n and end - t < self.CHUNK and same_l[end]:
                end += 1
            if counts_l[t] > 0:
                table = stride_l[t] * self.rows_per_detector
                assert table * (end - t) < (1 << 31), "tables of one detector chunk span more than 2^31 weight slots"
                chunks.append((t, end - t, starts_l[t], counts_l[t], stride_l[t], table,
                               wbase_l[t] & 0xFFFFFFFF, wbase_l[t] >> 32))
            t = end
        out = torch.tensor(chunks, dtype=torch.int64).reshape(-1, 8)
        out = torch.where(out >= (1 << 31), out - (1 << 32), out)  # low words above 2^31 wrap into int32
        return out.to(torch.int32).contiguous()

    _TENSORS = ("det_wbase", "det_stride", "det_count", "det_sstart", "syn_det", "syn_target", "chunk_info")

    @staticmethod
    def row_stride(count, group_size):
        return count + 2 * ((count + group_size - 1) // group_size)

    @classmethod
    def from_detector_targets(cls, targets, counts, rows_per_detector, group_size, n_outputs):
        """targets int64 [Nt, Pmax] padded with -1 (synapse order), counts [Nt]."""
        counts = counts.to(torch.int64)
        stride = cls.row_stride(counts, group_size)
        per_det = stride * rows_per_detector
        wbase = torch.cumsum(per_det, 0) - per_det      # the first header hole lies before index 0
        n_weights = int(per_det.sum().item()) - 2
        mask = torch.arange(targets.shape[1]).view(1, -1) < counts.view(-1, 1)
        return cls(wbase, stride, counts, targets[mask], group_size, n_weights, n_outputs, rows_per_detector)

    @classmethod
    def from_export(cls, source_ids, weight_indices, target_ids, n_detectors, rows_per_detector, group_size,
                    n_outputs, n_weights):
        """Rebuild the index from a reference layer's synapse export: per synapse its lookup neuron, its
        slot in the flat weight array and its output index.  Checks the regularity the kernels rely on."""
        src = torch.as_tensor(source_ids, dtype=torch.int64)
        slot = torch.as_tensor(weight_indices, dtype=torch.int64)
        tgt = torch.as_tensor(target_ids, dtype=torch.int64)
        order = torch.argsort(src * (int(slot.max().item()) + 1) + slot)
        src, slot, tgt = src[order], slot[order], tgt[order]
        n_neurons = n_detectors * rows_per_detector
        counts_n = torch.bincount(src, minlength=n_neurons)
        counts_n = counts_n.view(n_detectors, rows_per_detector)
        if not bool((counts_n == counts_n[:, :1]).all()):
            raise ValueError("lookup neurons of one detector have different synapse counts; unsupported connectivity")
        counts = counts_n[:, 0]
        starts = torch.cumsum(counts_n.reshape(-1), 0) - counts_n.reshape(-1)
        first_slot = torch.full((n_neurons,), -1, dtype=torch.int64)
        has = counts_n.reshape(-1) > 0
        first_slot[has] = slot[starts[has]]
        first_slot = first_slot.view(n_detectors, rows_per_detector)
        stride = cls.row_stride(counts, group_size)
        wbase = first_slot[:, 0]
        expect = wbase.view(-1, 1) + torch.arange(rows_per_detector).view(1, -1) * stride.view(-1, 1)
        if not bool(((first_slot == expect) | (counts.view(-1, 1) == 0)).all()):
            raise ValueError("weight slots of a detector's rows are not evenly spaced; unsupported layout")
        p = torch.arange(src.numel()) - starts[src]
        if not bool((slot == first_slot.reshape(-1)[src] + p + 2 * (p // group_size)).all()):
            raise ValueError("synapse slots do not follow the grouped layout")
        # the target list of row 0 stands for the detector; every other row must repeat it
        tmax = int(counts.max().item())
        tl = torch.full((n_neurons, max(tmax, 1)), -1, dtype=torch.int64)
        tl[src, p] = tgt
        tl = tl.view(n_detectors, rows_per_detector, -1)
        if not bool((tl == tl[:, :1]).all()):
            raise ValueError("lookup neurons of one detector have different target lists; unsupported connectivity")
        det_targets = tl[:, 0]
        mask = torch.arange(det_targets.shape[1]).view(1, -1) < counts.view(-1, 1)
        return cls(wbase, stride, counts, det_targets[mask], group_size, n_weights, n_outputs, rows_per_detector)

    def synapses_of(self, neuron_ids):
        """Per synapse of the given lookup neurons (table rows; id = detector * rows_per_detector + row), in the
        order given and in synapse order inside a row: (lookup neuron, slot in the flat weight array, output index),
        all int64 on the index's device.  Inverse of ``from_export``."""
        dev = self.det_wbase.device
        ids = torch.as_tensor(neuron_ids, device=dev).to(torch.int64).reshape(-1)
        n_neurons = self.det_count.numel() * self.rows_per_detector
        if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= n_neurons):
            raise ValueError("lookup neuron id out of range")
        det = ids // self.rows_per_detector
        row = ids - det * self.rows_per_detector
        counts = self.det_count.to(torch.int64)[det]
        which = torch.repeat_interleave(torch.arange(ids.numel(), device=dev), counts)
        p = torch.arange(which.numel(), device=dev) - (torch.cumsum(counts, 0) - counts)[which]
        d = det[which]
        slot = self.det_wbase[d] + row[which] * self.det_stride.to(torch.int64)[d] + p + 2 * (p // self.group_size)
        target = self.syn_target.to(torch.int64)[self.det_sstart.to(torch.int64)[d] + p]
        return ids[which], slot, target

    def chunk_weight_bounds(self):
        """int64 [n_chunks + 1]: chunk c's tables occupy the weight slots [bounds[c], bounds[c + 1]); the ranges are
        contiguous, disjoint and cover every synapse slot (the last one ends at n_weights)."""
        info = self.chunk_info.cpu().to(torch.int64)
        low = torch.where(info[:, 6] < 0, info[:, 6] + (1 << 32), info[:, 6])
        start = (info[:, 7] << 32) | low
        return torch.cat([start, torch.tensor([self.n_weights], dtype=torch.int64)])

    def shard_chunks(self, world):
        """Splits the chunks into ``world`` consecutive ranges of about equal table size; returns the world + 1
        chunk boundaries (a range may be empty when there are fewer chunks than ranks)."""
        bounds = self.chunk_weight_bounds()
        total = int(bounds[-1] - bounds[0])
        cuts = [0]
        for r in range(1, world):
            want = int(bounds[0]) + (total * r) // world
            c = int(torch.searchsorted(bounds, torch.tensor(want), right=False))
            cuts.append(min(max(c, cuts[-1]), self.n_chunks))
        cuts.append(self.n_chunks)
        return cuts

    def initial_weights(self, synapse_meta, seed=None):
        """fp32 [n_weights]: noise * U[0,1) + initial weight, clipped to the meta's range; holes are zero."""
        gen = None
        if seed is not None:
            gen = torch.Generator(device="cpu")
            gen.manual_seed(int(seed))
        w = torch.rand(self.n_weights, generator=gen, dtype=torch.float32)
        w.mul_(synapse_meta.initial_noise_level).add_(synapse_meta.initial_weight)
        w.clip_(synapse_meta.min_weight, synapse_meta.max_weight)
        w[~self.slot_mask()] = 0.0
        return w

    def slot_mask(self):
        """bool [n_weights]: True where a slot holds a synapse weight (False in header holes)."""
        dev = self.det_wbase.device
        mask = torch.zeros(self.n_weights, dtype=torch.bool, device=dev)
        counts = self.det_count.to(torch.int64)
        p = torch.arange(self.n_syn_per_sample, device=dev) - self.det_sstart.to(torch.int64)[self.syn_det.to(torch.int64)]
        base = self.det_wbase[self.syn_det.to(torch.int64)] + p + 2 * (p // self.group_size)
        stride = self.det_stride.to(torch.int64)[self.syn_det.to(torch.int64)]
        for row in range(self.rows_per_detector):
            mask[base + row * stride] = True
        del counts
        return mask

    def to_device(self, device_index):
        dev = torch.device("cpu") if device_index < 0 else torch.device("cuda", device_index)
        for name in self._TENSORS:
            setattr(self, name, getattr(self, name).to(dev))
        return self

    def c_struct(self):
        """ctypes view for the C ABI (valid while this object and its tensors are alive)."""
        from ._native import SparseIndexC

        return SparseIndexC(
            det_wbase=self.det_wbase.data_ptr(), det_stride=self.det_stride.data_ptr(),
            det_count=self.det_count.data_ptr(), det_sstart=self.det_sstart.data_ptr(),
            syn_det=self.syn_det.data_ptr(), syn_target=self.syn_target.data_ptr(),
            chunk_info=self.chunk_info.data_ptr(), n_chunks=self.n_chunks, n_syn_per_sample=self.n_syn_per_sample, n_weights=self.n_weights, group_size=self.group_size,
            max_count=self.max_count, max_table_slots=self.max_table_slots, tables_aligned16=self.tables_aligned16)

    def nbytes(self):
        return sum(getattr(self, n).numel() * getattr(self, n).element_size() for n in self._TENSORS)

    def numpy(self):
        return {n: getattr(self, n).cpu().numpy() for n in self._TENSORS}
