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
import torch


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
