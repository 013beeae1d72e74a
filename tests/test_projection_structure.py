"""ProjectionLUTLayer geometry against reference-built layers (fixtures recorded from the reference's
ProjectionLUTLayer): every group's target list must be the rectangle `structure.rectangle_members` produces for SOME
centre, rescaled from input to output coordinates the way the layer does it, and the anchors the reference sampled for
the group's detectors must lie in the receptive rectangle of that same centre.  The reference draws its centres from its
own random stream, so the centre is searched, per axis, on a fine grid."""
import numpy as np
import pytest
import torch

import golden_util
from spiky_b200 import structure


def axis_sets(candidates, scale, half, n):
    """For every candidate centre coordinate: the set of grid coordinates inside |k - c * scale| <= half, as a bool
    matrix [n_candidates, n], computed with structure.rectangle_members on a one-row grid."""
    centres = torch.stack([candidates * scale, torch.zeros_like(candidates)], dim=1)
    members, counts = structure.rectangle_members(centres, 0.5, half, 1, n)
    inside = torch.zeros(len(candidates), n, dtype=torch.bool)
    rows = torch.arange(len(candidates)).view(-1, 1).expand_as(members)
    valid = members >= 0
    inside[rows[valid], members[valid]] = True
    return inside


@pytest.mark.parametrize("name", golden_util.names("proj_"))
def test_reference_groups_are_rectangles_of_this_geometry(name):
    cfg, ref = golden_util.load(name)
    h, w = cfg["in_shape"]
    oh, ow = cfg["out_shape"]
    rh, rw = cfg["receptive"]
    ph, pw = cfg["projection"]
    groups, per = cfg["groups"], cfg["per_group"]
    Nt, rows = cfg["Nt"], cfg["n_lookup_neurons"] // cfg["Nt"]
    assert Nt == groups * per
    anchors = ref["anchors"].reshape(Nt, -1).astype(np.int64)
    src, tgt = ref["syn_source"].astype(np.int64), ref["syn_target"].astype(np.int64)
    cand_x = torch.arange(0.0, w + 1e-9, 0.02, dtype=torch.float64)
    cand_y = torch.arange(0.0, h + 1e-9, 0.02, dtype=torch.float64)
    out_x = axis_sets(cand_x, ow / w, pw / 2 + 1e-4, ow)
    out_y = axis_sets(cand_y, oh / h, ph / 2 + 1e-4, oh)
    in_x = axis_sets(cand_x, 1.0, (rw - 1) / 2 + 1e-4, w)
    in_y = axis_sets(cand_y, 1.0, (rh - 1) / 2 + 1e-4, h)
    for g in range(groups):
        lists = [np.sort(tgt[src == (g * per + d) * rows]) for d in range(per)]
        assert all(np.array_equal(lists[0], l) for l in lists), f"group {g}: detectors differ in targets"
        cells = lists[0]
        ys, xs = np.unique(cells // ow), np.unique(cells % ow)
        # a full rectangle (projection_prob is 1 in these fixtures)
        assert len(cells) == len(ys) * len(xs) and np.array_equal(cells, (ys[:, None] * ow + xs[None, :]).reshape(-1))
        a = anchors[g * per:(g + 1) * per].reshape(-1)
        a = a[a >= 0]
        ax, ay = torch.from_numpy(np.unique(a % w)), torch.from_numpy(np.unique(a // w))
        want_x = torch.zeros(ow, dtype=torch.bool)
        want_x[torch.from_numpy(xs)] = True
        want_y = torch.zeros(oh, dtype=torch.bool)
        want_y[torch.from_numpy(ys)] = True
        ok_x = (out_x == want_x).all(dim=1) & in_x[:, ax].all(dim=1)
        ok_y = (out_y == want_y).all(dim=1) & in_y[:, ay].all(dim=1)
        assert bool(ok_x.any()), f"group {g}: no centre x reproduces columns {xs.tolist()} with anchors at {ax.tolist()}"
        assert bool(ok_y.any()), f"group {g}: no centre y reproduces rows {ys.tolist()} with anchors at {ay.tolist()}"


def test_grid_centres_follow_the_sampling_policy():
    policy = structure.PointSamplingPolicy(structure.PointSamplingType.Grid, grid_h=3, grid_w=2, stride_h=2, stride_w=4,
                                           pad_h=1, pad_w=2)
    c = structure.sample_centers(policy, 6, 10, 10)
    assert c.tolist() == [[2.0, 1.0], [6.0, 1.0], [2.0, 3.0], [6.0, 3.0], [2.0, 5.0], [6.0, 5.0]]
    members, counts = structure.rectangle_members(c[:1], 1.0 + 1e-4, 1.0 + 1e-4, 10, 10)
    # 3x3 box around (x=2, y=1), row-major ids
    assert counts.tolist() == [9] and members[0].tolist() == [1, 2, 3, 11, 12, 13, 21, 22, 23]


def test_anchor_pairs_are_distinct_and_inside_their_pool():
    pools = torch.tensor([[4, 7, 9, 12, -1], [0, 1, 2, 3, 5]])
    counts = torch.tensor([4, 5])
    pairs = structure.sample_anchor_pairs(pools, counts, 6, seed=3).view(2, 6, 2)
    for t in range(2):
        allowed = set(pools[t, :counts[t]].tolist())
        for a1, a2 in pairs[t].tolist():
            assert a1 in allowed and a2 in allowed and a1 != a2
    again = structure.sample_anchor_pairs(pools, counts, 6, seed=3).view(2, 6, 2)
    assert torch.equal(pairs, again)
