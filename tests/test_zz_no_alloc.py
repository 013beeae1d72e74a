"""The backward entry point that allocates nothing (lutb_nonseq_fc_backward_noalloc).

Some callers cannot call cudaMalloc: a real-time loop that may not block on the allocator, a host callback,
a process whose device memory is owned and fully handed out by another component.  For them the library keeps
a fixed scratch array inside its own device image.  This test calls the entry point through the C ABI, twice in
a row (the second call finds the first call's leftovers in the shared array), and checks it against the
regular entry point that uses a caller-provided workspace.  It is collected last so that a run which stops at
the first failure has already executed every other test; it must also pass alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

import golden_util
import synth

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _problem(seed, B, I, Nt, Nc, O):
    from spiky_b200 import _native
    from spiky_b200.lut_data_manager import LUTDataManagerF

    dev = torch.device("cuda:0")
    dm = LUTDataManagerF(I, O, Nt, Nc, 1, 0, 0, 32, 32)
    dm.register_synapse_meta(learning_rate=1.0, min_synaptic_weight=-1.0, max_synaptic_weight=1.0,
                             initial_noise_level=0.0, initial_weight=0.0)
    dm.initialize_neurons(True)
    dm.to_device(0)
    W = torch.from_numpy(synth.normal(seed + 3, (Nt * (1 << Nc) * O,), 0.0, 0.02)).to(dev)
    x = torch.from_numpy(synth.uniform(seed + 1, (B, I))).reshape(-1).to(dev)
    a = torch.from_numpy(synth.anchor_pairs(seed + 2, Nt, Nc, I)).reshape(-1).to(dev)
    dY = torch.from_numpy(synth.normal(seed + 4, (B, O))).reshape(-1).to(dev)
    y = torch.zeros(B * O, device=dev)
    idx = torch.zeros(B * Nt, dtype=torch.int32, device=dev)
    md = torch.zeros(B * Nt, device=dev)
    mk = torch.zeros(B * Nt, dtype=torch.int32, device=dev)
    dm.forward_step(W, B, x, a, y, idx, 0.0, None, md, mk)
    return _native, dm._cfg(), dict(W=W, a=a, dY=dY, idx=idx, md=md, mk=mk, B=B, I=I, Nt=Nt, Nc=Nc, O=O)


def _run_regular(native, cfg, p):
    L = native.lib()
    dev = p["W"].device
    need = L.lutb_nonseq_fc_backward_workspace(ctypes.byref(cfg), p["B"], native.DW_SORTED)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    dX = torch.zeros(p["B"] * p["I"], device=dev)
    dW = torch.zeros_like(p["W"])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    native.check(L.lutb_nonseq_fc_backward(ctypes.byref(cfg), p["B"], _ptr(p["W"]), _ptr(p["dY"]), _ptr(p["a"]),
                                           _ptr(p["idx"]), _ptr(p["md"]), _ptr(p["mk"]), _ptr(dX), _ptr(dW), -1.0,
                                           native.DW_SORTED, _ptr(ws), need, stream))
    torch.cuda.synchronize()
    return dX.cpu().numpy(), dW.cpu().numpy()


def _run_noalloc(native, cfg, p, out=None):
    """out: (dX, dW) device buffers to reuse, so that the caller can watch the allocator around the call."""
    L = native.lib()
    dev = p["W"].device
    if out is None:
        dX = torch.zeros(p["B"] * p["I"], device=dev)
        dW = torch.zeros_like(p["W"])
    else:
        dX, dW = out
        dX.zero_()
        dW.zero_()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    native.check(L.lutb_nonseq_fc_backward_noalloc(ctypes.byref(cfg), p["B"], _ptr(p["W"]), _ptr(p["dY"]), _ptr(p["a"]),
                                                   _ptr(p["idx"]), _ptr(p["md"]), _ptr(p["mk"]), _ptr(dX), _ptr(dW), -1.0,
                                                   stream))
    torch.cuda.synchronize()
    return dX.cpu().numpy(), dW.cpu().numpy()


def _oracle(p):
    from oracle import lut_oracle as orc

    B = p["B"]
    return orc.nonseq_fc_backward(p["W"].cpu().numpy(), p["dY"].cpu().numpy().reshape(B, p["O"]),
                                  p["a"].cpu().numpy().reshape(p["Nt"], p["Nc"], 2), p["idx"].cpu().numpy().reshape(B, p["Nt"]),
                                  p["md"].cpu().numpy().reshape(B, p["Nt"]), p["mk"].cpu().numpy().reshape(B, p["Nt"]),
                                  p["I"], p["Nc"])


def test_noalloc_backward_matches_workspace_backward_twice_in_a_row():
    # two different problems back to back: the second call must not be disturbed by what the first one left
    # in the shared scratch array (different batch, different table shape)
    for seed, shape in ((10, (256, 784, 64, 6, 32)), (20, (97, 50, 9, 4, 12))):
        native, cfg, p = _problem(seed, *shape)
        ref_dX, ref_dW = _run_regular(native, cfg, p)
        orc_dX, orc_dW = _oracle(p)
        for _ in range(2):
            dX, dW = _run_noalloc(native, cfg, p)
            assert np.array_equal(dW, ref_dW), "table gradient: both paths add in the same fixed order"
            golden_util.assert_close(dX, ref_dX, 1e-5, "dX")
            # and directly against the CPU oracle, not only through the workspace variant
            golden_util.assert_close(dW, orc_dW.reshape(-1), 1e-5, "dW vs oracle")
            golden_util.assert_close(dX, orc_dX.reshape(-1), 1e-5, "dX vs oracle")


def test_noalloc_backward_leaves_device_memory_as_it_found_it():
    """The promise itself: once the first call on the device has loaded the kernels and looked the scratch array
    up, a call changes neither the driver's free-memory figure nor torch's allocator statistics."""
    native, cfg, p = _problem(40, 128, 96, 16, 5, 24)
    out = (torch.zeros(p["B"] * p["I"], device=p["W"].device), torch.zeros_like(p["W"]))
    _run_noalloc(native, cfg, p, out)   # first use: module / kernel loading and the symbol look-up happen here
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    stats_before = torch.cuda.memory_stats()
    _run_noalloc(native, cfg, p, out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    stats_after = torch.cuda.memory_stats()
    assert free_after == free_before, "the driver reports a different amount of free device memory"
    for key in ("allocation.all.allocated", "segment.all.allocated", "reserved_bytes.all.current"):
        # the host copies _run_noalloc makes of its results use pinned/pageable host memory, not the device pool
        assert stats_after[key] == stats_before[key], key


def test_noalloc_backward_refuses_problems_beyond_the_builtin_scratch():
    native, cfg, p = _problem(30, 8, 16, 4, 3, 4)
    L = native.lib()
    too_many = 1 << 22  # 4 detectors x 4 Mi samples of sorted lists alone exceed the 8 MiB array
    assert L.lutb_nonseq_fc_backward_workspace(ctypes.byref(cfg), too_many, native.DW_SORTED) > (8 << 20)
    rc = L.lutb_nonseq_fc_backward_noalloc(ctypes.byref(cfg), too_many, _ptr(p["W"]), _ptr(p["dY"]), _ptr(p["a"]),
                                           _ptr(p["idx"]), _ptr(p["md"]), _ptr(p["mk"]), _ptr(p["dY"]), _ptr(p["W"]), -1.0,
                                           None)
    assert rc == -4 and b"built-in array" in L.lutb_last_error()
    cfg.int_mode = 1
    rc = L.lutb_nonseq_fc_backward_noalloc(ctypes.byref(cfg), 8, _ptr(p["W"]), _ptr(p["dY"]), _ptr(p["a"]), _ptr(p["idx"]),
                                           _ptr(p["md"]), _ptr(p["mk"]), _ptr(p["dY"]), _ptr(p["W"]), -1.0, None)
    assert rc == -3
