"""The C-ABI library loads and exports every entry point include/spiky_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "spiky_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lutb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "lutb_nonseq_fc_forward" in syms and "lutb_nonseq_fc_backward" in syms


def test_library_exports_every_declared_symbol():
    from spiky_b200 import build, _native

    path = build.build()
    handle = ctypes.CDLL(path)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
        assert name in _native.SIGNATURES, f"{name} has no ctypes signature in spiky_b200/_native.py"
    assert handle.lutb_version() >= 100


def test_argument_errors_do_not_need_a_gpu():
    """Validation happens before any CUDA call: status < 0 and a readable message."""
    from spiky_b200 import _native

    L = _native.lib()
    cfg = _native.LayerCfg(n_inputs=4, n_outputs=4, n_detectors=0, n_anchors=2, seq_len=1, pos_dim=0,
                           forward_group=32, backward_group=32, int_mode=0, sliced_product=0, cmp_eps=0.0,
                           reserved0=0.0, int_rescaler=1.0, lr_meta=1.0)
    rc = L.lutb_nonseq_fc_forward(ctypes.byref(cfg), 1, None, None, None, None, None, None, None, None)
    assert rc < 0 and b"n_detectors" in L.lutb_last_error()
    with pytest.raises(ValueError):
        _native.check(rc)


def test_data_manager_argument_errors():
    from spiky_b200.lut_data_manager import LUTDataManagerF, LUTDataManagerI

    with pytest.raises(ValueError):
        LUTDataManagerF(0, 4, 4, 2, 1, 0, 0, 32, 32)
    dm = LUTDataManagerI(8, 4, 4, 2, 1, 0, 0, 32, 32, 0.001)
    assert dm.get_summations_data_type() == "int32"
    assert dm.get_number_of_lookup_neurons() == 16
    with pytest.raises(ValueError):
        dm.register_synapse_meta(learning_rate=2.0, min_synaptic_weight=0, max_synaptic_weight=1,
                                 initial_noise_level=0, initial_weight=0)
    with pytest.raises(ValueError):
        dm.initialize_neurons(True)  # no synapse meta registered yet
