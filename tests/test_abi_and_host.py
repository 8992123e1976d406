"""The C ABI library loads and exports every symbol include/m26b_expert.h declares (no compute calls),
the host-side mirror validates its arguments like the reference wrapper, and the product fails loudly
without a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def header_symbols():
    text = open(os.path.join(ROOT, "include", "m26b_expert.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(m26b_[a-z_0-9]+)\s*\(", text)))


def test_header_cites_the_reference_interface():
    text = open(os.path.join(ROOT, "include", "m26b_expert.h")).read()
    for cite in ("b1_serve.cu:214-574", "b1_serve.cu:312-572", "b1_serve.cu:218-265", "src/b1.rs:21-49"):
        assert cite in text, cite


def test_library_exports_every_declared_symbol():
    from mimo26f_afd_b200 import _native

    assert os.path.exists(_native.LIB_PATH), "build the library first: python -c 'import __graft_entry__ as g; g.build()'"
    lib = ctypes.CDLL(_native.LIB_PATH)
    declared = header_symbols()
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(_native.SYMBOLS) == declared
    assert _native.lib().m26b_version().decode().startswith("m26b-expert")


def test_argument_errors_come_before_any_cuda_call():
    import mimo26f_afd_b200 as M

    class Fake:  # handles are not touched when the extents are wrong
        _h = None

    bf = np.zeros(2 * 4096, np.uint16)
    with pytest.raises(M.ExpertError) as e:
        M.ffn(Fake(), Fake(), np.zeros(4096, np.uint8), np.zeros(128, np.uint8), np.zeros(16, np.int32),
              np.zeros(16, np.float32), 2, bf)
    assert e.value.code == 1 and "extents do not match 2 rows" in e.value.message
    with pytest.raises(M.ExpertError) as e:
        M.ffn_strided(Fake(), Fake(), np.zeros(4224, np.uint8), 4000, np.zeros(8, np.int32), np.zeros(8, np.float32), 1,
                      bf[:4096])
    assert e.value.code == 1 and "hidden rows do not match" in e.value.message


def test_null_handles_are_bad_arguments():
    from mimo26f_afd_b200 import _native

    L = _native.lib()
    err = ctypes.create_string_buffer(256)
    rc = L.m26b_ffn(None, None, None, 4096, None, 128, None, None, 1, None, None, err, 256)
    assert rc == 1 and b"bad rows/handles/pitch" in err.value
    out = ctypes.c_void_p()
    rc = L.m26b_layer_new_tp(None, 0, 0, 3, ctypes.byref(out), err, 256)
    assert rc == 1 and b"bad canonical extent/rank" in err.value
    assert L.m26b_layer_all_normal(None) == 0
    L.m26b_layer_free(None)
    L.m26b_scratch_free(None)


def test_no_gpu_means_a_loud_failure_not_a_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import mimo26f_afd_b200 as M

    with pytest.raises(M.ExpertError) as e:
        M.Scratch()
    assert e.value.code == 2


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "mimo26f_afd_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, f


def test_synth_numpy_and_torch_agree():
    import torch

    from mimo26f_afd_b200 import synth

    t = synth.layer_torch(0x51, torch.device("cpu"), n_experts=2)
    for name in synth.TENSORS:
        for e in range(2):
            assert np.array_equal(t[name][e].numpy(), synth.expert_tensor_np(0x51, name, e)), (name, e)
    s = synth.expert_tensor_np(0x51, "gate_s", 0)
    assert s.min() >= 118 and s.max() <= 122
    ids, w = synth.routing(3, 64, 1.2)
    assert ids.shape == (64, 8) and all(len(set(r)) == 8 for r in ids)
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6) and (w >= 0).all()
    img = synth.canonical_rank_image_np(synth.layer_np(0x51, [0]), [0], 1, 4)
    assert img.shape == (256, 3342336)
