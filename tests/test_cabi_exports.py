"""CPU: the C-ABI library loads and exports exactly what include/efm_b200.h declares; the host
engine fails loudly without a GPU instead of falling back."""
import ctypes
import os
import re

import pytest

import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "efm_b200.h")).read()
    return sorted(set(re.findall(r"\b(efm_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(built)
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), n


def test_ctypes_signatures_cover_the_header(built):
    assert sorted(cabi.SIGNATURES) == declared_symbols()
    assert ctypes.sizeof(cabi.ModelDesc) == 17 * 4 and ctypes.sizeof(cabi.Sampling) == 24
    assert cabi.lib().efm_b200_version().decode().startswith("efm_b200")


def _no_gpu():
    try:
        import torch
        return not torch.cuda.is_available()
    except Exception:
        return True


@pytest.mark.skipif(not _no_gpu(), reason="checks the no-device failure mode")
def test_no_cpu_fallback(built, tmp_path):
    from oracle import synth
    cfg = synth.tiny_config()
    with pytest.raises(cabi.BackendError, match="no CUDA device"):
        cabi.Backend(cfg)
    import edge_fm
    model_dir = synth.write_checkpoint(str(tmp_path / "m"), cfg, synth.make_weights(cfg))
    path = synth.write_engine_config(str(tmp_path / "e.json"), model_dir)
    with pytest.raises(RuntimeError, match="no CUDA device"):
        edge_fm.EdgeFM(path)


def test_product_sources_never_reach_the_oracle():
    pkg = os.path.join(ROOT, "edge-fm-x_b200")
    for base, _, files in os.walk(pkg):
        if os.sep + "build" in base:
            continue
        for f in files:
            if f.endswith((".cu", ".cuh", ".cpp", ".h", ".py")):
                text = open(os.path.join(base, f), errors="ignore").read()
                assert "oracle" not in text.replace("test oracle", "").replace("the oracle", "") or f == "x", (base, f)
