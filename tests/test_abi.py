"""CPU-side checks of the C-ABI boundary: the header and the library agree."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "wr_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wr_cuda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from wayruntime_b200 import _build, binding
    _build.build()
    lib = ctypes.CDLL(binding.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), f"{name} declared in wr_cuda.h but not exported"
    assert sorted(binding.EXPORTS) == names


def test_status_codes_match_reference_enum():
    """include/wayruntime/wayruntime.h:82-107."""
    text = open(HEADER).read()
    want = {"OK": 0, "ERR_UNSUPPORTED": -3, "ERR_INVAL": -4, "ERR_NOMEM": -5, "ERR_CTX_FULL": -6,
            "ERR_STATE": -7, "ERR_LIMIT": -8, "ERR_INTERNAL": -10}
    for name, val in want.items():
        m = re.search(rf"#define WR_CUDA_{name}\s+\(?(-?\d+)\)?", text)
        assert m and int(m.group(1)) == val, name


def test_no_device_is_an_explicit_error():
    """No B200 bound -> WR_ERR_UNSUPPORTED from the probe and from context
    creation; nothing falls back to the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import wayruntime_b200 as wr
    assert wr.device_check(0) == -3
    with pytest.raises(wr.WrCudaError) as e:
        wr.Context(0)
    assert e.value.status == -3


def test_missing_library_fails_loudly(monkeypatch):
    from wayruntime_b200 import binding
    monkeypatch.setattr(binding, "_lib", None)
    monkeypatch.setattr(binding, "LIB_PATH", "/nonexistent/libwr_cuda.so")
    with pytest.raises(RuntimeError, match="no CPU path"):
        binding.load_library()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "wayruntime_b200")
    for dirpath, _dirs, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".c", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, f"{f} mentions the oracle"


def test_dropin_engine_create_refuses_a_host_without_b200():
    """The drop-in library's wr_engine_create is the gate (reference contract:
    include/wayruntime/wayruntime.h:181-185, probe at src/core/engine.c:130):
    with no compute-capability-10.x device it returns WR_ERR_UNSUPPORTED, writes
    one line to the caller's log sink, and creates nothing."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    path = os.path.join(ROOT, "wayruntime_b200", "lib", "libwayruntime_b200.so")
    if not os.path.exists(path):
        pytest.skip("drop-in library not built on this machine (needs the reference checkout)")
    L = ctypes.CDLL(path)
    L.wr_engine_create.restype = ctypes.c_int
    engine = ctypes.c_void_p()
    cfg = (ctypes.c_uint8 * 512)()                     # zeroed wr_engine_config: default sink (stderr)
    assert L.wr_engine_create(cfg, ctypes.byref(engine)) == -3
    assert not engine.value
    assert L.wr_engine_create(None, ctypes.byref(engine)) == -3
    assert L.wr_engine_create(cfg, None) == -4
    # the session objects refuse as well when driven without an engine
    assert L.wri_self_test_llm_step() == -2
