"""The C ABI: every function include/monarch_muon_b200.h declares is exported by
the shared library and bound by the ctypes layer, and nothing else is bound.
No kernel is launched here, so this runs without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "monarch_muon_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)          # drop comments
    names = re.findall(r"\b(mmb_[a-z0-9_]+)\s*\(", text)
    return sorted(set(n for n in names if not n.endswith("_seg")))


def test_header_declares_functions():
    names = declared_functions()
    assert "mmb_momentum_step" in names and "mmb_newton_schulz" in names and len(names) >= 15


def test_library_exports_every_declared_symbol():
    from monarch_muon_b200 import build
    path = build.build()                                       # no-op when up to date
    lib = ctypes.CDLL(path)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_ctypes_layer_binds_exactly_the_header():
    from monarch_muon_b200 import _lib
    assert sorted(_lib.SYMBOLS) == declared_functions()
    lib = _lib.load()
    assert lib.mmb_version() >= 100
    assert lib.mmb_last_error() is not None


def test_struct_layouts_match_the_header():
    """Field order and sizes of the ctypes structures against the C structs (LP64)."""
    from monarch_muon_b200 import _lib
    assert ctypes.sizeof(_lib.MomentumSeg) == 9 * 8
    assert ctypes.sizeof(_lib.UpdateSeg) == 3 * 8
    assert ctypes.sizeof(_lib.AdamWSeg) == 5 * 8 + 8
    assert ctypes.sizeof(_lib.GradSeg) == 2 * 8 + 8
    assert ctypes.sizeof(_lib.MasterUpdateSeg) == 4 * 8
    assert ctypes.sizeof(_lib.AdamWFp8Seg) == 11 * 8 + 8
    assert ctypes.sizeof(_lib.MasterAdamWSeg) == 6 * 8 + 8
    text = open(HEADER).read()
    for struct, cls in (("mmb_momentum_seg", _lib.MomentumSeg), ("mmb_update_seg", _lib.UpdateSeg),
                        ("mmb_adamw_seg", _lib.AdamWSeg), ("mmb_grad_seg", _lib.GradSeg),
                        ("mmb_master_update_seg", _lib.MasterUpdateSeg),
                        ("mmb_adamw_fp8_seg", _lib.AdamWFp8Seg),
                        ("mmb_master_adamw_seg", _lib.MasterAdamWSeg)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = re.findall(r"\b([a-z_0-9]+)\s*;", body)
        assert fields == [f[0] for f in cls._fields_], struct


def test_calls_validate_arguments_without_a_gpu():
    """Argument errors are reported through the return code and mmb_last_error, never by crashing."""
    from monarch_muon_b200 import _lib
    lib = _lib.load()
    rc = lib.mmb_newton_schulz(None, None, None, 1, 8, 8, None, 0, 0, None, None)
    assert rc == -1 and b"null pointer" in lib.mmb_last_error()
    rc = lib.mmb_gemm_bf16(None, None, None, 1, 8, 8, 8, 0, 0, 0, 1.0, 0.0, None, 0, 0, None, None)
    assert rc == -1
    assert lib.mmb_ns_workspace_bytes(4, 1024, 1024) > 4 * 1024 * 1024 * 2 * 4
    assert lib.mmb_momentum_static_max_floats() == 1 << 20


def test_launch_options_are_validated_and_per_thread():
    """mmb_set_stream_ctas_per_sm sizes grids whose reductions have scratch for 32 CTAs per SM: larger
    values are refused (they would index past that scratch), 0..32 accepted.  The options act on the
    calling thread only."""
    import threading
    from monarch_muon_b200 import _lib
    lib = _lib.load()
    assert lib.mmb_set_stream_ctas_per_sm(33) == -1 and b"outside 0..32" in lib.mmb_last_error()
    assert lib.mmb_set_stream_ctas_per_sm(-1) == -1
    assert lib.mmb_set_stream_ctas_per_sm(32) == 0 and lib.mmb_set_stream_ctas_per_sm(0) == 0
    with pytest.raises(RuntimeError):
        _lib.set_stream_ctas_per_sm(64)
    seen = {}

    def other():
        # a fresh thread starts from the defaults whatever this thread has set
        with _lib.launch_options(stream_ctas_per_sm=1, dynamic_schedule=True):
            seen["inside"] = True
        seen["done"] = True
    with _lib.launch_options(stream_ctas_per_sm=2):
        t = threading.Thread(target=other)
        t.start()
        t.join()
    assert seen == {"inside": True, "done": True}
    # the context manager restores the defaults even when the body raises
    with pytest.raises(ZeroDivisionError):
        with _lib.launch_options(sm_limit=100, dynamic_schedule=True, stream_ctas_per_sm=1):
            1 / 0
    assert lib.mmb_wait_probe(0, None, None) == -1               # argument check comes before any launch


def test_staged_reference_is_unmodified():
    """oracle/_ref/ (when present) holds the reference's files byte for byte: every file still has the hash
    recorded when it was staged, and the files the GPU tests and the benchmark import are there."""
    from oracle import make_ref, ref_loader
    if not ref_loader.available():
        pytest.skip("oracle/_ref/ not staged (python oracle/make_ref.py <reference checkout>)")
    assert make_ref.verify()
    for rel in ("pretrain/src/models/monarch/coat_state_muon.py", "pretrain/src/models/monarch/monarch_muon.py",
                "membench/src/models/monarch/monarch_muon.py", "pretrain/third_party/coat/optimizer/triton_kernels.py",
                "pretrain/src/main.py", "pretrain/src/optim/base.py", "pretrain/tests/test_coat_state_muon.py"):
        assert os.path.exists(os.path.join(ref_loader.ROOT, rel)), rel
    twin = ref_loader.membench_twin()
    assert hasattr(twin, "MonarchMuonOptimizer") and hasattr(twin, "_newton_schulz_batched")
