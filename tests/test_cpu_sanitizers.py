"""The C++ host runtime (checkpoint codec, tokenizer, parsers, tiered-store files, TCP store, CPU kernels) under
AddressSanitizer + UndefinedBehaviorSanitizer: the library is rebuilt with -fsanitize=address,undefined and the tests that
drive it are re-run in a child interpreter that preloads the sanitizer runtime. Any heap overflow, use after free or
undefined arithmetic in the native code aborts the child."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _asan_runtime():
    sys.path.insert(0, str(ROOT))
    from rust_neural_network_b200 import _build
    try:
        return _build.asan_runtime(_build._sanitizer_cxx())
    except RuntimeError:
        return None


@pytest.mark.skipif(_asan_runtime() is None, reason="no libasan on this machine")
def test_host_runtime_is_clean_under_asan_and_ubsan():
    sys.path.insert(0, str(ROOT))
    from rust_neural_network_b200 import _build
    lib = _build.build_host_sanitized()
    env = dict(os.environ)
    env.update({"LD_PRELOAD": _asan_runtime(), "B200NN_HOST_LIB": str(lib), "OMP_NUM_THREADS": "1",
                "ASAN_OPTIONS": "detect_leaks=0:abort_on_error=1:handle_segv=0", "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1"})
    tests = ["tests/test_cpu_ref.py", "tests/test_cpu_tokenizer_data.py",
             "tests/test_cpu_core.py::test_rnnb_golden_bytes_and_roundtrip", "tests/test_cpu_core.py::test_safetensors_roundtrip_skips_metadata",
             "tests/test_cpu_production.py", "tests/test_cpu_tooling.py::test_ssd_tensor_format_and_store",
             "tests/test_cpu_modules.py::test_tcp_store_set_get_add_barrier_timeout", "tests/test_cpu_modules.py::test_message_framing_is_byte_exact"]
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider"] + tests, cwd=str(ROOT), env=env,
                       capture_output=True, text=True, timeout=1500)
    tail = (r.stdout[-3000:] + r.stderr[-3000:])
    assert r.returncode == 0, tail
    assert "ERROR: AddressSanitizer" not in tail and "runtime error:" not in tail, tail
