"""The host-side lock-free code (SPSC ring in process and over POSIX shared memory, signal-pad epoch
protocol) under ThreadSanitizer and AddressSanitizer: ``native/selftest.cpp`` is compiled with the
sanitizer and run as a plain executable.  Skipped where the compiler has no sanitizer runtime."""
import pytest

from chaoscontrol_b200 import _build


@pytest.mark.parametrize("sanitizer", ["none", "thread", "address"])
def test_ring_shm_and_pad_protocol_selftest(sanitizer):
    rc, out = _build.build_and_run_selftest(sanitizer)
    if rc == 127:
        pytest.skip(out)
    assert rc == 0, out[-3000:]
    assert "selftest: ok" in out
