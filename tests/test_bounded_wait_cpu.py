"""The give-up branch of the device-side waits, without a GPU.

Every wait in the kernels (mbarrier waits, the shared-memory slot poll) is one loop,
``fa::bounded_wait`` in ``csrc/bounded_wait.h``, written so that it also compiles for the host.
No test makes a GPU wait run out; instead the same code is built with g++ here and driven with
polls that never succeed and a fake clock (``tests/cpu/bounded_wait_host.cpp``).  The second
test checks the host's mapping from a recorded status word to the error code of the C ABI."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "flash-attention-ptx-cuda_b200", "csrc")


def test_give_up_branch_on_the_host(tmp_path):
    exe = tmp_path / "bounded_wait_host"
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", CSRC,
                    os.path.join(ROOT, "tests", "cpu", "bounded_wait_host.cpp"), "-o", str(exe)], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0 and res.stdout.strip() == "ok", res.stdout + res.stderr


def test_status_word_maps_to_device_timeout():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    fa = ge.load_package()
    lib = fa.lib()
    assert lib.fa_status_word_to_error(0) == fa.FA_OK
    for barrier_id in (1, 14, 0x41, 0x4F):
        assert lib.fa_status_word_to_error((1 << 16) | barrier_id) == fa.FA_ERR_DEVICE_TIMEOUT
    assert fa.error_string(fa.FA_ERR_DEVICE_TIMEOUT) == "a kernel gave up on a bounded wait"
