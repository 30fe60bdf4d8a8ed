"""CPU: the host-side half of tensor-parallel failure detection.  The wait that every synchronising call of a
tensor-parallel context uses (efm_b200_tp_host_wait) is driven here with a stand-in libnccl (tests/fake_nccl) and a
Python `ready` callback, in a child process so that the stand-in never meets a real NCCL: a stream that becomes
ready, an asynchronous NCCL error, and a rank that never answers (timeout).  No GPU is involved; the device-side
half (a kernel's bounded wait) is tests/test_gpu_ops.py::test_peer_wait_runs_out_and_the_device_stays_usable."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("fake_nccl") / "libnccl_fake.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", out, os.path.join(ROOT, "tests", "fake_nccl", "fake_nccl.c")], check=True)
    return out


CHILD = textwrap.dedent("""
    import ctypes as C, sys, time
    sys.path.insert(0, {tests!r})
    import cabi
    L = cabi.lib()
    READY = C.CFUNCTYPE(C.c_int, C.c_void_p)
    t0 = time.perf_counter()
    ready_after = float(sys.argv[1])
    cb = READY(lambda arg: 1 if time.perf_counter() - t0 >= ready_after else 0)
    st = L.efm_b200_tp_host_wait(C.c_void_p(1), cb, None, float(sys.argv[2]))
    print(st, round(time.perf_counter() - t0, 3), L.efm_b200_last_error(None).decode())
""")


def run_child(fake, tmp_path, ready_after, timeout_s, fail_after=None):
    env = dict(os.environ, EFM_NCCL_LIB=fake, FAKE_NCCL_ABORT_FILE=str(tmp_path / "aborts"))
    if fail_after is not None:
        env["FAKE_NCCL_FAIL_AFTER"] = str(fail_after)
    r = subprocess.run([sys.executable, "-c", CHILD.format(tests=os.path.join(ROOT, "tests")), str(ready_after), str(timeout_s)],
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    st, secs, msg = (r.stdout.strip() + "  ").split(" ", 2)
    aborts = open(tmp_path / "aborts").read().count("abort") if (tmp_path / "aborts").exists() else 0
    return int(st), float(secs), msg, aborts


def test_wait_returns_when_the_stream_is_ready(built, fake_nccl, tmp_path):
    st, secs, _, aborts = run_child(fake_nccl, tmp_path, ready_after=0.05, timeout_s=5.0)
    assert st == 0 and secs < 2.0 and aborts == 0


def test_wait_surfaces_an_asynchronous_nccl_error_and_aborts_the_communicator(built, fake_nccl, tmp_path):
    st, secs, msg, aborts = run_child(fake_nccl, tmp_path, ready_after=60.0, timeout_s=30.0, fail_after=5)
    assert st == 2 and "asynchronous error" in msg and "system error" in msg      # EFM_ERR_CUDA
    assert secs < 5.0 and aborts == 1


def test_wait_times_out_on_a_rank_that_never_answers(built, fake_nccl, tmp_path):
    st, secs, msg, aborts = run_child(fake_nccl, tmp_path, ready_after=60.0, timeout_s=0.3)
    assert st == 6 and "timed out" in msg                                        # EFM_ERR_DEVICE_WAIT
    assert 0.25 <= secs < 5.0 and aborts == 1
