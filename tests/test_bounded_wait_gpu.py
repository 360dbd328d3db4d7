"""A bounded wait that runs out: the kernels' waits on barriers give up after a limit, set a status
word and return, so that a broken pipeline ends the kernel instead of hanging the GPU.  Here a
test-only kernel (tests/csrc/wait_probe.cu), built with a limit of 2 ms, waits through the
package's own wait (``bw::mbar_wait``) for a barrier nobody arrives at.  Nothing faults, traps or
spins without end; the context stays usable."""
import ctypes
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def build_probe(out_dir):
    from blackwellllm_b200.kernels import build
    out = os.path.join(out_dir, "wait_probe.so")
    cmd = [build.find_nvcc()] + build.ARCH_FLAGS + build.BASE_FLAGS + \
          ["-DBW_WAIT_NS=2000000ull", "-DBW_SPIN_LIMIT=4096u", "-I", build.CSRC, "-o", out,
           os.path.join(HERE, "csrc", "wait_probe.cu")]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    assert proc.returncode == 0, proc.stdout.decode(errors="replace")
    return ctypes.CDLL(out)


def test_a_wait_that_nothing_satisfies_gives_up_sets_the_status_and_returns(tmp_path):
    lib = build_probe(str(tmp_path))
    lib.bw_wait_probe.argtypes = [ctypes.c_void_p] * 4
    lib.bw_wait_probe.restype = ctypes.c_int
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    result = torch.full((2,), -1, dtype=torch.int32, device="cuda:0")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    rc = lib.bw_wait_probe(status.data_ptr(), result.data_ptr(), waited.data_ptr(),
                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()                                   # the kernel ended by itself
    assert result.tolist() == [0, 1]                           # gave up; then, with the phase complete, succeeded
    assert int(status) == 77                                   # the first wait's code; the second set nothing
    assert int(waited) < 1_000_000_000                         # within its limit (2 ms or 4,096 probes), not the default 1.5 s
    x = torch.arange(8, device="cuda:0")
    assert int((x * 2).sum()) == 56                            # the context is alive
