"""The bounded waits of the kernels, exercised on purpose: a one-warp self-test kernel waits, with a limit
of about a millisecond, on a barrier that nobody arrives on.  The wait must run out, the kernel must end
normally (nothing faults, nothing hangs), the device status word must carry the self-test bit, the status
check must turn it into an error exactly once, and the context must stay usable."""
import pytest
import torch

import simplicial_attention_b200 as sa
from simplicial_attention_b200 import _lib
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable():
    lib = _lib.lib()
    assert sa.device_status() == 0
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sa2_selftest_wait(2_000_000, stream) == 0          # ~1 ms at 2 GHz
    torch.cuda.synchronize()
    assert sa.device_status(reset=False) & _lib.SELFTEST_WAIT_BIT
    with pytest.raises(_lib.Sa2Error) as err:
        sa.check_device()
    assert err.value.status == _lib.SA2_ERR_DEVICE
    assert sa.device_status() == 0                                  # the check cleared the word
    sa.check_device()                                               # and passes now
    # the context still works: a real kernel runs and reports no error
    ins = [t.cuda() for t in O.make_inputs(1, 64, 2, 2, 64, seed=3, dtype=torch.bfloat16)]
    out, _ = sa.sa2_forward(*ins[:5], 16, 4)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all() and sa.device_status() == 0


def test_selftest_rejects_limits_outside_its_range():
    lib = _lib.lib()
    assert lib.sa2_selftest_wait(0, None) == 1
    assert lib.sa2_selftest_wait(3_000_000_000, None) == 1
