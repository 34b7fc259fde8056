"""The bounded device-side wait: a probe kernel waits on an mbarrier that nobody arrives on, with a
limit of a few milliseconds.  The wait must give up and the kernel return (no hang, no fault), the
status word must carry the probe's code, gb200_device_sync must report GB200_ERR_TIMEOUT once, and
the context must stay usable."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(ctx, oracle):
    from gern_b200 import api
    ctx.sync()
    returned = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = api.lib.gb200_selftest_bounded_wait(ctx.handle, 3_000_000, returned.data_ptr(), None)   # 3 ms
    assert rc == 0
    with pytest.raises(api.GernB200Error) as e:
        ctx.sync()
    assert e.value.code == -5 and "status code 901" in str(e.value)
    assert int(returned.item()) == 1, "the probe's wait must give up, not complete"
    ctx.sync()                                  # the status word was cleared by the report
    # the same context still computes
    x = np.random.default_rng(0).random((66, 130), dtype=np.float32)
    out = torch.empty((64, 128), device="cuda")
    ctx.blur3x3(torch.from_numpy(x).cuda(), out)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.blur_xy(x))


def test_a_host_entry_point_reports_the_timeout_itself(ctx):
    """The `_host` forms read the status word behind their own work."""
    from gern_b200 import api
    returned = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert api.lib.gb200_selftest_bounded_wait(ctx.handle, 1_000_000, returned.data_ptr(), None) == 0
    torch.cuda.synchronize()
    x = np.ones((40, 40), np.float32)
    out = np.zeros((38, 38), np.float32)
    with pytest.raises(api.GernB200Error) as e:
        ctx.blur3x3_host(x, out)
    assert e.value.code == -5
    ctx.blur3x3_host(x, out)                    # reported once; the next call is clean
    assert (out == 1.0).all()


def test_a_flag_wait_that_runs_out_is_reported_too(ctx):
    """The one wait on a word in global memory (the blur's halo block row waits for the flag its
    context's copy stream sets): a probe waits 2 ms for a value nobody writes."""
    from gern_b200 import api
    ctx.sync()
    returned = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert api.lib.gb200_selftest_bounded_flag_wait(ctx.handle, 2_000_000, returned.data_ptr(), None) == 0
    with pytest.raises(api.GernB200Error) as e:
        ctx.sync()
    assert e.value.code == -5 and "status code 902" in str(e.value)
    assert int(returned.item()) == 1
    ctx.sync()
