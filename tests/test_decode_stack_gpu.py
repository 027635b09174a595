"""The benchmark's decode stack: the host-to-host step (activations copied up every step, beside the first layer's launches
from the second layer on; the last output read back) gives the bits of the device-resident step, and really copies."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_host_step_equals_device_step_and_copies(ctx):
    import torch
    from makepad_b200.decode_stack import DecodeStack
    stack = DecodeStack(ctx, layers=3, M=1, shapes=[("a", 1024, 512), ("b", 512, 1024)], seed=5).capture()
    with torch.cuda.stream(stack.stream):
        stack.step()
    stack.stream.synchronize()
    want = stack.output(len(stack.weights) - 1).cpu().numpy().copy()
    got = stack.step_host().numpy().reshape(want.shape).copy()
    assert np.array_equal(got, want)
    # new host activations for the LAST projection (the part copied on the second stream): what the device-resident step
    # gives for them is what the host step must give after the device copy has been wiped
    i = len(stack.weights) - 1
    off, n = stack.x_off[i], stack.weights[i].K
    stack.x_host[off:off + n] = torch.randn(n)
    stack.x.copy_(stack.x_host)
    with torch.cuda.stream(stack.stream):
        stack.step()
    stack.stream.synchronize()
    want2 = stack.output(i).cpu().numpy().copy()
    assert not np.array_equal(want2, want)
    stack.x.zero_()
    torch.cuda.synchronize()
    got2 = stack.step_host().numpy().reshape(want.shape).copy()
    assert np.array_equal(got2, want2)
    assert torch.equal(stack.x.cpu(), stack.x_host)
    assert stack.h2d_bytes_per_step == stack.x.numel() * 4 and stack.d2h_bytes_per_step == want.size * 4
    stack.destroy()
