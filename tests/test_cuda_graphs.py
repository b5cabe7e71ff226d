"""The operators inside CUDA graphs.

The entry points take the stream they launch on and do nothing else to the device (no allocation, no
synchronisation, no host read), so a launch-bound loop over them can be captured once and replayed.  Checked here:
a captured forward + in-place backward replays on new input values with the bits of the eager calls, for the flat,
packed and ragged-row kernels and for the GeGLU sibling; the fused projection through the entry point that needs
no device allocation is captured too.  On the smallest benchmark shape (256 x 1024 fp32, a few microseconds of
kernel time) the replay must not be slower than the eager launches it replaces.
"""
from __future__ import annotations

import time

import pytest
import torch

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def _capture(step, warmups: int = 3):
    """Runs `step` on a side stream a few times (first-launch set-up happens outside the capture), then captures it."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmups):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = step()
    return graph, out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(256, 1024), (37, 1001), (4, 5, 11008)])
def test_forward_and_in_place_backward_replay_bit_for_bit(dtype, shape):
    from kernels.swiglu import swiglu_backward, swiglu_forward

    g = torch.Generator(device=DEVICE).manual_seed(21)
    draw = lambda: torch.randn(*shape, generator=g, device=DEVICE).to(dtype)
    gate_in, up_in, dout_in = draw(), draw(), draw()
    gate_buf, up_buf = torch.empty_like(gate_in), torch.empty_like(up_in)

    def step():
        gate_buf.copy_(gate_in)
        up_buf.copy_(up_in)
        h, gate_2d, up_2d = swiglu_forward(gate_buf, up_buf, 0.7, 1.3)
        dgate, dup = swiglu_backward(dout_in, gate_2d, up_2d, 0.7, 1.3)
        return h, dgate, dup

    graph, outs = _capture(step)
    for _ in range(3):  # new values in the static input buffers, same graph
        for t in (gate_in, up_in, dout_in):
            t.copy_(draw())
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in outs]
        want = step()
        torch.cuda.synchronize()
        for name, a, b in zip(("h", "dgate", "dup"), got, want):
            assert torch.equal(a.view(-1), b.reshape(-1)), name


def test_packed_ragged_and_geglu_replay():
    from kernels.geglu import geglu_backward, geglu_forward
    from kernels.swiglu import swiglu_packed_backward, swiglu_packed_forward

    g = torch.Generator(device=DEVICE).manual_seed(22)
    rows, half = 333, 1001  # odd half-width: the ragged-row kernels
    packed_in = torch.randn(rows, 2 * half, generator=g, device=DEVICE).bfloat16()
    dout = torch.randn(rows, half, generator=g, device=DEVICE).bfloat16()
    gate_in = torch.randn(64, 2048, generator=g, device=DEVICE).bfloat16()
    up_in = torch.randn(64, 2048, generator=g, device=DEVICE).bfloat16()
    dout2 = torch.randn(64, 2048, generator=g, device=DEVICE).bfloat16()
    packed_buf, gate_buf, up_buf = torch.empty_like(packed_in), torch.empty_like(gate_in), torch.empty_like(up_in)

    def step():
        packed_buf.copy_(packed_in)
        gate_buf.copy_(gate_in)
        up_buf.copy_(up_in)
        h, flat = swiglu_packed_forward(packed_buf)
        d_packed = swiglu_packed_backward(dout, flat, packed_buf.shape)
        hg, g2, u2 = geglu_forward(gate_buf, up_buf, "none")
        dg, du = geglu_backward(dout2, g2, u2, "none")
        return h, d_packed, hg, dg, du

    graph, outs = _capture(step)
    packed_in.mul_(0.5)
    gate_in.add_(0.25)
    graph.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in outs]
    want = step()
    torch.cuda.synchronize()
    for name, a, b in zip(("h", "d_packed", "geglu h", "geglu dgate", "geglu dup"), got, want):
        assert torch.equal(a.view(-1), b.reshape(-1)), name


def test_projection_without_device_allocation_is_capturable():
    from kernel_pocs_b200 import _lib
    from kernel_pocs_b200 import fused_mlp as F

    lib = _lib.load()
    m, n, k = 512, 768, 256
    g = torch.Generator(device=DEVICE).manual_seed(23)
    x = torch.randn(m, k, generator=g, device=DEVICE).bfloat16()
    wg = (torch.randn(n, k, generator=g, device=DEVICE) * k ** -0.5).bfloat16()
    wu = (torch.randn(n, k, generator=g, device=DEVICE) * k ** -0.5).bfloat16()
    h = torch.zeros(m, n, device=DEVICE, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32).pin_memory()

    def step():
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.swiglu_b200_gemm_fwd_noalloc(h.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), m, n, k, 1.0, 1.0,
                                              status.data_ptr(), x.device.index, stream)
        assert rc == 0
        return h

    graph, _ = _capture(step)
    want = F.gate_up_swiglu_forward(x, wg, wu)
    F.check_status(x.device)
    h.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert torch.equal(h, want)
    x.mul_(-1.0)  # new values, same graph
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(h, F.gate_up_swiglu_forward(x, wg, wu))


def test_replay_is_not_slower_than_eager_launches_on_the_smallest_shape():
    """256 x 1024 fp32 (the reference's CPU-runnable configuration): forward + in-place backward are a few
    microseconds of kernel time each, so the step is bound by its launches; a graph of 16 steps replays in no more
    host + device time than the 16 eager steps take."""
    from kernels.swiglu import swiglu_backward, swiglu_forward

    g = torch.Generator(device=DEVICE).manual_seed(24)
    gate0 = torch.randn(256, 1024, generator=g, device=DEVICE)
    up0 = torch.randn(256, 1024, generator=g, device=DEVICE)
    dout = torch.randn(256, 1024, generator=g, device=DEVICE)
    gate, up = gate0.clone(), up0.clone()

    def steps():
        for _ in range(16):
            h, g2, u2 = swiglu_forward(gate, up)
            swiglu_backward(dout, g2, u2)
        return h

    graph, _ = _capture(steps)

    def wall(fn, reps=30):
        fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            best = min(best, time.perf_counter() - t0)
        return best

    eager, replay = wall(steps), wall(graph.replay)
    assert replay <= eager * 1.05, f"graph replay {replay * 1e6:.1f} us against {eager * 1e6:.1f} us eager"
