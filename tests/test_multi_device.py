"""Several host threads driving several GPUs through the C ABI at once (one thread per device, the layout
of a row-partitioned multi-GPU run inside one process): results must equal the single-device results bit for
bit, whatever device is current in the calling thread.  Skipped when fewer than two GPUs are visible."""
import threading

import pytest
import torch

from kernel_pocs_b200 import _lib
from kernel_pocs_b200 import workloads as W

pytestmark = pytest.mark.gpu


def test_threads_on_different_devices_do_not_interfere():
    n_dev = torch.cuda.device_count()
    if n_dev < 2:
        pytest.skip("needs at least two GPUs")
    n_dev = min(n_dev, 4)
    w = W.Workload("t", 4096 * n_dev, 2048, torch.bfloat16, 6)
    shards = [W.row_shard(w.tokens, n_dev, r) for r in range(n_dev)]
    # reference result on device 0, whole matrix
    gate, up, dh = W.generate_rows(w, 0, w.tokens, "cuda:0")
    from kernels.swiglu import swiglu_backward, swiglu_forward

    h_ref = swiglu_forward(gate, up)[0]
    dg_ref, du_ref = swiglu_backward(dh, gate, up, preserve_inputs=True)
    torch.cuda.synchronize(0)

    results, errors = [None] * n_dev, []

    def worker(r):
        try:
            dev = torch.device("cuda", r)
            lo, hi = shards[r]
            g, u, d = W.generate_rows(w, lo, hi, dev)
            h = torch.empty_like(g)
            stream = torch.cuda.Stream(device=dev)
            # the generator wrote g, u, d on the device's default stream: order the side stream after it
            stream.wait_stream(torch.cuda.current_stream(dev))
            rows, cols = g.shape
            for _ in range(20):  # the calling thread's current device stays 0: the call switches and restores
                rc = _lib.lib.swiglu_b200_fwd(h.data_ptr(), g.data_ptr(), u.data_ptr(), rows, cols, cols, cols,
                                              _lib.BF16, 1.0, 1.0, r, stream.cuda_stream)
                assert rc == 0, rc
            gc, uc = g.clone(), u.clone()
            stream.wait_stream(torch.cuda.current_stream(dev))
            rc = _lib.lib.swiglu_b200_bwd(gc.data_ptr(), uc.data_ptr(), d.data_ptr(), gc.data_ptr(), uc.data_ptr(), rows,
                                          cols, cols, cols, cols, _lib.BF16, 1.0, 1.0, r, stream.cuda_stream)
            assert rc == 0, rc
            stream.synchronize()
            assert torch.cuda.current_device() == 0
            results[r] = (h.cpu(), gc.cpu(), uc.cpu())
        except Exception as exc:  # surfaced in the main thread
            errors.append((r, repr(exc)))

    threads = [threading.Thread(target=worker, args=(r,)) for r in range(n_dev)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert torch.equal(torch.cat([r[0] for r in results]), h_ref.cpu())
    assert torch.equal(torch.cat([r[1] for r in results]), dg_ref.cpu())
    assert torch.equal(torch.cat([r[2] for r in results]), du_ref.cpu())
