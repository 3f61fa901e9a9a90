"""The allocation-free entry point ``ssd_b200_forward_static_scratch``.

Some users of the library cannot allocate device memory: a plugin that runs inside a
host runtime owning the whole device heap (cudaMalloc is forbidden on its request path,
and would fail once the host has reserved the memory), or a plain FFI client with no
allocator.  They call this entry point, whose scratch is a fixed 16 MiB array inside the
library.  The test drives it through the C ABI with ctypes, gives it only inputs and
outputs, and checks the result against the ordinary entry point (which takes a
caller-provided workspace) on two consecutive calls, since the shared scratch still holds
the first call's data when the second one starts.

Collected last on purpose (file name), so that a failure here cannot hide other tests in
a run that stops at the first failure.
"""
import ctypes as C

import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(lib, W, d, chunk, nsegments, Y, kernel="scan_f32"):
    from workloadsuite_b200 import _lib
    from workloadsuite_b200.ssd import _fill

    args = _lib.SsdArgs()
    _fill(args, d["X"], d["A"], d["B"], d["C"], None, d.get("initial_states"), Y, None, None, chunk, kernel,
          nsegments, False)
    assert args.workspace is None and args.workspace_bytes == 0     # the caller passes no scratch
    with torch.cuda.device(Y.device):
        return lib.ssd_b200_forward_static_scratch(C.byref(args),
                                                   C.c_void_p(torch.cuda.current_stream(Y.device).cuda_stream))


def test_static_scratch_entry_matches_workspace_entry_twice():
    import workloadsuite_b200 as W
    from workloadsuite_b200 import _lib

    lib = _lib.load()
    assert lib.ssd_b200_static_scratch_capacity() == 16 << 20
    for seed, dtype, tol in [(31, torch.bfloat16, 2e-2), (32, torch.float32, 1e-4)]:
        first = O.make_inputs(b=2, s=1024, h=3, p=64, n=64, g=1, dtype=dtype, init=True, seed=seed, decay_scale=0.02)
        second = O.make_inputs(b=2, s=1024, h=3, p=64, n=64, g=1, dtype=dtype, init=True, seed=seed + 100,
                               decay_scale=0.05)
        for inp in (first, second):           # two calls in a row on the same scratch
            d = {k: v.to(DEV) for k, v in inp.items()}
            want = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 128, initial_states=d["initial_states"],
                                 kernel="scan_f32", nsegments=4)
            got = torch.empty_like(want)
            rc = _call_static(lib, W, d, 128, 4, got)
            assert rc == 0, _lib.strerror(rc)
            torch.cuda.synchronize()
            per_bh, fro = O.error_metrics(got.cpu(), want.cpu())
            assert per_bh < tol and fro < tol, (dtype, per_bh, fro)
            # and both agree with the definition
            Yr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"])
            assert O.error_metrics(got.cpu(), Yr)[0] < tol


@pytest.mark.parametrize("mode", ["look_back", "chained"])
def test_static_scratch_entry_with_the_tensor_core_kernels_twice(mode):
    """The tensor-core kernel passes states from CTA to CTA through the shared array, in two ways: with fewer
    sequences than SMs every CTA publishes the state of its last piece scanned from zero and later pieces fold
    those ("look-back"); with more, a piece hands its final state to the next ("chained").  Both need their ready
    flags cleared, which the entry point does itself.  Two calls in a row on different data, against the ordinary
    entry point."""
    import workloadsuite_b200 as W
    from workloadsuite_b200 import _lib

    lib = _lib.load()
    if mode == "look_back":     # 4 head pairs of 16 tiles for 148 SMs
        shape, nseg = dict(b=2, s=2048, h=4, p=64, n=128, g=1), 4
    else:                       # 160 head pairs: tiles dealt out evenly inside one launch
        shape, nseg = dict(b=40, s=512, h=8, p=64, n=128, g=2), 2
    for seed in (61, 62):
        inp = O.make_inputs(dtype=torch.bfloat16, init=True, seed=seed, decay_scale=0.02, **shape)
        d = {k: v.to(DEV) for k, v in inp.items()}
        plan = W.plan(d["X"], d["A"], d["B"], d["C"], 256, kernel="tcgen05", nsegments=nseg)
        assert plan["launches"] == 1 and 0 < plan["workspace_bytes"] <= 16 << 20
        want = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, initial_states=d["initial_states"],
                             kernel="tcgen05", nsegments=nseg)
        got = torch.empty_like(want)
        rc = _call_static(lib, W, d, 256, nseg, got, kernel="tcgen05")
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        assert W.device_status(DEV) == 0
        per_bh, fro = O.error_metrics(got.cpu(), want.cpu())
        assert per_bh < 2e-2 and fro < 2e-2, (mode, seed, per_bh, fro)
        Yr = O.ssd_recurrence(inp["X"][:1], inp["A"][:1], inp["B"][:1], inp["C"][:1],
                              initial_states=inp["initial_states"][:1])
        assert O.error_metrics(got[:1].cpu(), Yr)[0] < 2e-2


def test_static_scratch_entry_rejects_oversized_problems():
    import workloadsuite_b200 as W
    from workloadsuite_b200 import _lib

    lib = _lib.load()
    # 64 units x 16 segments x (128*64+1) floats = 33.6 MB of segment states > 16 MiB
    d = {k: v.to(DEV) for k, v in
         O.make_inputs(b=2, s=4096, h=32, p=64, n=128, g=1, dtype=torch.bfloat16, seed=33).items()}
    Y = torch.empty_like(d["X"])
    rc = _call_static(lib, W, d, 256, 16, Y)
    assert rc == -8 and b"limit" in lib.ssd_b200_strerror(rc)
