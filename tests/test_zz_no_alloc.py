"""The embedding scatter-add for callers that cannot allocate device memory.

`dyb200_lookup_accumulate_grads_noalloc` keeps its sort/segment tables in a fixed array inside the
library instead of the context's growable arena, for hosts whose device memory is reserved once at
start-up (as DyNet's pools are) and that must not hit cudaMalloc in the training loop.  It has to
give what `dyb200_lookup_accumulate_grads` gives: here both are called through the C ABI on the same
inputs, twice in a row (the second call reuses the array the first one left behind), and the size
limit is checked.  Both add the rows of one id in ascending position; the regular entry point sums a
very frequent id chunk-wise, so the two agree to rounding (the 1e-4 class of the other gradient
tests) and bit for bit on ids that occur once.  The allocation-free entry point adds strictly one row
after the other, so it is also compared bit for bit with the CPU oracle's sequential loop, for every id.
This file sorts last so a run that stops at the first failure has already covered everything else."""
import subprocess
import sys
import os
import numpy as np
import pytest

from util import TOL_REDUCE, assert_close, randn, rng, zipf_ids

pytestmark = pytest.mark.gpu


def _run(ctx, fn, ids, grad, acc0):
    import torch
    acc = torch.from_numpy(acc0).cuda()
    ids_dev = torch.from_numpy(ids.view(np.int32)).cuda()
    g = torch.from_numpy(grad).cuda()
    fn(ids, ids_dev.data_ptr(), g.data_ptr(), acc.data_ptr(), grad.shape[1], acc0.shape[0])
    torch.cuda.synchronize()
    return acc.cpu().numpy()


def _same(got, want, ids, what):
    counts = np.bincount(ids, minlength=want.shape[0])
    once = counts <= 1
    assert np.array_equal(got[once], want[once]), what
    assert_close(got, want, TOL_REDUCE, floor=max(1.0, float(np.sqrt(counts.max()))), what=what)


def test_noalloc_scatter_add_matches_regular_entry_point():
    import torch
    from dynet_b200 import capi
    ctx = capi.Context(0)
    r = rng(900)
    first = None
    for call, (E, V, n) in enumerate([(512, 5000, 4096), (64, 300, 777)]):   # two calls in a row
        ids = zipf_ids(r, n, V)
        grad = randn(r, n, E)
        acc0 = randn(r, V, E)
        want = _run(ctx, ctx.lookup_accumulate_grads, ids, grad, acc0)
        got = _run(ctx, ctx.lookup_accumulate_grads_noalloc, ids, grad, acc0)
        _same(got, want, ids, "call %d vs dyb200_lookup_accumulate_grads" % call)
        if first is None:
            first = (ids, grad, acc0, want)
    # the first problem again, after the array was reused by a different one
    ids, grad, acc0, want = first
    acc = torch.from_numpy(acc0).cuda()
    ids_dev = torch.from_numpy(ids.view(np.int32)).cuda()
    g = torch.from_numpy(grad).cuda()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]      # driver-level free memory: sees any cudaMalloc
    ctx.lookup_accumulate_grads_noalloc(ids, ids_dev.data_ptr(), g.data_ptr(), acc.data_ptr(), grad.shape[1], acc0.shape[0])
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    _same(acc.cpu().numpy(), want, ids, "third call")
    assert ctx.device_errors() == 0
    ctx.close()


@pytest.mark.parametrize("E,V,n", [(512, 5000, 4096), (30, 211, 4096), (64, 300, 777), (7, 5, 33)])
def test_noalloc_scatter_add_is_the_sequential_cpu_sum(oracle, E, V, n):
    """All ids, repeated ones included, bit for bit against the reference's CPU loop (dynet/model.cc:735-741);
    E = 30 and E = 7 take the scalar path (rows that are not whole 16-byte vectors), n = 4096 fills the array."""
    from dynet_b200 import capi
    ctx = capi.Context(0)
    r = rng(901 + E)
    ids = zipf_ids(r, n, V)
    grad = randn(r, n, E)
    acc0 = randn(r, V, E)
    want = oracle.lookup_accumulate_grads(acc0.copy(), ids, grad)
    for call in range(2):
        got = _run(ctx, ctx.lookup_accumulate_grads_noalloc, ids, grad, acc0)
        assert np.array_equal(got, want), "call %d: %d elements differ" % (call, int((got != want).sum()))
    assert ctx.device_errors() == 0
    ctx.close()


_CAPTURE_PROBE = r"""
import numpy as np, torch
from dynet_b200 import capi
s = torch.cuda.Stream()
ctx = capi.Context(0, s.cuda_stream)
ids = np.arange(8, dtype=np.uint32)
ids_dev = torch.from_numpy(ids.view(np.int32)).cuda()
g = torch.ones(8, 4, device="cuda"); acc = torch.zeros(8, 4, device="cuda")
torch.cuda.synchronize()
graph = torch.cuda.CUDAGraph()
err = None
with torch.cuda.graph(graph, stream=s):
    try:
        ctx.lookup_accumulate_grads_noalloc(ids, ids_dev.data_ptr(), g.data_ptr(), acc.data_ptr(), 4, 8)
    except capi.RuntimeErr as e:
        err = str(e)
assert err and "before any stream capture" in err, err
# outside a capture the same call works, and the gradient rows arrive
ctx.lookup_accumulate_grads_noalloc(ids, ids_dev.data_ptr(), g.data_ptr(), acc.data_ptr(), 4, 8)
torch.cuda.synchronize()
assert float(acc.sum()) == 32.0
print("ok")
"""


def test_noalloc_first_call_inside_a_capture_is_refused():
    """The one-time set-up of the first call on a device must not happen while a stream capture is open: the entry
    point says so with a status instead of breaking the capture.  Runs in a fresh process, where no earlier test has
    done the set-up."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-c", _CAPTURE_PROBE], cwd=root, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "ok" in p.stdout, p.stdout + p.stderr


def test_noalloc_needs_the_contexts_device_current():
    import torch
    from dynet_b200 import capi
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = capi.Context(0)
    ids = np.zeros(4, np.uint32)
    ids_dev = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    g = torch.zeros(4, 4, device="cuda:0")
    acc = torch.zeros(8, 4, device="cuda:0")
    torch.cuda.set_device(1)
    try:
        with pytest.raises(capi.InvalidArgument, match="current device"):
            ctx.lookup_accumulate_grads_noalloc(ids, ids_dev.data_ptr(), g.data_ptr(), acc.data_ptr(), 4, 8)
    finally:
        torch.cuda.set_device(0)
    ctx.close()


def test_noalloc_rejects_sizes_beyond_the_fixed_array():
    import torch
    from dynet_b200 import capi
    ctx = capi.Context(0)
    n = 4097
    ids = np.zeros(n, np.uint32)
    ids_dev = torch.zeros(n, dtype=torch.int32, device="cuda")
    g = torch.zeros(n, 4, device="cuda")
    acc = torch.zeros(8, 4, device="cuda")
    with pytest.raises(capi.InvalidArgument, match="DYB200_NOALLOC_MAX_IDS"):
        ctx.lookup_accumulate_grads_noalloc(ids, ids_dev.data_ptr(), g.data_ptr(), acc.data_ptr(), 4, 8)
    assert float(acc.abs().max()) == 0.0
    ctx.close()
