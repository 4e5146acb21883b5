"""The allocation-free compaction entry point against the regular one (through the C ABI).

Some callers of libv1g.so cannot let it allocate: framework op kernels have to take device memory
from the framework's allocator, and fixed-budget programs have nothing to allocate from.
``v1g_compact_spikes_noalloc`` keeps its scratch in a fixed array inside the library instead.  This
file is collected last, so a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, handle, x, cap):
    rows, cols = x.shape
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = []
    for noalloc in (False, True):
        coords = torch.full((max(cap, 1), 2), -1, dtype=torch.int64, device="cuda")
        count = torch.full((1,), -7, dtype=torch.int32, device="cuda")
        if noalloc:
            rc = lib.v1g_compact_spikes_noalloc(x.data_ptr(), rows, cols, coords.data_ptr(), cap,
                                                count.data_ptr(), stream)
        else:
            rc = lib.v1g_compact_spikes(handle, x.data_ptr(), rows, cols, coords.data_ptr(), cap,
                                        count.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        out.append((int(count.item()), coords.cpu()))
    return out


def test_noalloc_compaction_equals_regular_on_consecutive_calls():
    from util import make_case
    from v1_glif_model_b200 import _lib
    from v1_glif_model_b200.models import V1Column
    lib = _lib.load()
    cfg, dicts, _ = make_case("tiny")
    cell = V1Column(*dicts)           # only to obtain a handle for the regular entry point
    g = torch.Generator().manual_seed(123)
    # two calls in a row with different shapes and densities: the second must not see leftovers
    for shape, p in (((5, 20000), 0.02), ((3, 4097), 0.4), ((2, 50), 0.0), ((4, 9000), 1.0)):
        x = (torch.rand(shape, generator=g) < p).float().cuda().contiguous()
        cap = shape[0] * shape[1]
        (n_ref, c_ref), (n_new, c_new) = _both(lib, cell._libh, x, cap)
        want = torch.nonzero(x.cpu() > 0)
        assert n_ref == n_new == want.shape[0]
        assert torch.equal(c_new[:n_new], c_ref[:n_ref])      # bit-exact, same order
        assert torch.equal(c_new[:n_new], want)


def test_noalloc_rejects_oversized_input():
    from v1_glif_model_b200 import _lib
    lib = _lib.load()
    rc = lib.v1g_compact_spikes_noalloc(None, 70000, 4096, None, 0, None, None)
    assert rc == _lib.EINVAL          # null input with a non-empty shape
    x = torch.zeros(1, device="cuda")
    rc = lib.v1g_compact_spikes_noalloc(x.data_ptr(), 70000, 4096, None, 0, None, None)
    assert rc == _lib.ERANGE          # 70000 segments > 65536
    assert b"exceed the fixed scratch" in lib.v1g_last_error(None)
