"""The allocation-free histogram entry point, called the way a C caller would: through
its exported symbol, with caller-owned device buffers and a raw stream handle.

Kept in a file that sorts last, so a run that stops at the first failure has already run
every other test.  It passes alone in a fresh process and after the rest of the suite:
the entry point looks up its scratch address itself on first use and re-zeroes what it
needs on every call."""

import ctypes

import pytest
import torch

from lplb_b200 import Planner, _native, topology

pytestmark = pytest.mark.gpu

MAX_CTAS, MAX_EXPERTS = 160, 1024


@pytest.fixture(scope="module")
def entry():
    _native.load()
    lib = ctypes.CDLL(str(_native._so_path()))
    fn = lib.lplb_count_tokens_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [
        ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t,
    ]
    return fn


def _call(fn, idx, n_logical, n_cta, out):
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(idx.data_ptr(), int(idx.dtype == torch.int64), idx.numel(), n_logical, n_cta, out.data_ptr(), stream, err, 256)
    return rc, err.value.decode()


def test_two_calls_in_a_row_match_the_allocating_entry_point(entry):
    torch.cuda.set_device(0)
    # first call: 256 experts on every SM; second call right behind it: a smaller problem on
    # fewer CTAs, so rows and ticket left by the first call would show up if they mattered
    cases = [(256, 32, 148, (4096, 8), torch.int64), (64, 8, 5, (777,), torch.int32)]
    prepared = []
    for n_logical, ep, n_cta, shape, dtype in cases:
        planner = Planner(topology.cube(), n_logical + 2 * ep, n_logical, ep, device="cuda")
        idx = torch.randint(-1, n_logical, shape, device="cuda", generator=torch.Generator("cuda").manual_seed(n_cta)).to(dtype)
        out = torch.full((n_logical,), -7, dtype=torch.int32, device="cuda")
        prepared.append((planner, idx, n_logical, n_cta, out))
    torch.cuda.synchronize()
    for _, idx, n_logical, n_cta, out in prepared:  # back to back on one stream, nothing in between
        rc, msg = _call(entry, idx, n_logical, n_cta, out)
        assert rc == 0, msg
    torch.cuda.synchronize()
    for planner, idx, n_logical, n_cta, out in prepared:
        want, _ = planner.count_workload(idx, n_cta)
        assert torch.equal(out, want)  # integer counts: the tolerance is zero
        assert int(out.sum()) == int((idx >= 0).sum())


def test_sizes_beyond_the_fixed_scratch_are_refused(entry):
    torch.cuda.set_device(0)
    idx = torch.zeros(16, dtype=torch.int64, device="cuda")
    out = torch.full((MAX_EXPERTS + 1,), -7, dtype=torch.int32, device="cuda")
    rc, msg = _call(entry, idx, MAX_EXPERTS + 1, 8, out)
    assert rc < 0 and "n_logical" in msg and "1024" in msg
    rc, msg = _call(entry, idx, 64, MAX_CTAS + 1, out)
    assert rc < 0 and "n_cta" in msg and "160" in msg
    torch.cuda.synchronize()
    assert int((out != -7).sum()) == 0  # nothing was launched
    rc, msg = _call(entry, idx, MAX_EXPERTS, MAX_CTAS, out)  # the limits themselves are fine
    assert rc == 0, msg
    torch.cuda.synchronize()
    assert out[:MAX_EXPERTS].tolist()[:2] == [16, 0]


def test_a_call_after_the_warm_up_leaves_device_memory_as_it_was(entry):
    """The claim a caller with its own memory pool relies on: once the first call on the device
    has run (it loads the library's device image, array included), later calls take no device
    memory, neither from the driver nor from the framework's allocator."""
    torch.cuda.set_device(0)
    idx = torch.randint(-1, 256, (4096, 8), device="cuda")
    out = torch.zeros(256, dtype=torch.int32, device="cuda")
    rc, msg = _call(entry, idx, 256, 148, out)  # warm-up
    assert rc == 0, msg
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for n_cta in (148, 7):
        rc, msg = _call(entry, idx, 256, n_cta, out)
        assert rc == 0, msg
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_before
    assert int(out.sum()) == int((idx >= 0).sum())
