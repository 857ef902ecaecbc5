"""The allocation-free grouping entry point (gptoss_moe_build_offsets_noalloc) against the context-based
one.  Some hosts cannot allocate device memory once they are running: an engine that reserves the whole
GPU for its own pool at start-up leaves nothing for a later cudaMalloc, and a serving loop cannot afford
the device-wide synchronisation an allocation may imply.  For them the library keeps the scratch of the
counting sort in a fixed device array; this test checks that the result is identical to the regular entry
point, on two calls in a row (the second must not see anything of the first in the shared scratch), and
that batches beyond the fixed scratch are refused.  Runs last so a failure here hides no other result."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_noalloc_build_offsets_matches_context_entry_point_twice_in_a_row():
    from gptoss_b200 import capi, moe
    lib = capi.load()
    torch.cuda.set_device(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(1234)
    for E, k, T in [(32, 4, 1000), (128, 4, 333)]:  # second call: other sizes, stale scratch from the first
        p = 1.0 / np.arange(1, E + 1) ** 1.2
        ids = rng.choice(E, size=(T, k), p=p / p.sum()).astype(np.int32)
        ids[3, 1] = -7  # an id outside [0,E) is skipped by both entry points
        ids_dev = torch.from_numpy(ids).cuda()
        blk = moe.MoEBlock(hidden=64, intermediate=64, n_experts=E, top_k=k, max_tokens=T)
        want_off, want_srt = blk.moe_build_offsets(ids_dev)
        off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
        srt = torch.full((T * k,), -1, dtype=torch.int32, device="cuda")
        rc = lib.gptoss_moe_build_offsets_noalloc(T, E, k, _ptr(ids_dev), _ptr(off), _ptr(srt), stream)
        assert rc == capi.OK, lib.gptoss_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(off, want_off)
        assert torch.equal(srt, want_srt)
        blk.close()


def test_noalloc_call_leaves_free_device_memory_unchanged():
    """What the entry point promises: after its one-time set-up on a device, a call allocates nothing — the free
    device memory reported by the driver is the same before and after."""
    from gptoss_b200 import capi
    lib = capi.load()
    torch.cuda.set_device(0)
    E, k, T = 32, 4, 4096
    ids_dev = torch.from_numpy(np.random.default_rng(5).integers(0, E, size=(T, k), dtype=np.int32)).cuda()
    off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    srt = torch.empty(T * k, dtype=torch.int32, device="cuda")
    call = lambda: lib.gptoss_moe_build_offsets_noalloc(T, E, k, _ptr(ids_dev), _ptr(off), _ptr(srt), None)  # noqa: E731
    assert call() == capi.OK  # the first call on the device resolves the scratch array's address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert call() == capi.OK
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_noalloc_rejects_batches_beyond_the_static_scratch():
    from gptoss_b200 import capi
    lib = capi.load()
    torch.cuda.set_device(0)
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = lib.gptoss_moe_build_offsets_noalloc(8192 * 2 + 8, 128, 4, _ptr(dummy), _ptr(dummy), _ptr(dummy), None)
    assert rc == capi.ERR_BAD_ARG
    assert b"static scratch" in lib.gptoss_noalloc_last_error()
    assert lib.gptoss_moe_build_offsets_noalloc(16, 300, 4, _ptr(dummy), _ptr(dummy), _ptr(dummy), None) == capi.ERR_BAD_ARG
