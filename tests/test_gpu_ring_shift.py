"""The in-place ring-shift kernel (rotate-only kernel of the library) on ONE GPU: N emulated ranks in one cooperative
launch, each with its own buffer and staging area; N shifts bring every buffer home bit-exact."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(world, lanes):
    from rtp_b200.ops import _lib
    L = _lib.lib()
    stg = []
    for _ in range(world):
        p = C.c_void_p()
        assert L.rtp_shift_staging_create(lanes, C.byref(p)) == 0, L.rtp_shift_last_error()
        stg.append(p.value)
    return L, stg


def _shift(L, bufs, stg, direction, lanes, status, timeout_ns=500_000_000):
    from rtp_b200.ops import _lib
    world = len(bufs)
    arr = C.c_void_p * world
    d = 0 if direction == "down" else 1
    dst = [stg[(r - 1) % world] if d == 0 else stg[(r + 1) % world] for r in range(world)]
    src = [stg[(r + 1) % world] if d == 0 else stg[(r - 1) % world] for r in range(world)]
    nbytes = bufs[0].numel() * bufs[0].element_size()
    rc = L.rtp_ring_shift(world, arr(*[b.data_ptr() for b in bufs]), nbytes, arr(*stg), arr(*dst), arr(*src), d, lanes,
                          arr(*[status.data_ptr()] * world), timeout_ns, _lib.stream_ptr())
    assert rc == 0, L.rtp_shift_last_error()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("nbytes", [48, 32768 * 3 + 1024, 5 * 1024 * 1024 + 16])
def test_ring_shift_rotates_bit_exact(world, nbytes):
    from rtp_b200.ops import _lib
    lanes = 16
    L, stg = _setup(world, lanes)
    status = _lib.status_word()
    torch.manual_seed(0)
    orig = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(world)]
    bufs = [o.clone() for o in orig]
    try:
        # down: rank r receives the buffer of rank r+1
        for step in range(1, world + 1):
            _shift(L, bufs, stg, "down", lanes, status)
            torch.cuda.synchronize()
            _lib.check_status()
            for r in range(world):
                assert torch.equal(bufs[r], orig[(r + step) % world]), (step, r)
        # up undoes it hop by hop; counters keep growing across calls and directions
        for step in range(1, world + 1):
            _shift(L, bufs, stg, "up", lanes, status)
            torch.cuda.synchronize()
            _lib.check_status()
            for r in range(world):
                assert torch.equal(bufs[r], orig[(r - step) % world]), (step, r)
    finally:
        torch.cuda.synchronize()
        for p in stg:
            L.rtp_shift_staging_destroy(p)


def test_ring_shift_missing_neighbour_times_out_and_returns():
    """A rank whose source never sends: the bounded wait runs out, the kernel records the status and returns."""
    from rtp_b200.ops import _lib
    lanes = 4
    L, stg = _setup(2, lanes)
    status = _lib.status_word()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    arr = C.c_void_p * 1
    try:
        # only "rank 0" is launched; its source (stg[1]) is never driven by anyone
        rc = L.rtp_ring_shift(1, arr(buf.data_ptr()), 4096, arr(stg[0]), arr(stg[1]), arr(stg[1]), 0, lanes,
                              arr(status.data_ptr()), 50_000_000, _lib.stream_ptr())
        assert rc == 0
        torch.cuda.synchronize()
        with pytest.raises(_lib.RotationTimeout):
            _lib.check_status()
    finally:
        torch.cuda.synchronize()
        for p in stg:
            L.rtp_shift_staging_destroy(p)
    # the context is still usable
    assert int((torch.ones(8, device="cuda") * 2).sum().item()) == 16
