"""GPU (one device is enough): the segment-copy kernel behind the peer-memory dispatch / combine and the
row-gather kernel, through the C ABI, against index arithmetic done on the host."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from primus_turbo_b200 import _lib  # noqa: E402
from primus_turbo_b200.pytorch.dist.peer_exchange import segment_tables  # noqa: E402
from primus_turbo_b200.pytorch.kernels.quantization_impl import gather_rows  # noqa: E402

DEV = "cuda"


def _copy(src, dsts, segs, row_bytes, num_ctas=0):
    arr = (ctypes.c_void_p * len(dsts))(*[d.data_ptr() for d in dsts])
    _lib.call("ptb_copy_segments", src.data_ptr(), arr, len(dsts), segs.data_ptr(), segs.shape[0], row_bytes, num_ctas,
              torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("world,E,width", [(2, 6, 64), (4, 8, 7168), (8, 256, 512)])
def test_dispatch_and_combine_of_all_ranks_on_one_device(world, E, width):
    """Every rank's dispatch and combine run as separate launches into buffers of one GPU (the kernels
    wait on nothing, so this is safe): rows must land expert-major and come back where they started."""
    g = torch.Generator().manual_seed(world)
    counts = torch.randint(0, 40 if width > 1000 else 300, (world, E), generator=g)
    counts[:, 1] = 0
    xs = [torch.randn(int(counts[r].sum()), width, generator=g).to(torch.bfloat16).to(DEV) for r in range(world)]
    tabs = [segment_tables(counts, r) for r in range(world)]
    recv = [torch.full((max(t.rows_out, 1), width), float("nan"), dtype=torch.bfloat16, device=DEV) for t in tabs]
    row_bytes = width * 2
    for r in range(world):
        _copy(xs[r], recv, tabs[r].dispatch.to(DEV), row_bytes, num_ctas=(0, 7, 32)[r % 3])
    torch.cuda.synchronize()
    e_loc = E // world
    for r in range(world):
        want = [xs[s][int(counts[s, :e].sum()) : int(counts[s, : e + 1].sum())]
                for e in range(r * e_loc, (r + 1) * e_loc) for s in range(world)]
        want = torch.cat(want)
        assert torch.equal(recv[r][: want.shape[0]].view(torch.int16), want.view(torch.int16))
    back = [torch.full_like(x, float("nan")) if x.shape[0] else x for x in xs]
    for r in range(world):
        _copy(recv[r], back, tabs[r].combine.to(DEV), row_bytes)
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(back[r].view(torch.int16), xs[r].view(torch.int16))
    assert _lib.copy_segments_status() == 0


@pytest.mark.parametrize("world,E,width", [(2, 6, 64), (8, 64, 512)])
def test_signalled_copies_of_all_ranks_on_one_device(world, E, width):
    """The arrival-flag form, every rank emulated on one GPU.  All copies are enqueued before any wait, on
    one stream, so no wait kernel ever runs beside a kernel it depends on: each finds its flags set.
    Checks the slot arithmetic (rank r's copy sets slot r of every destination's row), that an exchange
    with nothing to send still signals, that the CTA counters are left at zero, and two rounds of
    growing sequence numbers."""
    g = torch.Generator().manual_seed(world + 100)
    counts = torch.randint(0, 30, (world, E), generator=g)
    counts[world - 1] = 0  # the last rank sends nothing and must signal all the same
    xs = [torch.randn(int(counts[r].sum()), width, generator=g).to(torch.bfloat16).to(DEV) for r in range(world)]
    tabs = [segment_tables(counts, r) for r in range(world)]
    recv = [torch.zeros((max(t.rows_out, 1), width), dtype=torch.bfloat16, device=DEV) for t in tabs]
    flags = [torch.zeros(world, dtype=torch.int32, device=DEV) for _ in range(world)]  # flags[d][s]: source s -> destination d
    done = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    dst = (ctypes.c_void_p * world)(*[d.data_ptr() for d in recv])
    for seq in (1, 2):
        for r in range(world):
            segs = tabs[r].dispatch.to(DEV)
            slots = (ctypes.c_void_p * world)(*[flags[d].data_ptr() + 4 * r for d in range(world)])
            n = segs.shape[0] if xs[r].shape[0] else 0
            _lib.call("ptb_copy_segments_signal", xs[r].data_ptr() if n else None, dst, world, segs.data_ptr() if n else None, n,
                      width * 2, (0, 5)[r % 2], slots, done[r].data_ptr(), seq, stream)
        for d in range(world):
            _lib.call("ptb_wait_flags", flags[d].data_ptr(), world, seq, stream)
        torch.cuda.synchronize()
        assert _lib.copy_segments_status() == 0
        for d in range(world):
            assert flags[d].tolist() == [seq] * world and int(done[d]) == 0
    e_loc = E // world
    for r in range(world):
        want = torch.cat([xs[s][int(counts[s, :e].sum()) : int(counts[s, : e + 1].sum())]
                          for e in range(r * e_loc, (r + 1) * e_loc) for s in range(world)])
        assert torch.equal(recv[r][: want.shape[0]].view(torch.int16), want.view(torch.int16))
    # a wait for a number that has already been passed returns at once as well
    _lib.call("ptb_wait_flags", flags[0].data_ptr(), world, 1, stream)
    torch.cuda.synchronize()
    assert _lib.copy_segments_status() == 0


def test_copy_segments_argument_checks_and_bad_rank_flag():
    src = torch.zeros(4, 16, dtype=torch.uint8, device=DEV)
    dst = torch.zeros(4, 16, dtype=torch.uint8, device=DEV)
    segs = torch.tensor([[0, 0, 2, 5]], dtype=torch.int64, device=DEV)  # destination 5 of 1
    _copy(src + 1, [dst], segs, 16)
    torch.cuda.synchronize()
    assert _lib.copy_segments_status(reset=True) == 1 and _lib.copy_segments_status() == 0
    assert int(dst.sum()) == 0  # the bad segment was skipped
    arr = (ctypes.c_void_p * 1)(dst.data_ptr())
    rc = _lib.lib.ptb_copy_segments(src.data_ptr(), arr, 1, segs.data_ptr(), 1, 24, 0, None)
    assert rc == -3  # row size not a multiple of 16 bytes
    rc = _lib.lib.ptb_copy_segments(src.data_ptr(), arr, 17, segs.data_ptr(), 1, 16, 0, None)
    assert rc == -5


@pytest.mark.parametrize("rows,width,dtype", [(1000, 7168, torch.bfloat16), (77, 8, torch.bfloat16), (513, 4096, torch.float8_e4m3fn),
                                              (64, 36, torch.float32)])
def test_gather_rows(rows, width, dtype):
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, width, generator=g).to(dtype).to(DEV)
    idx = torch.randint(0, rows, (rows + 13,), generator=g).to(DEV)
    idx[5] = -1
    idx[6] = rows  # out of range on both sides: zero rows
    out = gather_rows(x, idx)
    view = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[x.element_size()]
    ref = x.view(view)[idx.clamp(0, rows - 1)]
    ref[5] = 0
    ref[6] = 0
    assert torch.equal(out.view(view), ref)
