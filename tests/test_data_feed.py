"""Data feed (the first row past the training step): token bins and the epoch sampler against the reference's own pinned
window starts and test properties (ojas-data/tests/sampler.rs), and the device-resident feed against the host sampler.
Integer paths: every comparison is exact."""
import struct

import numpy as np
import pytest

from ojas_b200.data import (BatchSampler, DataCursor, DataError, SamplerRngState, SplitMix64, TokenBin, FINEWEB_HEADER_BYTES)


def write_bin(path, n, width=2, fineweb=False, magic=None, version=None):
    tokens = (np.arange(n, dtype=np.uint64) * 7 + 3) % (60000 if width == 2 else 100000)
    body = tokens.astype("<u2" if width == 2 else "<u4").tobytes()
    if fineweb:
        header = np.zeros(256, "<i4")
        header[0] = magic if magic is not None else (20240520 if width == 2 else 20240801)
        header[1] = version if version is not None else (1 if width == 2 else 7)
        header[2] = n
        body = header.tobytes() + body
    path.write_bytes(body)
    return tokens.astype(np.uint32)


def test_splitmix64_reference_values():
    r = SplitMix64(0)   # ojas-data/src/rng.rs: reference_splitmix64_values_and_counter_wraparound
    assert [r.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    top = SplitMix64((1 << 64) - 1)
    assert top.next_u64() == 0xE4D971771B652C20 and top.state == 0x9E3779B97F4A7C14


PINNED = [  # ojas-data/tests/sampler.rs:238-256: (seed, epoch, first eight window starts) for 1001 tokens, T = 10 (W = 100)
    (42, 0, [460, 450, 170, 260, 80, 430, 60, 970]),
    (42, 1, [310, 260, 960, 460, 810, 110, 470, 30]),
    (42, 7, [830, 50, 290, 530, 740, 820, 630, 260]),
    (0xDEADBEEF, 0, [570, 750, 980, 610, 430, 990, 840, 310]),
    (0xDEADBEEF, 1, [410, 710, 390, 780, 250, 940, 800, 140]),
    (0xDEADBEEF, 7, [630, 990, 250, 200, 900, 170, 360, 130]),
]


@pytest.mark.parametrize("seed,epoch,want", PINNED)
def test_permutation_is_pinned(seed, epoch, want):
    s = BatchSampler(1001, 10, 1, seed)
    assert s.windows_per_epoch() == 100
    assert [s.window_start(epoch, o) for o in range(8)] == want


def test_every_window_exactly_once_per_epoch_and_independent_of_batch(tmp_path):
    tokens = write_bin(tmp_path / "t.bin", 1237)
    bin_ = TokenBin.open(tmp_path / "t.bin", "headerless_u16")
    assert len(bin_) == 1237
    for seed in (0, 5):
        streams = []
        for batch in (1, 3, 8):
            s = BatchSampler(len(bin_), 16, batch, seed)
            w = s.windows_per_epoch()
            assert w == (1237 - 1) // 16
            starts = []
            while len(starts) < 3 * w:
                starts += list(s.next_starts())
            streams.append(starts[: 3 * w])
            for e in range(3):   # each epoch is a permutation of all windows
                assert sorted(starts[e * w:(e + 1) * w]) == [k * 16 for k in range(w)]
        assert streams[0] == streams[1] == streams[2]
        assert streams[0][:w] != streams[0][w:2 * w]       # epochs differ
    s = BatchSampler(len(bin_), 16, 4, 9)
    x, y = s.next_batch(bin_)
    assert x.shape == y.shape == (4, 16) and x.dtype == np.uint32
    assert np.array_equal(x[:, 1:], y[:, :-1])
    first = BatchSampler(len(bin_), 16, 4, 9).window_start(0, 0)
    assert np.array_equal(x[0], tokens[first:first + 16]) and y[0, -1] == tokens[first + 16]
    bin_.close()


def test_resume_from_a_cursor_and_refusals(tmp_path):
    write_bin(tmp_path / "t.bin", 500)
    bin_ = TokenBin.open(tmp_path / "t.bin", "headerless_u16")
    a = BatchSampler(len(bin_), 8, 5, 3)
    for _ in range(7):
        a.next_starts()
    cur = a.cursor()
    b = BatchSampler(len(bin_), 8, 5, 3, cur)
    assert list(a.next_starts()) == list(b.next_starts()) and a.cursor() == b.cursor()
    with pytest.raises(DataError):
        BatchSampler(len(bin_), 8, 5, 3, DataCursor(0, a.windows_per_epoch()))
    with pytest.raises(DataError):
        BatchSampler(len(bin_), 0, 5, 3)
    with pytest.raises(DataError):
        BatchSampler(8, 8, 1, 3)            # a window needs T + 1 tokens
    assert BatchSampler(9, 8, 1, 3).windows_per_epoch() == 1
    with pytest.raises(DataError):
        bin_.read_u32(495, 6)
    bin_.close()


def test_rng_state_layout_is_exact_and_refuses_anything_else():
    state = SamplerRngState(0x0123456789ABCDEF)
    raw = state.encode()
    assert raw == struct.pack("<IIQ", 1, 1, 0x0123456789ABCDEF) and SamplerRngState.decode(raw) == state
    for n in (0, 1, 8, 15, 17, 32):
        with pytest.raises(DataError, match="bytes"):
            SamplerRngState.decode(raw[:n].ljust(n, b"\0"))
    with pytest.raises(DataError, match="version"):
        SamplerRngState.decode(struct.pack("<IIQ", 2, 1, 5))
    with pytest.raises(DataError, match="generator"):
        SamplerRngState.decode(struct.pack("<IIQ", 1, 2, 5))


def test_token_bin_layouts(tmp_path):
    t16 = write_bin(tmp_path / "a.bin", 300, 2, fineweb=True)
    t32 = write_bin(tmp_path / "b.bin", 300, 4, fineweb=True)
    a, b = TokenBin.open(tmp_path / "a.bin", "fineweb"), TokenBin.open(tmp_path / "b.bin", "fineweb")
    assert (a.width, b.width, len(a), len(b), a.data_offset) == (2, 4, 300, 300, FINEWEB_HEADER_BYTES)
    assert np.array_equal(a.read_u32(10, 20), t16[10:30]) and np.array_equal(b.read_u32(280, 20), t32[280:300])
    assert np.array_equal(b.raw_tokens(), t32) and np.array_equal(b.raw_tokens(), t32)   # positioned: a second read starts at token 0 too
    with pytest.raises(DataError, match="expected u16"):
        TokenBin.open(tmp_path / "b.bin", "fineweb_u16")
    write_bin(tmp_path / "c.bin", 10, 2, fineweb=True, magic=123)
    with pytest.raises(DataError, match="magic"):
        TokenBin.open(tmp_path / "c.bin", "fineweb")
    write_bin(tmp_path / "d.bin", 10, 2, fineweb=True, version=2)
    with pytest.raises(DataError, match="version"):
        TokenBin.open(tmp_path / "d.bin", "fineweb")
    (tmp_path / "e.bin").write_bytes(b"\0" * 7)
    with pytest.raises(DataError, match="multiple"):
        TokenBin.open(tmp_path / "e.bin", "headerless_u16")
    (tmp_path / "f.bin").write_bytes((tmp_path / "a.bin").read_bytes()[:-2])
    with pytest.raises(DataError, match="size mismatch"):
        TokenBin.open(tmp_path / "f.bin", "fineweb")
    with pytest.raises(DataError, match="not a regular file"):
        TokenBin.open(tmp_path, "headerless_u16")
    a.close(); b.close()


@pytest.mark.gpu
@pytest.mark.parametrize("width", [2, 4])
def test_device_feed_matches_the_host_sampler(tmp_path, width):
    """The HBM-resident feed gives exactly the host sampler's batches; two ranks read disjoint rows whose union is the global batch."""
    from ojas_b200 import CudaBackend, OjasError
    from ojas_b200.data import DeviceFeed
    tokens = write_bin(tmp_path / "t.bin", 20011, width)
    bin_ = TokenBin.open(tmp_path / "t.bin", "headerless_u16" if width == 2 else "headerless_u32")
    be = CudaBackend(0, 1 << 30)
    feed = DeviceFeed(be, bin_, 64, 6, seed=11)
    host = BatchSampler(len(bin_), 64, 6, 11)
    for _ in range(60):        # runs across an epoch boundary (312 windows per epoch)
        ids, tgt = feed.next()
        x, y = host.next_batch(bin_)
        assert np.array_equal(ids.numpy(), x) and np.array_equal(tgt.numpy(), y)
    assert feed.cursor() == host.cursor()
    ranks = [DeviceFeed(be, bin_, 64, 3, seed=11, rank=r, world=2) for r in range(2)]
    host = BatchSampler(len(bin_), 64, 6, 11)
    for _ in range(5):
        x, y = host.next_batch(bin_)
        got = [f.next() for f in ranks]
        assert np.array_equal(np.concatenate([g[0].numpy() for g in got]), x) and np.array_equal(np.concatenate([g[1].numpy() for g in got]), y)
    # a window past the end is refused before any launch
    import ctypes as C
    from ojas_b200._lib import lib
    from ojas_b200.backend import _check, _p
    bad = np.array([len(bin_) - 64], np.int64)
    with pytest.raises(OjasError):
        _check(lib.ojc_gather_token_windows(be._handle, C.c_void_p(feed._tokens.ptr), C.c_int32(width), C.c_uint64(len(bin_)), bad.ctypes.data_as(C.POINTER(C.c_int64)),
                                            C.c_int64(1), C.c_int64(64), _p(be.empty((1, 64), feed._ids[0].dtype)), _p(be.empty((1, 64), feed._ids[0].dtype))))
    del ranks, feed
    be.close(); bin_.close()
