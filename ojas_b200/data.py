"""Data feed for the training step: token bins, the epoch sampler, and a device-resident feed.

Mirrors ojas-data's `TokenBin` (ojas-data/src/tokens.rs) and `BatchSampler` (ojas-data/src/sampler.rs): windows of T + 1
tokens that do not overlap, every window exactly once per epoch, in an order that is a 4-round Feistel permutation of
0..W keyed by (seed, epoch) with SplitMix64 as round function and key schedule, cycle-walked into range. The cursor
(epoch, ordinal of the next window) and the 16-byte rng state are what a checkpoint stores.

`DeviceFeed` is the B200 form: the whole token stream is uploaded to HBM once (a 10-billion-token u16 shard is 20 GB of
the 180), each step sends only the batch's window starts, and `ojc_gather_token_windows` writes ids and targets on the
device. Under data parallelism every rank holds the same sampler with the global batch and takes its own rows, so the
ranks read disjoint windows and the union is the single-process stream.
"""
from __future__ import annotations

import ctypes as C
import os
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_MASK64 = (1 << 64) - 1
FINEWEB_MAGIC, FINEWEB_VERSION = 20240520, 1
FINEWEB_U32_MAGIC, FINEWEB_U32_VERSION = 20240801, 7
FINEWEB_HEADER_BYTES = 256 * 4
ROUNDS = 4                                   # Feistel rounds (sampler.rs:36)
EPOCH_STEP = 0xD1B54A32D192ED03              # per-epoch key spacing (sampler.rs:41)
RNG_STATE_VERSION, RNG_GENERATOR_FEISTEL4_SPLITMIX64, RNG_STATE_BYTES = 1, 1, 16


class DataError(Exception):
    """ojas-data's DataError: a refusal with a detail string."""


class SplitMix64:
    """The counter generator ojas calls CounterRng (ojas-kernels/src/rng.rs): state += gamma, then the two-multiply mix."""

    def __init__(self, seed: int):
        self.state = seed & _MASK64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        return z ^ (z >> 31)


@dataclass(frozen=True)
class DataCursor:
    """Checkpoint cursor: `shard` is the epoch, `token_index` the ordinal of the next window in it (not a token offset)."""
    shard: int = 0
    token_index: int = 0


@dataclass(frozen=True)
class SamplerRngState:
    """The sampler's identity in a checkpoint's rng_state: u32 version, u32 generator, u64 seed, little endian (sampler.rs:56-113)."""
    seed: int

    def encode(self) -> bytes:
        return struct.pack("<IIQ", RNG_STATE_VERSION, RNG_GENERATOR_FEISTEL4_SPLITMIX64, self.seed & _MASK64)

    @staticmethod
    def decode(data: bytes) -> "SamplerRngState":
        if len(data) != RNG_STATE_BYTES:
            raise DataError(f"rng_state: {len(data)} bytes, the v{RNG_STATE_VERSION} layout is {RNG_STATE_BYTES}")
        version, generator, seed = struct.unpack("<IIQ", data)
        if version != RNG_STATE_VERSION:
            raise DataError(f"rng_state: version {version}, expected {RNG_STATE_VERSION}")
        if generator != RNG_GENERATOR_FEISTEL4_SPLITMIX64:
            raise DataError(f"rng_state: generator {generator}, this sampler is {RNG_GENERATOR_FEISTEL4_SPLITMIX64}")
        return SamplerRngState(seed)


class TokenBin:
    """A token file read with positioned reads: headerless little-endian u16 / u32, or a FineWeb shard (256 x i32 header:
    magic 20240520 -> u16 version 1, magic 20240801 -> u32 version 7 or 1, token count at word 2; tokens.rs:1-6,156-214)."""

    def __init__(self, fd: int, data_offset: int, len_tokens: int, width: int):
        self._fd, self.data_offset, self.len_tokens, self.width = fd, data_offset, len_tokens, width

    @staticmethod
    def open(path, layout: str = "headerless_u16") -> "TokenBin":
        """layout: headerless_u16 | headerless_u32 | fineweb | fineweb_u16 | fineweb_u32. Anything but a regular file is refused."""
        path = Path(path)
        try:
            st = os.stat(path)
        except OSError as e:
            raise DataError(f"{path}: {e.strerror}") from None
        import stat as _stat
        if not _stat.S_ISREG(st.st_mode):
            raise DataError(f"{path}: not a regular file")
        fd = os.open(path, os.O_RDONLY)
        try:
            return TokenBin._from_fd(fd, os.fstat(fd).st_size, layout)
        except DataError as e:
            os.close(fd)
            raise DataError(f"{path}: {e}") from None

    @staticmethod
    def _from_fd(fd: int, length: int, layout: str) -> "TokenBin":
        if layout.startswith("headerless"):
            width = {"headerless_u16": 2, "headerless_u32": 4}.get(layout)
            if width is None:
                raise DataError(f"unknown layout {layout}")
            if length % width:
                raise DataError(f"truncated token bin, {length} bytes is not a multiple of {width}")
            return TokenBin(fd, 0, length // width, width)
        if layout not in ("fineweb", "fineweb_u16", "fineweb_u32"):
            raise DataError(f"unknown layout {layout}")
        if length < FINEWEB_HEADER_BYTES:
            raise DataError(f"truncated FineWeb header, {length} bytes")
        magic, version, count = struct.unpack("<iii", os.pread(fd, 12, 0))
        if magic == FINEWEB_MAGIC:
            if version != FINEWEB_VERSION:
                raise DataError(f"version {version} != {FINEWEB_VERSION}")
            width = 2
        elif magic == FINEWEB_U32_MAGIC:
            if version not in (FINEWEB_U32_VERSION, 1):
                raise DataError(f"version {version} != {FINEWEB_U32_VERSION}")
            width = 4
        else:
            raise DataError(f"magic {magic} != {FINEWEB_MAGIC}")
        if count < 0:
            raise DataError(f"token count {count} is negative")
        expect = FINEWEB_HEADER_BYTES + count * width
        if length != expect:
            raise DataError(f"size mismatch, expected {expect} bytes, got {length}")
        want = {"fineweb_u16": 2, "fineweb_u32": 4}.get(layout)
        if want is not None and want != width:
            raise DataError(f"expected {'u16' if want == 2 else 'u32'} FineWeb bin, found {'U16' if width == 2 else 'U32'}")
        return TokenBin(fd, FINEWEB_HEADER_BYTES, count, width)

    def __len__(self) -> int:
        return self.len_tokens

    def close(self) -> None:
        if self._fd >= 0:
            os.close(self._fd)
            self._fd = -1

    def read_u32(self, index: int, count: int) -> np.ndarray:
        """`count` tokens from `index`, widened to u32; a window past the end is refused (tokens.rs:283-296)."""
        end = index + count
        if index < 0 or end > self.len_tokens:
            raise DataError(f"token window [{index}, {end}) past length {self.len_tokens}")
        raw = os.pread(self._fd, count * self.width, self.data_offset + index * self.width)
        if len(raw) != count * self.width:
            raise DataError("token read: short read")
        return np.frombuffer(raw, dtype="<u2" if self.width == 2 else "<u4").astype(np.uint32)

    def raw_tokens(self) -> np.ndarray:
        """The whole stream in its stored width (for the device-resident feed). Positioned reads, in 256 MB pieces:
        the file's own cursor is neither used nor moved."""
        out = np.empty(self.len_tokens, dtype="<u2" if self.width == 2 else "<u4")
        view, total, done, piece = out.view(np.uint8), self.len_tokens * self.width, 0, 256 << 20
        while done < total:
            raw = os.pread(self._fd, min(piece, total - done), self.data_offset + done)
            if not raw:
                raise DataError("token read: short read")
            view[done:done + len(raw)] = np.frombuffer(raw, np.uint8)
            done += len(raw)
        return out


class BatchSampler:
    """Epoch sampler over `len_tokens` tokens (sampler.rs:138-318). It owns no file: `next_starts` gives the token offsets of
    the next B windows and moves the cursor; `next_batch(bin)` also reads them."""

    def __init__(self, len_tokens: int, seq_len: int, batch: int, seed: int, cursor: DataCursor = DataCursor()):
        if seq_len <= 0 or batch <= 0:
            raise DataError(f"sampler: seq_len {seq_len} and batch {batch} must be non-zero")
        if len_tokens < seq_len + 1:
            raise DataError(f"sampler: a window needs {seq_len + 1} tokens, the bin has {len_tokens}")
        self.seq_len, self.batch, self.seed = seq_len, batch, seed & _MASK64
        self.windows = (len_tokens - 1) // seq_len
        if cursor.token_index >= self.windows:
            raise DataError(f"sampler: cursor window {cursor.token_index} is past the {self.windows} windows of an epoch")
        bits = (self.windows - 1).bit_length()
        self.half_bits = max((bits + 1) // 2, 1)
        self.epoch, self.ordinal = cursor.shard, cursor.token_index
        self._keys_epoch, self._keys = None, None

    def windows_per_epoch(self) -> int:
        return self.windows

    def cursor(self) -> DataCursor:
        return DataCursor(self.epoch, self.ordinal)

    def rng_state(self) -> SamplerRngState:
        return SamplerRngState(self.seed)

    def _round_keys(self, epoch: int):
        if self._keys_epoch != epoch:
            rng = SplitMix64(self.seed ^ ((epoch * EPOCH_STEP) & _MASK64))
            self._keys, self._keys_epoch = [rng.next_u64() for _ in range(ROUNDS)], epoch
        return self._keys

    def _feistel(self, v: int, keys) -> int:
        h = self.half_bits
        mask = (1 << h) - 1
        left, right = (v >> h) & mask, v & mask
        for key in keys:
            f = SplitMix64(right ^ key).next_u64() & mask
            left, right = right, left ^ f
        return (left << h) | right

    def window_start(self, epoch: int, ordinal: int) -> int:
        """Token offset of the `ordinal`-th window of `epoch`: the permutation, cycle-walked back into 0..W."""
        if ordinal >= self.windows:
            raise DataError(f"sampler: window {ordinal} past {self.windows} per epoch")
        keys, v = self._round_keys(epoch), ordinal
        while True:
            v = self._feistel(v, keys)
            if v < self.windows:
                return v * self.seq_len

    def next_starts(self) -> np.ndarray:
        """The next B window starts; a batch runs on into the next epoch when one ends, so the stream does not depend on B."""
        epoch, ordinal, starts = self.epoch, self.ordinal, np.empty(self.batch, np.int64)
        for i in range(self.batch):
            starts[i] = self.window_start(epoch, ordinal)
            ordinal += 1
            if ordinal == self.windows:
                ordinal, epoch = 0, epoch + 1
        self.epoch, self.ordinal = epoch, ordinal
        return starts

    def next_batch(self, bin_: TokenBin):
        """(x, y) as u32 [B, T]: y[r][i] == x[r][i + 1], y[r][T - 1] is the token after the window. The cursor moves only on success."""
        saved = (self.epoch, self.ordinal)
        try:
            starts = self.next_starts()
            rows = [bin_.read_u32(int(s), self.seq_len + 1) for s in starts]
        except DataError:
            self.epoch, self.ordinal = saved
            raise
        x = np.stack([r[:-1] for r in rows])
        y = np.stack([r[1:] for r in rows])
        return x, y


class DeviceFeed:
    """The token stream resident in HBM plus the sampler: `next()` returns device ids / targets [B, T] for this rank.

    world > 1: every rank constructs the feed with the same seed and the per-rank batch; the sampler runs with the global
    batch world * B and rank r takes rows [r B, (r + 1) B)."""

    def __init__(self, be, bin_: TokenBin, seq_len: int, batch: int, seed: int, rank: int = 0, world: int = 1, cursor: DataCursor = DataCursor()):
        from ._lib import lib
        from .backend import DType
        if not (0 <= rank < world):
            raise DataError(f"feed: rank {rank} outside world {world}")
        self._lib, self.be, self.rank, self.world, self.batch, self.seq_len = lib, be, rank, world, batch, seq_len
        self.sampler = BatchSampler(len(bin_), seq_len, batch * world, seed, cursor)
        self.width, self.len_tokens = bin_.width, len(bin_)
        tokens = bin_.raw_tokens()
        # stored width on the device too; the upload goes through a byte view of whatever the file holds
        padded = np.zeros((tokens.nbytes + 3) // 4, np.uint32)
        padded.view(np.uint8)[: tokens.nbytes] = tokens.view(np.uint8)
        self._tokens = be.upload(padded, DType.U32)
        self._ids = [be.empty((batch, seq_len), DType.U32) for _ in range(2)]      # two batches in flight: the step reads one
        self._tgt = [be.empty((batch, seq_len), DType.U32) for _ in range(2)]      # while the next is gathered
        self._slot = 0

    def cursor(self) -> DataCursor:
        return self.sampler.cursor()

    def next(self):
        from .backend import _check, _p
        starts = self.sampler.next_starts()[self.rank * self.batch:(self.rank + 1) * self.batch]
        starts = np.ascontiguousarray(starts, np.int64)
        ids, tgt = self._ids[self._slot], self._tgt[self._slot]
        self._slot ^= 1
        _check(self._lib.ojc_gather_token_windows(self.be._handle, C.c_void_p(self._tokens.ptr), C.c_int32(self.width), C.c_uint64(self.len_tokens),
                                                  starts.ctypes.data_as(C.POINTER(C.c_int64)), C.c_int64(self.batch), C.c_int64(self.seq_len), _p(ids), _p(tgt)))
        return ids, tgt
