"""Flint token files and the batches a data-parallel training job draws from them.

The file format is the one the reference's data preparation writes
(``scripts/fineweb.py:27-37`` states it, ``:251-308`` writes and checks it): a
64-byte little-endian header -- magic ``FLINTTOK``, uint32 version 1, uint32
tokenizer id 1 (tiktoken "gpt2", 50,257 tokens), uint64 token count, 40 zero
bytes -- followed by the tokens as uint16 with no padding, so a file is exactly
``64 + 2 * count`` bytes. ``read_token_file`` applies the reference's checks in
its order and with its messages; ``write_token_file`` produces byte-identical
files, atomically.

``TokenBatches`` turns a list of such shards into the (tokens, targets) pairs
``flint_gpt2_forward`` takes: uint16 arrays of ``sequences x length``, the
targets being the tokens one position later. The walk over a shard is the one
llm.c-style loaders use (and the reference's shards are cut for,
``scripts/fineweb.py:39-50``): rank r of w starts at r * sequences * length,
every step advances all ranks by w * sequences * length, and a shard is left
when it cannot give every rank a full batch plus the one extra token the last
target needs. The position is plain data (``state()`` / ``restore()``), so a
checkpoint can resume the stream exactly.
"""

import hashlib
import os
import struct
from pathlib import Path

import numpy as np

MAGIC = b"FLINTTOK"
FORMAT_VERSION = 1
TOKENIZER_ID = 1   # tiktoken "gpt2"
HEADER_BYTES = 64
_FIELDS = struct.Struct("<8s2IQ")  # magic, version, tokenizer id, token count
_WRITE_BYTES = 16 << 20


class TokenFileError(ValueError):
    """A token file whose header, size or contents are not what the format says."""


def _replace_atomically(path: Path, fill):
    """fill(file) writes a temporary neighbour of path, which then takes path's place; if
    anything fails, neither file is left."""
    scratch = path.parent / (path.name + ".tmp")
    try:
        with open(scratch, "wb") as out:
            result = fill(out)
            out.flush()
            os.fsync(out.fileno())
        os.replace(scratch, path)
        return result
    except BaseException:
        scratch.unlink(missing_ok=True)
        raise


def _as_uint16(tokens) -> np.ndarray:
    values = np.asarray(tokens).reshape(-1)
    if values.dtype == np.uint16:
        return np.ascontiguousarray(values, dtype="<u2")
    if values.size and not (0 <= int(values.min()) and int(values.max()) <= 0xFFFF):
        raise ValueError("a token doesn't fit in uint16")
    return np.ascontiguousarray(values.astype(np.uint16), dtype="<u2")


def write_token_file(path, tokens) -> str:
    """Writes tokens (values that fit uint16) as a token file and returns the sha256 of
    the whole file."""
    values = _as_uint16(tokens)
    header = bytearray(HEADER_BYTES)
    _FIELDS.pack_into(header, 0, MAGIC, FORMAT_VERSION, TOKENIZER_ID, values.size)
    payload = values.view(np.uint8)

    def fill(out):
        sha = hashlib.sha256()
        for piece in [bytes(header)] + [payload[at:at + _WRITE_BYTES]
                                        for at in range(0, payload.size, _WRITE_BYTES)]:
            sha.update(piece)
            out.write(piece)
        return sha.hexdigest()

    return _replace_atomically(Path(path), fill)


def parse_header(header: bytes, file_size: int) -> int:
    """The token count a 64-byte header states. Raises TokenFileError, checking in the
    reference's order: length, magic, version, tokenizer id, reserved bytes, file size."""
    if len(header) < HEADER_BYTES:
        raise TokenFileError("token file is shorter than its header")
    magic, version, tokenizer, count = _FIELDS.unpack_from(header)
    expected_size = HEADER_BYTES + 2 * count
    problems = (
        (magic != MAGIC, "token file has the wrong magic"),
        (version != FORMAT_VERSION, f"token file version {version} isn't {FORMAT_VERSION}"),
        (tokenizer != TOKENIZER_ID, f"token file tokenizer id {tokenizer} isn't {TOKENIZER_ID}"),
        (bytes(header[_FIELDS.size:HEADER_BYTES]).strip(b"\0") != b"",
         "token file header's reserved bytes aren't zero"),
        (file_size != expected_size,
         f"token file is {file_size} bytes, but {count} tokens need {expected_size}"),
    )
    for wrong, message in problems:
        if wrong:
            raise TokenFileError(message)
    return count


def read_token_count(path) -> int:
    with open(path, "rb") as f:
        return parse_header(f.read(HEADER_BYTES), os.fstat(f.fileno()).st_size)


def read_token_file(path):
    """The tokens of a token file as a read-only uint16 array (a memory map unless the
    file is empty), after the header and size checks."""
    count = read_token_count(path)
    if count:
        return np.memmap(path, dtype="<u2", mode="r", offset=HEADER_BYTES, shape=(count,))
    nothing = np.zeros(0, dtype="<u2")
    nothing.setflags(write=False)
    return nothing


class TokenBatches:
    """(tokens, targets) micro-batches for one rank of a data-parallel job, drawn from
    token-file shards in order, epoch after epoch."""

    def __init__(self, paths, sequences: int, length: int, rank: int = 0, world: int = 1,
                 vocab: int = 50257):
        if sequences <= 0 or length <= 0:
            raise ValueError("sequences and length must be positive")
        if world <= 0 or not 0 <= rank < world:
            raise ValueError(f"rank {rank} is not in a world of {world}")
        self.paths = [Path(p) for p in paths]
        if not self.paths:
            raise ValueError("no token files")
        self.sequences, self.length = sequences, length
        self.rank, self.world = rank, world
        self.vocab = vocab
        self.per_rank = sequences * length
        self.per_step = self.per_rank * world
        self.counts = [read_token_count(p) for p in self.paths]
        self.usable = [i for i, count in enumerate(self.counts) if count >= self.per_step + 1]
        if not self.usable:
            raise TokenFileError(
                f"no token file holds the {self.per_step + 1} tokens one step of {world} ranks needs")
        self.epoch = 0
        self.cursor = 0      # index into self.usable
        self.position = 0    # first token of rank 0's next batch in the current shard
        self._tokens = None
        self._open = None

    # -- the stream's position ----------------------------------------------------------------

    def state(self) -> dict:
        """The stream's position: enough to continue it in another process."""
        return {"epoch": self.epoch, "shard": self.paths[self.usable[self.cursor]].name,
                "cursor": self.cursor, "position": self.position,
                "sequences": self.sequences, "length": self.length, "world": self.world}

    def restore(self, state: dict) -> None:
        for key in ("sequences", "length", "world"):
            if state[key] != getattr(self, key):
                raise ValueError(f"the saved stream's {key} is {state[key]}, not {getattr(self, key)}")
        cursor = int(state["cursor"])
        if not 0 <= cursor < len(self.usable) or self.paths[self.usable[cursor]].name != state["shard"]:
            raise ValueError("the saved stream's shard is not in this list of token files")
        position = int(state["position"])
        if position < 0 or position % self.per_step != 0:
            raise ValueError(f"the saved stream's position {position} is not a whole step")
        self.epoch, self.cursor, self.position = int(state["epoch"]), cursor, position

    def steps_per_epoch(self) -> int:
        return sum((self.counts[i] - 1) // self.per_step for i in self.usable)

    # -- batches ------------------------------------------------------------------------------

    def _shard(self):
        index = self.usable[self.cursor]
        if self._open != index:
            self._tokens = read_token_file(self.paths[index])
            self._open = index
        return self._tokens

    def next_batch(self, tokens_out=None, targets_out=None):
        """This rank's next (tokens, targets), each uint16 of sequences x length; written
        into the given arrays (for instance views of pinned host buffers) when they are
        passed."""
        shard = self._shard()
        if self.position + self.per_step + 1 > len(shard):
            self.cursor += 1
            self.position = 0
            if self.cursor == len(self.usable):
                self.cursor = 0
                self.epoch += 1
            shard = self._shard()
        begin = self.position + self.rank * self.per_rank
        window = np.asarray(shard[begin:begin + self.per_rank + 1])
        if self.vocab and window.size and int(window.max()) >= self.vocab:
            raise TokenFileError(
                f"{self.paths[self.usable[self.cursor]].name}: a token at or above the vocabulary "
                f"size {self.vocab} near position {begin}")
        shape = (self.sequences, self.length)
        if tokens_out is None:
            tokens_out = np.empty(shape, dtype=np.uint16)
        if targets_out is None:
            targets_out = np.empty(shape, dtype=np.uint16)
        if tuple(tokens_out.shape) != shape or tuple(targets_out.shape) != shape:
            raise ValueError(f"output arrays must be {shape}")
        tokens_out[...] = window[:-1].reshape(shape)
        targets_out[...] = window[1:].reshape(shape)
        self.position += self.per_step
        return tokens_out, targets_out
