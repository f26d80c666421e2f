"""Checkpoint files for the trainer: named arrays plus a JSON record, in one file.

The reference has no checkpoint format of its own (its C API moves weights
through ``flint_gpt2_parameter`` + ``flint_copy`` under PyTorch's parameter
names, ``include/flint/flint.h:533-573``; its roadmap lists the long training
run that needs resuming, ``README.md:147``). This container keeps those names,
so ``read_checkpoint(path)[1]`` with the ``param/`` prefix stripped is a
PyTorch ``state_dict`` of FP32 arrays.

Layout, everything little-endian:

    bytes  0-7    magic b"FLINTCKP"
    bytes  8-11   uint32 version = 1
    bytes 12-15   uint32 length of the JSON record
    bytes 16-     the JSON record (UTF-8), zero-padded to a multiple of 64 bytes
    ...           each array's bytes at the 64-byte-aligned offset the record gives
    last 32 bytes sha256 of everything before them

The record is ``{"meta": <the caller's dict>, "arrays": [{"name", "dtype",
"shape", "offset", "nbytes"}, ...]}``. Files are written to a temporary
neighbour and renamed into place, so a killed writer never leaves a half
checkpoint under the final name.
"""

import hashlib
import json
import os
import struct
from pathlib import Path

import numpy as np

MAGIC = b"FLINTCKP"
VERSION = 1
ALIGN = 64
_PREFIX = struct.Struct("<8s2I")
_PIECE = 16 << 20


class CheckpointError(ValueError):
    """A checkpoint file that is damaged or not in this format."""


def _padded(size: int) -> int:
    return -(-size // ALIGN) * ALIGN


def _plan(meta: dict, arrays: dict):
    """The JSON record, the offset of the first array and the end of the last."""
    names = list(arrays)
    entries = [{"name": n, "dtype": arrays[n].dtype.str, "shape": list(arrays[n].shape),
                "offset": 0, "nbytes": int(arrays[n].nbytes)} for n in names]
    total = sum(_padded(e["nbytes"]) for e in entries)

    def encode(base):
        at = base
        for e in entries:
            e["offset"] = at
            at += _padded(e["nbytes"])
        return json.dumps({"meta": meta, "arrays": entries}, sort_keys=True).encode()

    # The record's length depends on the digits of the offsets it states: iterate to the
    # fixed point (lengths only grow, so this ends after a few rounds).
    base = 0
    while True:
        record = encode(base)
        needed = _padded(_PREFIX.size + len(record))
        if needed == base:
            break
        base = needed
    return record, base, base + total


def write_checkpoint(path, meta: dict, arrays: dict) -> str:
    """Writes the arrays (name -> numpy array) and the JSON-serialisable meta to path;
    returns the file's trailing sha256 as hex."""
    arrays = {name: np.ascontiguousarray(a) for name, a in arrays.items()}
    for name, a in arrays.items():
        if a.dtype.byteorder == ">" or a.dtype.hasobject:
            raise ValueError(f"{name}: arrays must be little-endian plain data")
    record, base, end = _plan(meta, arrays)
    path = Path(path)
    scratch = path.parent / (path.name + ".tmp")
    sha = hashlib.sha256()
    try:
        with open(scratch, "wb") as out:
            def put(data):
                sha.update(data)
                out.write(data)

            put(_PREFIX.pack(MAGIC, VERSION, len(record)))
            put(record)
            put(bytes(base - _PREFIX.size - len(record)))
            for a in arrays.values():
                flat = a.reshape(-1).view(np.uint8)
                for at in range(0, flat.size, _PIECE):
                    put(flat[at:at + _PIECE])
                put(bytes(_padded(flat.size) - flat.size))
            out.write(sha.digest())
            out.flush()
            os.fsync(out.fileno())
        os.replace(scratch, path)
    except BaseException:
        scratch.unlink(missing_ok=True)
        raise
    return sha.hexdigest()


def read_checkpoint(path, verify: bool = False):
    """(meta, {name: read-only array}) of a checkpoint; the arrays are memory maps into
    the file. verify=True also rereads the whole file against its sha256."""
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as f:
        prefix = f.read(_PREFIX.size)
        if len(prefix) < _PREFIX.size:
            raise CheckpointError("checkpoint is shorter than its prefix")
        magic, version, length = _PREFIX.unpack(prefix)
        if magic != MAGIC:
            raise CheckpointError("checkpoint has the wrong magic")
        if version != VERSION:
            raise CheckpointError(f"checkpoint version {version} isn't {VERSION}")
        if _PREFIX.size + length + 32 > size:
            raise CheckpointError("checkpoint is shorter than its record")
        try:
            record = json.loads(f.read(length).decode())
            meta, entries = record["meta"], record["arrays"]
        except (ValueError, KeyError, TypeError) as error:
            raise CheckpointError(f"checkpoint record can't be read: {error}") from None
        if verify:
            f.seek(0)
            sha = hashlib.sha256()
            left = size - 32
            while left > 0:
                piece = f.read(min(_PIECE, left))
                if not piece:
                    break
                sha.update(piece)
                left -= len(piece)
            if sha.digest() != f.read(32):
                raise CheckpointError("checkpoint's sha256 doesn't match its contents")
    arrays = {}
    end = _padded(_PREFIX.size + length)
    for e in entries:
        dtype = np.dtype(e["dtype"])
        shape = tuple(e["shape"])
        nbytes = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
        if nbytes != e["nbytes"] or e["offset"] % ALIGN or e["offset"] < end:
            raise CheckpointError(f"checkpoint array {e['name']} has an inconsistent entry")
        end = e["offset"] + _padded(nbytes)
        if end + 32 > size:
            raise CheckpointError(f"checkpoint is too short for array {e['name']}")
        if nbytes == 0:
            arrays[e["name"]] = np.zeros(shape, dtype=dtype)
            arrays[e["name"]].setflags(write=False)
        else:
            arrays[e["name"]] = np.memmap(path, dtype=dtype, mode="r", offset=e["offset"], shape=shape)
    if end + 32 != size:
        raise CheckpointError(f"checkpoint is {size} bytes, but its record describes {end + 32}")
    return meta, arrays
