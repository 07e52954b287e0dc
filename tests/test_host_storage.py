"""The EXL3 virtual pack reader (storage_exl3) and the map upload without a GPU: the cases of the reference's own test
(tests/storage_exl3_test.c:216-330: mapped data, zero holes, bounds, outputs kept on a refusal, read modes that
agree), more refusals of source/storage_exl3_linux.c:185-279, and, where the reference's reader was compiled
(oracle/_ref), the same verdicts and the same bytes on random maps."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from anemone_b200 import api, exl3_map
from anemone_b200.exl3_map import BLOCK, MapReader, StorageOperations, write_map

OK, INVALID, IO_ERROR, CORRUPT, UNSUPPORTED = 0, 1, 3, 4, 7


@pytest.fixture()
def folder(tmp_path):
    return str(tmp_path)


def source_file(folder, name, data):
    path = os.path.join(folder, name)
    with open(path, "wb") as file:
        file.write(bytes(data))
    return path


def open_status(ops, path, copies=1):
    handle = C.c_void_p(0x1234)
    paths = (C.c_char_p * copies)(*([os.fsencode(path)] * copies))
    status = ops.reader_open(paths, copies, C.byref(handle))
    if status == OK:
        ops.reader_close(handle)
    else:
        assert handle.value == 0x1234  # untouched on a refusal
    return status


def test_the_reference_case(folder):
    ops = exl3_map.storage()
    source = source_file(folder, "source", b"\x5a" * BLOCK)
    path = os.path.join(folder, "pack.exl3map")
    write_map(path, 3 * BLOCK, [source], [(BLOCK, BLOCK, 0, 1)])
    reader = MapReader(path)
    assert reader.byte_count == 3 * BLOCK
    data = reader.read(0, 3 * BLOCK)
    assert not data[:BLOCK].any() and (data[BLOCK:2 * BLOCK] == 0x5A).all() and not data[2 * BLOCK:].any()
    buffer = np.zeros(2 * BLOCK, dtype=np.uint8)
    aligned = buffer.ctypes.data + (-buffer.ctypes.data) % BLOCK
    assert ops.reader_read(reader.handle, 1, 0, aligned, BLOCK) == INVALID        # no second copy
    assert ops.reader_read(reader.handle, 0, 3 * BLOCK, aligned, BLOCK) == INVALID  # beyond the pack
    assert ops.reader_read(reader.handle, 0, 0, aligned, 0) == INVALID
    assert ops.reader_read(reader.handle, 0, 512, aligned, BLOCK) == INVALID       # off the block alignment
    assert ops.reader_read(reader.handle, 0, 0, aligned + 8, BLOCK) == INVALID
    assert ops.reader_read(reader.handle, 0, 0, None, BLOCK) == INVALID
    assert ops.reader_read(None, 0, 0, aligned, BLOCK) == INVALID
    description = exl3_map.StorageDescription()
    assert ops.reader_describe(reader.handle, None) == INVALID and ops.reader_describe(None, C.byref(description)) == INVALID
    assert ops.reader_describe(reader.handle, C.byref(description)) == OK
    assert (description.copy_count, description.block_alignment_bytes) == (1, BLOCK)
    assert description.first_inode == os.stat(path).st_ino
    reader.close()
    ops.reader_close(None)
    # a segment beyond its source, then a reserved header byte
    write_map(path, 3 * BLOCK, [source], [(BLOCK, BLOCK, BLOCK, 1)])
    assert open_status(ops, path) == CORRUPT
    write_map(path, 3 * BLOCK, [source], [(BLOCK, BLOCK, 0, 1)])
    with open(path, "r+b") as file:
        file.seek(24)
        file.write(b"\x01")
    assert open_status(ops, path) == CORRUPT


def test_for_path_and_copies(folder):
    lib = api.library()
    ops = exl3_map.storage()
    assert C.addressof(lib.storage_for_path(b"weights.exl3map").contents) == C.addressof(ops)
    for other in (b"weights.anemone", b"map", None):
        assert not lib.storage_for_path(other)
    source = source_file(folder, "s", b"\x01" * BLOCK)
    path = os.path.join(folder, "p.exl3map")
    write_map(path, BLOCK, [source], [(0, BLOCK, 0, 1)])
    assert open_status(ops, path, copies=2) == UNSUPPORTED and open_status(ops, path, copies=9) == INVALID
    handle = C.c_void_p()
    assert ops.reader_open(None, 1, C.byref(handle)) == INVALID
    assert ops.reader_open((C.c_char_p * 1)(os.fsencode(path)), 1, None) == INVALID
    assert open_status(ops, os.path.join(folder, "absent.exl3map")) == IO_ERROR


def malformed(folder):
    """(name, writer) pairs: each writes a map that must be refused, with the status it must be refused with."""
    source = source_file(folder, "src", bytes(range(256)) * 64)  # 4 blocks
    good = [(0, BLOCK, 0, 1), (2 * BLOCK, 100, 5, 1)]
    cases = {
        "bad magic": (CORRUPT, lambda p: (write_map(p, 4 * BLOCK, [source], good), patch(p, 0, b"X"))),
        "zero bytes": (CORRUPT, lambda p: write_map(p, 0, [source], good)),
        "ragged bytes": (CORRUPT, lambda p: write_map(p, 4 * BLOCK + 1, [source], good)),
        "no segment": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, [source], [])),
        "overlap": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, [source], [(0, BLOCK, 0, 1), (BLOCK - 1, 8, 0, 1)])),
        "unsorted": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, [source], [(BLOCK, 8, 0, 1), (0, 8, 0, 1)])),
        "empty segment": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, [source], [(0, 0, 0, 1)])),
        "beyond the pack": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, [source], [(3 * BLOCK, BLOCK + 1, 0, 1)])),
        "source index": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, [source], [(0, 8, 0, 2)])),
        "beyond the source": (CORRUPT, lambda p: write_map(p, 8 * BLOCK, [source], [(0, 4 * BLOCK + 1, 0, 1)])),
        "the manifest as data": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, [source], [(0, 8, 64, 0)])),
        "relative source": (CORRUPT, lambda p: write_map(p, 4 * BLOCK, ["src"], good)),
        "segment reserved": (CORRUPT, lambda p: (write_map(p, 4 * BLOCK, [source], good),
                                                 patch(p, 64 + 2 * 512 + 28, b"\x01"))),
        "named first source": (CORRUPT, lambda p: (write_map(p, 4 * BLOCK, [source], good), patch(p, 64, b"/x"))),
        "missing source": (IO_ERROR, lambda p: write_map(p, 4 * BLOCK, [os.path.join(folder, "gone")], good)),
        "a folder as source": (IO_ERROR, lambda p: write_map(p, 4 * BLOCK, [folder], good)),
        "truncated": (CORRUPT, lambda p: (write_map(p, 4 * BLOCK, [source], good), os.truncate(p, 64 + 2 * 512 + 40))),
    }
    return cases


def patch(path, offset, data):
    with open(path, "r+b") as file:
        file.seek(offset)
        file.write(data)


def test_refusals_and_the_reference_verdicts(folder):
    ops = exl3_map.storage()
    theirs = reference_storage()
    path = os.path.join(folder, "bad.exl3map")
    for name, (expected, write) in malformed(folder).items():
        write(path)
        assert open_status(ops, path) == expected, name
        if theirs is not None:
            assert open_status(theirs, path) == expected, name


def reference_storage():
    from oracle.binding import REFERENCE_SO
    if not os.path.exists(REFERENCE_SO):
        return None
    lib = C.CDLL(REFERENCE_SO)
    if not hasattr(lib, "storage_exl3"):
        return None
    lib.storage_exl3_read_mode.argtypes = [C.c_int]
    lib.storage_exl3_read_mode(exl3_map.READS_BUFFERED)
    return StorageOperations.in_dll(lib, "storage_exl3")


def random_map(folder, rng, name):
    blocks = int(rng.integers(8, 40))
    total = blocks * BLOCK
    sources, datas = [], []
    for index in range(int(rng.integers(1, 4))):
        data = rng.integers(0, 256, int(rng.integers(1, 6)) * BLOCK + int(rng.integers(0, 100)), dtype=np.uint8)
        sources.append(source_file(folder, "%s-source-%d" % (name, index), data))
        datas.append(data)
    own = rng.integers(0, 256, 3000, dtype=np.uint8)
    cuts = np.sort(rng.choice(np.arange(1, total), size=int(rng.integers(2, 14)) * 2, replace=False))
    segments, image = [], np.zeros(total, dtype=np.uint8)
    path = os.path.join(folder, name + ".exl3map")
    own_at = 64 + 512 * (1 + len(sources)) + 32 * (len(cuts) // 2)
    for begin, end in zip(cuts[::2], cuts[1::2]):
        source = int(rng.integers(0, len(sources) + 1))
        data, base = (own, own_at) if source == 0 else (datas[source - 1], 0)
        count = int(min(end - begin, data.size))
        at = int(rng.integers(0, data.size - count + 1))
        segments.append((int(begin), count, base + at, source))
        image[begin:begin + count] = data[at:at + count]
    assert write_map(path, total, sources, segments, own.tobytes()) == own_at
    return path, image


def test_random_maps_read_like_their_image_and_like_the_reference(folder):
    rng = np.random.default_rng(21)
    theirs = reference_storage()
    lib = api.library()
    for trial in range(6):
        path, image = random_map(folder, rng, "map%d" % trial)
        reader = MapReader(path)
        handle = C.c_void_p()
        if theirs is not None:
            assert theirs.reader_open((C.c_char_p * 1)(os.fsencode(path)), 1, C.byref(handle)) == OK
        for mode in range(4):
            lib.storage_exl3_read_mode(mode)
            assert np.array_equal(reader.read(0, image.size), image)
            for _ in range(12):
                first = int(rng.integers(0, image.size // BLOCK))
                count = int(rng.integers(1, image.size // BLOCK - first + 1))
                got = reader.read(first * BLOCK, count * BLOCK)
                assert np.array_equal(got, image[first * BLOCK:(first + count) * BLOCK])
                if theirs is not None and mode == 0:
                    raw = np.zeros((count + 1) * BLOCK, dtype=np.uint8)
                    shift = (-raw.ctypes.data) % BLOCK
                    assert theirs.reader_read(handle, 0, first * BLOCK, raw.ctypes.data + shift, count * BLOCK) == OK
                    assert np.array_equal(raw[shift:shift + count * BLOCK], got)
        lib.storage_exl3_read_mode(exl3_map.READS_DIRECT)
        reader.close()
        if theirs is not None:
            theirs.reader_close(handle)


def test_device_path(folder):
    lib = api.library()
    exl3_map.storage()
    small = source_file(folder, "small", b"\x01" * BLOCK)
    large = source_file(folder, "large", b"\x02" * 4 * BLOCK)
    path = os.path.join(folder, "d.exl3map")
    write_map(path, 8 * BLOCK, [small, large], [(0, BLOCK, 0, 1), (BLOCK, 3 * BLOCK, 0, 2)])
    output = C.create_string_buffer(512)
    assert lib.storage_device_path(os.fsencode(path), output) == os.fsencode(large)
    assert lib.storage_device_path(b"/some/where.bin", output) == b"/some/where.bin"
    own = bytes(5 * BLOCK)
    at = write_map(path, 8 * BLOCK, [small], [(0, BLOCK, 0, 1)], own)
    write_map(path, 8 * BLOCK, [small], [(0, BLOCK, 0, 1), (BLOCK, 4 * BLOCK, at + 32, 0)], own)
    assert lib.storage_device_path(os.fsencode(path), output) == os.fsencode(path)  # the map itself holds the most


class ArenaBackend:
    """upload_begin copies into a host array at once; upload_wait counts. Nothing else of the table is set."""

    def __init__(self, arena_bytes):
        self.arena = np.zeros(arena_bytes, dtype=np.uint8)
        self.begun, self.waited = [], []
        self.table = api.BackendOperations()
        fields = dict(api.BackendOperations._fields_)

        def begin(card, offset, source, count, ticket_out):
            self.arena[offset:offset + count] = np.ctypeslib.as_array(C.cast(source, C.POINTER(C.c_ubyte)), (count,))
            self.begun.append((offset, count))
            ticket_out[0] = len(self.begun)
            return 0

        def wait(card, ticket, limit):
            self.waited.append(ticket)
            return 0
        self.callbacks = (fields["upload_begin"](begin), fields["upload_wait"](wait))
        self.table.upload_begin, self.table.upload_wait = self.callbacks


def test_upload_through_a_fake_card(folder):
    rng = np.random.default_rng(2)
    path, image = random_map(folder, rng, "up")
    reader = MapReader(path)
    fake = ArenaBackend(1 << 20)
    raw = np.zeros(5 * BLOCK, dtype=np.uint8)
    staging = raw.ctypes.data + (-raw.ctypes.data) % BLOCK
    lib = api.library()
    ops, card = C.byref(reader.ops), C.c_void_p(0x10)
    count = image.size - 3 * BLOCK - 77  # a ragged tail
    assert lib.exl3_map_upload(ops, reader.handle, 2 * BLOCK, count, C.byref(fake.table), card, 4096, staging, 4 * BLOCK,
                               10 ** 9) == OK
    assert np.array_equal(fake.arena[4096:4096 + count], image[2 * BLOCK:2 * BLOCK + count])
    assert not fake.arena[4096 + count:].any() and not fake.arena[:4096].any()
    assert sum(c for _, c in fake.begun) == count and all(c <= 2 * BLOCK for _, c in fake.begun)
    assert sorted(fake.waited) == list(range(1, len(fake.begun) + 1))  # every upload waited for, once
    for bad in (dict(offset=BLOCK + 1), dict(count=0), dict(count=image.size), dict(staging_bytes=BLOCK),
                dict(staging=staging + 8)):
        arguments = dict(offset=2 * BLOCK, count=count, staging=staging, staging_bytes=4 * BLOCK)
        arguments.update(bad)
        assert lib.exl3_map_upload(ops, reader.handle, arguments["offset"], arguments["count"], C.byref(fake.table), card,
                                   4096, arguments["staging"], arguments["staging_bytes"], 10 ** 9) == INVALID
    reader.close()
