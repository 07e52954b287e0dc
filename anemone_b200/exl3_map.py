"""The read-only EXL3 virtual pack (".exl3map"), host side: writing a map over source files, reading through the
C-ABI's storage table (storage_exl3) and loading a run of its logical bytes into a card's arena (exl3_map_upload).
The file format is the reference's (source/storage_exl3_linux.c:27-40; its converter tools/convert/make_virtual_pack.py
writes the same header, path table and segments)."""
import ctypes as C
import os
import struct

import numpy as np

from . import api

BLOCK, PATH_BYTES, HEADER_BYTES, SEGMENT_BYTES = 4096, 512, 64, 32
MAGIC = b"ANEXL3\0\0"
READS_BUFFERED, READS_DROPPED, READS_DIRECT, READS_DIRECT_DROPPED = range(4)


class StorageDescription(C.Structure):
    _fields_ = [("byte_count", C.c_uint64), ("copy_count", C.c_uint32), ("block_alignment_bytes", C.c_uint32),
                ("first_device", C.c_uint64), ("first_inode", C.c_uint64)]


_status = C.c_int
_reader = C.c_void_p


class StorageOperations(C.Structure):
    _fields_ = [("name", C.c_char_p),
                ("reader_open", C.CFUNCTYPE(_status, C.POINTER(C.c_char_p), C.c_uint32, C.POINTER(_reader))),
                ("reader_close", C.CFUNCTYPE(None, _reader)),
                ("reader_describe", C.CFUNCTYPE(_status, _reader, C.POINTER(StorageDescription))),
                ("reader_read", C.CFUNCTYPE(_status, _reader, C.c_uint32, C.c_uint64, C.c_void_p, C.c_uint64))]


def storage():
    lib = api.library()
    lib.storage_for_path.restype = C.POINTER(StorageOperations)
    lib.storage_for_path.argtypes = [C.c_char_p]
    lib.storage_exl3_read_mode.restype = None
    lib.storage_exl3_read_mode.argtypes = [C.c_int]
    lib.storage_device_path.restype = C.c_char_p
    lib.storage_device_path.argtypes = [C.c_char_p, C.c_char_p]
    lib.exl3_map_upload.argtypes = [C.POINTER(StorageOperations), _reader, C.c_uint64, C.c_uint64,
                                    C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64,
                                    C.c_uint64]
    return StorageOperations.in_dll(lib, "storage_exl3")


def write_map(path, byte_count, sources, segments, own_data=b""):
    """sources: absolute paths of sources 1..; segments: (logical offset, byte count, source offset, source index),
    sorted and disjoint; own_data: bytes kept in the map file itself behind the manifest (source 0), whose source
    offsets count from the start of the file. Returns the offset at which own_data begins."""
    header = MAGIC + struct.pack("<QII", byte_count, 1 + len(sources), len(segments)) + bytes(40)
    table = bytes(PATH_BYTES) + b"".join(os.fsencode(p).ljust(PATH_BYTES, b"\0") for p in sources)
    body = b"".join(struct.pack("<QQQII", *segment, 0) for segment in segments)
    with open(path, "wb") as file:
        file.write(header + table + body + own_data)
    return len(header) + len(table) + len(body)


class MapReader:
    def __init__(self, path):
        self.ops = storage()
        self.handle = _reader()
        paths = (C.c_char_p * 1)(os.fsencode(path))
        api.check(self.ops.reader_open(paths, 1, C.byref(self.handle)), "reader_open")
        description = StorageDescription()
        api.check(self.ops.reader_describe(self.handle, C.byref(description)), "reader_describe")
        self.byte_count = description.byte_count

    def close(self):
        if self.handle:
            self.ops.reader_close(self.handle)
            self.handle = _reader()

    def read(self, offset, byte_count):
        """Whole blocks into a block-aligned buffer (a copy is returned)."""
        raw = np.zeros(byte_count + BLOCK, dtype=np.uint8)
        shift = (-raw.ctypes.data) % BLOCK
        view = raw[shift:shift + byte_count]
        api.check(self.ops.reader_read(self.handle, 0, offset, view.ctypes.data, byte_count), "reader_read")
        return view.copy()

    def upload(self, card, pack_offset, byte_count, arena_offset, staging_bytes=8 << 20, wait_ns=60_000_000_000):
        """byte_count logical bytes from pack_offset into the card's arena at arena_offset, through the card's
        page-locked staging (its first staging_bytes bytes)."""
        api.check(api.library().exl3_map_upload(C.byref(self.ops), self.handle, pack_offset, byte_count,
                                                card.ops_pointer, card.handle, arena_offset, card.staging,
                                                staging_bytes, wait_ns), "exl3_map_upload")
