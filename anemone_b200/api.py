"""Thin ctypes binding of libanemone_b200.so: the card table and the preparers, as the tests and the benchmark call them.

Nothing here computes: every result comes from the library's kernels on a CUDA device. Loading raises if the library
was not built (python -m anemone_b200.build); opening a card raises without a CUDA device.
"""
import ctypes as C
import os

import numpy as np

from . import records as R

HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(HERE, "lib", "libanemone_b200.so")
WAIT_NANOSECONDS = 120 * 10 ** 9

_status = C.c_int
_card = C.c_void_p


class BackendOperations(C.Structure):
    """struct backend_operations of include/anemone_b200_backend.h, member for member."""
    _fields_ = [
        ("name", C.c_char_p),
        ("card_count", C.CFUNCTYPE(_status, C.POINTER(C.c_uint32))),
        ("card_describe", C.CFUNCTYPE(_status, C.c_uint32, C.POINTER(R.CardDescription))),
        ("card_open", C.CFUNCTYPE(_status, C.c_uint32, C.c_uint64, C.POINTER(_card))),
        ("card_close", C.CFUNCTYPE(None, _card, C.c_uint64)),
        ("staging_allocate", C.CFUNCTYPE(_status, C.c_uint64, C.POINTER(C.c_void_p))),
        ("staging_free", C.CFUNCTYPE(None, C.c_void_p)),
        ("upload_begin", C.CFUNCTYPE(_status, _card, C.c_uint64, C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64))),
        ("upload_wait", C.CFUNCTYPE(_status, _card, C.c_uint64, C.c_uint64)),
        ("digest", C.c_void_p),
        ("download_begin", C.CFUNCTYPE(_status, _card, C.c_uint64, C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64))),
        ("kernel_prepare", C.CFUNCTYPE(_status, _card, C.c_char_p, C.c_char_p, C.c_uint32, C.POINTER(C.c_uint32))),
        ("launch_run", C.CFUNCTYPE(_status, _card, C.POINTER(R.KernelLaunch), C.c_uint32)),
        ("launch_wait", C.CFUNCTYPE(_status, _card, C.c_uint64)),
        ("format_supported", C.CFUNCTYPE(C.c_bool, C.c_uint32, C.c_int)),
        ("exchange_allocate", C.c_void_p),
        ("exchange_free", C.c_void_p),
        ("exchange_attach", C.c_void_p),
        ("peer_attach", C.c_void_p),
        ("graph_capture", C.CFUNCTYPE(_status, _card, C.POINTER(R.KernelLaunch), C.c_uint32, C.POINTER(C.c_uint32))),
        ("graph_run", C.CFUNCTYPE(_status, _card, C.c_uint32)),
        ("mark_record", C.CFUNCTYPE(_status, _card, C.c_uint32)),
        ("mark_follow", C.CFUNCTYPE(_status, _card, _card, C.c_uint32)),
        ("staging_retire", C.c_void_p),
        ("peer_connect", C.CFUNCTYPE(_status, _card, _card, C.c_uint64, C.c_uint64)),
        ("measure_begin", C.CFUNCTYPE(_status, _card)),
        ("measure_end", C.CFUNCTYPE(_status, _card)),
        ("measure_elapsed_us", C.CFUNCTYPE(_status, _card, C.c_uint64, C.POINTER(C.c_double))),
    ]


class StatusError(RuntimeError):
    def __init__(self, what, status):
        self.status = status
        name = R.STATUS_NAMES[status] if 0 <= status < len(R.STATUS_NAMES) else str(status)
        super().__init__("%s: %s" % (what, name))


def check(status, what):
    if status != R.STATUS_OK:
        raise StatusError(what, status)


_library = None


def library():
    """The loaded C-ABI library. Raises if it has not been built: there is no fallback."""
    global _library
    if _library is None:
        if not os.path.exists(LIBRARY):
            raise RuntimeError("libanemone_b200.so is not built: run `python -m anemone_b200.build`")
        lib = C.CDLL(LIBRARY)
        lib.backend_b200_operations.restype = C.POINTER(BackendOperations)
        lib.status_text.restype = C.c_char_p
        lib.status_text.argtypes = [C.c_int]
        lib.exl3_width_name.restype = C.c_char_p
        lib.exl3_width_name.argtypes = [C.c_uint32]
        lib.exl3_scratch_byte_count.restype = C.c_uint64
        lib.exl3_scratch_byte_count.argtypes = [C.c_uint32, C.c_uint32]
        lib.backend_b200_launch_count.restype = C.c_uint64
        lib.backend_b200_launch_count.argtypes = [_card]
        lib.backend_b200_arena_address.restype = C.c_uint64
        lib.backend_b200_arena_address.argtypes = [_card]
        lib.backend_b200_image_register.argtypes = [C.c_char_p, C.c_void_p, C.c_uint64]
        lib.backend_b200_waits_expired.argtypes = [_card, C.POINTER(C.c_uint32)]
        lib.backend_b200_fill.argtypes = [_card, C.c_uint64, C.c_ubyte, C.c_uint64]
        lib.backend_b200_step_run.argtypes = [_card, C.c_uint32, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint64,
                                              C.c_void_p, C.c_uint64]
        lib.backend_b200_step_capture.argtypes = [_card, C.POINTER(R.KernelLaunch), C.c_uint32, C.c_uint64, C.c_void_p,
                                                  C.c_uint64, C.c_uint64, C.c_void_p, C.c_uint64,
                                                  C.POINTER(C.c_uint32)]
        lib.backend_b200_graph_run_wait.argtypes = [_card, C.c_uint32]
        lib.backend_b200_ipc_export.argtypes = [_card, C.c_char_p]
        lib.backend_b200_ipc_connect.argtypes = [_card, C.c_char_p, C.c_uint64, C.c_uint64]
        lib.exl3_reconstruct_prepare.argtypes = [C.POINTER(R.Exl3Reconstruct), C.c_uint64, C.c_uint32,
                                                 C.POINTER(R.KernelLaunch)]
        for name in ("exl3_experts_prepare", "exl3_experts_fast_prepare", "exl3_experts_relaxed_prepare"):
            getattr(lib, name).argtypes = [C.POINTER(R.Exl3Expert), C.c_uint64, C.POINTER(BackendOperations), _card,
                                           C.c_uint32, C.POINTER(R.KernelLaunch)]
        lib.exl3_moe_prepare.argtypes = [C.POINTER(R.Exl3Moe), C.c_uint64, C.POINTER(BackendOperations), _card,
                                         C.POINTER(R.KernelLaunch)]
        lib.exl3_prefill_prepare.argtypes = [C.POINTER(R.Exl3Prefill), C.c_uint64, C.POINTER(BackendOperations),
                                             _card, C.POINTER(R.KernelLaunch)]
        lib.exl3_prefill_sizes.restype = None
        lib.exl3_prefill_sizes.argtypes = [C.c_uint32] * 6 + [C.POINTER(R.Exl3PrefillParts)]
        lib.exl3_moe_sizes.restype = None
        lib.exl3_moe_sizes.argtypes = [C.c_uint32] * 4 + [C.POINTER(R.Exl3MoeSizes)]
        lib.exl3_layer_sizes.restype = None
        lib.exl3_layer_sizes.argtypes = [C.c_uint32] * 4 + [C.POINTER(R.Exl3MoeSizes)]
        lib.exl3_layer_prepare.argtypes = [C.POINTER(R.Exl3LayerDescription), C.POINTER(BackendOperations), _card,
                                           C.POINTER(R.KernelLaunch)]
        lib.bb_exl3_row_sum_prepare.argtypes = [C.POINTER(R.ExpertRowSum), C.c_uint32, C.c_uint64,
                                                C.POINTER(BackendOperations), _card, C.POINTER(R.KernelLaunch)]
        lib.backend_b200_launch_order.argtypes = [C.POINTER(R.KernelLaunch), C.c_uint32, C.POINTER(R.LaunchOrder)]
        lib.ring_exchange_bank_bytes.restype = C.c_uint64
        lib.ring_exchange_bank_bytes.argtypes = [C.c_uint32] * 4
        lib.ring_exchange_prepare.argtypes = [C.POINTER(R.RingExchangeDescription), C.POINTER(BackendOperations),
                                              _card, C.POINTER(R.KernelLaunch)]
        _library = lib
    return _library


def operations():
    return library().backend_b200_operations()


def image_register(file_name, image_bytes):
    """One more kernel file for kernel_prepare: an sm_100a cubin the caller built (backend_b200_image_register)."""
    data = bytes(image_bytes)
    check(library().backend_b200_image_register(file_name.encode(), data, len(data)), "image_register")


def card_count():
    count = C.c_uint32(0)
    check(operations().contents.card_count(C.byref(count)), "card_count")
    return count.value


def moe_sizes(pair_count, job_count, input_size, inner_size):
    """Scratch sizes of the fused launches for these shapes (exl3_moe_sizes)."""
    sizes = R.Exl3MoeSizes()
    library().exl3_moe_sizes(pair_count, job_count, input_size, inner_size, C.byref(sizes))
    return sizes


def layer_sizes(pair_count, job_count, input_size, inner_size):
    """Scratch sizes of the decode step's four launches for these shapes (exl3_layer_sizes)."""
    sizes = R.Exl3MoeSizes()
    library().exl3_layer_sizes(pair_count, job_count, input_size, inner_size, C.byref(sizes))
    return sizes


def prefill_parts(row_capacity, picks, shared_count, expert_count, input_size, inner_size):
    """Workspace layout of the prefill launches for these shapes (exl3_prefill_sizes)."""
    parts = R.Exl3PrefillParts()
    library().exl3_prefill_sizes(row_capacity, picks, shared_count, expert_count, input_size, inner_size,
                                 C.byref(parts))
    return parts


def align(value, alignment):
    return (value + alignment - 1) // alignment * alignment


class Layout:
    """A bump allocator of arena offsets (the caller owns all placement, as in the reference)."""

    def __init__(self, begin=0):
        self.cursor = begin

    def take(self, byte_count, alignment=256):
        offset = align(self.cursor, alignment)
        self.cursor = offset + byte_count
        return offset


class Card:
    """One opened card: an arena, a staging block, and the table's calls with statuses turned into exceptions."""

    def __init__(self, index, arena_bytes, staging_bytes=64 << 20):
        self.ops = operations().contents
        self.ops_pointer = operations()
        self.handle = _card()
        self.arena_bytes = arena_bytes
        check(self.ops.card_open(index, arena_bytes, C.byref(self.handle)), "card_open")
        self.staging = C.c_void_p()
        self.staging_bytes = staging_bytes
        check(self.ops.staging_allocate(staging_bytes, C.byref(self.staging)), "staging_allocate")
        self.staging_view = np.ctypeslib.as_array(C.cast(self.staging, C.POINTER(C.c_ubyte)), shape=(staging_bytes,))

    def close(self):
        if self.handle:
            self.ops.card_close(self.handle, WAIT_NANOSECONDS)
            self.ops.staging_free(self.staging)
            self.handle = _card()

    # ---- transfers through the staging block ----
    def upload(self, offset, array):
        data = np.ascontiguousarray(array).reshape(-1).view(np.uint8)
        for begin in range(0, data.size, self.staging_bytes):
            chunk = data[begin:begin + self.staging_bytes]
            self.staging_view[:chunk.size] = chunk
            ticket = C.c_uint64()
            check(self.ops.upload_begin(self.handle, offset + begin, self.staging, chunk.size, C.byref(ticket)),
                  "upload_begin")
            check(self.ops.upload_wait(self.handle, ticket.value, WAIT_NANOSECONDS), "upload_wait")

    def download(self, offset, byte_count, dtype=np.uint8):
        out = np.empty(byte_count, dtype=np.uint8)
        for begin in range(0, byte_count, self.staging_bytes):
            size = min(self.staging_bytes, byte_count - begin)
            ticket = C.c_uint64()
            check(self.ops.download_begin(self.handle, offset + begin, self.staging, size, C.byref(ticket)),
                  "download_begin")
            check(self.ops.upload_wait(self.handle, ticket.value, WAIT_NANOSECONDS), "download wait")
            out[begin:begin + size] = self.staging_view[:size]
        return out.view(dtype)

    def upload_async(self, offset, staging_offset, byte_count):
        """Queue a copy of staging bytes [staging_offset, +byte_count) into the arena; returns the ticket."""
        ticket = C.c_uint64()
        check(self.ops.upload_begin(self.handle, offset, C.c_void_p(self.staging.value + staging_offset), byte_count,
                                    C.byref(ticket)), "upload_begin")
        return ticket.value

    def download_async(self, offset, staging_offset, byte_count):
        ticket = C.c_uint64()
        check(self.ops.download_begin(self.handle, offset, C.c_void_p(self.staging.value + staging_offset),
                                      byte_count, C.byref(ticket)), "download_begin")
        return ticket.value

    def transfer_wait(self, ticket):
        check(self.ops.upload_wait(self.handle, ticket, WAIT_NANOSECONDS), "upload_wait")

    def fill(self, offset, value, byte_count):
        check(library().backend_b200_fill(self.handle, offset, value, byte_count), "fill")

    # ---- kernels ----
    def kernel(self, file_name, function_name, argument_bytes):
        handle = C.c_uint32(R.BACKEND_NO_KERNEL)
        check(self.ops.kernel_prepare(self.handle, file_name.encode(), function_name.encode(), argument_bytes,
                                      C.byref(handle)), "kernel_prepare %s/%s" % (file_name, function_name))
        return handle.value

    def run(self, launches):
        table = launches if isinstance(launches, C.Array) else (R.KernelLaunch * len(launches))(*launches)
        check(self.ops.launch_run(self.handle, table, len(table)), "launch_run")

    def wait(self):
        check(self.ops.launch_wait(self.handle, WAIT_NANOSECONDS), "launch_wait")

    def graph(self, launches):
        table = launches if isinstance(launches, C.Array) else (R.KernelLaunch * len(launches))(*launches)
        graph = C.c_uint32()
        check(self.ops.graph_capture(self.handle, table, len(table), C.byref(graph)), "graph_capture")
        return graph.value

    def graph_run(self, graph):
        check(self.ops.graph_run(self.handle, graph), "graph_run")

    def step_run(self, graph, input_offset, input_staging_offset, input_bytes, output_offset, output_staging_offset,
                 output_bytes):
        """Copy in, run the graph, copy out and wait, in one call of the library (backend_b200_step_run)."""
        check(library().backend_b200_step_run(self.handle, graph, input_offset,
                                              C.c_void_p(self.staging.value + input_staging_offset), input_bytes,
                                              output_offset,
                                              C.c_void_p(self.staging.value + output_staging_offset), output_bytes),
              "step_run")

    def step_capture(self, launches, input_offset, input_staging_offset, input_bytes, output_offset,
                     output_staging_offset, output_bytes):
        """The copy in, a chain of launches and the copy out as ONE graph (backend_b200_step_capture); None if the
        table is not a plain chain. Run it with graph_run_wait."""
        table = launches if isinstance(launches, C.Array) else (R.KernelLaunch * len(launches))(*launches)
        graph = C.c_uint32()
        status = library().backend_b200_step_capture(self.handle, table, len(table), input_offset,
                                                     C.c_void_p(self.staging.value + input_staging_offset), input_bytes,
                                                     output_offset,
                                                     C.c_void_p(self.staging.value + output_staging_offset),
                                                     output_bytes, C.byref(graph))
        if status == R.STATUS_UNSUPPORTED:
            return None
        check(status, "step_capture")
        return graph.value

    def graph_run_wait(self, graph):
        check(library().backend_b200_graph_run_wait(self.handle, graph), "graph_run_wait")

    def measure_begin(self):
        check(self.ops.measure_begin(self.handle), "measure_begin")

    def measure_end(self):
        check(self.ops.measure_end(self.handle), "measure_end")

    def measure_elapsed_us(self):
        value = C.c_double()
        check(self.ops.measure_elapsed_us(self.handle, WAIT_NANOSECONDS, C.byref(value)), "measure_elapsed_us")
        return value.value

    def expired_bits(self):
        """Waits for the queue; the bits the card's kernels set when they gave up: 1 a bounded wait ran out, 2 a
        sequence was replayed, 4 a step named more rows than were prepared (push and exchange kernels)."""
        expired = C.c_uint32()
        check(library().backend_b200_waits_expired(self.handle, C.byref(expired)), "waits_expired")
        return expired.value

    def waits_expired(self):
        """Waits for the queue; True if a kernel gave up a bounded wait (its CTA then stored nothing more)."""
        return self.expired_bits() != 0

    def launch_count(self):
        return library().backend_b200_launch_count(self.handle)

    def peer_connect(self, owner, owner_offset, address_word_offset):
        check(self.ops.peer_connect(self.handle, owner.handle, owner_offset, address_word_offset), "peer_connect")

    def ipc_export(self):
        handle = C.create_string_buffer(64)
        check(library().backend_b200_ipc_export(self.handle, handle), "ipc_export")
        return handle.raw

    def ipc_connect(self, handle_bytes, owner_offset, address_word_offset):
        check(library().backend_b200_ipc_connect(self.handle, handle_bytes, owner_offset, address_word_offset),
              "ipc_connect")
