"""The reference's own EXL3 kernels on the card: its retained and fast kernel files, compiled for sm_100a from its
sources by oracle/Makefile into oracle/_ref, registered with the library's backend under names of their own, and
launched through the reference's own preparers (oracle/_ref/libanemone_ref.so). Test infrastructure: the GPU checker of
the card tests and the "reference kernels on the same card" baseline of bench.py; never a product path."""
import ctypes as C
import os

from anemone_b200 import api
from anemone_b200 import records as R

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = {"kernel_exl3": "reference_kernel_exl3", "kernel_exl3_wide": "reference_kernel_exl3_wide"}
_registered = False


def available():
    return all(os.path.exists(os.path.join(HERE, "_ref", name + ".cubin")) for name in FILES) and \
        os.path.exists(os.path.join(HERE, "_ref", "libanemone_ref.so"))


def register():
    global _registered
    if not _registered:
        for name, registered_name in FILES.items():
            with open(os.path.join(HERE, "_ref", name + ".cubin"), "rb") as handle:
                api.image_register(registered_name, handle.read())
        _registered = True


class RenamingBackend:
    """The library's backend table with one change: a kernel file the reference's preparers name is looked up under
    the name its image was registered with."""

    def __init__(self):
        register()
        real = api.operations().contents
        self.table = api.BackendOperations()
        C.memmove(C.byref(self.table), C.byref(real), C.sizeof(real))
        prototype = dict(api.BackendOperations._fields_)["kernel_prepare"]

        def prepare(card, file_name, function_name, argument_bytes, kernel_out):
            renamed = FILES.get(file_name.decode(), file_name.decode()).encode()
            return real.kernel_prepare(card, renamed, function_name, argument_bytes, kernel_out)
        self.callback = prototype(prepare)
        self.table.kernel_prepare = self.callback


def chain_launches(reference, backend, card, record, arena_bytes, fast):
    """The five launches of the reference's chain for class 80 (retained products) or its fast form."""
    launches = (R.KernelLaunch * 5)()
    function = reference.exl3_experts_fast_prepare if fast else reference.exl3_experts_prepare
    function.argtypes = [C.POINTER(R.Exl3Expert), C.c_uint64, C.POINTER(api.BackendOperations), C.c_void_p, C.c_uint32,
                         C.POINTER(R.KernelLaunch)]
    status = function(C.byref(record), arena_bytes, C.byref(backend.table), card.handle, 80, launches)
    if status != 0:
        raise RuntimeError("the reference's preparer refused: status %d" % status)
    return launches
