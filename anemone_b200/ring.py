"""The output-axis exchanges between the ranks of a tensor-parallel group, host side: a gather of every owner's packs,
the BF16 sum in the order the reference's ring visits the ranks (plain or with the lossless wire code), and the
round-once sum (reference: include/anemone/exact_ring_records.h:17-56, round_once_ring_records.h,
compressed_ring_records.h; the reference's model program fills these launches at source/model_v41_program.c:8445).

A RingExchange lays out one rank's ranges in its card's arena, prepares the launch through the C-ABI
(ring_exchange_prepare) and reads the bank's status word. There is no CPU path here: the kernels run on the card."""
import ctypes as C

import numpy as np

from . import api
from . import records as R

KINDS = {"exact": R.RING_EXCHANGE_EXACT, "compressed": R.RING_EXCHANGE_COMPRESSED,
         "round_once": R.RING_EXCHANGE_ROUND_ONCE}
STATUS_TEXT = {1: "a wait ran past its deadline", 2: "the generation counter is exhausted",
               3: "the record is malformed"}


def bank_bytes(kind, mode, ranks, packs_per_owner):
    return api.library().ring_exchange_bank_bytes(KINDS[kind], mode, ranks, packs_per_owner)


class RingLayout:
    """peer table | input | output | bank, the same offsets on every rank (peer_bank_delta = bank - region)."""

    def __init__(self, kind, mode, ranks, packs_per_owner, begin=0):
        layout = api.Layout(begin)
        self.peer_table = layout.take(ranks * 32)
        self.plane_bytes = ranks * packs_per_owner * R.EXACT_RING_PACK_BYTES
        self.input = layout.take(self.plane_bytes)
        self.output = layout.take(self.plane_bytes)
        self.bank_bytes = bank_bytes(kind, mode, ranks, packs_per_owner)
        self.bank = layout.take(self.bank_bytes)
        self.arena_bytes = layout.take(0, 4096) + 4096


class RingExchange:
    def __init__(self, card, kind, mode, rank, ranks, packs_per_owner, vectors=0, blocks=0, layout=None,
                 deadline_cycles=2_000_000_000, in_place=False):
        self.card, self.kind, self.mode, self.rank, self.ranks = card, kind, mode, rank, ranks
        self.packs, self.vectors = packs_per_owner, vectors
        self.layout = L = layout or RingLayout(kind, mode, ranks, packs_per_owner)
        self.arguments = R.ExactRing(L.input, L.input if in_place else L.output, L.bank, L.peer_table, 0,
                                     deadline_cycles, packs_per_owner, vectors, rank, mode)
        self.arguments.reserved_words[0] = ranks
        description = R.RingExchangeDescription(self.arguments, card.arena_bytes, KINDS[kind], blocks)
        self.launch = R.KernelLaunch()
        api.check(api.library().ring_exchange_prepare(C.byref(description), card.ops_pointer, card.handle,
                                                      C.byref(self.launch)), "ring_exchange_prepare")
        card.fill(L.bank, 0, L.bank_bytes)

    def connect_local(self, exchanges):
        """Peers in this process: every rank's arena address into this rank's table; a peer's bank is its region."""
        peers = (R.OrderedPeer * self.ranks)()
        for peer, other in enumerate(exchanges):
            peers[peer].region_offset = other.layout.bank
        self.card.upload(self.layout.peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
        for peer, other in enumerate(exchanges):
            self.card.peer_connect(other.card, 0, self.layout.peer_table + 32 * peer)

    def load(self, values):
        self.card.upload(self.layout.input, np.ascontiguousarray(values))

    def run(self):
        self.card.run([self.launch])

    def status(self):
        return int(self.card.download(self.layout.bank + R.EXACT_RING_STATUS_OFFSET, 4, np.uint32)[0])

    def result(self, dtype=np.uint16):
        status = self.status()
        if status != 0:
            raise RuntimeError("ring exchange on rank %d: %s" % (self.rank, STATUS_TEXT.get(status, status)))
        return self.card.download(self.arguments.output_offset, self.layout.plane_bytes, dtype)
