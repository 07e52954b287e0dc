"""The output-axis exchanges on one card, through the C-ABI, against the CPU oracle. One rank of the group is real; what
the other ranks would have stored into its bank by now (their packs, their flags, their packets) is written by the
host from the oracle, and their banks are further ranges of the same arena, so that what the real rank stores for them
can be read back (kernels that wait on one another never share a GPU). Bit for bit: the work is integer and bfloat16."""
import numpy as np
import pytest

from anemone_b200 import records as R
from anemone_b200.ring import RingExchange, RingLayout
from oracle.binding import pointer_array, ptr, u16p, u32p

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from anemone_b200 import api as module
    assert module.card_count() >= 1, "no CUDA device: the CUDA path cannot run and there is no fallback"
    return module


def values_for(rng, ranks, packs, kind):
    """bfloat16 bits with zeros of both signs, an infinity and a far exponent here and there"""
    count = ranks * packs * 8
    spread = 40 if kind == "wide" else 9
    inputs = []
    for _ in range(ranks):
        x = (rng.integers(0, 128, count) | rng.integers(0, 2, count) << 15 |
             (120 - rng.integers(0, spread, count)) << 7).astype(np.uint16)
        x[::17], x[1::17], x[5::131] = 0, 0x8000, 0x0003
        inputs.append(x)
    inputs[0][2::4099] = 0x7F80
    return inputs


def expected_for(oracle, kind, mode, inputs, ranks, packs, vectors):
    if mode == R.EXACT_RING_GATHER:
        out = np.zeros_like(inputs[0])
        oracle.orc_ring_gather(pointer_array(inputs, u16p), ranks, packs, vectors, ptr(out, u16p))
        return [out] * ranks
    if kind == "round_once":
        out = np.zeros_like(inputs[0])
        oracle.orc_ring_round_once(pointer_array(inputs, u16p), ranks, out.size, ptr(out, u16p))
        return [out] * ranks
    outputs = [np.zeros_like(inputs[0]) for _ in range(ranks)]
    oracle.orc_ring_bf16_sum(pointer_array(inputs, u16p), ranks, packs, vectors if mode == 2 else 0,
                             pointer_array(outputs, u16p))
    return outputs


def part(values, ranks, packs, row_packs, owner):
    """owner's packs of a plane of [ranks * packs] packs, in pack order, as [packs][8]"""
    table = values.reshape(-1, 8)
    if row_packs == 0:
        return table[owner * packs:(owner + 1) * packs]
    return table.reshape(packs // row_packs, ranks, row_packs, 8)[:, owner].reshape(packs, 8)


def encode(oracle, group_values):
    packet = np.zeros(136, dtype=np.uint32)
    oracle.orc_ring_packet_encode(ptr(np.ascontiguousarray(group_values).reshape(-1), u16p), ptr(packet, u32p))
    return packet


def decode(oracle, packet):
    values = np.zeros(256, dtype=np.uint16)
    oracle.orc_ring_packet_decode(ptr(np.ascontiguousarray(packet), u32p), ptr(values, u16p))
    return values.reshape(32, 8)


class Emulated:
    def __init__(self, api, kind, mode, rank, ranks, packs, vectors, blocks=0, deadline=2_000_000_000):
        self.kind, self.mode, self.rank, self.ranks, self.packs, self.vectors = kind, mode, rank, ranks, packs, vectors
        self.layout = L = RingLayout(kind, mode, ranks, packs)
        self.banks = [L.bank if peer == rank else L.arena_bytes + peer * api.align(L.bank_bytes, 256)
                      for peer in range(ranks)]
        self.card = api.Card(0, L.arena_bytes + ranks * api.align(L.bank_bytes, 256) + 4096)
        self.exchange = RingExchange(self.card, kind, mode, rank, ranks, packs, vectors, blocks, layout=L,
                                     deadline_cycles=deadline)
        peers = (R.OrderedPeer * ranks)()
        for peer in range(ranks):
            peers[peer].region_offset = self.banks[peer]
            self.card.fill(self.banks[peer], 0, L.bank_bytes)
        self.card.upload(L.peer_table, np.frombuffer(bytes(peers), dtype=np.uint8))
        for peer in range(ranks):
            self.card.peer_connect(self.card, 0, L.peer_table + 32 * peer)
        self.planes = 1 if mode == R.EXACT_RING_GATHER else 2
        self.row_packs = packs // vectors if (vectors and mode != R.EXACT_RING_BF16_SUM) else 0

    def plane(self, bank, plane, source):
        return bank + 128 + ((plane * self.ranks + source) * self.packs) * 16

    def flags(self, bank, phase, source):
        return bank + 128 + self.planes * self.ranks * self.packs * 16 + ((phase * self.ranks + source) * 16) * 4

    def packet(self, bank, slot, group):
        return bank + 128 + (slot * (self.packs // 32) + group) * 544

    def peers_plain(self, inputs, expected, generation):
        mine, row_packs = self.banks[self.rank], self.row_packs
        for source in range(self.ranks):
            if source == self.rank:
                continue
            if self.mode == R.EXACT_RING_GATHER:
                sent = part(inputs[source], self.ranks, self.packs, 0, source)
            else:
                sent = part(inputs[source], self.ranks, self.packs, row_packs, self.rank)
                result = part(expected[self.rank], self.ranks, self.packs, row_packs, source)
                self.card.upload(self.plane(mine, 1, source), np.ascontiguousarray(result))
            self.card.upload(self.plane(mine, 0, source), np.ascontiguousarray(sent))
            for phase in (0, 1):
                self.card.upload(self.flags(mine, phase, source), np.full(16, generation, dtype=np.uint32))

    def peers_coded(self, oracle, inputs, expected, generation):
        mine, ranks = self.banks[self.rank], self.ranks
        for slot in range(2 * (ranks - 1)):
            sender = (self.rank + 1 + slot % (ranks - 1)) % ranks
            if slot < ranks - 1:
                sent = part(inputs[sender], ranks, self.packs, self.row_packs, self.rank)
            else:
                sent = part(expected[self.rank], ranks, self.packs, self.row_packs, sender)
            for group in range(self.packs // 32):
                packet = encode(oracle, sent[32 * group:32 * group + 32])
                packet[R.COMPRESSED_RING_READY_WORD] = generation
                packet[R.COMPRESSED_RING_ACK_WORD] = generation - 1  # the receiver took the call before
                self.card.upload(self.packet(mine, slot, group), packet)

    def close(self):
        self.card.close()


CASES = [("exact", 0, 1, 4, 64, 0), ("exact", 0, 2, 4, 96, 4), ("exact", 1, 0, 4, 96, 0), ("exact", 2, 3, 4, 128, 4),
         ("exact", 1, 1, 2, 64, 0), ("exact", 1, 5, 8, 64, 0), ("exact", 0, 7, 8, 32, 2),
         ("round_once", 1, 2, 4, 96, 0), ("round_once", 2, 0, 4, 64, 2), ("round_once", 1, 6, 8, 64, 0),
         ("round_once", 1, 0, 2, 32, 0)]


@pytest.mark.parametrize("kind,mode,rank,ranks,packs,vectors", CASES)
def test_plain_exchanges(api, oracle, kind, mode, rank, ranks, packs, vectors):
    world = Emulated(api, kind, mode, rank, ranks, packs, vectors)
    try:
        rng = np.random.default_rng(hash((kind, mode, rank, ranks)) & 0xFFFF)
        for generation in (1, 2, 3):
            inputs = values_for(rng, ranks, packs, "near")
            expected = expected_for(oracle, kind, mode, inputs, ranks, packs, vectors)
            world.peers_plain(inputs, expected, generation)
            world.exchange.load(inputs[rank])
            world.card.fill(world.layout.output, 0xEE, world.layout.plane_bytes)
            world.exchange.run()
            world.card.wait()
            assert np.array_equal(world.exchange.result(), expected[rank])
            for peer in range(ranks):
                if peer == rank:
                    continue
                bank = world.banks[peer]
                got = world.card.download(world.plane(bank, 0, rank), packs * 16, np.uint16).reshape(packs, 8)
                if mode == R.EXACT_RING_GATHER:
                    assert np.array_equal(got, part(inputs[rank], ranks, packs, 0, rank))
                else:
                    assert np.array_equal(got, part(inputs[rank], ranks, packs, world.row_packs, peer))
                    got = world.card.download(world.plane(bank, 1, rank), packs * 16, np.uint16).reshape(packs, 8)
                    assert np.array_equal(got, part(expected[peer], ranks, packs, world.row_packs, rank))
                for phase in (0, 1):
                    assert (world.card.download(world.flags(bank, phase, rank), 64, np.uint32) == generation).all()
    finally:
        world.close()


@pytest.mark.parametrize("mode,rank,ranks,packs,vectors,kind", [(1, 0, 4, 96, 0, "near"), (2, 2, 4, 128, 4, "wide"),
                                                                 (1, 1, 2, 64, 0, "wide"), (1, 4, 8, 64, 0, "near")])
def test_compressed_exchange(api, oracle, mode, rank, ranks, packs, vectors, kind):
    world = Emulated(api, "compressed", mode, rank, ranks, packs, vectors)
    try:
        rng = np.random.default_rng(77 + rank)
        for generation in (1, 2):
            inputs = values_for(rng, ranks, packs, kind)
            expected = expected_for(oracle, "compressed", mode, inputs, ranks, packs, vectors)
            world.peers_coded(oracle, inputs, expected, generation)
            world.exchange.load(inputs[rank])
            world.card.fill(world.layout.output, 0xEE, world.layout.plane_bytes)
            world.exchange.run()
            world.card.wait()
            assert np.array_equal(world.exchange.result(), expected[rank])
            coded = 0
            for away in range(1, ranks):  # what this rank put on the wire: its packs, then its part's sum
                peer = (rank - away) % ranks
                for slot, sent in ((away - 1, part(inputs[rank], ranks, packs, world.row_packs, peer)),
                                   (ranks - 2 + away, part(expected[peer], ranks, packs, world.row_packs, rank))):
                    for group in range(packs // 32):
                        packet = world.card.download(world.packet(world.banks[peer], slot, group), 544, np.uint32)
                        assert packet[R.COMPRESSED_RING_READY_WORD] == generation
                        assert np.array_equal(decode(oracle, packet), sent[32 * group:32 * group + 32])
                        want = encode(oracle, sent[32 * group:32 * group + 32])
                        used = 4 + 96 + bin(int(want[1])).count("1")
                        assert np.array_equal(packet[:used], want[:used])  # the same words on the wire
                        coded += 32 - bin(int(want[1])).count("1")
            assert coded > 0 or kind == "wide"  # near exponents: most lanes travel as three words
            for slot in range(2 * (ranks - 1)):  # and it told every sender that its packet was taken
                sender = (rank + 1 + slot % (ranks - 1)) % ranks
                for group in range(packs // 32):
                    word = world.packet(world.banks[sender], slot, group) + 4 * R.COMPRESSED_RING_ACK_WORD
                    assert int(world.card.download(word, 4, np.uint32)[0]) == generation
    finally:
        world.close()


@pytest.mark.parametrize("kind", ["exact", "compressed", "round_once"])
def test_a_wait_that_runs_out_sets_the_status(api, oracle, kind):
    """No peer ever answers: the kernel gives up after its deadline, says so in the bank and returns; the bank is then
    refused until the host clears it."""
    world = Emulated(api, kind, 1, 0, 4, 64, 0, deadline=2_000_000)
    try:
        world.exchange.load(values_for(np.random.default_rng(1), 4, 64, "near")[0])
        world.exchange.run()
        world.card.wait()
        assert world.exchange.status() == 1
        with pytest.raises(RuntimeError):
            world.exchange.result()
        world.exchange.run()  # returns at once
        world.card.wait()
        assert world.exchange.status() == 1
    finally:
        world.close()
