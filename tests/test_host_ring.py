"""ring_exchange_prepare and ring_exchange_bank_bytes without a GPU: the launches written, the bank sizes against the
reference's reservations for four ranks (include/anemone/exact_ring_records.h, round_once_ring_records.h,
compressed_ring_records.h), and the refusals."""
import ctypes as C

import pytest

from anemone_b200 import api
from anemone_b200 import records as R
from tests.test_host_preparers import FakeBackend

PACKS, RANKS = 96, 4
TABLE, INPUT = 0, 256
PLANE = RANKS * PACKS * 16
OUTPUT, BANK = INPUT + PLANE, INPUT + 2 * PLANE
ARENA = BANK + 128 + 2 * PLANE + 4096
INVALID = 1


def description(kind=R.RING_EXCHANGE_EXACT, mode=R.EXACT_RING_BF16_SUM, blocks=0, arena=ARENA, ranks=RANKS, **changes):
    arguments = R.ExactRing(INPUT, OUTPUT, BANK, TABLE, 0, 1_000_000, PACKS, 0, 1, mode)
    arguments.reserved_words[0] = ranks
    for name, value in changes.items():
        setattr(arguments, name, value)
    return R.RingExchangeDescription(arguments, arena, kind, blocks)


def prepare(value, fake):
    launch = R.KernelLaunch()
    status = api.library().ring_exchange_prepare(C.byref(value), C.byref(fake.table), fake.card, C.byref(launch))
    return status, launch


def test_launches():
    fake = FakeBackend()
    names = [("kernel_exact_ring", "exact_ring"), ("kernel_bf16_compressed_ring", "bf16_compressed_ring"),
             ("kernel_bf16_round_once_ring", "bf16_round_once_ring")]
    for kind, (file_name, name) in enumerate(names):
        status, launch = prepare(description(kind=kind), fake)
        assert status == 0 and fake.asked[-1] == (file_name, name, 80)
        assert tuple(launch.grid) == (16, 1, 1) and tuple(launch.block) == (256, 1, 1)
        assert launch.argument_byte_count == 80 and launch.dynamic_shared_byte_count == 0
        assert bytes(launch.argument[:80]) == bytes(description(kind=kind).arguments)
    status, launch = prepare(description(blocks=3), fake)
    assert status == 0 and launch.grid[0] == 3
    # the gather and its [vector][channels] order; in place for the sums; the reference's rank count as 0
    assert prepare(description(mode=R.EXACT_RING_GATHER, vectors=4), fake)[0] == 0
    assert prepare(description(mode=R.EXACT_RING_BF16_SUM_COLUMNS, vectors=4), fake)[0] == 0
    assert prepare(description(output_offset=INPUT), fake)[0] == 0
    assert prepare(description(ranks=0), fake)[0] == 0


def test_bank_bytes_fit_the_reference_reservations():
    bank = api.library().ring_exchange_bank_bytes
    for packs in (32, 960, 7680):
        assert bank(R.RING_EXCHANGE_ROUND_ONCE, 1, 4, packs) == 128 + 128 * packs + 512
        assert bank(R.RING_EXCHANGE_EXACT, 1, 4, packs) <= 128 + 192 * packs + 512
        assert bank(R.RING_EXCHANGE_EXACT, 0, 4, packs) <= 128 + 120 * packs
        assert bank(R.RING_EXCHANGE_COMPRESSED, 1, 4, packs) == 128 + 6 * (packs // 32) * 544
    assert bank(R.RING_EXCHANGE_EXACT, 1, 8, 64) == 128 + 2 * 8 * 64 * 16 + 2 * 8 * 16 * 4


@pytest.mark.parametrize("fault", [
    dict(ranks=3), dict(ranks=16), dict(rank=4), dict(mode=3), dict(packs_per_owner=0), dict(packs_per_owner=33),
    dict(mode=R.EXACT_RING_BF16_SUM_COLUMNS), dict(mode=R.EXACT_RING_BF16_SUM_COLUMNS, vectors=5),
    dict(mode=R.EXACT_RING_BF16_SUM, vectors=1), dict(mode=R.EXACT_RING_GATHER, vectors=5), dict(deadline_cycles=0),
    dict(kind=R.RING_EXCHANGE_COMPRESSED, mode=R.EXACT_RING_GATHER),
    dict(kind=R.RING_EXCHANGE_ROUND_ONCE, mode=R.EXACT_RING_GATHER), dict(kind=3), dict(blocks=17),
    dict(input_offset=INPUT + 8), dict(output_offset=INPUT + 16), dict(bank_offset=OUTPUT), dict(arena=ARENA - 4096 - 1),
    dict(mode=R.EXACT_RING_GATHER, output_offset=INPUT), dict(peer_table_offset=INPUT),
])
def test_refusals(fault):
    fake = FakeBackend()
    status, launch = prepare(description(**fault), fake)
    assert status == INVALID and not fake.asked
    assert launch.kernel == 0 and launch.argument_byte_count == 0  # nothing written
