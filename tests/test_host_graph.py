"""The order a table's branches give its launches in a graph (backend_b200_launch_order), without a card: the grammar of
the reference's launch record (include/anemone/backend_seam.h:183-195; the walk of
source/backend_cuda_launch.c:486-632) and its refusals."""
import ctypes as C

import pytest

from anemone_b200 import api
from anemone_b200 import records as R

CHAIN, SIDE, RESUME, JOIN, MORE = range(5)


def order_of(branches):
    table = (R.KernelLaunch * len(branches))()
    for launch, branch in zip(table, branches):
        launch.branch = branch
    order = (R.LaunchOrder * len(branches))()
    C.memset(order, 0xA5, C.sizeof(order))
    status = api.library().backend_b200_launch_order(table, len(branches), order)
    if status != 0:
        assert bytes(order) == b"\xA5" * C.sizeof(order)  # a refusal writes nothing
        return status
    return [list(entry.behind[:entry.behind_count]) for entry in order]


def test_chain_and_fork_join():
    assert order_of([CHAIN, CHAIN, CHAIN]) == [[], [0], [1]]
    # a side run of two behind launch 0, the main run resumes behind 0, the join takes both ends
    assert order_of([CHAIN, SIDE, SIDE, RESUME, CHAIN, JOIN]) == [[], [0], [1], [0], [3], [2, 4]]
    # copies to three peers at once: three side runs of one launch each
    assert order_of([CHAIN, SIDE, MORE, MORE, RESUME, JOIN]) == [[], [0], [0], [0], [0], [1, 2, 3, 4]]
    # four runs is the most; a join right behind a side run names that run once
    assert order_of([CHAIN, SIDE, MORE, MORE, MORE, JOIN]) == [[], [0], [0], [0], [0], [1, 2, 3, 4]]
    assert order_of([CHAIN, SIDE, SIDE, JOIN, CHAIN]) == [[], [0], [1], [2], [3]]
    # a side run at the head forks at the graph's root
    assert order_of([SIDE, RESUME, JOIN]) == [[], [], [0, 1]]
    assert order_of([SIDE, MORE, RESUME, CHAIN, JOIN, CHAIN]) == [[], [], [], [2], [0, 1, 3], [4]]
    # a second fork after a join
    assert order_of([CHAIN, SIDE, RESUME, JOIN, SIDE, RESUME, JOIN]) == [[], [0], [0], [1, 2], [3], [3], [4, 5]]


@pytest.mark.parametrize("branches", [[CHAIN, SIDE, MORE, SIDE], [CHAIN, MORE], [CHAIN, RESUME], [CHAIN, JOIN],
                                      [CHAIN, SIDE, MORE, MORE, MORE, MORE], [CHAIN, SIDE, JOIN, JOIN], [CHAIN, 5],
                                      [CHAIN, SIDE, RESUME, RESUME]])
def test_tables_outside_the_grammar(branches):
    assert order_of(branches) == R.STATUS_INVALID_ARGUMENT


def test_a_launch_that_may_overlap_the_one_before_it_is_a_chain_launch():
    overlap = 0x100  # LAUNCH_OVERLAPS_PREVIOUS
    assert order_of([CHAIN, CHAIN | overlap, CHAIN | overlap]) == [[], [0], [1]]
    assert order_of([CHAIN, SIDE, RESUME | overlap]) == R.STATUS_INVALID_ARGUMENT  # the bit goes with CHAIN alone
    assert order_of([CHAIN | overlap, SIDE, RESUME, JOIN]) == [[], [0], [0], [1, 2]]


def test_null_and_empty():
    lib = api.library()
    table, order = (R.KernelLaunch * 1)(), (R.LaunchOrder * 1)()
    assert lib.backend_b200_launch_order(None, 1, order) == R.STATUS_INVALID_ARGUMENT
    assert lib.backend_b200_launch_order(table, 0, order) == R.STATUS_INVALID_ARGUMENT
    assert lib.backend_b200_launch_order(table, 1, None) == R.STATUS_INVALID_ARGUMENT
