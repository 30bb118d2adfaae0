"""CPU-side checks of the ring library's C ABI (include/darkforest_ring.h): it loads, exports every symbol the
header declares, and its host-only schedule equals the schedule the gloo-tested Python ring uses."""
import importlib
import re

import pytest

from helpers import pkg


def _rc():
    pkg()
    return importlib.import_module("dark_forest_b200.ring_c")


def test_ring_library_exports_every_declared_symbol():
    rc = _rc()
    text = open(rc.RING_HEADER_PATH).read()
    names = re.findall(r"DF_API\s+[\w\s\*]+?\b(df_ring_\w+)\s*\(", text)
    assert len(names) >= 9
    L = rc.ring_lib()
    for n in names:
        assert n in rc.RING_PROTOTYPES, f"{n} declared in the header but not bound"
        getattr(L, n)
    assert set(rc.RING_PROTOTYPES) == set(names)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
@pytest.mark.parametrize("causal", [True, False])
def test_library_schedule_equals_the_python_schedule(world, layout, causal):
    """Same blocks per hop as dark-forest_b200/ring.py (which the gloo tests run at world 2, 4 and 8); the library
    additionally fuses two fully visible key chunks of one query chunk into a single call."""
    rc = _rc()
    ring = importlib.import_module("dark_forest_b200.ring")
    for rank in range(world):
        for hop in range(world):
            src = (rank - hop) % world
            want = set()
            for op in ring.hop_blocks(rank, src, world, layout, causal):
                want.add((op.q_slot, op.k_slot, int(op.diagonal)))
            got = set()
            for q_slot, k_slot, k_chunks, diagonal in rc.hop_blocks(rank, world, layout, causal, hop):
                assert k_chunks in (1, 2)
                assert not (diagonal and k_chunks == 2)
                for j in range(k_chunks):
                    got.add((q_slot, k_slot + j, diagonal))
            assert got == want, (world, layout, causal, rank, hop)
    assert rc.ring_lib().df_ring_hop_blocks(2, 2, 0, 1, 0, None) == -1
    # "balanced" runs the zigzag schedule
    assert rc.hop_blocks(0, 4, "balanced", True, 1) == rc.hop_blocks(0, 4, "zigzag", True, 1)
