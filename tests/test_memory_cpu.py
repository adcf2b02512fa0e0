"""Block allocator and block-table helpers behind the C ABI against the semantics the reference's own
tests pin (memory/memory_test.go:9-50 reference counting, :90-137 cover and map, :215-end grow
rollback) and against the oracle's Table.Map."""
import numpy as np
import pytest

from oracle import pyoracle as yo
from yuuka_b200 import cuda


def test_reference_counting_like_the_reference_test():
    a = cuda.Allocator(2, 4)
    first, second = a.acquire(), a.acquire()
    assert (first, second) == (0, 1)  # descending free list popped from the back: block 0 first
    with pytest.raises(cuda.YuukaError) as e:
        a.acquire()
    assert e.value.status == 4  # ErrOutOfBlocks
    a.retain(first)
    assert a.refs(first) == 2
    a.release(first)
    assert a.refs(first) == 1
    a.release(second)
    with pytest.raises(cuda.YuukaError):
        a.release(second)  # double release must fail
    a.release(first)
    st = a.stats()
    assert (st.free, st.used, st.shared, st.total, st.block_size) == (2, 0, 0, 2, 4)
    assert (st.allocated, st.released) == (2, 3)
    # a released block is the next one handed out (LIFO)
    assert a.acquire() == first
    assert a.refs(99) == 0 and a.refs(-1) == 0
    with pytest.raises(cuda.YuukaError):
        a.retain(second)  # free block
    with pytest.raises(cuda.YuukaError):
        a.release(7)      # invalid id
    a.close()
    for bad in ((0, 4), (4, 0), (-1, 16)):
        with pytest.raises(cuda.YuukaError):
            cuda.Allocator(*bad)


def test_table_cover_map_and_rollback():
    a = cuda.Allocator(6, 16)
    t = cuda.Table(a, 8)
    t.cover(0)
    assert t.blocks().size == 0
    t.cover(17)
    assert t.blocks().tolist() == [0, 1]
    t.cover(20)   # already covered
    assert t.blocks().tolist() == [0, 1]
    t.cover(33)
    assert t.blocks().tolist() == [0, 1, 2]
    assert t.map(0) == (0, 0) and t.map(16) == (1, 0) and t.map(47) == (2, 15)
    with pytest.raises(cuda.YuukaError):
        t.map(48)
    with pytest.raises(cuda.YuukaError):
        t.map(-1)
    # a second table takes the rest; growing past the pool fails and leaves table and pool unchanged
    u = cuda.Table(a, 8)
    u.cover(32)
    assert u.blocks().tolist() == [3, 4]
    free_before = a.stats().free
    with pytest.raises(cuda.YuukaError) as e:
        u.cover(16 * 4)   # needs two more blocks, one is left
    assert e.value.status == 4
    assert u.blocks().tolist() == [3, 4] and a.stats().free == free_before == 1
    # the same positions through the oracle's Table.Map
    blocks = t.blocks()
    for pos in (0, 5, 16, 31, 32, 47):
        assert t.map(pos) == tuple(yo.table_map(blocks, 16, pos))
    a.close()
