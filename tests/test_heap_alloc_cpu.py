"""The symmetric heap's range allocator: deterministic first fit with coalescing (pure Python, no GPU)."""
import pytest

from maco_b200.parallel.symm_heap import RangeAllocator


def test_bump_then_reuse_of_freed_ranges():
    a = RangeAllocator(16 * 1024, align=1024)
    x, y, z = a.alloc(1000), a.alloc(2048), a.alloc(1)
    assert (x, y, z) == (0, 1024, 3072)
    assert a.free(y) == (1024, 2048)
    assert a.alloc(1500) == 1024            # first fit into the hole
    assert a.alloc(10) == 4096              # the remaining 0-byte hole cannot serve it: bump
    assert a.free_bytes == 16 * 1024 - 5 * 1024


def test_coalescing_and_return_to_bump_region():
    a = RangeAllocator(8 * 1024, align=1024)
    blocks = [a.alloc(1024) for _ in range(4)]
    a.free(blocks[1])
    a.free(blocks[2])                        # adjacent holes merge
    assert a.holes == [(1024, 2048)]
    assert a.alloc(2048) == 1024
    a.free(blocks[3])                        # top block rejoins the bump region
    assert a.cursor == 3072 and a.holes == []
    with pytest.raises(ValueError):
        a.free(blocks[3])                    # double free
    with pytest.raises(MemoryError):
        a.alloc(6 * 1024)


def test_same_call_sequence_gives_same_offsets():
    def run():
        a = RangeAllocator(1 << 20)
        out = []
        live = []
        for i in range(50):
            live.append(a.alloc(1000 * (1 + i % 7)))
            out.append(live[-1])
            if i % 3 == 2:
                a.free(live.pop(i % len(live)))
        return out
    assert run() == run()
