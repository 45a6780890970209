"""The block cache of ``qutai_b200.storage`` on a fake allocator (no GPU): released blocks are reused by size, and over
the limit the blocks that have waited longest are the ones given back to the device."""
import ctypes

import pytest

from qutai_b200 import lib, storage


class FakeDevice:
    def __init__(self):
        self.next, self.live, self.freed = 0x1000, set(), []

    def qmoe_free(self, address):
        self.live.discard(address)
        self.freed.append(address)
        return 0

    def malloc(self, out, size):
        address = self.next
        self.next += 1 << 32
        self.live.add(address)
        ctypes.cast(out, ctypes.POINTER(ctypes.c_uint64))[0] = address


@pytest.fixture
def fake(monkeypatch):
    device = FakeDevice()
    monkeypatch.setattr(lib, "load", lambda: device)
    monkeypatch.setattr(lib, "call", lambda name, *args: device.malloc(*args) if name == "qmoe_malloc" else None)
    monkeypatch.setattr(storage, "_cache", {})
    monkeypatch.setattr(storage, "_cached_bytes", 0)
    monkeypatch.setattr(storage, "CACHE_LIMIT_BYTES", 3 << 20)
    return device


def test_released_blocks_are_reused_by_size(fake):
    a = storage.DeviceStorage(1 << 18, "float32")            # 1 MiB
    address = a.ptr
    del a
    assert storage._cached_bytes == 1 << 20 and not fake.freed
    b = storage.DeviceStorage(1 << 18, "float32")
    assert b.ptr == address and storage._cached_bytes == 0
    c = storage.DeviceStorage(1 << 17, "float32")            # another size: a new block
    assert c.ptr != address


def test_over_the_limit_the_oldest_blocks_go_first(fake):
    blocks = [storage.DeviceStorage(1 << 18, "float32") for _ in range(3)]      # 3 x 1 MiB
    addresses = [b.ptr for b in blocks]
    small = storage.DeviceStorage(1 << 16, "float32")                           # 256 KiB
    del blocks[0], blocks[0], blocks[0]
    assert storage._cached_bytes == 3 << 20 and not fake.freed
    kept = small.ptr
    del small                                                                   # does not fit: the oldest MiB block leaves
    assert fake.freed == [addresses[0]]
    assert storage._cached_bytes == (2 << 20) + (1 << 18)
    again = storage.DeviceStorage(1 << 16, "float32")                           # the block just released is still there
    assert again.ptr == kept


def test_a_block_larger_than_the_limit_is_not_kept(fake):
    big = storage.DeviceStorage(1 << 20, "float32")                             # 4 MiB > 3 MiB
    address = big.ptr
    del big
    assert fake.freed == [address] and storage._cached_bytes == 0
