"""Sleep-mode allocator bookkeeping against a host-memory fake of the driver."""
import ctypes

import pytest

from fake_vmm_driver import FakeDriver
from omni_npu_b200.worker.mem_pool import B200MemAllocator


@pytest.fixture()
def pool():
    alloc = B200MemAllocator.get_instance()
    drv = FakeDriver()
    alloc.lib.omni_vmm_set_driver(ctypes.cast(drv.table, ctypes.c_void_p))
    yield alloc, drv
    alloc.lib.omni_vmm_set_driver(None)


def _malloc(alloc, tag, size):
    alloc.lib.omni_vmm_set_tag(tag.encode())
    p = alloc.lib.omni_vmm_malloc(size, 0, None)
    assert p
    return p


def test_sleep_offloads_tagged_and_discards_the_rest(pool):
    alloc, drv = pool
    base = alloc.stats()
    w = _malloc(alloc, "weights", 3 << 20)         # rounds up to 4 MiB
    kv = _malloc(alloc, "kv_cache", 2 << 20)
    assert alloc.get_current_usage("weights") == 4 << 20 and alloc.get_current_usage("kv_cache") == 2 << 20
    assert alloc.get_current_usage() == 6 << 20 and drv.physical_bytes() == 6 << 20
    drv.write(w, b"model weights!")
    drv.write(kv, b"old kv")
    released = alloc.sleep(offload_tags="weights")
    assert released == 6 << 20 and drv.physical_bytes() == 0 and not drv.mapped
    st = alloc.stats()
    assert st["sleeping_bytes"] == 6 << 20 and st["host_backup_bytes"] == 4 << 20 and st["mapped_bytes"] == 0
    assert set(drv.reserved) == {w, kv}                # addresses stay reserved
    # wake only the weights first, then everything
    assert alloc.wake_up(tags=["weights"]) == 4 << 20
    assert drv.read(w, 14) == b"model weights!" and kv not in drv.mapped
    assert alloc.wake_up() == 2 << 20
    assert drv.read(kv, 6) == b"\0" * 6                 # discarded content comes back empty
    st = alloc.stats()
    assert st["sleeping_bytes"] == 0 and st["host_backup_bytes"] == 0 and not drv.host
    assert st["sleeps"] == base["sleeps"] + 1
    alloc.lib.omni_vmm_free(w, 0, 0, None)
    alloc.lib.omni_vmm_free(kv, 0, 0, None)
    assert alloc.stats()["allocations"] == base["allocations"] and not drv.reserved and drv.physical_bytes() == 0


def test_free_while_asleep_and_double_sleep(pool):
    alloc, drv = pool
    a = _malloc(alloc, "default", 1 << 20)
    b = _malloc(alloc, "default", 1 << 20)
    drv.write(a, b"aaaa")
    alloc.sleep()
    assert alloc.sleep() == 0                           # nothing left to release
    alloc.lib.omni_vmm_free(b, 0, 0, None)               # freed while asleep: backup dropped, range returned
    assert b not in drv.reserved and len(drv.host) == 1
    alloc.wake_up()
    assert drv.read(a, 4) == b"aaaa"
    alloc.lib.omni_vmm_free(a, 0, 0, None)
    alloc.lib.omni_vmm_free(a, 0, 0, None)               # unknown pointer: ignored
    assert not drv.reserved and not drv.host


def test_driver_errors_are_reported(pool):
    alloc, drv = pool
    drv.fail_create = True
    alloc.lib.omni_vmm_set_tag(b"default")
    assert not alloc.lib.omni_vmm_malloc(1 << 20, 0, None)
    assert "create" in alloc.last_error() and not drv.reserved      # the reserved range was given back
    drv.fail_create = False
    p = _malloc(alloc, "default", 1 << 20)
    alloc.sleep()
    drv.fail_create = True
    with pytest.raises(RuntimeError, match="create"):
        alloc.wake_up()
    drv.fail_create = False
    alloc.wake_up()
    alloc.lib.omni_vmm_free(p, 0, 0, None)
