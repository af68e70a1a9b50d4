"""A host-memory stand-in for the CUDA virtual-memory driver calls, installed into
the native allocator through its driver table.  Virtual ranges are plain integers,
physical handles are bytearrays; ``map`` binds a handle to a range, copies go through
whatever handle is mapped at the address (an unmapped address is an error, as on a GPU)."""
import ctypes

ULL, SZ, CI, VP = ctypes.c_ulonglong, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p


class FakeDriver:
    GRAN = 2 << 20

    def __init__(self) -> None:
        self.next_va = 0x7000_0000_0000
        self.next_handle = 1
        self.reserved = {}      # va -> size
        self.handles = {}       # handle -> bytearray
        self.mapped = {}        # va -> handle
        self.host = {}          # addr -> ctypes buffer
        self.fail_create = False
        self.calls = []
        F = ctypes.CFUNCTYPE
        self._fns = [
            F(CI, ctypes.POINTER(ULL), SZ, SZ)(self.address_reserve),
            F(CI, ULL, SZ)(self.address_free),
            F(CI, ctypes.POINTER(ULL), SZ, CI)(self.create),
            F(CI, ULL)(self.release),
            F(CI, ULL, SZ, ULL)(self.map),
            F(CI, ULL, SZ, CI)(self.set_access_rw),
            F(CI, ULL, SZ)(self.unmap),
            F(CI, ctypes.POINTER(SZ), CI)(self.granularity),
            F(CI, ctypes.POINTER(VP), SZ)(self.host_alloc),
            F(CI, VP)(self.host_free),
            F(CI, VP, ULL, SZ)(self.copy_d2h),
            F(CI, ULL, VP, SZ)(self.copy_h2d),
            F(CI)(self.sync),
        ]
        self.table = (VP * len(self._fns))(*[ctypes.cast(f, VP) for f in self._fns])

    # --- driver entry points
    def address_reserve(self, out, size, align):
        assert size % self.GRAN == 0
        out[0] = self.next_va
        self.reserved[self.next_va] = size
        self.next_va += size + self.GRAN
        return 0

    def address_free(self, va, size):
        assert va not in self.mapped
        del self.reserved[va]
        return 0

    def create(self, out, size, device):
        if self.fail_create:
            return 2            # out of memory
        out[0] = self.next_handle
        self.handles[self.next_handle] = bytearray(size)
        self.next_handle += 1
        return 0

    def release(self, h):
        del self.handles[h]
        return 0

    def map(self, va, size, h):
        assert va in self.reserved and va not in self.mapped
        self.mapped[va] = h
        return 0

    def set_access_rw(self, va, size, device):
        return 0 if va in self.mapped else 1

    def unmap(self, va, size):
        del self.mapped[va]
        return 0

    def granularity(self, out, device):
        out[0] = self.GRAN
        return 0

    def host_alloc(self, out, size):
        buf = ctypes.create_string_buffer(size)
        addr = ctypes.addressof(buf)
        self.host[addr] = buf
        out[0] = addr
        return 0

    def host_free(self, p):
        del self.host[p]
        return 0

    def copy_d2h(self, dst, va, size):
        if va not in self.mapped:
            return 700
        ctypes.memmove(dst, bytes(self.handles[self.mapped[va]][:size]), size)
        return 0

    def copy_h2d(self, va, src, size):
        if va not in self.mapped:
            return 700
        self.handles[self.mapped[va]][:size] = ctypes.string_at(src, size)
        return 0

    def sync(self):
        return 0

    # --- helpers for tests
    def write(self, va, data: bytes):
        self.handles[self.mapped[va]][: len(data)] = data

    def read(self, va, n: int) -> bytes:
        return bytes(self.handles[self.mapped[va]][:n])

    def physical_bytes(self) -> int:
        return sum(len(b) for b in self.handles.values())
