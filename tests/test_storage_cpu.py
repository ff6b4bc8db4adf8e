"""The tiered store's residency logic through the C ABI with host memory standing in for device memory (no GPU needed):
budget, pins, least-recently-used eviction order, the reference's error texts (src/storage.cu:8-9), prefetch, the
pinned-host cache tier and budget reservations."""
import ctypes as C
import os
import sys
import time

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

LAYER0 = "language_model.model.layers.0."
QKV, Z, OUT = (LAYER0 + "linear_attn." + n + ".weight" for n in ("in_proj_qkv", "in_proj_z", "out_proj"))
GATE, UP = (LAYER0 + "mlp." + n + ".weight" for n in ("gate_proj", "up_proj"))
MiB = 1 << 20
# sizes in the 4-layer golden checkpoint: qkv 16 MiB, z / out 8 MiB, gate / up 24 MiB


class Store:
    def __init__(self, idx, budget):
        from insignia_b200 import _lib

        self.L = _lib.lib()
        self.h = self.L.insg_storage_open(idx.encode(), budget, 1)
        assert self.h, self.L.insg_last_error()

    def close(self):
        self.L.insg_storage_close(self.h)

    def err(self):
        return self.L.insg_last_error().decode()

    def acquire(self, name):
        p, n = C.c_void_p(), C.c_uint64()
        rc = self.L.insg_storage_acquire(self.h, name.encode(), C.byref(p), C.byref(n))
        return rc, p.value, n.value

    def release(self, name):
        return self.L.insg_storage_release(self.h, name.encode())

    def tier(self, name):
        return self.L.insg_storage_tier(self.h, name.encode())

    def stats(self):
        out = (C.c_uint64 * 6)()
        assert self.L.insg_storage_stats(self.h, out) == 0
        return dict(zip(("uploads", "upload_bytes", "evictions", "hits", "pinned_cache_hits", "prefetches"), list(out)))

    def used(self):
        return self.L.insg_storage_device_bytes(self.h)


@pytest.fixture
def store(golden_ckpt):
    s = Store(golden_ckpt[1], 60 * MiB)
    yield s
    s.close()


def test_upload_is_the_files_bytes_and_pins_hold(store, golden_ckpt):
    from insignia_b200.checkpoint_io import SafetensorsReader

    rc, p, n = store.acquire(QKV)
    assert rc == 0 and n == 8192 * 512 * 4 and store.tier(QKV) == 2
    got = np.ctypeslib.as_array((C.c_uint32 * (n // 4)).from_address(p))
    want = SafetensorsReader(golden_ckpt[0]).get(QKV).reshape(-1).view(np.uint32)
    assert np.array_equal(got, want)
    assert store.acquire(QKV)[1] == p and store.stats()["hits"] == 1  # second pin: the same copy
    assert store.used() == n
    assert store.acquire("no.such.tensor")[0] == -4 and store.err() == "tensor not found: no.such.tensor"


def test_lru_eviction_order_and_budget_errors(store):
    # 16 + 8 + 8 + 24 = 56 MiB fit the 60 MiB budget
    for name in (QKV, Z, OUT, GATE):
        assert store.acquire(name)[0] == 0
    # everything pinned: the next tensor cannot be made room for
    assert store.acquire(UP)[0] == -4 and store.err() == "device budget exhausted by pinned tensors"
    for name in (QKV, Z, OUT, GATE):
        store.release(name)
    # use order is now QKV, Z, OUT, GATE; touching QKV makes Z the oldest
    assert store.acquire(QKV)[0] == 0 and store.release(QKV) == 0
    assert store.acquire(UP)[0] == 0  # needs 24 MiB: 4 free, evicts Z (8), OUT (8) and GATE (24), not QKV
    assert [store.tier(n) for n in (QKV, Z, OUT, GATE, UP)] == [2, 0, 0, 0, 2]
    assert store.stats()["evictions"] == 3 and store.used() == 40 * MiB
    store.release(UP)


def test_single_tensor_beyond_budget(golden_ckpt):
    s = Store(golden_ckpt[1], 4 * MiB)
    try:
        assert s.acquire(QKV)[0] == -4 and s.err() == "tensor exceeds device budget"
        assert s.used() == 0
    finally:
        s.close()


def test_prefetch_then_acquire_is_a_hit(store):
    assert store.L.insg_storage_prefetch(store.h, GATE.encode()) == 1
    assert store.L.insg_storage_prefetch(store.h, b"no.such.tensor") == 0
    for _ in range(200):  # the uploader thread works in the background
        if store.tier(GATE) == 2:
            break
        time.sleep(0.01)
    assert store.tier(GATE) == 2
    st = store.stats()
    assert st["prefetches"] == 1 and st["uploads"] == 1
    assert store.acquire(GATE)[0] == 0
    assert store.stats()["hits"] == 1 and store.stats()["uploads"] == 1
    # an unpinned prefetched tensor is evictable like any other
    store.release(GATE)
    for name in (QKV, Z, OUT, UP):
        assert store.acquire(name)[0] == 0
    assert store.tier(GATE) == 0


def test_pinned_host_cache_tier(store):
    assert store.L.insg_storage_set_host_cache(store.h, 64 * MiB) == 0
    assert store.acquire(QKV)[0] == 0 and store.release(QKV) == 0
    for name in (GATE, UP):  # 16 + 24 + 24 > 60: QKV is evicted from the device and stays in pinned host memory
        assert store.acquire(name)[0] == 0
    assert store.tier(QKV) == 1
    store.release(GATE), store.release(UP)
    assert store.acquire(QKV)[0] == 0 and store.tier(QKV) == 2
    assert store.stats()["pinned_cache_hits"] == 1


def test_reservations_share_the_budget(store):
    assert store.acquire(QKV)[0] == 0 and store.release(QKV) == 0
    assert store.L.insg_storage_reserve(store.h, 50 * MiB) == 0  # evicts the unpinned tensor
    assert store.tier(QKV) == 0 and store.L.insg_storage_reserved_bytes(store.h) == 50 * MiB
    assert store.acquire(QKV)[0] == -4 and store.err() == "device budget exhausted by pinned tensors"
    assert store.L.insg_storage_reserve(store.h, 61 * MiB) == -4 and store.err() == "tensor exceeds device budget"
    assert store.L.insg_storage_unreserve(store.h, 50 * MiB) == 0
    assert store.acquire(QKV)[0] == 0
    assert store.L.insg_storage_clear(store.h) == 0 and store.used() == 0 and store.tier(QKV) == 0
