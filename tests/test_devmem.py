"""Growable device buffers (virtual memory management), pinned staging and the threaded loader.  The logic runs against
an in-process fake of the driver API on CPU; the GPU tests use the real driver."""
import os

import pytest
import torch

from spark_engine_b200 import runtime as rt
from spark_engine_b200.utils.devmem import GrowableDeviceBuffer, load_file_range_to


def test_vmm_region_grows_and_shrinks_in_place_fake():
    L = rt.rt()
    before = L.fake_driver_mapped_bytes()
    b = GrowableDeviceBuffer(0, 10 << 20, fake=True)
    g = b.region.granularity
    assert b.size == 0 and b.region.capacity >= 10 << 20
    assert b.resize(3 * g + 1) == 4 * g
    ptr = b.region.ptr
    t = b.view(0, (4 * g // 4,), torch.int32)
    t.copy_(torch.arange(t.numel(), dtype=torch.int32))
    assert b.resize(6 * g) == 6 * g and b.region.ptr == ptr            # same address after growing
    assert torch.equal(b.view(0, (4 * g // 4,), torch.int32), torch.arange(4 * g // 4, dtype=torch.int32))
    assert b.resize(2 * g) == 2 * g
    assert L.fake_driver_mapped_bytes() - before == 2 * g
    with pytest.raises(ValueError):
        b.view(0, (3 * g,), torch.uint8)
    with pytest.raises(RuntimeError):
        b.resize(11 << 20)
    del b, t
    assert L.fake_driver_mapped_bytes() == before


def test_fast_load_through_staging_ring_fake(tmp_path):
    data = torch.randint(0, 256, (5 * 1000 * 1000 + 123,), dtype=torch.uint8)
    p = tmp_path / "blob.bin"
    p.write_bytes(b"HEAD" + data.numpy().tobytes())
    dst = torch.zeros_like(data)
    st = load_file_range_to(dst, str(p), 4, chunk=1 << 20, n_buffers=3, n_threads=3)
    assert torch.equal(dst, data) and st.bytes == data.numel() and st.copies == 5
    with pytest.raises(RuntimeError):
        load_file_range_to(torch.zeros(10, dtype=torch.uint8), str(tmp_path / "missing"), 0)
    pb = rt.rt().PinnedBuffer(100000, False, True)
    assert pb.size >= 100000 and memoryview(pb).nbytes == pb.size
    # O_DIRECT reads: unaligned offset and size, chunks that are not multiples of 4 KiB, the tail past the last aligned
    # block of the file; the bytes are the same whether or not the file system takes the flag
    for off, n, chunk in ((4, data.numel(), 1 << 20), (4099, 777777, 300001), (8192, 4096, 1 << 16), (1, data.numel() + 3, 999983)):
        dst2 = torch.zeros(n, dtype=torch.uint8)
        raw = (b"HEAD" + data.numpy().tobytes())[off: off + n]
        st2 = load_file_range_to(dst2, str(p), off, chunk=chunk, n_buffers=2, n_threads=2, direct=True)
        assert bytes(dst2.numpy().tobytes()) == raw and st2.bytes == n
        assert isinstance(st2.direct, bool)


@pytest.mark.gpu
def test_vmm_region_and_loader_on_device(tmp_path):
    assert rt.rt().cuda_driver_available()
    torch.zeros(1, device="cuda")                                        # primary context
    b = GrowableDeviceBuffer(0, 64 << 20)
    g = b.region.granularity
    b.resize(g)
    t = b.view(0, (g // 4,), torch.float32)
    t.fill_(3.0)
    ptr = b.region.ptr
    b.resize(4 * g)
    assert b.region.ptr == ptr and float(b.view(0, (g // 4,), torch.float32).sum()) == 3.0 * (g // 4)
    u = b.view(3 * g, (1024,), torch.int64)
    u.copy_(torch.arange(1024, device="cuda"))
    assert int(u.sum()) == 1023 * 1024 // 2
    b.resize(g)
    torch.cuda.synchronize()
    data = torch.randint(0, 256, (9 * 1000 * 1000 + 7,), dtype=torch.uint8)
    p = tmp_path / "w.bin"
    p.write_bytes(data.numpy().tobytes())
    dst = torch.empty_like(data, device="cuda")
    st = load_file_range_to(dst, str(p), 0, chunk=2 << 20)
    assert torch.equal(dst.cpu(), data) and st.bytes == data.numel()
    pb = rt.rt().PinnedBuffer(1 << 20, True, False)
    assert pb.registered


def _kv_backed_generation(device, fake):
    """Tiny hybrid model whose KV tensors grow on demand: leases back their rows first, tokens equal the dense model's,
    the backing follows the highest live lease up and down."""
    import torch
    from spark_engine_b200.cache.kv import KvBacking, KvManager
    from spark_engine_b200.config import tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights, to_device
    cfg = tiny_hybrid()
    cfg.mtp_layers = 0
    W = init_weights(cfg, seed=0)
    dt = torch.float32 if device == "cpu" else torch.bfloat16
    if device != "cpu":
        W = to_device(W, device)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (2, 40), generator=g).tolist()
    dense = Model(cfg, W, device=device, dtype=dt, n_slots=2, kv_tokens=1 << 16, slot_tokens=1 << 15)
    backing = KvBacking(device, fake=fake)
    m = Model(cfg, W, device=device, dtype=dt, n_slots=2, kv_tokens=1 << 16, kv_backing=backing)
    kv = KvManager(m, granule=256)
    import pytest
    with pytest.raises(RuntimeError):                   # no lease, no region: refused on the host, nothing is touched
        m.forward(make_plan([(0, ids[0][:8], 0)], device=device))
    assert kv.assign(0, 512) and kv.assign(1, 40000)
    b1 = backing.backed_bytes()
    assert backing.tokens >= 40512 - 512 and b1 > 0
    for s in (0, 1):
        a = dense.forward(make_plan([(s, ids[s][:32], 0)], device=device))
        b = m.forward(make_plan([(s, ids[s][:32], 0)], device=device))
        assert torch.equal(a, b)
        for t in range(32, 40):
            a = dense.forward(make_plan([(s, [ids[s][t]], t)], device=device))
            b = m.forward(make_plan([(s, [ids[s][t]], t)], device=device))
            assert torch.equal(a, b)
    kv.release(1)                                        # the high lease goes away: the backing shrinks under it
    assert backing.backed_bytes() < b1 and backing.tokens <= 2048
    assert kv.grow(0, 1024) and backing.tokens >= 1024   # in place, now that the neighbour is gone
    b = m.forward(make_plan([(0, [ids[0][0]], 40)], device=device))      # slot 0 still works after the shrink
    a = dense.forward(make_plan([(0, [ids[0][0]], 40)], device=device))
    assert torch.equal(a, b)
    assert "kv_backed_bytes" in kv.stats()


def test_kv_tensors_grow_on_demand_fake_driver():
    _kv_backed_generation("cpu", True)


import pytest


@pytest.mark.gpu
def test_kv_tensors_grow_on_demand_on_the_device():
    """The same through the CUDA virtual-memory calls: a few MB mapped, grown and unmapped; no row outside a backed
    lease is ever addressed."""
    _kv_backed_generation("cuda", False)
