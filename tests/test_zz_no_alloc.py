"""The allocation-free decode-attention entry point against the regular one.

Some callers of this library cannot allocate device memory while they run (inside a stream capture, in a
fixed-budget embedding, from plain C without a caching allocator), so `spark_attn_decode_noalloc` keeps its
split partials in an array built into the library.  It must give the same output as `spark_attn_decode`,
also on a second call that finds the first call's leftovers in the shared array, and must refuse a problem
that does not fit."""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, R, Hq, Hkv, D, ctx):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qbuf = torch.randn(R, Hq, D, device="cuda", generator=g).bfloat16()
    kc = torch.randn(ctx + 8, Hkv, D, device="cuda", generator=g).bfloat16()
    vc = torch.randn(ctx + 8, Hkv, D, device="cuda", generator=g).bfloat16()
    pos = torch.tensor([ctx - 1 - 3 * r for r in range(R)], dtype=torch.int32, device="cuda")
    row_kv = torch.zeros(R, dtype=torch.int64, device="cuda")
    qkv = torch.randn(R, Hq * 2 * D, device="cuda", generator=g).bfloat16()      # per head [q | gate]
    return qbuf, kc, vc, pos, row_kv, qkv


def test_noalloc_entry_point_matches_regular_one_twice():
    from spark_engine_b200.ops import cuda as cu
    dll = cu.lib()._dll
    fn = dll.spark_attn_decode_noalloc
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    fn.argtypes = [vp, vp, vp, vp, vp, i32, vp, vp, vp, vp, i32, i32, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp]
    fn.restype = i32
    for seed, (R, Hq, Hkv, D, ctx) in enumerate([(4, 16, 2, 256, 700), (2, 4, 2, 64, 130)]):   # two calls in a row
        qbuf, kc, vc, pos, row_kv, qkv = _problem(seed, R, Hq, Hkv, D, ctx)
        nsplit = (ctx + 63) // 64
        scale = 1.0 / math.sqrt(D)
        part_o = torch.empty(R * Hq * nsplit * D, device="cuda")
        part_ml = torch.empty(R * Hq * nsplit * 2, device="cuda")
        ref = torch.empty(R, Hq * D, dtype=torch.bfloat16, device="cuda")
        out = torch.full_like(ref, float("nan"))
        rc = cu.lib().spark_attn_decode(qbuf.data_ptr(), kc.data_ptr(), vc.data_ptr(), None, None, 0, pos.data_ptr(),
                                        row_kv.data_ptr(), None, None, 0, part_o.data_ptr(), part_ml.data_ptr(), nsplit,
                                        qkv.data_ptr(), qkv.stride(0), 1, R, Hq, Hkv, D, scale, ref.data_ptr(), cu.stream(),
                                        None, None, None, 1)
        assert rc == 0
        rc = fn(qbuf.data_ptr(), kc.data_ptr(), vc.data_ptr(), None, None, 0, pos.data_ptr(), row_kv.data_ptr(), None, None,
                0, nsplit, qkv.data_ptr(), qkv.stride(0), 1, R, Hq, Hkv, D, scale, out.data_ptr(), cu.stream())
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-3)
        assert torch.equal(out, ref)        # same kernels, same order of operations
        # and against plain fp32 attention
        k = kc.float().repeat_interleave(Hq // Hkv, 1)
        v = vc.float().repeat_interleave(Hq // Hkv, 1)
        for r in range(R):
            n = int(pos[r]) + 1
            s = torch.einsum("hd,shd->hs", qbuf[r].float(), k[:n]) * scale
            o = torch.einsum("hs,shd->hd", torch.softmax(s, -1), v[:n])
            gate = qkv[r].float().view(Hq, 2 * D)[:, D:]
            want = (o * torch.sigmoid(gate)).reshape(-1)
            assert ((out[r].float() - want).norm() / want.norm()) < 2e-2
    # a request beyond the built-in scratch is refused, nothing runs
    rc = fn(None, None, None, None, None, 0, None, None, None, None, 0, 4096, None, 0, 0, 64, 64, 8, 256, 1.0, None, cu.stream())
    assert rc == -22
