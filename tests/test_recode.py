"""Load-time re-codings of dense weights: exactness / error bounds of every codec on CPU, and the device GEMVs."""
import pytest
import torch

from spark_engine_b200.quant import recode as RC


def _w(n=64, k=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.05
    w[3, 7] = 3.0e4          # outliers with rare exponents: exercise the escape list
    w[5, 100] = 1.0e-30
    w[9, :] = 0.0
    w[11] = w[11] * torch.exp(torch.randn(k, generator=g) * 6)     # > 15 distinct exponents in one row
    return w


def test_c12_is_lossless_on_bf16_values():
    w = _w()
    c = RC.C12Weight.encode(w)
    assert torch.equal(c.dequant_bf16().view(torch.int16), w.bfloat16().view(torch.int16))
    assert c.ptr[-1] > 0                                         # some escapes were needed
    assert c.nbytes() < 0.85 * w.numel() * 2                     # 0.75 of the bf16 bytes + tables and escapes


def test_q8_q4_fp8_error_bounds():
    w = _w()[:, :256]
    w[3, 7] = 0.2
    q8 = RC.Q8Weight.encode(w)
    step = q8.scales.repeat_interleave(128, 1)
    assert ((q8.dequant() - w).abs() <= step * 0.5 + 1e-9).all()
    q4 = RC.Q4Weight.encode(w)
    step4 = q4.sm[..., 0].repeat_interleave(64, 1)
    assert ((q4.dequant() - w).abs() <= step4 * 0.5 + 1e-7).all()
    f8 = RC.Fp8RowWeight.encode(w)
    assert ((f8.dequant() - w).abs() <= w.abs() * 2 ** -3 + f8.scales.unsqueeze(1) * 2 ** -9 + 1e-9).all()


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 8])
def test_spx_bitstream_rotation_and_product(bits):
    w = _w(32, 256, 2)
    w[3, 7] = 0.1
    s = RC.SpxWeight.encode(w, bits=bits)
    codes = RC.unpack_bits(s.q, bits, 256)
    assert torch.equal(RC.pack_bits(codes, bits), s.q) and int(codes.max()) < 2 ** bits
    x = torch.randn(5, 256, generator=torch.Generator().manual_seed(3))
    y_rot = s.rotate_input(x) @ s.w_rot().t()                   # decode-path form: rotate the input once
    y_deq = x @ s.dequant().t()                                 # equivalent weight-side form
    assert torch.allclose(y_rot, y_deq, atol=1e-4, rtol=1e-4)
    if bits == 8:
        assert ((y_deq - x @ w.t()).norm() / (x @ w.t()).norm()) < 2e-2


def test_recode_dense_replaces_only_large_projections():
    from spark_engine_b200.config import tiny_hybrid
    from spark_engine_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    W = init_weights(cfg, seed=0)
    Wq = RC.recode_dense(W, "q8", min_numel=1 << 12)
    kinds = {type(v).__name__ for lw in Wq["layers"] for v in lw["mix"].values()}
    assert "Q8Weight" in kinds
    assert isinstance(Wq["embed"], torch.Tensor)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["q8", "q4", "fp8"])
@pytest.mark.parametrize("R", [1, 4, 11, 16])
def test_coded_gemv_on_device(kind, R):
    from spark_engine_b200 import ops
    g = torch.Generator().manual_seed(7)
    w = torch.randn(512, 1024, generator=g) * 0.05
    cw = RC.RECODERS[kind](w).to("cuda")
    x = torch.randn(R, 1024, generator=g).bfloat16().cuda()
    y = ops.linear(x, cw).float().cpu()
    ref = x.float().cpu() @ cw.dequant().t()
    assert ((y - ref).norm() / ref.norm()) < 6e-3
    assert torch.equal(ops.linear(x, cw), ops.linear(x, cw))
    y1 = ops.linear(x[:1].contiguous(), cw)
    assert torch.equal(y1[0], ops.linear(x, cw)[0])


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["c12", "fp8", "spx"])
def test_other_codings_run_on_device(kind):
    from spark_engine_b200 import ops
    g = torch.Generator().manual_seed(8)
    w = torch.randn(256, 512, generator=g) * 0.05
    cw = RC.RECODERS[kind](w).to("cuda")
    x = torch.randn(40, 512, generator=g).bfloat16().cuda()
    y = ops.linear(x, cw).float().cpu()
    ref = x.float().cpu() @ cw.dequant().bfloat16().float().t()
    assert ((y - ref).norm() / ref.norm()) < 1e-2


def test_latent_fp8_rows_round_trip():
    """Packed FP8 latent cache rows: e4m3 codes with a scale per tile of 128, four scale slots, rope dims in bf16."""
    import torch
    from spark_engine_b200.models.model import pack_latent_fp8, unpack_latent_fp8
    g = torch.Generator().manual_seed(0)
    for L, r in ((512, 64), (256, 32), (32, 16)):
        x = torch.randn(7, L + r, generator=g) * 3
        x[3, :L] = 0                                            # an all-zero tile keeps scale 1
        p = pack_latent_fp8(x, L)
        assert p.dtype == torch.uint8 and p.shape == (7, L + 16 + 2 * r)
        b = unpack_latent_fp8(p, L)
        assert ((b - x).norm() / x.norm()).item() < 3e-2
        assert torch.equal(b[3, :L], torch.zeros(L))
        assert (b[:, L:] - x[:, L:]).abs().max().item() < 2e-2 * x.abs().max().item()
