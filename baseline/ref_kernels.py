"""Kernel-level comparison against the reference's own CUDA kernels on the same GPU.

The reference engine as a whole is a Rust binary and cannot be installed here; its decode kernels for the Qwen-style
model, however, are plain CUDA C++ behind a C ABI that the reference's own Python tests drive through ctypes
(reference/qwen38/kern.py:20-53).  `build()` copies the UNMODIFIED kernel sources (engine-rs/shim/qwen_exl3.cu,
qwen_exl3.cuh, qwen_gdn.cu) out of a reference checkout into baseline/_ref/shim, compiles them with the reference's own
flags (engine-rs/build.rs:79: -O3 -std=c++17 --fmad=false) for sm_100, and links one stub for a host symbol of the
reference's runtime.  `bench()` then (1) checks the reference kernels against themselves and against this repo's fp32
oracle on the box, (2) times them and this repo's kernels at the same shapes, cold (L2 flushed before every launch),
with CUDA events.  Only kernels without device-side waits are used: the EXL3 GEMV family (had_in / gemv / finish and
the one-launch `qwen_exl3_linear`, whose only cross-CTA step is a last-arriver ticket) and the GDN conv + recurrence.

    python -m baseline.ref_kernels build [--reference DIR]      # here (nvcc cross-compiles)
    python -m baseline.ref_kernels bench [--out FILE.md]        # on a B200
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SO = os.path.join(REF, "libref_qwen_kernels.so")
SOURCES = ["qwen_exl3.cu", "qwen_gdn.cu"]
HEADERS = ["qwen_exl3.cuh"]


def build(reference_dir: str) -> str:
    shim = os.path.join(reference_dir, "engine-rs", "shim")
    dst = os.path.join(REF, "shim")
    os.makedirs(dst, exist_ok=True)
    for f in SOURCES + HEADERS:
        shutil.copyfile(os.path.join(shim, f), os.path.join(dst, f))          # byte-for-byte copies
    cmd = ["nvcc", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "--fmad=false",
           "-gencode=arch=compute_100,code=sm_100", *[os.path.join(dst, f) for f in SOURCES],
           os.path.join(HERE, "ref_stubs.cpp"), "-o", SO]
    subprocess.check_call(cmd)
    return SO


# ------------------------------------------------------------------------------------------------ bench (GPU)
def _flusher(torch):
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    return lambda: buf.zero_()


def _time(torch, fn, flush, n=30):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(n):
        flush()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def bench(out_path: str) -> int:
    import torch
    sys.path.insert(0, os.path.dirname(HERE))
    from spark_engine_b200.ops import cuda as cu
    from spark_engine_b200.oracle import layers as L
    from spark_engine_b200.quant import formats as Q
    lib = C.CDLL(SO)
    st = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    i64 = C.c_int64
    flush = _flusher(torch)
    g = torch.Generator(device="cuda").manual_seed(0)
    lines = ["| op | shape | rows | reference kernels (us) | this repo (us) | ratio |", "|---|---|---|---|---|---|"]
    checks = []

    # ---- EXL3 4-bit linear
    for (K, N) in ((2560, 640), (2560, 10240), (6144, 2560), (2048, 8192)):
        tr = torch.randint(-32768, 32767, (K // 16, N // 16, 64), dtype=torch.int16, device="cuda", generator=g)
        suh = (torch.randint(0, 2, (K,), device="cuda", generator=g) * 2 - 1).half()
        svh = (torch.randint(0, 2, (N,), device="cuda", generator=g) * 2 - 1).half()
        ours_w = Q.random_exl3(N, K, 4, 0, 0.02, 1, "cuda")
        for M in (1, 4, 16):
            x = torch.randn(M, K, device="cuda", generator=g)
            S = max(1, min(16, (K // 16) // 8, 96 // max(1, N // 128)))          # the reference tests' slice rule
            xh = torch.empty(M, K, dtype=torch.half, device="cuda")
            part = torch.empty(S, M, N, dtype=torch.float32, device="cuda")
            y3 = torch.empty(M, N, dtype=torch.float32, device="cuda")
            y1 = torch.empty(M, N, dtype=torch.float32, device="cuda")
            cnt = torch.zeros(N // 128, dtype=torch.int32, device="cuda")

            def three():
                assert lib.qwen_exl3_had_in(p(x), 1, i64(x.stride(0)), p(suh), p(xh), M, K, st()) == 0
                assert lib.qwen_exl3_gemv(p(xh), p(tr), p(part), M, K, N, 4, S, st()) == 0
                assert lib.qwen_exl3_finish(p(part), S, p(svh), p(y3), 1, i64(N), M, N, st()) == 0

            def one():
                assert lib.qwen_exl3_linear(p(x), i64(x.stride(0)), p(suh), p(tr), p(svh), p(part), p(y1), i64(N), p(cnt), M, K, N,
                                            4, S, st()) == 0
            three()
            one()
            if M == 4:                                   # the reference against itself: folded dense weight
                Wt = torch.empty(N, K, dtype=torch.half, device="cuda")
                assert lib.qwen_exl3_fold(p(tr), p(suh), p(svh), K, N, 4, p(Wt), i64(K), st()) == 0
                ref = x.double() @ Wt.double().t()
                e3 = float((y3.double() - ref).abs().max() / ref.abs().max())
                e1 = float((y1.double() - ref).abs().max() / ref.abs().max())
                checks.append(f"EXL3 {K}->{N}: three-launch vs folded dense {e3:.2e}, one-launch vs folded dense {e1:.2e}")
                assert e3 < 2e-2 and e1 < 2e-2, (e3, e1)
            xb = x.to(torch.bfloat16)
            t3, t1 = _time(torch, three, flush), _time(torch, one, flush)
            to = _time(torch, lambda: cu.quant_linear(xb, ours_w), flush)
            best = min(t3, t1)
            lines.append(f"| EXL3 4 bpw linear | {K}->{N} | {M} | {t3:.1f} (3 launches) / {t1:.1f} (fused) | {to:.1f} | {best / to:.2f}x |")

    # ---- GDN conv + recurrence, 16 key heads, 48 value heads of 128
    Hk, Hv, D, Cc = 16, 48, 128, 10240
    for T in (1, 4, 16):
        qkv = torch.randn(T, Cc, device="cuda", generator=g)
        z = torch.randn(T, Hv * D, device="cuda", generator=g)
        ab = torch.randn(T, 2 * Hv, device="cuda", generator=g)           # reference layout: a | b
        conv_w = (torch.rand(Cc, 4, device="cuda", generator=g) - 0.5).to(torch.bfloat16)
        conv_state = torch.randn(Cc, 3, device="cuda", generator=g)
        A_log = torch.log(torch.rand(Hv, device="cuda", generator=g) * 7 + 1).to(torch.bfloat16)
        dtb = (torch.rand(Hv, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
        nw = (torch.rand(D, device="cuda", generator=g) + 0.5).to(torch.bfloat16)
        S0 = torch.randn(Hv, D, D, device="cuda", generator=g) * 0.1
        Sr = S0.clone()
        y = torch.empty(T, Cc, device="cuda")
        out = torch.empty(T, Hv * D, device="cuda")

        def ref_gdn():
            assert lib.qwen_gdn_conv(p(qkv), i64(Cc), p(conv_state), p(conv_w), p(y), T, st()) == 0
            assert lib.qwen_gdn_recur(p(y), p(ab), i64(2 * Hv), p(z), i64(Hv * D), p(A_log), p(dtb), p(nw), p(Sr), p(out), T, 0,
                                      st()) == 0
        ref_gdn()
        # this repo's kernel on the same numbers: proj = q | k | v | z in bf16, ab = b | a, conv history oldest first
        class _M:
            pass
        mx = _M()
        mx.c = _M()
        mx.c.n_k_heads, mx.c.n_v_heads, mx.c.head_dim = Hk, Hv, D
        mx.cfg = _M()
        mx.cfg.norm_eps = 1e-6
        mx.w = {"conv": conv_w.float().contiguous(), "A_log": A_log.float(), "dt_bias": dtb.float(), "norm": nw.float()}
        mx.S = S0.clone().unsqueeze(0).contiguous()
        tail = torch.zeros(1, 3, Hv, 3 * D, device="cuda")
        cs = conv_state.t().contiguous()                                   # [3, C] oldest first
        rep = Hv // Hk
        for j in range(3):
            for h in range(Hv):
                hk = h // rep
                tail[0, j, h, :D] = cs[j, hk * D:(hk + 1) * D]
                tail[0, j, h, D:2 * D] = cs[j, 2048 + hk * D: 2048 + (hk + 1) * D]
                tail[0, j, h, 2 * D:] = cs[j, 4096 + h * D: 4096 + (h + 1) * D]
        mx.tail = tail
        proj = torch.cat((qkv, z), 1).to(torch.bfloat16).contiguous()
        ab_ours = torch.cat((ab[:, Hv:], ab[:, :Hv]), 1).to(torch.bfloat16).contiguous()
        from spark_engine_b200.models.plan import make_plan
        plan = make_plan([(0, [0] * T, 0)], device="cuda")
        o = cu.gdn_mixer(mx, proj, ab_ours, plan, False)
        # both kernels against the fp32 formulas (bf16 inputs for ours, so compare each to its own rounding of the inputs)
        rel = float((o.float() - out).norm() / out.norm())
        checks.append(f"GDN T={T}: this repo's kernel vs the reference kernel on the same inputs (ours reads bf16 projections): "
                      f"relative difference {rel:.2e}")
        assert rel < 3e-2, rel
        tr_ = _time(torch, ref_gdn, flush)
        to = _time(torch, lambda: cu.gdn_mixer(mx, proj, ab_ours, plan, False), flush)
        lines.append(f"| GDN conv + recurrence (16/48 heads x 128) | state 48x128x128 fp32 | {T} | {tr_:.1f} (2 launches) | {to:.1f} | "
                     f"{tr_ / to:.2f}x |")
    text = "\n".join(lines) + "\n\nChecks on this GPU:\n" + "\n".join("- " + c for c in checks) + "\n"
    print(text)
    if out_path:
        with open(out_path, "w") as f:
            f.write(text)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=["build", "bench"])
    ap.add_argument("--reference", default=os.environ.get("SPARK_REFERENCE_DIR", os.path.join(os.path.dirname(HERE), "..", "reference")))
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    if a.cmd == "build":
        print(build(os.path.abspath(a.reference)))
        return 0
    if not os.path.exists(SO):
        print("reference kernels not built: run `python -m baseline.ref_kernels build` first")
        return 1
    return bench(a.out)


if __name__ == "__main__":
    sys.exit(main())
