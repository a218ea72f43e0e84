"""`python -m spark_engine_b200 <command> [args]`: one entry point for the package's tools.

    serve | engine | status | stop     the launcher (serving/launch.py): one engine rank per GPU + the HTTP front end
    front                              the OpenAI-compatible front end alone (serving/openai_server.py)
    build                              compile the CUDA kernels and the C++ runtime in-tree
    bench-gemm | bench-decode | bench-prefill | bench-mx | bench-fused | bench-http | profile-round
                                       kernel and serving microbenchmarks
    ref-kernels                        the reference's own kernels on this GPU (baseline/ref_kernels.py, repo checkout only)
    configs                            the model presets as JSON
    version

Every command forwards its remaining arguments to the module it names.  Library GEMMs run with fp32 accumulation and
without reduced-precision reductions (utils/precision.py); SPARK_TF32=1 allows TF32.
Reference: engine-rs/src/main.rs:85-273 (subcommand dispatch, global precision setup)."""
from __future__ import annotations

import json
import runpy
import sys

MODULES = {
    "front": "spark_engine_b200.serving.openai_server",
    "build": "spark_engine_b200.build",
    "bench-gemm": "spark_engine_b200.ops.bench_gemm",
    "bench-decode": "spark_engine_b200.ops.bench_decode_kernels",
    "bench-prefill": "spark_engine_b200.ops.bench_prefill_kernels",
    "bench-mx": "spark_engine_b200.ops.bench_mx_experts",
    "bench-fused": "spark_engine_b200.parallel.bench_fused",
    "bench-http": "spark_engine_b200.serving.bench_http",
    "profile-round": "spark_engine_b200.serving.profile_round",
    "ref-kernels": "baseline.ref_kernels",
}
LAUNCHER = ("serve", "engine", "status", "stop")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(__doc__)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "version":
        from .serving.openai_server import VERSION
        print(VERSION)
        return 0
    if cmd == "configs":
        from .config import PRESETS
        print(json.dumps({k: json.loads(f().to_json()) for k, f in PRESETS.items()}, indent=1))
        return 0
    from .utils import precision
    precision.set_fp32_accum()
    if cmd in LAUNCHER:
        sys.argv = ["spark_engine_b200.serving.launch", cmd] + rest
        runpy.run_module("spark_engine_b200.serving.launch", run_name="__main__")
        return 0
    if cmd in MODULES:
        sys.argv = [MODULES[cmd]] + rest
        runpy.run_module(MODULES[cmd], run_name="__main__")
        return 0
    print(f"unknown command {cmd!r}\n{__doc__}", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
