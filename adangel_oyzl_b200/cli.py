"""Command-line entry point: ``python -m adangel_oyzl_b200 {doctor,verify-layout,show-config,run,analyze}``.

Mirrors the reference CLI (``python/adangel/cli.py:12-18,46-53,56-91``) for the commands that belong
to the native hot path.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path


def _doctor(args) -> None:
    from .ops.extension import native_status, require_native

    status = native_status()
    print(json.dumps({"available": status.available, "reason": status.reason,
                      "capabilities": status.capabilities}, indent=2))
    if args.require_native:
        require_native()


def _verify_layout(args) -> None:
    from .ops.extension import require_sm100_extension

    native = require_sm100_extension()
    result = dict(native.verify_layout())
    print(json.dumps(result, indent=2))
    if not result.get("passed", False):
        raise RuntimeError("SM100 microscale layout verification failed")


def _show_config(args) -> None:
    import yaml

    config = yaml.safe_load(Path(args.config).read_text(encoding="utf-8"))
    print(yaml.safe_dump(config, sort_keys=False))


def _run(args) -> None:
    from .benchmark.runner import run_experiment

    print(run_experiment(args.config, args.output, sample_limit=args.samples, warmup_override=args.warmup,
                         repeats_override=args.repeats, prepared_dir=args.prepared))


def _audit(args) -> None:
    from .audit import audit

    result = audit(args.output)
    print("\n".join(result["lines"]))
    print(f"status={result['status']}")
    if result["status"] != "PASS":
        raise SystemExit(1)


def _prepare(args) -> None:
    from .trace.prepare import prepare_synthetic, prepare_trace

    if args.input:
        if not (args.config and args.trace_config):
            raise SystemExit("--input needs --config (experiment YAML) and --trace-config (trace selection YAML)")
        records = prepare_trace(args.input, args.output, args.config, args.trace_config)
    else:
        import yaml

        from .benchmark.runner import _shapes

        config = yaml.safe_load(open(args.config, encoding="utf-8"))
        records = prepare_synthetic(_shapes(config), args.output, seed=config["experiment"]["seed"])
    print(f"prepared {len(records)} samples")


def _analyze(args) -> None:
    from .analysis import generate_report

    print(generate_report(args.run, args.output, allow_unstable=args.allow_unstable))


def _validate(args) -> None:
    import json

    from .synthetic import canonical_inputs
    from .validate import validate_variant

    inputs = canonical_inputs(args.m, args.n, args.k, device="cuda")
    failed = False
    for variant in args.variant:
        report = validate_variant(variant, inputs, warmup=args.warmup, repeats=args.repeats,
                                  max_compute_ms=args.max_compute_ms, max_cv_percent=args.max_cv_percent)
        print(json.dumps(report, indent=2))
        failed |= not report["passed"]
    if failed:
        raise SystemExit(1)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="adangel_oyzl_b200")
    commands = parser.add_subparsers(dest="command", required=True)

    doctor = commands.add_parser("doctor", help="inspect CUDA/GPU/native backend readiness")
    doctor.add_argument("--require-native", action="store_true")
    doctor.set_defaults(func=_doctor)

    verify = commands.add_parser("verify-layout", help="run the block-scaled MMA scale-layout known-answer test")
    verify.add_argument("--require-native", action="store_true")
    verify.set_defaults(func=_verify_layout)

    show = commands.add_parser("show-config", help="parse and print a YAML config")
    show.add_argument("--config", required=True)
    show.set_defaults(func=_show_config)
    run = commands.add_parser("run", help="run the interleaved O0/O1/O2 experiment on synthetic samples")
    run.add_argument("--config", required=True)
    run.add_argument("--output", required=True)
    run.add_argument("--samples", type=int)
    run.add_argument("--warmup", type=int)
    run.add_argument("--repeats", type=int)
    run.add_argument("--require-native", action="store_true", help="kept for explicit scripts; a run always requires native")
    run.add_argument("--prepared", help="directory of prepared samples (manifest.json) to run instead of synthetic ones")
    run.set_defaults(func=_run)

    audit = commands.add_parser("audit", help="check that every production kernel contains its TMA / tensor-core instruction family")
    audit.add_argument("--output", help="directory for summary.txt")
    audit.set_defaults(func=_audit)

    prepare = commands.add_parser("prepare", help="quantize samples on the GPU into a prepared directory")
    prepare.add_argument("--output", required=True)
    prepare.add_argument("--config", required=True, help="experiment YAML (shapes and seed; formal YAML with --input)")
    prepare.add_argument("--input", help="directory of a raw FP16 prefill trace (24 sample files + trace_manifest.json)")
    prepare.add_argument("--trace-config", help="trace selection YAML (with --input)")
    prepare.set_defaults(func=_prepare)

    validate = commands.add_parser("validate", help="acceptance check of one or more variants: stage contract, cross-mode "
                                               "consistency and, at 4096^3, the compute-only median / CV gate")
    validate.add_argument("--variant", nargs="+", default=["o0", "o1", "o2"], choices=["o0", "o1", "o2", "o1x"])
    validate.add_argument("--m", type=int, default=4096)
    validate.add_argument("--n", type=int, default=4096)
    validate.add_argument("--k", type=int, default=4096)
    validate.add_argument("--warmup", type=int, default=10)
    validate.add_argument("--repeats", type=int, default=50)
    validate.add_argument("--max-compute-ms", type=float, default=None)
    validate.add_argument("--max-cv-percent", type=float, default=3.0)
    validate.set_defaults(func=_validate)

    analyze = commands.add_parser("analyze", help="generate the four tables of a finished run")
    analyze.add_argument("--run", required=True)
    analyze.add_argument("--output", required=True)
    analyze.add_argument("--allow-unstable", action="store_true", help="include records that failed the CV gate")
    analyze.set_defaults(func=_analyze)
    return parser


def main(argv=None) -> None:
    args = build_parser().parse_args(argv)
    args.func(args)
