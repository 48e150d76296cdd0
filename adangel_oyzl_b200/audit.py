"""Instruction audit of the production kernels.

The reference ships ``scripts/audit_instructions.sh``, which checks that every production kernel of
the built extension contains both TMA copies and the tensor-core instruction family of its variant.
This is the sm_100a counterpart.  It does not look into a binary: each kernel source is compiled to
PTX with ``nvcc -ptx`` (the compiler's own output for this project's sources), every ``.entry`` is
scanned for the instruction families it must and must not contain, and only the verdict is kept
(``summary.txt``: ``status=PASS`` or ``status=FAIL`` plus one line per kernel); the PTX text is
discarded.
"""

from __future__ import annotations

import re
import subprocess
import tempfile
from pathlib import Path

from .build import ARCH_FLAGS, CSRC, INCLUDE, _nvcc

# kernel name pattern (regular expression on the mangled entry name) -> (required instruction patterns, description)
REQUIRED = {
    "gemm_acc_kernelILi0E": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global", r"tcgen05\.mma\.cta_group::1\.kind::f16",
                              r"tcgen05\.ld\.sync\.aligned\.32x32b", r"cp\.async\.bulk\.tensor\.2d\.global\.shared::cta"],
                             "O0 GEMM: TMA loads, kind::f16 MMA, tensor-memory loads, TMA stores"),
    "gemm_o1_kernel": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global", r"tcgen05\.mma\.cta_group::1\.kind::i8",
                        r"tcgen05\.ld\.sync\.aligned\.32x32b", r"setmaxnreg"],
                       "O1 GEMM: TMA loads, kind::i8 MMA, tensor-memory loads, register re-balancing"),
    "gemm_acc_kernelILi2E": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global",
                              r"tcgen05\.mma\.cta_group::1\.kind::mxf4\.block_scale", r"tcgen05\.cp\.cta_group::1\.32x128b\.warpx4",
                              r"tcgen05\.ld\.sync\.aligned\.32x32b"],
                             "O2 GEMM: TMA loads, block-scaled MXFP4 MMA, scale-factor copies, tensor-memory loads"),
    "gemm_o1_bf16_kernel": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global", r"tcgen05\.mma\.cta_group::1\.kind::f16",
                             r"tcgen05\.ld\.sync\.aligned\.32x32b", r"setmaxnreg"],
                            "O1 GEMM on BF16 operands: TMA loads, kind::f16 MMA, tensor-memory loads, register re-balancing"),
    "gemm_pair_kernelILi0E": ([r"cp\.async\.bulk\.tensor\.2d\.cta_group::2\.shared::cluster\.global",
                               r"tcgen05\.mma\.cta_group::2\.kind::f16", r"tcgen05\.commit\.cta_group::2",
                               r"barrier\.cluster\.arrive", r"cp\.async\.bulk\.tensor\.2d\.global\.shared::cta"],
                              "O0 GEMM on CTA pairs: pair TMA loads, cta_group::2 MMA and commits, cluster barrier, TMA stores"),
    "gemm_pair_kernelILi2E": ([r"cp\.async\.bulk\.tensor\.2d\.cta_group::2\.shared::cluster\.global",
                               r"tcgen05\.mma\.cta_group::2\.kind::mxf4\.block_scale",
                               r"tcgen05\.cp\.cta_group::2\.32x128b\.warpx4", r"tcgen05\.commit\.cta_group::2"],
                              "O2 GEMM on CTA pairs: pair TMA loads, cta_group::2 block-scaled MMA, scale-factor copies, commits"),
    "gemm_o2_skinny_kernel": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global",
                               r"tcgen05\.mma\.cta_group::1\.kind::mxf4\.block_scale"],
                              "O2 decode GEMM: TMA loads, block-scaled MXFP4 MMA"),
    "gemm_o1_decode_kernel": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global", r"dp4a\.s32\.s32", r"elect\.sync"],
                              "O1 decode GEMM for M <= 16: TMA loads issued by an elected lane, dp4a dot products"),
    "gemm_o1_skinny_kernel": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global", r"tcgen05\.mma\.cta_group::1\.kind::i8"],
                              "O1 decode GEMM: TMA loads, kind::i8 MMA"),
    r"gemm_acc_kernelILi1E": ([r"cp\.async\.bulk\.tensor\.2d\.shared::cluster\.global", r"tcgen05\.mma\.cta_group::1\.kind::i8",
                               r"tcgen05\.ld\.sync\.aligned\.32x32b", r"cvt\.rn\.f32\.s32"],
                              "o1x GEMM: TMA loads, kind::i8 MMA over all of K, tensor-memory loads, one INT32 -> FP32 conversion"),
    r"gemm_(acc|pair)_kernelILi[02]E(Li\d+E)?Lb1E": ([r"setmaxnreg", r"red\.release\.gpu\.global\.add", r"ld\.acquire\.gpu\.global",
                                                        r"fence\.proxy\.async"],
                                                       "O0 / O2 GEMMs with converter warps: register re-balancing, row counters "
                                                       "published with release / read with acquire, proxy fences around them"),
    "o2_quantize_kernel": ([r"cvt\.rn\.satfinite\.e2m1x2\.f32"], "O2 activation re-quantization: hardware E2M1 conversion"),
    "mxfp4_to_fp16_kernel": ([r"cvt\.rn\.f16x2\.e2m1x2"], "O0 weight conversion: hardware E2M1 decode"),
}
# legacy / Hopper-only tensor-core paths and library entry points must not appear in any kernel
FORBIDDEN = [r"\bmma\.sync", r"\bwmma\.", r"\bwgmma\.", r"cublas", r"cutlass"]


def _entries(ptx: str) -> dict:
    """Map entry symbol -> body text."""
    out = {}
    for match in re.finditer(r"\.entry\s+(\w+)\s*\(", ptx):
        start = match.start()
        nxt = ptx.find(".entry", match.end())
        out[match.group(1)] = ptx[start: nxt if nxt != -1 else len(ptx)]
    return out


def audit(output_dir=None) -> dict:
    """Compile every kernel source to PTX, check the contract, return (and optionally write) the verdict."""
    entries = {}
    with tempfile.TemporaryDirectory() as tmp:
        for src in sorted(CSRC.glob("*.cu")):
            ptx_path = Path(tmp) / (src.stem + ".ptx")
            arch = ["-gencode", ARCH_FLAGS[1].replace("code=sm_100a", "code=compute_100a")]
            proc = subprocess.run([_nvcc(), *arch, "-ptx", "-std=c++17", "-I", str(INCLUDE), str(src), "-o", str(ptx_path)],
                                  capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc -ptx failed for {src.name}:\n{proc.stderr}")
            entries.update(_entries(ptx_path.read_text()))
    lines, ok = [], True
    for fragment, (patterns, what) in REQUIRED.items():
        bodies = [body for name, body in entries.items() if re.search(fragment, name)]
        found = bool(bodies) and all(all(re.search(p, body) for p in patterns) for body in bodies)
        ok &= found
        lines.append(f"{'PASS' if found else 'FAIL'} {fragment} ({len(bodies)} entries): {what}")
    for name, body in entries.items():
        bad = [p for p in FORBIDDEN if re.search(p, body)]
        if bad:
            ok = False
            lines.append(f"FAIL {name}: forbidden instruction family {bad}")
    result = {"status": "PASS" if ok else "FAIL", "kernels": len(entries), "lines": lines}
    if output_dir is not None:
        output_dir = Path(output_dir)
        output_dir.mkdir(parents=True, exist_ok=True)
        (output_dir / "summary.txt").write_text(
            f"status={result['status']}\nkernels={len(entries)}\n" + "\n".join(lines) + "\n", encoding="utf-8")
    return result
