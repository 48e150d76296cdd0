"""Generate the golden vectors under tests/golden/ by running the reference's own Python code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference's ``python/`` directory is put on ``sys.path`` and its semantic reference
(``adangel.reference.run_o{0,1,2}_reference``) and codecs (``adangel.quantization``) are called on
seeded inputs.  Results are written as small ``.npz`` / ``.json`` fixtures that travel with the
repository; nothing else reads the reference checkout.
"""

from __future__ import annotations

import hashlib
import json
import math
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "python"))
    import torch

    from adangel.benchmark.metrics import mse_fp64
    from adangel.quantization import mxfp4 as rq
    from adangel.quantization.int8 import dequantize_int8_per_row, quantize_int8_per_row
    from adangel.reference import run_o0_reference, run_o1_reference, run_o2_reference
    from adangel.trace.schema import PreparedInputs

    torch.set_num_threads(8)

    # ---- scalar known answers (pure-Python helpers of the reference) -------------------------
    sweep = [i / 64.0 for i in range(-8 * 64, 8 * 64 + 1)] + [100.0, -100.0, -0.0, 1e-40, -1e-40, 1e30]
    scalar = {
        "encode_values": sweep,
        "encode_codes": [rq.encode_e2m1(v) for v in sweep],
        "decode": [rq.decode_e2m1(c) for c in range(16)],
        "int8_base": [rq.e2m1_to_int8_base(c) for c in range(16)],
        "pack_1_2": list(rq.pack_e2m1([1, 2])),
        "scale_inputs": [],
        "scale_codes": [],
    }
    for e in range(-140, 130, 3):
        for mant in (1.0, 1.0 + 2.0 ** -23, 1.5, 2.0 - 2.0 ** -23):
            v = math.ldexp(mant, e)
            if v == 0.0 or math.isinf(v) or v > 3.4e38:
                continue
            v = float(np.float32(v))
            if v == 0.0 or math.isinf(v):
                continue
            scalar["scale_inputs"].append(v.hex())
            scalar["scale_codes"].append(rq.choose_ue8m0_scale_code(v))
    (HERE / "scalar_codec.json").write_text(json.dumps(scalar))

    # ---- tensor cases -------------------------------------------------------------------------
    def canonical(m, n, k, seed=20250805):
        g = torch.Generator().manual_seed(seed)
        a = torch.randn(m, k, generator=g, dtype=torch.float32)
        idx = torch.randperm(k, generator=g)[: max(1, round(0.005 * k))]
        a[:, idx] *= 20.0
        w = torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02
        a_int8, a_scale = quantize_int8_per_row(a)
        w_mx, w_sc = rq.quantize_mxfp4(w)
        return a_int8, a_scale, w_mx, w_sc

    def fp16_case(m, n, k, seed, pattern="random"):
        # the input construction of the reference's own integration tests
        # (tests/integration/test_sm120_o2.py:6-28)
        g = torch.Generator().manual_seed(seed)
        if pattern == "random":
            act = torch.randn((m, k), generator=g, dtype=torch.float16)
            a_int8, a_scale = quantize_int8_per_row(act)
        else:
            if pattern == "zero":
                a_int8 = torch.zeros((m, k), dtype=torch.int8)
            elif pattern == "alternating":
                a_int8 = torch.tensor([-127, 127], dtype=torch.int8).repeat(k // 2).repeat(m, 1)
            else:
                a_int8 = torch.full((m, k), 127, dtype=torch.int8)
                a_int8[:, 1::2] = -127
            a_scale = torch.linspace(2.0 ** -8, 2.0 ** 4, m, dtype=torch.float32)
        w = torch.randn((n, k), generator=g, dtype=torch.float16)
        w_mx, w_sc = rq.quantize_mxfp4(w)
        return a_int8.contiguous(), a_scale, w_mx, w_sc

    def run_all(tensors):
        inputs = PreparedInputs("golden", *tensors)
        o0 = run_o0_reference(inputs)
        o1 = run_o1_reference(inputs)
        o2 = run_o2_reference(inputs)
        return o0, o1, o2

    def full_record(name, tensors):
        a_int8, a_scale, w_mx, w_sc = tensors
        o0, o1, o2 = run_all(tensors)
        np.savez_compressed(
            HERE / f"{name}.npz",
            A_int8=a_int8.numpy(), A_scale=a_scale.numpy(), W_mxfp4=w_mx.numpy(), W_scale=w_sc.numpy(),
            o0_output=o0["output"].numpy(),
            o0_weight=o0["converted_weight"].numpy(), o0_activation=o0["converted_activation"].numpy(),
            o1_output=o1["output"].numpy(), o1_weight=o1["converted_weight"].numpy(),
            o2_output=o2["output"].numpy(),
            o2_codes=o2["converted_activation"][0].numpy(), o2_scales=o2["converted_activation"][1].numpy(),
            mse_o1=np.float64(mse_fp64(o1["output"], o0["output"])),
            mse_o2=np.float64(mse_fp64(o2["output"], o0["output"])),
        )

    full_record("canonical_128x128x128", canonical(128, 128, 128))
    full_record("canonical_68x36x64", canonical(68, 36, 64))
    full_record("fp16_seed2026_128x128x256", fp16_case(128, 128, 256, 2026))
    full_record("fp16_seed2026_132x132x256", fp16_case(132, 132, 256, 2026))
    for pattern in ("zero", "alternating", "saturated"):
        full_record(f"edge_{pattern}_128x128x256", fp16_case(128, 128, 256, 2026, pattern))

    # reference/tests/integration/test_reference_variants.py: seed 7, A 16x64, W 8x64, randn
    g = torch.Generator().manual_seed(7)
    a = torch.randn(16, 64, generator=g)
    w = torch.randn(8, 64, generator=g)
    a_int8, a_scale = quantize_int8_per_row(a)
    w_mx, w_sc = rq.quantize_mxfp4(w)
    np.savez_compressed(HERE / "seed7_floats.npz", a=a.numpy(), w=w.numpy())
    full_record("seed7_16x8x64", (a_int8, a_scale, w_mx, w_sc))

    # larger canonical grid points: digests + a strided sample of the outputs
    digests = {}
    for (m, n, k) in ((256, 512, 1024), (1000, 768, 2048)):
        tensors = canonical(m, n, k)
        o0, o1, o2 = run_all(tensors)
        key = f"{m}x{n}x{k}"
        digests[key] = {
            "A_int8": sha(tensors[0].numpy()), "A_scale": sha(tensors[1].numpy()),
            "W_mxfp4": sha(tensors[2].numpy()), "W_scale": sha(tensors[3].numpy()),
            "o0_weight": sha(o0["converted_weight"].numpy()),
            "o0_activation": sha(o0["converted_activation"].numpy()),
            "o1_weight": sha(o1["converted_weight"].numpy()),
            "o2_codes": sha(o2["converted_activation"][0].numpy()),
            "o2_scales": sha(o2["converted_activation"][1].numpy()),
            "mse_o1": mse_fp64(o1["output"], o0["output"]),
            "mse_o2": mse_fp64(o2["output"], o0["output"]),
        }
        np.savez_compressed(
            HERE / f"canonical_{key}_sample.npz",
            o0=o0["output"].numpy()[::8, ::8], o1=o1["output"].numpy()[::8, ::8],
            o2=o2["output"].numpy()[::8, ::8],
        )
    (HERE / "canonical_digests.json").write_text(json.dumps(digests, indent=1))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
