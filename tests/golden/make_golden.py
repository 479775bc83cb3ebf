"""Generates tests/golden/quant_golden.npz from the reference's own pure-torch quantisers
(tools/ref/oracle/kernel.py: act_quant, fp4_act_quant) and tests/golden/hadamard_golden.npz from its matrix-form
Hadamard transform (tools/ref/oracle/fast_hadamard_transform.py: x.float() @ H, scaled, back to bf16), both imported
from the reference checkout.

    python tests/golden/make_golden.py [/path/to/reference]

Runs only where the checkout exists (it cannot travel to the GPU box); the .npz it writes is committed. Inputs are
seeded synthetic bf16 rows: N(0,1), N(0,1) with +-20 outliers, per-row magnitudes 2^[-3,3], and rounding edge cases.
Outputs per input set: fp8 codes (e4m3 bytes) and scales (e8m0 exponent bytes) for blocks 32/64/128, the fp8
fake-quantised bf16 values, and the fp4 fake-quantised bf16 values (block 32)."""
import sys
from pathlib import Path

import numpy as np
import torch

ref = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
sys.path.insert(0, str(ref / "tools" / "ref" / "oracle"))
import fast_hadamard_transform as ref_hadamard  # noqa: E402  (the reference's module)
import kernel as ref_kernel  # noqa: E402  (the reference's module)


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def make_inputs():
    g = torch.Generator().manual_seed(20261125)
    rows, cols = 32, 256
    sets = {}
    sets["normal"] = torch.randn(rows, cols, generator=g).to(torch.bfloat16)
    x = torch.randn(rows, cols, generator=g)
    m = torch.rand(rows, cols, generator=g) < 0.01
    x[m] = torch.where(torch.rand(int(m.sum()), generator=g) < 0.5, -20.0, 20.0)
    sets["outliers"] = x.to(torch.bfloat16)
    mag = torch.ldexp(torch.ones(rows, 1), torch.randint(-3, 4, (rows, 1), generator=g))
    sets["octaves"] = (torch.randn(rows, cols, generator=g) * mag).to(torch.bfloat16)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 7.0, 448.0, 480.0,
                         416.0, 0.001953125, 0.0009765625, 0.0029296875, 17.0, 19.0, 0.0])
    t = ties[torch.randint(0, len(ties), (rows, cols), generator=g)]
    t = t * torch.ldexp(torch.ones(rows, 1), torch.randint(-12, 12, (rows, 1), generator=g))
    t = t * (torch.randint(0, 2, (rows, cols), generator=g) * 2 - 1)
    t[0] = 0.0
    sets["ties"] = t.to(torch.bfloat16)
    return sets


def main():
    out = {}
    for name, x in make_inputs().items():
        out[f"{name}/x"] = bits(x)
        for block in (32, 64, 128):
            q, s = ref_kernel.act_quant(x, block, "ue8m0")
            out[f"{name}/fp8_codes_b{block}"] = q.view(torch.uint8).numpy().copy()
            # scales are exact powers of two: store the e8m0 exponent byte
            out[f"{name}/fp8_scales_b{block}"] = ((s.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8).numpy().copy()
            out[f"{name}/fp8_fake_b{block}"] = bits(ref_kernel.act_quant(x.clone(), block, "ue8m0", inplace=True))
        out[f"{name}/fp4_fake_b32"] = bits(ref_kernel.fp4_act_quant(x.clone(), 32, inplace=True))
    dst = Path(__file__).resolve().parent / "quant_golden.npz"
    np.savez_compressed(dst, **out)
    print(dst, {k: v.shape for k, v in list(out.items())[:4]}, dst.stat().st_size)
    # hadamard128: 96 segments of 128 values (N(0,1), per-row octaves, a zero row, a one-hot row)
    g = torch.Generator().manual_seed(20261126)
    x = torch.randn(96, 128, generator=g) * torch.ldexp(torch.ones(96, 1), torch.randint(-6, 7, (96, 1), generator=g))
    x[0] = 0.0
    x[1] = 0.0
    x[1, 77] = 3.0
    x = x.to(torch.bfloat16)
    y = ref_hadamard.hadamard_transform(x, scale=128 ** -0.5)
    dst = Path(__file__).resolve().parent / "hadamard_golden.npz"
    np.savez_compressed(dst, x=bits(x), y=bits(y))
    print(dst, dst.stat().st_size)


if __name__ == "__main__":
    main()
