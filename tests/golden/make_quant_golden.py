"""Generate the quantizer golden vectors from the REFERENCE's own Triton kernels, run by Triton's CPU interpreter.

    TRITON_INTERPRET=1 python tests/golden/make_quant_golden.py /path/to/reference

Runs the reference's `kmean_frozen`, `kmean_m17`, `_quant_kernel` (MODE 0 / 1 / 2) and `_doq_m17_kernel` on small seeded
inputs on the CPU and stores inputs' seed, scales, k-mean, codes and the stale delta in tests/golden/quant_d{128,256}.npz.
The interpreter's float8 cast has a known defect (some values land one binade low); the codes are stored as produced and
the test that reads them states exactly which mismatches it tolerates.  The reference tree is only needed to regenerate.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np
import torch


def main(ref_root):
    sys.path.insert(0, ref_root)
    from delta_matching import producers as P
    from delta_matching import quant as FQ
    from delta_matching.core import blocks

    here = os.path.dirname(os.path.abspath(__file__))
    for D in (128, 256):
        B, H, Hk, N = 1, 2, 1, 256
        seed = 4000 + D
        g = torch.Generator("cpu").manual_seed(seed)
        q = torch.randn(B, H, N, D, generator=g).to(torch.bfloat16)
        k = (torch.randn(B, Hk, N, D, generator=g) + 0.25).to(torch.bfloat16)
        v = torch.randn(B, Hk, N, D, generator=g).to(torch.bfloat16)
        dO = (torch.randn(B, N, H, D, generator=g) * 1e-3).to(torch.bfloat16)
        O = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
        q[0, 0, :64] = 0                      # an all-zero block: the scale floor path
        dO[0, :128, 0] = 0
        v[0, 0, 64:96, 5] = 3.0e4             # a block whose amax is far above the rest
        rq, rk = blocks(D)
        sm = D ** -0.5
        kc = k.reshape(B * Hk, N, D).contiguous()
        km_frozen = P.kmean_frozen(kc)
        km_split = P.kmean_m17(kc)
        out = {"seed": np.int64(seed), "shape": np.array([B, H, Hk, N, D]), "km_frozen": km_frozen.numpy(),
               "km_split": km_split.numpy()}
        for name, x, mode, blk, bh, h in (("q", q.reshape(B * H, N, D).contiguous(), 0, rq, B * H, H),
                                          ("k", kc, 1, rk, B * Hk, Hk),
                                          ("v", v.reshape(B * Hk, N, D).contiguous(), 2, rk, B * Hk, Hk)):
            x8 = torch.empty(bh, N, D, dtype=torch.float8_e4m3fn)
            x8s = torch.empty(bh, N // blk, dtype=torch.float32)
            FQ._quant_kernel[(N // blk, bh)](x, km_frozen, x8, x8s, x8, x8, x8, N, h, SM=sm, BLK=blk, D=D, MODE=mode,
                                             WANT_T16=False, T16_IS_FP8=False, WANT_F16=False, T16_IS_BF16=False,
                                             F16_IS_BF16=False, WANT_T8=False, num_warps=8)
            out[name + "8"] = x8.view(torch.uint8).numpy()
            out[name + "8s"] = x8s.numpy()
        dO8, dO8s, dlt, _ = P.doq_m17(dO, O, H, rq, want_delta=True, want_twin=False)
        out["do8"] = dO8.view(torch.uint8).numpy()
        out["do8s"] = dO8s.numpy()
        out["delta_stale"] = dlt.numpy()
        np.savez_compressed(os.path.join(here, f"quant_d{D}.npz"), **out)
        print("wrote", f"quant_d{D}.npz", {kk: getattr(vv, "shape", None) for kk, vv in out.items()})


def golden_inputs(D):
    """The inputs the fixtures were generated from (shared with the test so both see identical bits)."""
    B, H, Hk, N = 1, 2, 1, 256
    g = torch.Generator("cpu").manual_seed(4000 + D)
    q = torch.randn(B, H, N, D, generator=g).to(torch.bfloat16)
    k = (torch.randn(B, Hk, N, D, generator=g) + 0.25).to(torch.bfloat16)
    v = torch.randn(B, Hk, N, D, generator=g).to(torch.bfloat16)
    dO = (torch.randn(B, N, H, D, generator=g) * 1e-3).to(torch.bfloat16)
    O = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    q[0, 0, :64] = 0
    dO[0, :128, 0] = 0
    v[0, 0, 64:96, 5] = 3.0e4
    return q, k, v, dO, O


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_quant_golden.py <checkout of the reference project>")
    main(sys.argv[1])
