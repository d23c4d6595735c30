"""Generates tests/golden/*.npz by IMPORTING the reference's CPU implementation
(tests/test_reference.py of kkontosis/LayerStoRmGemmKernels) and running it on small
seeded inputs.  Run once where the reference checkout exists:

    python tests/golden/make_golden.py /path/to/reference

The .npz files are committed; the tests read only them.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.path.insert(0, ref_root)
    from tests import test_reference as R  # the reference's own module, unmodified

    # --- Q4_K: packer bytes, dequant, dequant-GEMM --------------------------------
    g = torch.Generator().manual_seed(1234)
    w = torch.randn(24, 512, generator=g) * 0.02
    w[3, :256] = 0.0            # an all-zero super-block
    w[5, 256:288] = 0.37        # a constant sub-block
    packed = R.quantize_to_q4k(w)
    deq = R.ref_q4k_dequant(packed).numpy()
    x = torch.randn(5, 512, generator=g).to(torch.bfloat16)
    y = R.ref_q4k_gemm(x, packed).numpy()
    sc = np.array([1, 2, 3, 4, 5, 10, 15, 20], dtype=np.uint8)
    mn = np.array([2, 4, 6, 8, 10, 20, 30, 40], dtype=np.uint8)
    sc2 = np.array([63, 0, 17, 33, 48, 63, 1, 32], dtype=np.uint8)
    mn2 = np.array([0, 63, 31, 16, 63, 47, 32, 1], dtype=np.uint8)
    np.savez_compressed(
        os.path.join(HERE, "q4k_reference.npz"),
        w=w.numpy(), packed=packed, dequant=deq,
        x_bf16=x.view(torch.int16).numpy().view(np.uint16), gemm=y,
        ka_sc=sc, ka_mn=mn, ka_packed=R._pack_q4k_scales(sc, mn),
        ka_sc2=sc2, ka_mn2=mn2, ka_packed2=R._pack_q4k_scales(sc2, mn2))

    # --- FP8 block quantizer -------------------------------------------------------
    g = torch.Generator().manual_seed(77)
    xi = (torch.randn(6, 384, generator=g) * 3.0).to(torch.bfloat16)
    xi[2, 128:256] = 0.0        # an all-zero block (scale 1.0 branch)
    q, s = R.ref_dynamic_fp8_quant(xi)
    np.savez_compressed(
        os.path.join(HERE, "fp8_reference.npz"),
        x_bf16=xi.view(torch.int16).numpy().view(np.uint16),
        scaled=q.numpy(), scales=s.numpy())

    # --- NVFP4: table, weight quantizer, dequant, GEMM -----------------------------
    g = torch.Generator().manual_seed(4321)
    wn = (torch.randn(16, 128, generator=g) * 0.02)
    w_u8, w_sc, w_s2 = R.quantize_to_nvfp4(wn)
    w_deq = R.ref_nvfp4_dequant(w_u8, w_sc, w_s2).numpy()
    xn = torch.randn(4, 128, generator=g)
    yn = R.ref_nvfp4_gemm(xn, w_u8, w_sc, w_s2).numpy()
    np.savez_compressed(
        os.path.join(HERE, "nvfp4_reference.npz"),
        table=R.FP4_E2M1_TABLE.numpy(), w=wn.numpy(), w_u8=w_u8.numpy(),
        w_scale=w_sc.numpy(), w_scale2=np.float32(w_s2.item()), dequant=w_deq,
        x=xn.numpy(), gemm=yn)
    print("wrote", sorted(n for n in os.listdir(HERE) if n.endswith(".npz")))


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LSG_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_golden.py <reference checkout>   (or set LSG_REFERENCE_ROOT)")
    main(root)
