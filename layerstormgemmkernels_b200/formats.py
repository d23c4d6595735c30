"""GGUF type ids and block sizes (include/lsg.h; ids 0..6 are the reference's GgufType values,
csrc/sm120/gemm/gguf/gguf_dequant_gemm.h:23-31).  Pure Python: importing this module loads
no shared library, so host-only code (weight packers, the CPU baseline) can use it."""

Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_0, MXFP4, Q4_0 = range(8)
GGUF_TYPES = {"Q2_K": Q2_K, "Q3_K": Q3_K, "Q4_K": Q4_K, "Q5_K": Q5_K, "Q6_K": Q6_K,
              "Q8_0": Q8_0, "MXFP4": MXFP4, "Q4_0": Q4_0}
BLOCK_BYTES = {Q2_K: 84, Q3_K: 110, Q4_K: 144, Q5_K: 176, Q6_K: 210, Q8_0: 34, MXFP4: 17, Q4_0: 18}
BLOCK_VALUES = {Q2_K: 256, Q3_K: 256, Q4_K: 256, Q5_K: 256, Q6_K: 256, Q8_0: 32, MXFP4: 32, Q4_0: 32}

DTYPE_BF16, DTYPE_F32, DTYPE_F16 = 0, 1, 2
