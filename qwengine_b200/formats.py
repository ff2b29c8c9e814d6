"""GGUF block formats handled by the matvec / prefill path.

Type ids are the ggml type ids the reference uses verbatim (include/q38rt/q38rt_types.h:36-67 of
the reference project); block sizes follow its quant_block_info (:80-110).
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class BlockFormat:
    name: str
    type_id: int
    block_elems: int   # weights per block
    block_bytes: int

    def row_bytes(self, K: int) -> int:
        if K % 256:
            raise ValueError(f"K={K} is not a multiple of 256")
        return K // self.block_elems * self.block_bytes


Q8_0 = BlockFormat("Q8_0", 8, 32, 34)
Q4_K = BlockFormat("Q4_K", 12, 256, 144)
Q5_K = BlockFormat("Q5_K", 13, 256, 176)
Q6_K = BlockFormat("Q6_K", 14, 256, 210)
IQ3_XXS = BlockFormat("IQ3_XXS", 18, 256, 98)
IQ3_S = BlockFormat("IQ3_S", 21, 256, 110)
IQ4_XS = BlockFormat("IQ4_XS", 23, 256, 136)

FORMATS = {f.name: f for f in (IQ3_XXS, IQ3_S, IQ4_XS, Q4_K, Q5_K, Q6_K, Q8_0)}

# The reference's other six matvec formats (src/cuda/gemv.cu:206-213): decoded by the one-column kernel, the exact
# dequantizer and the prefill GEMM; calls with several columns run one column after the other (no tensor-core fragment
# builders for them).
Q2_K = BlockFormat("Q2_K", 10, 256, 84)
IQ2_XXS = BlockFormat("IQ2_XXS", 16, 256, 66)
IQ2_XS = BlockFormat("IQ2_XS", 17, 256, 74)
IQ1_S = BlockFormat("IQ1_S", 19, 256, 50)
IQ2_S = BlockFormat("IQ2_S", 22, 256, 82)
IQ1_M = BlockFormat("IQ1_M", 29, 256, 56)
ONE_COLUMN = {f.name: f for f in (IQ2_XXS, IQ2_XS, IQ2_S, IQ1_S, IQ1_M, Q2_K)}
ALL_FORMATS = {**FORMATS, **ONE_COLUMN}

BY_ID = {f.type_id: f for f in list(FORMATS.values()) + list(ONE_COLUMN.values())}

Q8K_BLOCK_BYTES = 292   # float d, int8 qs[256], int16 bsums[16] (src/quant/quant_formats.h:95)


def get(fmt) -> BlockFormat:
    if isinstance(fmt, BlockFormat):
        return fmt
    if isinstance(fmt, str):
        return ALL_FORMATS[fmt.upper()]
    return BY_ID[int(fmt)]
