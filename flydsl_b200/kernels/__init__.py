"""Factory functions with the reference's names (FlyDSL ``kernels/`` directory)."""
from .blockscale_preshuffle_gemm import compile_blockscale_preshuffle_gemm  # noqa: F401
from .preshuffle_gemm import compile_preshuffle_gemm_a8  # noqa: F401
from .moe_blockscale_2stage import (  # noqa: F401
    MoeGemm2Mode,
    compile_moe_blockscale_gemm1,
    compile_moe_blockscale_gemm2,
    compile_moe_blockscale_gemm2_ex,
    compile_moe_reduction,
)
from .moe_gemm_2stage import (  # noqa: F401
    compile_moe_gemm1,
    compile_moe_gemm2,
    compile_moe_gemm2_ex,
)
from .int4_gemm import (  # noqa: F401
    compile_int4_weight_only_gemm,
    pack_int4_weight,
    quantize_int4_groupwise,
)
