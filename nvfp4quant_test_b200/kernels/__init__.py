"""Drop-in counterparts of the reference's `kernels` package."""
from .kernel_ScaleSweep_MSE import (  # noqa: F401
    scalesweep_mse_nvfp4_quant_impl,
    scalesweep_mse_nvfp4_quant_out,
    scalesweep_mse_round_nvfp4_quant_impl,
    scalesweep_mse_round_nvfp4_quant_out,
)
from .kernel_ScaleSweep import (  # noqa: F401
    scalesweep_weighted_mse_nvfp4_quant_impl,
    scalesweep_weighted_mse_nvfp4_quant_out,
)
from .kernel_fused import scalesweep_nvfp4_quant_with_global_scale  # noqa: F401
from .kernel_amax import amax_nvfp4_quant_impl, amax_nvfp4_quant_out, scaled_fp4_quant  # noqa: F401
from .kernel_gemm import (PreparedWeight, cutlass_scaled_fp4_mm, nvfp4_scaled_mm, nvfp4_scaled_mm_grouped,  # noqa: F401
                          nvfp4_scaled_mm_prepared)
from .kernel_vllm import (  # noqa: F401
    create_fp4_output_tensors,
    round_up,
    swizzle_vllm_fp4_scale,
    unswizzle_vllm_fp4_scale,
)
from .linear import ActivationQuantizer, LinearGroup  # noqa: F401
