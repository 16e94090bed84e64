"""Blackwell (sm_100a) block-scaled GEMM: NVFP4 / MXFP8 operands, fp32 accumulation in
tensor memory, bf16 or fused-NVFP4 output; dense, batched, grouped (MoE) and
tensor-parallel forms.  The Python surface keeps the shape of the CUTLASS Python
Operator API; the work is done by hand-written CUDA behind a C ABI
(``include/bsgemm.h``, loaded by ``cutlass_b200.lib``)."""
from .arguments import (DenseTensor, EpilogueDescriptor, GemmArguments, GemmProblemSize, GroupedGemmArguments,
                        Mxfp8Quant, Nvfp4Quant, ScaledOperand, ScaleMode, ScaleSwizzleMode)
from .operator import (AllocationRequirement, BlockScaledGemmOperator, CompiledArtifact,
                       GroupedBlockScaledGemmOperator, NativeProvider, Operator, OperatorMetadata, Workspace, all_operators,
                       get_operators, to_cuda_stream)
from .quantize import quantize_blockscaled
from .status import Status

__all__ = [
    "AllocationRequirement", "BlockScaledGemmOperator", "CompiledArtifact", "DenseTensor", "EpilogueDescriptor",
    "GemmArguments", "GemmProblemSize", "GroupedBlockScaledGemmOperator", "GroupedGemmArguments", "Mxfp8Quant", "NativeProvider", "Nvfp4Quant",
    "Operator", "OperatorMetadata", "ScaleMode", "ScaleSwizzleMode", "ScaledOperand", "Status", "Workspace",
    "all_operators", "get_operators", "quantize_blockscaled", "to_cuda_stream",
]
__version__ = "0.1.0"
