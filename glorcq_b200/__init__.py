"""glorcq_b200: B200 (sm_100a) kernels behind the GLoRCQ real-quant inference API.

    from glorcq_b200.quantized_linear import GLoRCQLinear, GLoRCQExperts
    from glorcq_b200.moe_block import GraphCompatibleMoeBlock
    from glorcq_b200.graph_wrapper import GLoRCQGraphWrapper
    from glorcq_b200.kernels import turbo_dequant_matmul_fused, gptq_dequant_matmul_fused, ...

mirror the reference's ``inference`` package; the compute goes through libglorcq_b200.so
(include/glorcq_b200.h).  There is no CPU or PyTorch fallback.
"""

__version__ = "0.1.0"
