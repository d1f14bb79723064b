"""B200-native block-quantized (group-32) weight matmuls: packed weights, quantized linear,
lm_head, MoE dispatch / grouped experts / combine, tensor- and expert-parallel sharding.
All per-token compute runs in libb200q.so (hand-written CUDA for sm_100a)."""
from ._lib import (BqError, DT_BF16, DT_F32, FMT_Q4, FMT_Q8, PATH_AUTO, PATH_MMA, PATH_SIMT, PATH_TENSOR)
from .ops import (LMHead, MoEExperts, PackedWeight, PeerComm, PeerEP, QuantLinear, interleave_gate_up, moe_combine, moe_gather, moe_permute,
                  moe_route, shard)

__all__ = ["BqError", "DT_BF16", "DT_F32", "FMT_Q4", "FMT_Q8", "PATH_AUTO", "PATH_MMA", "PATH_SIMT",
           "PATH_TENSOR", "LMHead", "MoEExperts", "PackedWeight", "PeerComm", "PeerEP", "QuantLinear", "interleave_gate_up", "moe_combine", "moe_gather",
           "moe_permute", "moe_route", "shard"]
