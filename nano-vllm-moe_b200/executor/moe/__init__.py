"""MoE expert FFN on FP8 operands; mirrors nanovllm/executor/moe of the reference."""
from .config import MoEParallelConfig, make_ep_tp_groups, make_moe_parallel_config
from .experts import Fp8Experts, Fp8ExpertWeights
from .kernel import MoEKernel
from .prepare_finalize import (FixedCapacityAllToAllPrepareFinalize, NoEPPrepareFinalize, PrepareResult,
                               TorchAllToAllPrepareFinalize)
from .router import MoERouter, SoftmaxTopKRouter

__all__ = ["MoEParallelConfig", "make_moe_parallel_config", "make_ep_tp_groups", "Fp8Experts", "Fp8ExpertWeights", "MoEKernel",
           "NoEPPrepareFinalize", "TorchAllToAllPrepareFinalize", "FixedCapacityAllToAllPrepareFinalize", "PrepareResult", "MoERouter", "SoftmaxTopKRouter"]
