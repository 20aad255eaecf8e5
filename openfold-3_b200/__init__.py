"""B200-native (sm_100a) drop-in for OpenFold3's Pairformer hot path.

Import name ``openfold3_b200`` (the directory name is not a Python identifier; the
repository's ``__graft_entry__.load_package()`` registers it). Host code is Python/PyTorch
used for tensors, streams and ``torch.distributed`` only; every forward runs hand-written
CUDA kernels from the in-tree C-ABI library ``libof3b200.so``.
"""

from . import dap, init_config, lib, weights
from .patch import patch_openfold3, unpatch_openfold3
from .graphs import GraphedModule
from .modules import (
    AdaLN,
    Attention,
    AttentionPairBias,
    ConditionedTransitionBlock,
    DiffusionTransformer,
    DiffusionTransformerBlock,
    DropoutRowwise,
    LayerNorm,
    Linear,
    PairBlock,
    PairFormerBlock,
    PairFormerStack,
    PairStack,
    SwiGLU,
    SwiGLUTransition,
    TriangleAttention,
    TriangleAttentionEndingNode,
    TriangleAttentionStartingNode,
    TriangleMultiplicationIncoming,
    TriangleMultiplicationOutgoing,
    TriangleMultiplicativeUpdate,
)

__all__ = [n for n in dir() if not n.startswith("_")]
