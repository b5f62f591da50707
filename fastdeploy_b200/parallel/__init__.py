"""Multi-GPU layer: peer-memory communicator, fused GEMM + collective kernels, tensor-parallel
layers and the data-parallel serving scheduler."""
from .comm import Communicator, HeapBlock, HeapLayout, shard_rows  # noqa: F401
from .tp import ColumnParallelLinear, RowParallelLinear, TensorParallelMLP  # noqa: F401
from .vit import TensorParallelViT, VIT_SIZES, random_vit_weights, vit_reference  # noqa: F401
from .health import RankHealth, RankLostError  # noqa: F401
