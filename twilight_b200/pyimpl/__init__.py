"""``twilight_b200.pyimpl``: selector / pruner functions and statistics with the interface of the
reference's ``twilight.pyimpl`` (mask-returning), implemented on the CUDA kernels."""
from .attention import SparseDecodeAttention, enable_sparse_attention  # noqa: F401
from .quest import quest_selector  # noqa: F401
from .state import (CompressorType, HistoryBudgetInfo, IndexSelectorType,  # noqa: F401
                    WeightEstimatorType, WeightPrunerType)
from .top_k import oracle_topk_selector, top_k  # noqa: F401
from .top_p import top_p_unnormalized  # noqa: F401
