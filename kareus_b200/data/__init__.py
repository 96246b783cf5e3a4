"""Training data: Megatron-format indexed token files, GPT samples over them, per-rank batch iterator."""
from .gpt_dataset import (BlendedDataset, GPTDataset, GPTDatasetConfig, build_blend_index, build_sample_index,
                          split_documents)
from .indexed import IndexedDataset, IndexedDatasetWriter, best_dtype
from .loader import PretrainingBatches

__all__ = ["BlendedDataset", "build_blend_index", "GPTDataset", "GPTDatasetConfig", "IndexedDataset", "IndexedDatasetWriter", "PretrainingBatches",
           "best_dtype", "build_sample_index", "split_documents"]
