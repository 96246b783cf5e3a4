"""Training data: Megatron-format indexed token files, GPT samples over them, per-rank batch iterator."""
from .gpt_dataset import (BlendedDataset, GPTDataset, GPTDatasetConfig, build_blend_index, build_sample_index,
                          split_documents)
from .indexed import IndexedDataset, IndexedDatasetWriter, best_dtype
from .factory import TokenData, parse_data_path
from .loader import PretrainingBatches

__all__ = ["BlendedDataset", "build_blend_index", "GPTDataset", "GPTDatasetConfig", "IndexedDataset", "IndexedDatasetWriter", "PretrainingBatches", "TokenData", "parse_data_path",
           "best_dtype", "build_sample_index", "split_documents"]
