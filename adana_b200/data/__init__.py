"""Data layer: token-file readers, synthetic Zipf streams and dataset preparers."""
from .readers import AsyncFileLoader, DataReader, MultiFileDataReader, PinnedBatchStager
from .datasets import get_dataset, make_zipf_tokens, write_zipf_dataset

__all__ = ["AsyncFileLoader", "DataReader", "MultiFileDataReader", "PinnedBatchStager",
           "get_dataset", "make_zipf_tokens", "write_zipf_dataset"]
