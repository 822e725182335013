from .dataset import BlendedDataSource, DocumentDataSource
from .indexed_dataset import ArrayRecordDocDataset, MMapIndexedDataset
from .pipeline import ShiftTokens, create_eval_iterator, create_train_iterator
from .tokenizer import Tokenizer

__all__ = ["create_train_iterator", "create_eval_iterator", "ShiftTokens", "DocumentDataSource",
           "BlendedDataSource", "MMapIndexedDataset", "ArrayRecordDocDataset", "Tokenizer"]
