"""Data pipeline: datasets, permutations, mixtures, packing, the token cache and the resumable data loader."""
from .dataset import AsyncDataset, EpochDataset, ListAsyncDataset, MappedAsyncDataset, SyncDataset  # noqa: F401
from .loader import DataLoader  # noqa: F401
