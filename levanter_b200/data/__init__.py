"""Data pipeline: datasets, permutations, mixtures, packing, the token cache and the resumable data loader."""
from ._preprocessor import BatchProcessor  # noqa: F401
from .dataset import AsyncDataset, EpochDataset, ListAsyncDataset, MappedAsyncDataset, SyncDataset  # noqa: F401
from .loader import DataLoader  # noqa: F401
from .mixture import MixtureDataset, StopStrategy  # noqa: F401
from .permutation import EraShufflingDataset, PermutationDataset  # noqa: F401
from .sharded_datasource import ShardedDataSource, datasource_from_hf, datasource_from_json, datasource_from_jsonl  # noqa: F401
from .utils import batched  # noqa: F401
