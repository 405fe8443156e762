"""On-disk array stores: zarr arrays (checkpoints, token cache), jagged arrays, tree stores and the dataset cache."""
from .cache import SerialCacheWriter, TreeCache, build_or_load_cache  # noqa: F401
from .jagged_array import JaggedArrayStore  # noqa: F401
from .tree_store import TreeStore  # noqa: F401
