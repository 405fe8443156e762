"""On-disk array stores: zarr arrays (checkpoints, token cache), jagged arrays and tree stores."""
