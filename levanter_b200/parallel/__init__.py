"""Parallelism: the (replica, data, model) mesh, tensor-parallel regions, the sharded parameter engine (FSDP),
expert parallelism and the symmetric-memory communicator."""
