"""Job launch helpers: a single-node / SLURM launcher around ``torch.distributed.run`` and small command-line utilities.
The reference's TPU-VM, GCP and Ray-cluster tooling (src/levanter/infra/) has no counterpart on a GPU node."""
