#!/bin/bash
# One task per node under srun; each task starts one process per GPU.  Usage inside an sbatch script:
#   srun --ntasks-per-node=1 infra/run-slurm.sh levanter_b200.main.train_lm --config_path config/llama2_7b_b200.yaml
set -euo pipefail
export PYTHONPATH="${PYTHONPATH:-}:$(cd "$(dirname "$0")/.." && pwd)"
LOG_DIR="${LOG_DIR:-logs}"
mkdir -p "$LOG_DIR"
exec python -m levanter_b200.infra.launch -- "$@" > >(tee "$LOG_DIR/$(hostname).out") 2> >(tee "$LOG_DIR/$(hostname).err" >&2)
