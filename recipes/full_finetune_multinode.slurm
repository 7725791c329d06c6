#!/bin/bash
# Multi-node full fine-tuning under SLURM: one `tune run` (torchrun) launcher per node, eight ranks per node,
# c10d rendezvous on the first node of the allocation.  Adjust the #SBATCH lines and --nnodes to your node count.
#
#   sbatch recipes/full_finetune_multinode.slurm
#
#SBATCH --job-name=torchtune-b200-multi-node
#SBATCH --nodes=2
#SBATCH --ntasks=2
#SBATCH --gpus-per-task=8
#SBATCH --cpus-per-task=96
#SBATCH --partition=train

set -euo pipefail

# rendezvous endpoint = first host of the allocation
mapfile -t HOSTS < <(scontrol show hostnames "$SLURM_JOB_NODELIST")
HEAD_NODE="${HOSTS[0]}"
HEAD_IP="$(srun --nodes=1 --ntasks=1 -w "$HEAD_NODE" hostname --ip-address | awk '{print $1}')"
echo "rendezvous at ${HEAD_IP}:29500 over ${#HOSTS[@]} nodes"

# set these when the fabric needs an explicit interface:
# export NCCL_SOCKET_IFNAME=...
# export GLOO_SOCKET_IFNAME=...
export TORCH_DIST_INIT_BARRIER=1
export LOGLEVEL=INFO

# activate your environment here (conda / venv)

SHARED_FS=/mnt/slurm                       # a file system every node sees
CHECKPOINT_DIR="$SHARED_FS/Llama-3.3-70B-Instruct"
OUTPUT_DIR="$SHARED_FS/Llama3.3-70B-fft-output"

srun tune run --nnodes "${#HOSTS[@]}" --nproc_per_node 8 --rdzv_id 101 --rdzv_backend c10d --rdzv_endpoint "${HEAD_IP}:29500" \
    full_finetune_distributed --config llama3_3/70B_full \
    checkpointer.checkpoint_dir="$CHECKPOINT_DIR" tokenizer.path="$CHECKPOINT_DIR/original/tokenizer.model" output_dir="$OUTPUT_DIR"
