#!/bin/bash
# Mamba2-7B pre-training on 8xB200 nodes: TP=8 + sequence parallel + ZeRO-1, bf16, GBS 1024, MBS 1, seq 2048.
# Usage: ./tp_zero1_mamba2_7B_pretrain.sh DATA_DIR CHECKPOINT_DIR
# Hyper-parameters follow the reference launch script (tp_zero1_mamba2_7B_pretrain.sh:17-45,85-86,124-145);
# the Neuron compiler/runtime variables are replaced by NCCL ones.
set -euo pipefail
DATA_PATH=${1:?data dir}
CKPT_DIR=${2:?checkpoint dir}

export NCCL_NVLS_ENABLE=${NCCL_NVLS_ENABLE:-1}
export TORCH_NCCL_ASYNC_ERROR_HANDLING=1
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-8}
export MALLOC_ARENA_MAX=64

MODEL=${MODEL:-Mamba7B}
TP_DEGREE=${TP_DEGREE:-8}
GBS=${GBS:-1024}
MBS=${MBS:-1}
LR=${LR:-3e-4}
WARMUP_STEPS=${WARMUP_STEPS:-1500}
TOTAL_STEPS=${TOTAL_STEPS:-28000}
CKPT_FREQ=${CKPT_FREQ:-5000}
SEQ_LEN=${SEQ_LEN:-2048}
GPUS_PER_NODE=${GPUS_PER_NODE:-8}

if [ -n "${SLURM_NTASKS:-}" ]; then
  NODES=$SLURM_NTASKS
  NODE_RANK=$SLURM_NODEID
  MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
  DIST_ARGS="--nproc_per_node $GPUS_PER_NODE --nnodes $NODES --node_rank $NODE_RANK --master_addr $MASTER_ADDR --master_port 44000"
else
  NODES=1
  DIST_ARGS="--nproc_per_node $GPUS_PER_NODE --nnodes 1 --master_addr 127.0.0.1 --master_port 44000"
fi
WORLD=$((GPUS_PER_NODE * NODES))
DP=$((WORLD / TP_DEGREE))
ACC_STEPS=$((GBS / MBS / DP))
# CUDA graphs: every micro-step (forward + backward + fused collectives) and the optimizer update replay as captured
# graphs, which takes the host out of the loop (thousands of launches per micro-step); CUDA_GRAPH=0 runs eagerly.
# SSM_B200_FUSED_AG=0 / SSM_B200_FUSED_RS=0 (environment) run the all-gather GEMM / the reduce-scatter GEMM as NCCL
# collective + plain GEMM kernel; `python bench.py --gpus N` prints the step time of all four combinations on this machine.
GRAPH_FLAG=""
if [ "${CUDA_GRAPH:-1}" != "0" ]; then GRAPH_FLAG="--cuda_graph"; fi
echo "world=$WORLD tp=$TP_DEGREE dp=$DP acc_steps=$ACC_STEPS cuda_graph=${CUDA_GRAPH:-1}"

torchrun $DIST_ARGS train.py \
  --model $MODEL --tp $TP_DEGREE --use_zero_1 --sequence_parallel_enabled --rmsnorm_across_groups \
  --dtype bfloat16 --vocab_size 50288 --data_dir "$DATA_PATH" --batch $MBS --seq_len $SEQ_LEN \
  --grad_accum_usteps $ACC_STEPS --lr $LR --weight_decay 0.1 --beta1 0.9 --beta2 0.95 \
  --warmup_steps $WARMUP_STEPS --max_steps $TOTAL_STEPS --logging_interval 1 \
  --checkpoint_freq $CKPT_FREQ --checkpoint_dir "$CKPT_DIR" --num_kept_checkpoint 3 --save_last_step \
  $GRAPH_FLAG \
  --tag mamba2_7b "${@:3}"
