#!/bin/bash
# Starts one training process per GPU on every node of a multi-node job (one rank per GPU over NCCL).
#
# The job scheduler (or a loop over ssh) runs this script once on every node with the same variables:
#   NNODES                    number of nodes
#   NODE_RANK                 0 .. NNODES-1
#   JAX_COORDINATOR_ADDRESS   host name / IP of node 0 (also read as MASTER_ADDR)
#   JAX_COORDINATOR_PORT      rendezvous port on node 0 (also read as MASTER_PORT)
#   GPUS_PER_NODE             ranks to start on this node
#   COMMAND                   the training command, e.g.
#                             "python -m maxtext.train maxtext_b200/configs/base.yml model_name=llama3-8b hardware=gpu_multiprocess ..."
# The variable names are those of the reference's launcher (tools/orchestration/gpu_multi_process_run.sh), so job specs written
# for it keep working; the ranks themselves are started with torch.distributed.run, which exports RANK / LOCAL_RANK /
# WORLD_SIZE / MASTER_ADDR / MASTER_PORT for `parallel.mesh.init_distributed`.
# Optional: USE_GPUDIRECT=tcpx|fastrak|rdma selects NCCL network settings for multi-node fabrics; NCCL_DEBUG etc. pass through.
set -euo pipefail

: "${NNODES:?Must set NNODES}"
: "${NODE_RANK:?Must set NODE_RANK}"
: "${JAX_COORDINATOR_PORT:?Must set JAX_COORDINATOR_PORT}"
: "${JAX_COORDINATOR_ADDRESS:?Must set JAX_COORDINATOR_ADDRESS}"
: "${GPUS_PER_NODE:?Must set GPUS_PER_NODE}"
: "${COMMAND:?Must set COMMAND}"

case "${USE_GPUDIRECT:-none}" in
  tcpx|fastrak)
    export NCCL_CROSS_NIC=0 NCCL_NET_GDR_LEVEL=PIX NCCL_PROTO=Simple NCCL_SOCKET_IFNAME="${NCCL_SOCKET_IFNAME:-eth0}"
    export NCCL_P2P_NET_CHUNKSIZE=524288 NCCL_P2P_NVL_CHUNKSIZE=1048576 NCCL_P2P_PCI_CHUNKSIZE=524288
    ;;
  rdma)
    export NCCL_IB_DISABLE=0 NCCL_NET_GDR_LEVEL=SYS
    ;;
  none) ;;
  *) echo "unknown USE_GPUDIRECT=${USE_GPUDIRECT}" >&2; exit 2 ;;
esac
# one communicator per mesh axis is created at start-up: give NCCL enough connections, keep launch order deterministic
export CUDA_DEVICE_MAX_CONNECTIONS="${CUDA_DEVICE_MAX_CONNECTIONS:-8}"
export TORCH_NCCL_ASYNC_ERROR_HANDLING="${TORCH_NCCL_ASYNC_ERROR_HANDLING:-1}"
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"

# COMMAND is "python [-m module | script.py] args...": torch.distributed.run replaces the interpreter
read -r -a CMD <<< "${COMMAND}"
if [[ "${CMD[0]}" == python* ]]; then CMD=("${CMD[@]:1}"); fi

echo "node ${NODE_RANK}/${NNODES}: starting ${GPUS_PER_NODE} ranks, rendezvous ${JAX_COORDINATOR_ADDRESS}:${JAX_COORDINATOR_PORT}"
exec python -m torch.distributed.run --nnodes="${NNODES}" --node-rank="${NODE_RANK}" --nproc-per-node="${GPUS_PER_NODE}" \
  --master-addr="${JAX_COORDINATOR_ADDRESS}" --master-port="${JAX_COORDINATOR_PORT}" "${CMD[@]}"
