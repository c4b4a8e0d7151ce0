#!/bin/bash
#SBATCH --job-name=job-picotron-b200
#SBATCH --time=00:30:00
#SBATCH --nodes={{ nodes }}
#SBATCH --gres=gpu:{{ n_proc_per_node }}
#SBATCH --qos={{ qos }}
#SBATCH --ntasks-per-node=1
#SBATCH --cpus-per-task=96
#SBATCH --exclusive
#SBATCH --output={{ root_path }}/log_%j.out
#SBATCH --error={{ root_path }}/log_%j.out

# One torchrun per node, one rank per GPU. The job records its own state in status.txt:
#   pending -> running -> completed | oom | timeout | fail   (classified from the exit code and the log)

STATUS_FILE={{ root_path }}/status.txt

mark_running_when_started() {
    local job_id=$1
    while true; do
        local state
        state=$(squeue --job "$job_id" --noheader --format=%T)
        if [ -z "$state" ]; then break; fi
        if [ "$state" = "RUNNING" ]; then printf "running" > "$STATUS_FILE"; break; fi
        sleep 10
    done
}

echo "START TIME: $(date)"
export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
export MASTER_PORT=$((1024 + RANDOM % 64511))
export CUDA_DEVICE_MAX_CONNECTIONS="1"
export OMP_NUM_THREADS=1

REPO={{ repo_path }}
CMD="$REPO/train.py --config {{ config }}"
LAUNCHER="torchrun --nproc_per_node={{ n_proc_per_node }} --nnodes={{ nodes }} --node_rank=$SLURM_NODEID --rdzv_endpoint ${MASTER_ADDR}:${MASTER_PORT} --rdzv_backend c10d --max_restarts 0 --tee 3"

cd "$REPO"
mark_running_when_started "$SLURM_JOB_ID" &

echo "Running command: $CMD"
srun -u $LAUNCHER $CMD
exit_status=$?

LOG={{ root_path }}/log_${SLURM_JOB_ID}.out
if [ $exit_status -eq 0 ]; then
    printf "completed" > "$STATUS_FILE"
elif grep -q "OutOfMemoryError" "$LOG"; then
    printf "oom" > "$STATUS_FILE"
elif grep -q " CUDA error: an illegal memory access" "$LOG"; then
    printf "oom" > "$STATUS_FILE"
elif [ $exit_status -eq 124 ] || grep -q "Timeout" "$LOG"; then
    printf "timeout" > "$STATUS_FILE"
else
    printf "fail" > "$STATUS_FILE"
fi
echo "END TIME: $(date)"
