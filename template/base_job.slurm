#!/bin/bash
# Slurm job of one experiment directory ({{ root_path }}): one torchrun per node, one rank per GPU.
# The job keeps {{ root_path }}/status.txt up to date with the state machine that submit_slurm_jobs.py reads:
#   pending -> running -> completed | oom | timeout | fail
#SBATCH --job-name=picotron-b200
#SBATCH --qos={{ qos }}
#SBATCH --nodes={{ nodes }}
#SBATCH --ntasks-per-node=1
#SBATCH --gres=gpu:{{ n_proc_per_node }}
#SBATCH --cpus-per-task=96
#SBATCH --exclusive
#SBATCH --time=00:30:00
#SBATCH --output={{ root_path }}/log_%j.out
#SBATCH --error={{ root_path }}/log_%j.out

run_dir={{ root_path }}
repo_dir={{ repo_path }}
status_file="$run_dir/status.txt"
log_file="$run_dir/log_${SLURM_JOB_ID}.out"

set_status() { printf "%s" "$1" > "$status_file"; }

# Flip pending -> running once the scheduler reports the job as RUNNING (polled in the background).
watch_for_start() {
    while state=$(squeue --job "$SLURM_JOB_ID" --noheader --format=%T) && [ -n "$state" ]; do
        if [ "$state" = "RUNNING" ]; then set_status running; return; fi
        sleep 10
    done
}

# Final state from the exit code of srun and, for failures, from what the ranks printed.
classify() {
    local rc=$1
    if [ "$rc" -eq 0 ]; then echo completed; return; fi
    if grep -q -e "OutOfMemoryError" -e " CUDA error: an illegal memory access" "$log_file"; then echo oom; return; fi
    if [ "$rc" -eq 124 ] || grep -q "Timeout" "$log_file"; then echo timeout; return; fi   # 124: the step watchdog
    echo fail
}

echo "START TIME: $(date)"
head_node=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
rdzv_port=$((1024 + RANDOM % 64511))
export OMP_NUM_THREADS=1
export CUDA_DEVICE_MAX_CONNECTIONS=1        # kernel issue order = stream order (overlap of compute and collectives)

cd "$repo_dir"
watch_for_start &

launch="torchrun --nnodes={{ nodes }} --nproc_per_node={{ n_proc_per_node }} --node_rank=\$SLURM_NODEID \
--rdzv_backend c10d --rdzv_endpoint ${head_node}:${rdzv_port} --max_restarts 0 --tee 3"
target="$repo_dir/train.py --config {{ config }}"
echo "Running command: $target"
srun -u bash -c "$launch $target"
set_status "$(classify $?)"
echo "END TIME: $(date)"
