"""Render and submit one Slurm job per experiment directory, tracking each job's state in ``status.txt``.

    python submit_slurm_jobs.py --inp_dir tmp/sweep --qos high [--nb_slurm_array 4] [--only fail] --hf_token ...

State machine, CLI and resubmission filters follow the reference's ``submit_slurm_jobs.py:8-220``:
``init -> pending -> running -> {completed, fail, oom, timeout}``; ``--only`` resubmits one class, completed jobs
are never resubmitted, ``--nb_slurm_array N`` chains the jobs into N dependency lists (``afterany``). The job script
is rendered from ``template/base_job.slurm``; ``--dry_run`` renders the scripts without calling ``sbatch``.
"""
import argparse
import json
import os
import subprocess
from enum import Enum
from typing import List, Optional

from jinja2 import Template

HERE = os.path.dirname(os.path.abspath(__file__))
MAX_GPU_PER_NODE = 8


class Status(Enum):
    INIT = "init"
    PENDING = "pending"
    RUNNING = "running"
    FAIL = "fail"
    OOM = "oom"
    TIMEOUT = "timeout"
    COMPLETED = "completed"


class Job:
    def __init__(self, root_path: str, qos: str) -> None:
        self.root_path = root_path
        self.name = os.path.basename(root_path)
        self.config = os.path.join(root_path, "config.json")
        self.qos = qos
        if not os.path.exists(self._status_path()):
            self.set_status(Status.INIT)
        self.status = self.get_status()

    def _status_path(self) -> str:
        return os.path.join(self.root_path, "status.txt")

    def get_status(self) -> Status:
        with open(self._status_path(), "r") as f:
            text = f.read().strip()
        try:
            return Status(text)
        except ValueError:
            raise ValueError(f"Invalid status '{text}' in {self._status_path()}")

    def set_status(self, status: Status) -> Status:
        with open(self._status_path(), "w") as f:
            f.write(status.value)
        self.status = status
        return status


def world_layout(config: dict):
    d = config["distributed"]
    world = d["tp_size"] * d["cp_size"] * d["pp_size"] * d["dp_size"]
    assert world <= MAX_GPU_PER_NODE or world % MAX_GPU_PER_NODE == 0, f"world size {world} does not tile nodes of 8 GPUs"
    nodes = max(1, world // MAX_GPU_PER_NODE)
    per_node = min(MAX_GPU_PER_NODE, world // nodes)
    assert nodes * per_node == world
    return nodes, per_node


class Scheduler:
    def __init__(self, inp_dir: str, qos: str) -> None:
        paths = sorted(os.path.abspath(root) for root, dirs, files in os.walk(inp_dir)
                       if "config.json" in files)
        self.job_lists: List[Job] = [Job(p, qos) for p in paths]

    def keep_only_jobs(self, status: Status) -> List[Job]:
        return [j for j in self.job_lists if j.status == status]

    def filter_out_jobs(self, status: Status) -> List[Job]:
        return [j for j in self.job_lists if j.status != status]

    def create_slurm_script(self, job: Job) -> str:
        with open(job.config, "r") as f:
            config = json.load(f)
        nodes, per_node = world_layout(config)
        with open(os.path.join(HERE, "template", "base_job.slurm"), "r") as f:
            template = Template(f.read())
        out = os.path.join(job.root_path, "job.slurm")
        with open(out, "w") as f:
            f.write(template.render(nodes=nodes, n_proc_per_node=per_node, root_path=job.root_path, config=job.config,
                                    qos=job.qos, repo_path=HERE))
        print(f"Slurm script created at {out}")
        return out

    def launch_dependency(self, job_array: List[Job], env_vars, dry_run: bool = False) -> None:
        prev: Optional[str] = None
        for job in job_array:
            cmd = ["sbatch", "--parsable"] + ([f"--dependency=afterany:{prev}"] if prev else []) + \
                  [os.path.join(job.root_path, "job.slurm")]
            if dry_run:
                print("[dry run]", " ".join(cmd))
                prev = "0"
            else:
                prev = subprocess.run(cmd, env=env_vars, capture_output=True, text=True).stdout.strip()
            job.set_status(Status.PENDING)

    def check_status(self) -> dict:
        counts = {s.value: 0 for s in Status}
        for job in self.job_lists:
            counts[job.get_status().value] += 1
        print(f"{'Status':<10} | {'Count':<6}")
        print(f"{'-' * 10}-|-{'-' * 6}")
        for k, v in counts.items():
            print(f"{k.capitalize():<10} | {v:<6}")
        print(f"{'-' * 10}-|-{'-' * 6}")
        print(f"{'Total':<10} | {sum(counts.values()):<6}")
        return counts


def submit_jobs(inp_dir, qos, hf_token, nb_slurm_array, only: str = None, dry_run: bool = False):
    scheduler = Scheduler(inp_dir, qos)
    env_vars = os.environ.copy()
    if hf_token:
        env_vars["HUGGINGFACE_TOKEN"] = hf_token
    total = len(scheduler.job_lists)
    if only is not None:
        if only not in ("fail", "pending", "timeout", "running"):
            raise ValueError(f"--only must be one of fail|pending|timeout|running, got {only}")
        scheduler.job_lists = scheduler.keep_only_jobs(Status(only))
        if not scheduler.job_lists:
            print(f"No '{only}' jobs to resubmit")
            return scheduler
        print(f"Only {len(scheduler.job_lists)}/{total} jobs with status '{only}' will be resubmitted")
    scheduler.job_lists = scheduler.filter_out_jobs(Status.COMPLETED)

    if nb_slurm_array > 0:
        base, extra = divmod(len(scheduler.job_lists), nb_slurm_array)
        start = 0
        for i in range(nb_slurm_array):
            n = base + (1 if i < extra else 0)
            chunk = scheduler.job_lists[start:start + n]
            start += n
            print(f"Launching job Dependency array {i + 1} with {n} jobs")
            for job in chunk:
                scheduler.create_slurm_script(job)
            scheduler.launch_dependency(chunk, env_vars, dry_run)
    else:
        for job in scheduler.job_lists:
            script = scheduler.create_slurm_script(job)
            if dry_run:
                print("[dry run] sbatch", script)
            else:
                subprocess.run(["sbatch", script], env=env_vars)
            job.set_status(Status.PENDING)
    return scheduler


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Submit jobs to the cluster")
    parser.add_argument("--inp_dir", type=str, help="Input directory containing the jobs")
    parser.add_argument("--qos", type=str, help="QOS of the jobs")
    parser.add_argument("--nb_slurm_array", type=int, default=0, help="Number of slurm arrays")
    parser.add_argument("--only", type=str, default=None, help="Filter the jobs to submit")
    parser.add_argument("--hf_token", type=str, default=None, help="Huggingface token")
    parser.add_argument("--dry_run", action="store_true", help="render job scripts, do not call sbatch")
    parser.add_argument("--check_status", action="store_true", help="print a status table and exit")
    args = parser.parse_args()
    if args.check_status:
        Scheduler(args.inp_dir, args.qos).check_status()
    else:
        submit_jobs(args.inp_dir, args.qos, args.hf_token, args.nb_slurm_array, only=args.only, dry_run=args.dry_run)
