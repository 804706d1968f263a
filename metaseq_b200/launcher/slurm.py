"""Turns a sweep into runnable jobs: local ``python -m metaseq_b200.cli.train`` processes or SLURM
``sbatch`` submissions with requeue-on-signal (reference: metaseq/launcher/slurm.py:33-593).

Behaviours kept: save directory name from the sweep's ``save_dir_key`` fragments; a run whose
directory already holds a finished ``train.log`` is skipped unless ``--resume-finished``; the
sbatch script traps USR1 (sent 180 s before the time limit via ``--signal B:USR1@180``) and
requeues the job; ``NCCL_ASYNC_ERROR_HANDLING=1`` and Azure fabric settings are exported for the
job; code can be snapshotted so that queued jobs do not see later edits."""
from __future__ import annotations

import datetime
import fnmatch
import hashlib
import itertools
import os
import random
import shlex
import shutil
import subprocess
import sys
import textwrap
from collections import OrderedDict
from pathlib import Path
from typing import List

from .opt_job_constants import ComputeEnvs
from .sweep import grid_product
from .tombyard import tombstones


def main(get_grid, postprocess_hyperparams, args, scheduler_args=None):
    def dry_run(msg):
        if args.dry_run:
            print(f"| dry-run:  {msg}")
        return args.dry_run

    if args.local:
        args.num_nodes = 1
    grid = get_grid(args)
    configs = list(_expand(grid, args))
    sweep_config = {}
    save_dirs = []
    for i, hp_values in enumerate(configs):
        config = OrderedDict((hp.name, hp) for hp in hp_values)
        postprocess_hyperparams(args, config)
        if args.num_trials > 0 and i >= args.num_trials:
            break
        save_dir = launch_train(args, list(config.values()), dry_run)
        if save_dir is not None:
            save_dirs.append(save_dir)
    return save_dirs


def _expand(grid, args):
    import copy

    combos = []
    for g in grid_product(grid):
        combos.append(copy.deepcopy(g))
    if args.num_trials > 0:
        random.Random(args.seed).shuffle(combos)
    return combos


def set_env(args, env, dry_run):
    if "OMP_NUM_THREADS" not in env:
        env["OMP_NUM_THREADS"] = "2"
    env["NCCL_ASYNC_ERROR_HANDLING"] = "1"
    if args.local:
        if not dry_run("start training locally"):
            if "CUDA_VISIBLE_DEVICES" not in env:
                env["CUDA_VISIBLE_DEVICES"] = ",".join(map(str, range(args.num_gpus)))
            env["NCCL_DEBUG"] = env.get("NCCL_DEBUG", "WARN")
    else:
        env.setdefault("NCCL_SOCKET_IFNAME", "^docker0,lo")
        if getattr(args, "cluster_env", "") == ComputeEnvs.AZURE.value:
            env.update(get_azure_env())


def get_azure_env():
    """Fabric settings for Azure InfiniBand SKUs."""
    return {
        "NCCL_TOPO_FILE": "/opt/microsoft/ndv4-topo.xml",
        "NCCL_IB_PCI_RELAXED_ORDERING": "1",
        "UCX_IB_PCI_RELAXED_ORDERING": "on",
        "UCX_TLS": "tcp",
        "UCX_NET_DEVICES": "eth0",
        "CUDA_DEVICE_ORDER": "PCI_BUS_ID",
        "NCCL_SOCKET_IFNAME": "eth0",
        "NCCL_NET_GDR_LEVEL": "5",
    }


def is_job_valid(args, save_dir, dry_run):
    """Whether a run should be (re)submitted: not when it finished (unless ``--resume-finished``), not when its last
    job failed (unless ``--resume-failed``), not while it is in progress."""
    if is_finished(save_dir):
        if args.resume_finished:
            dry_run(f"restart previously finished run: {save_dir}")
        else:
            print(f"skip finished run (override with --resume-finished): {save_dir}")
            return False
    elif has_failed(save_dir):
        if getattr(args, "resume_failed", False):
            dry_run(f"resume failed run: {save_dir}")
        else:
            print(f"skip failed run (override with --resume-failed): {save_dir}")
            return False
    elif has_started(save_dir, args):
        print(f"skip in progress run: {save_dir}")
        return False
    return True


def has_failed(save_dir) -> bool:
    """The stderr file of the newest job (``train.stderr.<jobid>``) has any non-blank line."""
    if not os.path.isdir(save_dir):
        return False
    job_ids = [int(fn.rsplit(".", 1)[1]) for fn in os.listdir(save_dir)
               if fn.startswith("train.stderr.") and fn.rsplit(".", 1)[1].isdigit()]
    if not job_ids:
        return False
    with open(os.path.join(save_dir, f"train.stderr.{max(job_ids)}"), "r", errors="replace") as h:
        return any(line.strip() for line in h)


def has_started(save_dir, args=None) -> bool:
    return os.path.exists(os.path.join(save_dir, "train.log"))


def write_git_commit(train_log: str) -> None:
    """Appends the id of the checked-out commit to the training log (nothing outside a git checkout)."""
    try:
        commit = subprocess.check_output(["git", "rev-parse", "HEAD"], encoding="utf-8", stderr=subprocess.DEVNULL).strip()
    except (OSError, subprocess.CalledProcessError):
        return
    with open(train_log, "a") as h:
        print(f"commit {commit}", file=h)


def is_finished(save_dir):
    train_log = os.path.join(save_dir, "train.log")
    if not os.path.exists(train_log):
        return False
    with open(train_log, "r") as h:
        lines = h.readlines()
    if not lines:
        return False
    return "done training" in lines[-1]


has_finished = is_finished


def get_save_dir_name(args, hp_values) -> str:
    parts = [args.prefix]
    for hp in hp_values:
        key = hp.get_save_dir_key()
        if key is not None:
            parts.append(str(key))
    if args.num_nodes * args.num_gpus > 0:
        parts.append(f"ngpu{args.num_nodes * args.num_gpus}")
    return ".".join(p for p in parts if p)


def gen_train_command(args, env, hp_values, oss_destination, save_dir, save_dir_key):
    """Argument vector of one training process (module form: ``python -m <script>``)."""
    cmd = [args.python]
    script = args.script
    if script.endswith(".py"):
        cmd.append(os.path.join(oss_destination, script) if oss_destination else script)
    else:
        cmd += ["-m", script]
    cmd += ["--distributed-world-size", str(args.num_nodes * args.num_gpus)]
    if args.num_nodes > 1 or (args.num_gpus > 1 and not args.local):
        cmd += ["--distributed-port", str(get_random_port())]
    if getattr(args, "data", None) is not None and not any(hp.name == "--data" for hp in hp_values):
        cmd.append(args.data)  # positional, unless the grid already passes it by name
    run_name = save_dir_key  # <prefix>.<keys>.ngpu<N>, the basename of save_dir
    if not getattr(args, "no_save_dir", False):
        local_root = getattr(args, "local_checkpoints_dir", None)
        cmd += ["--save-dir", os.path.join(local_root, run_name) if local_root else save_dir]
    upload = getattr(args, "full_azure_upload_path", None)
    if upload is not None:
        if getattr(args, "azure_folder_auto_name", False):
            from urllib.parse import urlparse

            url = urlparse(upload)
            upload = url._replace(path=os.path.join(url.path, run_name) + "/").geturl()
        cmd += ["--save-async", "--cloud-upload-path", upload]
    if args.update_freq:
        cmd += ["--update-freq", str(args.update_freq)]
    if getattr(args, "log_tensorboard", False) or args.tensorboard_logdir:
        cmd += ["--tensorboard-logdir", args.tensorboard_logdir or os.path.join(save_dir, "tb")]
    for hp in hp_values:
        cmd += hp.get_cli_args()
    return cmd


def get_random_port():
    state = random.getstate()
    random.seed()
    port = random.randint(10000, 20000)
    random.setstate(state)
    return port


def gen_srun_command_and_str(args, env, save_dir_key, train_log, train_stderr, train_cmd, post_cmds=None):
    base = [
        "srun", "--job-name", f"{args.prefix}.{save_dir_key}", "--output", train_log, "--error", train_stderr,
        "--open-mode", "append", "--unbuffered", "--cpu-bind", getattr(args, "cpu_bind", "none"),
    ]
    if args.salloc:
        base += ["--nodes", str(args.num_nodes), "--ntasks-per-node", str(args.num_gpus), "--ntasks",
                 str(args.num_gpus * args.num_nodes), "--cpus-per-task", str(args.cpus_per_task)]
    srun_cmd = base + train_cmd
    srun_str = " ".join(map(shlex.quote, srun_cmd))
    for post in post_cmds or []:
        srun_str = f"( {srun_str} ) && {post}"
    return srun_cmd, srun_str


def gen_sbatch_command_and_str(args, job_name, train_log, train_stderr, oss_destination, srun_cmd_str, array_length=None):
    excluded = getattr(args, "exclude", None)
    sbatch_cmd = [
        "sbatch", "--job-name", job_name, "--gpus-per-node", str(args.num_gpus), "--nodes", str(args.num_nodes),
        "--ntasks-per-node", str(args.num_gpus), "--cpus-per-task", str(args.cpus_per_task),
        "--output", train_log, "--error", train_stderr, "--open-mode", "append",
        # USR1 three minutes before the limit: the job script traps it and requeues itself
        "--signal", "B:USR1@180",
    ]
    if args.constraint:
        sbatch_cmd += ["--constraint", args.constraint]
    if args.partition:
        sbatch_cmd += ["--partition", args.partition]
    if args.reservation:
        sbatch_cmd += ["--reservation", args.reservation]
    if args.exclusive:
        sbatch_cmd += ["--exclusive"]
    if args.comment:
        sbatch_cmd += ["--comment", args.comment]
    if args.time:
        sbatch_cmd += ["--time", str(args.time)]
    if args.mem is not None:
        sbatch_cmd += ["--mem", args.mem]
    else:
        sbatch_cmd += ["--mem", "0"]
    if args.dep is not None:
        sbatch_cmd += ["-d", str(args.dep)]
    if excluded:
        sbatch_cmd += ["-x", excluded]
    if array_length:
        sbatch_cmd += ["--array", f"0-{array_length - 1}"]
    wrapped = requeue_support() + "\n" + srun_cmd_str + " \n wait $! \n sleep 610 & \n wait $!"
    sbatch_cmd += ["--wrap", wrapped]
    return sbatch_cmd, " ".join(map(shlex.quote, sbatch_cmd))


def requeue_support():
    return textwrap.dedent("""
        trap_handler () {
           echo "Caught signal: " $1
           # SIGTERM must be bypassed
           if [ "$1" = "TERM" ]; then
               echo "bypass sigterm"
           else
             # Submit a new job to the queue
             echo "Requeuing " $SLURM_JOB_ID
             scontrol requeue $SLURM_JOB_ID
           fi
        }
        # Install signal handler
        trap 'trap_handler USR1' USR1
        trap 'trap_handler TERM' TERM
    """)


def local_run(args, env, train_cmd, post_cmds, dry_run):
    assert args.num_nodes == 1, "distributed training cannot be combined with --local"
    if not dry_run("start training locally"):
        if "CUDA_VISIBLE_DEVICES" not in env and args.num_gpus > 0:
            env["CUDA_VISIBLE_DEVICES"] = ",".join(map(str, range(args.num_gpus)))
        env["NCCL_DEBUG"] = env.get("NCCL_DEBUG", "WARN")
        train_proc = subprocess.Popen(train_cmd, env=env)
        train_proc.wait()
        for post in post_cmds or []:
            subprocess.Popen(post, shell=True, env=env).wait()
        return train_proc.returncode
    return 0


def run_batch(env, sbatch_cmd_str, sbatch_cmd):
    print(f"running command: {sbatch_cmd_str}\n")
    with subprocess.Popen(sbatch_cmd, stdout=subprocess.PIPE, env=env) as proc:
        stdout = proc.stdout.read().decode("utf-8")
        try:
            job_id = int(stdout.rstrip().split()[-1])
            print(f"Launched job {job_id}")
        except (IndexError, ValueError):
            job_id = None
            print(f"Could not parse job id from: {stdout!r}")
    return job_id, stdout


def dry_run_batch(env, train_log, train_stderr, sbatch_cmd_str, sbatch_cmd, dry_run):
    """Says what a submission would do and, where ``sbatch`` exists, asks the scheduler to validate the request
    without queueing it (``--test-only``)."""
    dry_run("start remote training")
    dry_run(f"- log stdout to: {train_log}")
    dry_run(f"- log stderr to: {train_stderr}")
    dry_run(f"- run command: {sbatch_cmd_str}")
    if shutil.which(sbatch_cmd[0]) is None:
        return None
    with subprocess.Popen(list(sbatch_cmd) + ["--test-only"], stdout=subprocess.PIPE, env=env) as proc:
        stdout = proc.stdout.read().decode("utf-8")
        print(stdout)
    return stdout


def run_setup(args, config, dry_run):
    """``(save_dir_key, save_dir)`` of one grid point (``config``: name -> hyperparam with its current value) and
    the directory made, unless this is a dry run."""
    keys = [hp.get_save_dir_key() for hp in config.values()]
    save_dir_key = ".".join(k for k in keys if k is not None and len(k) > 0).replace(",", "_")
    save_dir = os.path.join(args.checkpoints_dir, f"{args.prefix}.{save_dir_key}.ngpu{args.num_nodes * args.num_gpus}")
    if not os.path.exists(save_dir) and not dry_run(f"create directory: {save_dir}"):
        os.makedirs(save_dir)
    return save_dir_key, save_dir


def azure_support() -> str:
    """The Azure fabric settings as shell lines for a batch script (``get_azure_env`` is the dict form that
    ``set_env`` applies), plus loading the MPI module where the image has environment modules."""
    lines = [f"export {k}={v}" for k, v in get_azure_env().items()]
    lines += ["export OMPI_MCA_COLL_HCOLL_ENABLE=0",
              'if [ -e "/etc/profile.d/modules.sh" ]; then', "    . /etc/profile.d/modules.sh",
              "    module load mpi/hpcx", "fi"]
    return "\n" + "\n".join(lines) + "\n"


def copy_all_python_files(source, snapshot_main_dir, code_snapshot_hash, recurse_dirs="metaseq_b200"):
    """Snapshot of a source tree under ``<snapshot_main_dir>/<code_snapshot_hash>``: the ``*.py`` files directly in
    ``source`` and, for every directory named in the comma-separated ``recurse_dirs``, its ``*.py``, ``*.so``,
    ``*.yaml``, ``*.cu``, ``*.cuh``, ``*.cpp`` and ``*.h`` files at any depth.  Returns the snapshot directory."""
    destination = os.path.join(snapshot_main_dir, code_snapshot_hash)
    os.makedirs(destination, exist_ok=True)
    for name in os.listdir(source):
        if name.endswith(".py") and os.path.isfile(os.path.join(source, name)):
            shutil.copy2(os.path.join(source, name), os.path.join(destination, name))
    keep = (".py", ".so", ".yaml", ".cu", ".cuh", ".cpp", ".h")

    def ignore(path, names):
        return [n for n in names if n == "__pycache__" or
                (not os.path.isdir(os.path.join(path, n)) and not n.endswith(keep))]

    for d in filter(None, (x.strip() for x in recurse_dirs.split(","))):
        if os.path.isdir(os.path.join(source, d)):
            shutil.copytree(os.path.join(source, d), os.path.join(destination, d), ignore=ignore, dirs_exist_ok=True)
    return destination


def snapshot_code(args, destination: str) -> str:
    """Copies the package sources so that queued jobs run the code as it was at submission."""
    root = Path(args.snapshot_root).resolve()
    dst = Path(destination) / "code_snapshot"
    for rel in str(args.snapshot_recurse_dirs_oss).split(","):
        src = root / rel
        if src.is_dir():
            shutil.copytree(src, dst / rel, dirs_exist_ok=True,
                            ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "obj", "*.o"))
    return str(dst)


def launch_train(args, hp_values, dry_run):
    for hp in hp_values:
        if hp.current_value is None:
            hp.current_value = hp.values[0]
    save_dir_key = get_save_dir_name(args, hp_values)
    save_dir = os.path.join(args.checkpoints_dir, save_dir_key)
    if not os.path.exists(save_dir):
        if not dry_run(f"create directory: {save_dir}"):
            os.makedirs(save_dir, exist_ok=True)
    if not is_job_valid(args, save_dir, dry_run):
        return None
    env = os.environ.copy()
    set_env(args, env, dry_run)
    env["METASEQ_SAVE_DIR"] = save_dir
    oss_destination = ""
    if getattr(args, "snapshot_code", False) and not args.dry_run:
        oss_destination = snapshot_code(args, save_dir)
        env["PYTHONPATH"] = oss_destination + ":" + env.get("PYTHONPATH", "")
    train_cmd = gen_train_command(args, env, hp_values, oss_destination, save_dir, save_dir_key)
    post_cmds = list(args.post_steps) if args.post_steps else []
    train_log = os.path.join(save_dir, "train.log")
    train_stderr = os.path.join(save_dir, "train.stderr.%j")
    if dry_run("train command: " + " ".join(map(shlex.quote, train_cmd))):
        return save_dir
    with open(os.path.join(save_dir, "train.cmd"), "w") as f:
        f.write(" ".join(map(shlex.quote, train_cmd)) + "\n")
    if args.local:
        rc = local_run(args, env, train_cmd, post_cmds, dry_run)
        if rc not in (0, None):
            print(f"local run exited with code {rc}")
        return save_dir
    srun_cmd, srun_str = gen_srun_command_and_str(args, env, save_dir_key, train_log, train_stderr, train_cmd, post_cmds)
    if args.salloc:
        subprocess.Popen(srun_cmd, env=env).wait()
        return save_dir
    sbatch_cmd, sbatch_str = gen_sbatch_command_and_str(args, f"{args.prefix}.{save_dir_key}", train_log, train_stderr,
                                                        oss_destination, srun_str)
    job_id, _ = run_batch(env, sbatch_str, sbatch_cmd)
    if getattr(args, "tombstonable", False) and job_id is not None:
        print(f"tombstone file for job {job_id}: {os.path.join(save_dir, 'tombstone_' + str(job_id))}")
    return save_dir
