"""Hyper-parameter sweeps: a grid of ``hyperparam`` values expands into one training command
per combination, each with a save directory derived from the values that carry a
``save_dir_key`` (reference: metaseq/launcher/sweep.py)."""
from __future__ import annotations

import argparse
import datetime
import itertools
import os
import shlex
import subprocess
from typing import Any, Callable, List, Optional


class hyperparam:
    """One command-line flag with one value or a list of values to sweep over.

    ``binary_flag``: emit only the flag name (store_true) when the value is truthy.
    ``save_dir_key``: callable mapping the value to a fragment of the run's directory name.
    ``positional_arg``: emit the value without a flag name."""

    def __init__(self, name, values=None, binary_flag=False, save_dir_key: Optional[Callable] = None,
                 positional_arg=False):
        self.name = name
        if values is None:
            self.values = [True]
            self.binary_flag = True
        else:
            self.values = values if isinstance(values, list) else [values]
            self.binary_flag = binary_flag
        self.save_dir_key = save_dir_key
        self.positional_arg = positional_arg
        self.current_value = None
        if positional_arg and name.startswith("-"):
            raise ValueError(f"positional arguments must not start with a dash ({name})")
        if len(self.values) > 1 and self.save_dir_key is None:
            raise ValueError(f"{name} has more than one value but is missing a save_dir_key!")

    def get_cli_args(self) -> List[str]:
        if self.binary_flag:
            return [self.name] if self.current_value else []
        if self.positional_arg:
            return [str(self.current_value)]
        return [self.name, str(self.current_value)]

    def get_save_dir_key(self):
        if self.save_dir_key is None:
            return None
        if self.binary_flag:
            return self.save_dir_key(1) if self.current_value else None
        return self.save_dir_key(self.current_value)


def get_env_from_args(args):
    """The cluster named by the reference's switches (``--azure``, ``--aws``, ``--fair``, ``--rsc``) or by
    ``--cluster-env``."""
    from .opt_job_constants import ComputeEnvs

    for flag, env in (("azure", ComputeEnvs.AZURE), ("aws", ComputeEnvs.AWS), ("fair", ComputeEnvs.FAIR),
                      ("rsc", ComputeEnvs.RSC)):
        if getattr(args, flag, False):
            return env
    named = getattr(args, "cluster_env", None)
    if named:
        return ComputeEnvs(named)
    raise NotImplementedError("Env not passed in! Please pass in one of: --azure, --aws, --fair, --rsc")


def get_args(add_extra_options_func=None, input_args=None):
    parser = argparse.ArgumentParser("Script for launching hyperparameter sweeps")
    parser.add_argument("--grid", help="grid function to use, e.g. module:function")
    parser.add_argument("-p", "--prefix", required=True, help="save checkpoints and logs in <checkpoints-dir>/<prefix>.<save_dir_key>")
    parser.add_argument("-t", "--num-trials", default=-1, type=int, help="number of random hyperparam configurations to try (-1 for grid search)")
    parser.add_argument("-g", "--num-gpus", type=int, required=True, help="number of GPUs per node")
    parser.add_argument("-n", "--num-nodes", type=int, default=1, help="number of nodes for distributed training")
    parser.add_argument("--update-freq", type=int, default=0, help="update freq")
    parser.add_argument("--seed", type=int, default=1234)
    parser.add_argument("--resume-failed", action="store_true", help="resume any runs that failed")
    parser.add_argument("--resume-finished", action="store_true", help="force any runs that finished to begin again")
    parser.add_argument("--dry-run", action="store_true", help="output only a list of actions to perform without performing them")
    parser.add_argument("--local", action="store_true", help="run locally instead of submitting remote job")
    parser.add_argument("--debug", action="store_true", help="debug")
    parser.add_argument("--script", default="metaseq_b200.cli.train", help="module (python -m) or script to launch")
    parser.add_argument("--python", default="python", help="path to nonstandard python binary")
    parser.add_argument("--checkpoints-dir", default=os.path.join(os.path.expanduser("~"), "checkpoints",
                                                                  str(datetime.date.today())),
                        help="save checkpoints and logs in <checkpoints-dir>/<prefix>.<save_dir_key>")
    parser.add_argument("--cluster-env", default="local", help="cluster environment: fair / aws / azure / rsc / local")
    for env_name in ("azure", "aws", "fair", "rsc"):  # the reference's spelling of --cluster-env <name>
        parser.add_argument(f"--{env_name}", action="store_true", help=f"running on {env_name}")
    parser.add_argument("-d", "--data", help="path to data directory (appended to the training command)")
    parser.add_argument("--local-checkpoints-dir", default=None,
                        help="node-local directory for checkpoints (the job's save dir then holds logs only)")
    parser.add_argument("--full-azure-upload-path", default=None,
                        help="blob-store URL that checkpoints are uploaded to asynchronously")
    parser.add_argument("--azure-folder-auto-name", action="store_true",
                        help="append <prefix>.<save_dir_key>.ngpu<N>/ to the upload URL")
    parser.add_argument("--log-tensorboard", action="store_true")
    parser.add_argument("--tensorboard-logdir", default=None)
    parser.add_argument("--post-steps", nargs="+", help="additional steps to execute after the primary job is complete")
    # slurm
    parser.add_argument("--salloc", action="store_true", help="run agaist current allocation")
    parser.add_argument("--partition", help="partition to run on", default=None)
    parser.add_argument("--reservation", help="reservation to run on")
    parser.add_argument("--exclusive", action="store_true")
    parser.add_argument("--dep", metavar="JOBID", type=int, help="add JOBID as a dependency (i.e., wait for it to finish)")
    parser.add_argument("--sequential", action="store_true", help="schedule jobs to run sequentially")
    parser.add_argument("--time", default="4320", help="expected job duration in minutes")
    parser.add_argument("--mem", "--mem", help="memory to request")
    parser.add_argument("--constraint", metavar="CONSTRAINT")
    parser.add_argument("--comment", help="comment string")
    parser.add_argument("--snapshot-code", action="store_true", default=False, help="take a snapshot of the code")
    parser.add_argument("--snapshot-root", type=str, default=".")
    parser.add_argument("--snapshot-recurse-dirs-internal", default="metaseq_b200")
    parser.add_argument("--snapshot-recurse-dirs-oss", default="metaseq_b200")
    parser.add_argument("--no-wandb", action="store_true")
    parser.add_argument("--no-tensorboard", action="store_true", default=True)
    parser.add_argument("--cpus-per-task", type=int, default=12)
    parser.add_argument("--cpu-bind", default="none")
    parser.add_argument("--no-save-dir", action="store_true")
    parser.add_argument("-ts", "--tombstonable", type=bool, default=False, help="make the job killable by writing a tombstone file")
    parser.add_argument("--use-jobarray", action="store_true")
    parser.add_argument("--jobarray-name", type=str, default=None)
    if add_extra_options_func is not None:
        add_extra_options_func(parser)
    args = parser.parse_args(input_args)
    chosen = [n for n in ("azure", "aws", "fair", "rsc") if getattr(args, n)]
    if len(chosen) > 1:
        parser.error("pass only one of --azure, --aws, --fair, --rsc")
    if chosen:
        args.cluster_env = chosen[0]
    return args


def grid_product(grid: List[hyperparam]):
    """Every combination of the grid's values; each yielded list has ``current_value`` set."""
    for combo in itertools.product(*[hp.values for hp in grid]):
        for hp, val in zip(grid, combo):
            hp.current_value = val
        yield grid


def main(get_grid, postprocess_hyperparams, add_extra_options_func=None, scheduler_args=None, input_args=None):
    args = get_args(add_extra_options_func, input_args)
    from . import slurm

    return slurm.main(get_grid, postprocess_hyperparams, args)
