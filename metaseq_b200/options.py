"""Command-line parsers.

Every flag comes from a config dataclass (``metaseq_b200.dataclass.configs``) or from a
registered component's dataclass.  Parsing is two-pass (reference:
metaseq/options.py:76-193): a first pass over the generic groups discovers which task /
architecture / criterion / optimizer / lr-scheduler / bpe were selected, their flags are added,
the command line is parsed again, and finally the architecture function fills model defaults.
"""
from __future__ import annotations

import argparse
import importlib
import os
import sys
from typing import Callable, List, Optional

import torch

from metaseq_b200.dataclass.configs import (
    CheckpointConfig,
    CommonConfig,
    CommonEvalConfig,
    DatasetConfig,
    DistributedTrainingConfig,
    EMAConfig,
    EvalLMConfig,
    GenerationConfig,
    OptimizationConfig,
    ReshardConfig,
)
from metaseq_b200.dataclass.utils import gen_parser_from_dataclass


def get_training_parser(default_task="streaming_language_modeling"):
    parser = get_parser("Trainer", default_task)
    add_dataset_args(parser, train=True)
    add_distributed_training_args(parser)
    add_model_args(parser)
    add_optimization_args(parser)
    add_checkpoint_args(parser)
    add_ema_args(parser)
    return parser


def get_generation_parser(interactive=False, default_task="language_modeling"):
    parser = get_parser("Generation", default_task)
    add_dataset_args(parser, gen=True)
    add_distributed_training_args(parser, default_world_size=1)
    add_generation_args(parser)
    add_checkpoint_args(parser)
    return parser


def get_interactive_generation_parser(default_task="language_modeling"):
    return get_generation_parser(interactive=True, default_task=default_task)


def get_eval_lm_parser(default_task="language_modeling"):
    parser = get_parser("Evaluate Language Model", default_task)
    add_dataset_args(parser, gen=True)
    add_distributed_training_args(parser, default_world_size=1)
    add_eval_lm_args(parser)
    return parser


def get_validation_parser(default_task=None):
    parser = get_parser("Validation", default_task)
    add_dataset_args(parser, train=True)
    add_distributed_training_args(parser, default_world_size=1)
    group = parser.add_argument_group("Evaluation")
    gen_parser_from_dataclass(group, CommonEvalConfig())
    return parser


def get_reshard_parser(default_task=None):
    parser = get_parser("Reshard", default_task)
    add_dataset_args(parser, train=True)
    add_distributed_training_args(parser, default_world_size=1)
    group = parser.add_argument_group("Evaluation")
    gen_parser_from_dataclass(group, CommonEvalConfig())
    add_reshard_args(parser)
    return parser


def add_reshard_args(parser):
    """The options of checkpoint resharding at load time (metaseq/options.py:61)."""
    group = parser.add_argument_group("Reshard")
    gen_parser_from_dataclass(group, ReshardConfig())
    return group


def _import_user_module(args):
    path = getattr(args, "user_dir", None)
    if path is None:
        return
    path = os.path.abspath(path)
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    parent, name = os.path.split(path)
    if name not in sys.modules:
        sys.path.insert(0, parent)
        importlib.import_module(name)


def get_parser(desc, default_task="streaming_language_modeling"):
    # user modules may register components, so --user-dir is looked at before anything else
    usr = argparse.ArgumentParser(add_help=False, allow_abbrev=False)
    usr.add_argument("--user-dir", default=None)
    usr_args, _ = usr.parse_known_args()
    _import_user_module(usr_args)

    from metaseq_b200 import registry as _registry  # noqa: F401
    from metaseq_b200 import criterions, optim, tasks  # noqa: F401  (populate registries)
    from metaseq_b200.optim import lr_scheduler  # noqa: F401
    from metaseq_b200.data import encoders  # noqa: F401

    parser = argparse.ArgumentParser(allow_abbrev=False, description=desc)
    gen_parser_from_dataclass(parser, CommonConfig())
    for name, reg in _registry.REGISTRIES.items():
        parser.add_argument("--" + name.replace("_", "-"), default=reg["default"], choices=reg["registry"].keys())
    parser.add_argument("--task", metavar="TASK", default=default_task, choices=tasks.TASK_REGISTRY.keys(), help="task")
    return parser


def parse_args_and_arch(parser: argparse.ArgumentParser, input_args: Optional[List[str]] = None,
                        parse_known: bool = False, suppress_defaults: bool = False,
                        modify_parser: Optional[Callable[[argparse.ArgumentParser], None]] = None):
    if suppress_defaults:
        # second parser with every default suppressed: tells which flags were given explicitly
        args = parse_args_and_arch(parser, input_args=input_args, parse_known=parse_known, suppress_defaults=False)
        suppressed = argparse.ArgumentParser(add_help=False, parents=[parser])
        suppressed.set_defaults(**{k: None for k, v in vars(args).items()})
        args = suppressed.parse_args(input_args)
        return argparse.Namespace(**{k: v for k, v in vars(args).items() if v is not None})

    from metaseq_b200 import registry as _registry
    from metaseq_b200.models import ARCH_CONFIG_REGISTRY, ARCH_MODEL_REGISTRY, MODEL_REGISTRY
    from metaseq_b200.tasks import TASK_REGISTRY

    usr = argparse.ArgumentParser(add_help=False, allow_abbrev=False)
    usr.add_argument("--user-dir", default=None)
    usr_args, _ = usr.parse_known_args(input_args)
    _import_user_module(usr_args)

    if modify_parser is not None:
        modify_parser(parser)
    args, _ = parser.parse_known_args(input_args)

    if hasattr(args, "arch"):
        group = parser.add_argument_group("Model-specific configuration",
                                          argument_default=argparse.SUPPRESS)
        if args.arch in ARCH_MODEL_REGISTRY:
            ARCH_MODEL_REGISTRY[args.arch].add_args(group)
        elif args.arch in MODEL_REGISTRY:
            MODEL_REGISTRY[args.arch].add_args(group)
        else:
            raise RuntimeError(f"unknown --arch {args.arch}")
    if hasattr(args, "task"):
        TASK_REGISTRY[args.task].add_args(parser)
        # the data directory may also be given positionally, as on the reference's command lines
        # (metaseq/dataclass/utils.py:62-64: ``data`` is a positional argument there)
        if any(a.dest == "data" for a in parser._actions) and not any(a.dest == "data_positional" for a in parser._actions):
            parser.add_argument("data_positional", nargs="?", default=None, metavar="DATA",
                                help="path to the data directory (same as --data)")
    for name, reg in _registry.REGISTRIES.items():
        choice = getattr(args, name, None)
        if choice is not None:
            cls = reg["registry"][choice]
            if hasattr(cls, "add_args"):
                cls.add_args(parser)
            elif choice in reg["dataclass_registry"]:
                # a component registered with a config dataclass contributes that dataclass's flags
                gen_parser_from_dataclass(parser, reg["dataclass_registry"][choice]())
    if modify_parser is not None:
        modify_parser(parser)
    if parse_known:
        args, extra = parser.parse_known_args(input_args)
    else:
        args = parser.parse_args(input_args)
        extra = None

    if hasattr(args, "data_positional"):
        if args.data_positional is not None and getattr(args, "data", None) is None:
            args.data = args.data_positional
        del args.data_positional
    if (hasattr(args, "batch_size_valid") and args.batch_size_valid is None) or not hasattr(args, "batch_size_valid"):
        args.batch_size_valid = getattr(args, "batch_size", None)
    if hasattr(args, "max_tokens_valid") and args.max_tokens_valid is None:
        args.max_tokens_valid = getattr(args, "max_tokens", None)
    if getattr(args, "memory_efficient_fp16", False):
        args.fp16 = True
    if getattr(args, "seed", None) is None:
        args.seed = 1
        args.no_seed_provided = True
    else:
        args.no_seed_provided = False
    # architecture defaults are applied last so explicit flags win
    if hasattr(args, "arch") and args.arch in ARCH_CONFIG_REGISTRY:
        ARCH_CONFIG_REGISTRY[args.arch](args)
    if parse_known:
        return args, extra
    return args


def add_dataset_args(parser, train=False, gen=False):
    group = parser.add_argument_group("dataset_data_loading")
    gen_parser_from_dataclass(group, DatasetConfig())
    return group


def add_distributed_training_args(parser, default_world_size=None):
    group = parser.add_argument_group("distributed_training")
    if default_world_size is None:
        default_world_size = max(1, torch.cuda.device_count())
    dc = DistributedTrainingConfig()
    dc.distributed_world_size = default_world_size
    gen_parser_from_dataclass(group, dc)
    parser.set_defaults(distributed_world_size=default_world_size)
    return group


def add_optimization_args(parser):
    group = parser.add_argument_group("optimization")
    gen_parser_from_dataclass(group, OptimizationConfig())
    return group


def add_checkpoint_args(parser):
    group = parser.add_argument_group("checkpoint")
    gen_parser_from_dataclass(group, CheckpointConfig())
    return group


def add_ema_args(parser):
    group = parser.add_argument_group("EMA configuration")
    gen_parser_from_dataclass(group, EMAConfig())
    return group


def add_common_eval_args(group):
    gen_parser_from_dataclass(group, CommonEvalConfig())


def add_eval_lm_args(parser):
    group = parser.add_argument_group("LM Evaluation")
    add_common_eval_args(group)
    gen_parser_from_dataclass(group, EvalLMConfig())


def add_generation_args(parser):
    group = parser.add_argument_group("Generation")
    add_common_eval_args(group)
    gen_parser_from_dataclass(group, GenerationConfig())
    return group


def add_model_args(parser):
    group = parser.add_argument_group("Model configuration")
    from metaseq_b200.models import ARCH_MODEL_REGISTRY

    group.add_argument("--arch", "-a", metavar="ARCH", choices=ARCH_MODEL_REGISTRY.keys(), help="model architecture")
    return group
