"""``opt-baselines``: the canonical OPT training recipe as a sweep (reference:
metaseq/launcher/opt_baselines.py:43-352).  ``--model-size`` picks a row of ``MODEL_SIZES``;
``--benchmark`` swaps the data pipeline for ``dummy_lm`` and stops after 50 updates; ``--local``
runs in-process instead of through SLURM."""
from __future__ import annotations

import os

from .opt_job_constants import DATA_LOCATIONS, MODEL_SIZES, TOTAL_TRAIN_TOKENS, TOTAL_WARMUP_TOKENS, VALID_SUBSETS, ComputeEnvs
from .sweep import hyperparam
from .sweep import main as sweep_main

PREDEFINED_GRID_FUNCTION = {}


def add_extra_options_func(parser):
    parser.add_argument("--restore-file", help="load an existing checkpoint for continuing training")
    parser.add_argument("--reset-dataloader", action="store_true", help="reset the dataloader to epoch 1")
    parser.add_argument("--model-size", choices=MODEL_SIZES.keys(), required=True)
    # --data (directory with train/ and valid/) is an option of the sweep parser itself
    parser.add_argument("--vocab-filename", default=None)
    parser.add_argument("--merges-filename", default=None)
    parser.add_argument("--valid-subset", default=None)
    parser.add_argument("--max-update", "--mu", type=int, default=None)
    parser.add_argument("--max-epoch", "--me", type=int, default=None)
    parser.add_argument("--disable-validation", action="store_true")
    parser.add_argument("--circleci", action="store_true", help="running a test on circleci")
    parser.add_argument("--benchmark", action="store_true", help="use synthetic data and only train for 50 steps")
    parser.add_argument("--profile", action="store_true")
    parser.add_argument("--max-tokens-per-gpu", "--bs", type=int, default=None, help="overrides the default tokens per GPU")
    parser.add_argument("--sequence-parallel", action="store_true")
    parser.add_argument("--kernel-backend", default="auto", choices=["auto", "torch"])


def get_grid(args):
    size = MODEL_SIZES[args.model_size]
    SEQ_LEN = 2048
    num_gpus = args.num_gpus * args.num_nodes
    total_gpus = max(1, num_gpus)
    ddp_backend = "fully_sharded"
    mp = min(size.model_parallel, total_gpus)
    dp = max(1, total_gpus // mp)
    # batch size in the table is in tokens per update
    total_gpus_for_bsz = total_gpus
    bs_per_gpu = max(1, size.batch_size // SEQ_LEN // dp)
    if args.max_tokens_per_gpu:
        bs_per_gpu = max(1, args.max_tokens_per_gpu // SEQ_LEN)
    tokens_per_update = bs_per_gpu * SEQ_LEN * dp
    total_updates = int(TOTAL_TRAIN_TOKENS) // max(1, size.batch_size)
    warmup_updates = max(1, int(TOTAL_WARMUP_TOKENS) // max(1, size.batch_size))
    log_interval = 10 if not args.local else 1
    if args.max_update is not None:
        max_update = args.max_update
    else:
        max_update = total_updates

    grid = []

    def H(*a, **k):
        grid.append(hyperparam(*a, **k))

    if args.benchmark:
        H("--task", "dummy_lm", save_dir_key=lambda val: val)
        H("--dict-size", 51200 - 4 if not args.circleci else 50272 - 4 + 4)
        H("--save-interval-epochs", 0)
        H("--save-interval-updates", 0)
        H("--disable-validation")
        max_update = 50 if args.max_update is None else args.max_update
        log_interval = 5
    else:
        H("--task", "streaming_language_modeling")
        H("--sample-break-mode", "none", save_dir_key=lambda val: f"bm_{val}")
        H("--vocab-filename", args.vocab_filename or os.path.join(args.data or "", "gpt2-vocab.json"),
          save_dir_key=lambda _: "gpt2")
        H("--merges-filename", args.merges_filename or os.path.join(args.data or "", "gpt2-merges.txt"))
        H("--save-interval-updates", 2000)
        H("--train-subset", "train")
        H("--valid-subset", args.valid_subset or ",".join(f"valid/{s}" for s in VALID_SUBSETS))
        H("--ignore-unused-valid-subsets")
        H("--num-workers", 8)
        H("--num-workers-valid", 1)
        H("--validate-interval-updates", 2000)
        if args.data:
            H("--data", args.data)
    if args.profile:
        H("--profile")
    if not args.benchmark:
        H("--save-interval-epochs", 0)
    H("--memory-efficient-fp16", save_dir_key=lambda val: "me_fp16")
    H("--fp16-init-scale", 4)
    H("--ddp-backend", ddp_backend)
    H("--no-reshard-after-forward", save_dir_key=lambda _: "zero2")
    H("--use-sharded-state")
    H("--checkpoint-activations")
    H("--model-parallel-size", mp)
    H("--criterion", "vocab_parallel_cross_entropy")
    H("--distribute-checkpointed-activations")
    H("--tensor-parallel-init-model-on-gpu")
    H("--full-megatron-init")
    H("--megatron-init-sigma", 0.006)
    H("--activation-fn", "relu", save_dir_key=lambda x: x)
    H("--arch", "transformer_lm_megatron", save_dir_key=lambda val: val)
    H("--share-decoder-input-output-embed")
    H("--decoder-layers", size.n_layers, save_dir_key=lambda val: f"nlay{val}")
    H("--decoder-embed-dim", size.emb_size, save_dir_key=lambda val: f"emb{val}")
    H("--decoder-ffn-embed-dim", size.ffn_size)
    H("--decoder-attention-heads", size.n_heads)
    H("--decoder-learned-pos", save_dir_key=lambda _: "lrnpos")
    H("--no-scale-embedding", save_dir_key=lambda _: "0emb_scale")
    H("--tokens-per-sample", SEQ_LEN, save_dir_key=lambda val: f"tps{val}")
    H("--optimizer", "adam", save_dir_key=lambda val: val)
    H("--adam-betas", "(0.9, 0.95)", save_dir_key=lambda val: "b2_{}".format(val.split(",")[-1].strip(" )")))
    H("--adam-eps", 1e-8, save_dir_key=lambda val: f"eps{val}")
    H("--clip-norm", 1.0, save_dir_key=lambda val: f"cl{val}")
    H("--clip-norm-type", "l2")
    H("--lr-scheduler", "polynomial_decay")
    H("--lr", size.lr, save_dir_key=lambda val: f"lr{val:.3g}")
    H("--end-learning-rate", size.lr * 0.1, save_dir_key=lambda val: f"endlr{val:.3g}")
    H("--warmup-updates", warmup_updates, save_dir_key=lambda val: f"wu{val}")
    H("--total-num-update", total_updates)
    H("--dropout", 0.1 if not args.sequence_parallel else 0.0, save_dir_key=lambda val: f"dr{val}")
    H("--attention-dropout", 0.1 if not args.sequence_parallel else 0.0, save_dir_key=lambda val: f"atdr{val}")
    H("--no-emb-dropout", save_dir_key=lambda _: "0emb_dr")
    H("--weight-decay", 0.1, save_dir_key=lambda val: f"wd{val}")
    H("--batch-size", bs_per_gpu, save_dir_key=lambda val: f"ms{val}")
    H("--update-freq", 1, save_dir_key=lambda val: f"uf{val}")
    H("--max-update", max_update, save_dir_key=lambda val: f"mu{val}")
    H("--seed", 1, save_dir_key=lambda val: f"s{val}")
    H("--log-format", "json")
    H("--log-interval", log_interval)
    H("--required-batch-size-multiple", 1)
    H("--kernel-backend", args.kernel_backend)
    if args.sequence_parallel:
        H("--sequence-parallel", save_dir_key=lambda _: "sp")
    if args.restore_file:
        H("--restore-file", args.restore_file)
    if args.reset_dataloader:
        H("--reset-dataloader")
    if args.disable_validation and not args.benchmark:
        H("--disable-validation")
    return [g for g in grid if g is not None]


def postprocess_hyperparams(args, config):
    pass


def cli_main(input_args=None):
    return sweep_main(get_grid, postprocess_hyperparams, add_extra_options_func, input_args=input_args)


if __name__ == "__main__":
    cli_main()
