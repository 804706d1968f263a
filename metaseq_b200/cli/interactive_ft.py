"""Prompt loop for a model served by an external FasterTransformer build (reference: metaseq/cli/interactive_ft.py).

This entry point does not run this framework's model code: it loads weights exported by
``metaseq_b200.checkpoint.convert_metaseq_ft`` into the ``ParallelGptOp`` custom class of a FasterTransformer
shared library (path in ``FT_PATH``), one process per tensor-parallel rank, and reads prompts from stdin on
rank 0.  Without that library it exits with an explanatory error."""
from __future__ import annotations

import argparse
import os
import sys

import torch


def load_ft(path=None):
    path = path or os.environ.get("FT_PATH")
    if not path or not os.path.exists(path):
        raise ImportError("FasterTransformer is an external dependency: build it and point FT_PATH at "
                          "libth_transformer.so")
    torch.classes.load_library(path)
    return torch.classes.FasterTransformer


DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
BOS, PAD, EOS, UNK = 0, 1, 2, 3


def build_model(ft, weights_path: str, num_layers: int, num_heads: int, embed_size: int, vocab_size: int,
                tensor_para_size: int, dtype=torch.float16, int8_mode: int = 0, device="cuda"):
    """Weights written by ``convert_metaseq_ft`` (a flat list in the library's order, optionally with int8 copies
    and their scales) go to the library's op; ``int8_mode`` is honoured only when the file holds the int8 tensors."""
    state = torch.load(weights_path, map_location=device, weights_only=False)
    weights = state["weights"] if isinstance(state, dict) else state
    weights = [w.to(dtype) if torch.is_tensor(w) and w.is_floating_point() else w for w in weights]
    int8_w, int8_s = [], []
    if int8_mode != 0 and isinstance(state, dict) and {"int8_weights", "int8_scales"} <= state.keys():
        int8_w, int8_s = list(state["int8_weights"]), list(state["int8_scales"])
    head_dim = embed_size // num_heads
    return ft.ParallelGptOp(num_heads, head_dim, 4 * embed_size, num_layers, BOS, vocab_size, EOS, EOS, tensor_para_size,
                            1, int8_mode if int8_w else 0, 1e-5, "pre_layernorm", "relu", False, 0, weights, int8_w,
                            int8_s)


def _one(value, dtype):
    return None if value is None else torch.tensor([value], dtype=dtype)


def generate(model, token_ids, output_length: int, beam_width: int = 1, top_k=0, top_p=1.0, diversity_rate=None,
             temperature=1.0, len_penalty=None, repetition_penalty=1.0, presence_penalty=None, random_seed=0,
             min_length=None, bad_words_list=None, return_cum_log_probs: int = 0, device="cuda"):
    """Runs the library's decoding loop on a batch of prompts (each gets the EOS token in front, as in training) and
    returns, per prompt, the generated ids of the first beam without the prompt-side special tokens and cut at the
    first special token after the text.  Sampling parameters are passed as one-element tensors (``None`` = the
    library's default)."""
    rows = [torch.tensor([EOS] + list(t), dtype=torch.int32, device=device) for t in token_ids]
    lengths = torch.tensor([len(r) for r in rows], dtype=torch.int32, device=device)
    batch = torch.nn.utils.rnn.pad_sequence(rows, batch_first=True, padding_value=PAD)
    outputs, output_lengths = model.forward(
        batch, lengths, output_length, beam_width, _one(top_k, torch.int32), _one(top_p, torch.float32),
        _one(diversity_rate, torch.float32), _one(temperature, torch.float32), _one(len_penalty, torch.float32),
        _one(repetition_penalty, torch.float32), _one(presence_penalty, torch.float32), _one(min_length, torch.int64),
        _one(random_seed, torch.int64), bad_words_list, return_cum_log_probs)
    special = outputs.new_tensor([BOS, PAD, EOS, UNK])
    results = []
    for out, out_len in zip(outputs, output_lengths):
        seq, n = out[0], int(out_len[0])
        keep = ~torch.isin(seq, special)
        keep[1:] = keep[1:].cummin(dim=0)[0]  # nothing after the first special token past position 0
        results.append(seq[1:n][keep[1:n]].tolist())
    return results


def measure_time(fn, *args, **kwargs) -> float:
    """Device time of one call in milliseconds."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    fn(*args, **kwargs)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def get_parser():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--weight-path", required=True, help="pattern with {i} for the tensor-parallel rank")
    ap.add_argument("--vocab-file")
    ap.add_argument("--merges-file")
    ap.add_argument("--tokenizer-file", default=None, help="a tokenizers JSON file (used instead of vocab + merges)")
    ap.add_argument("--num-layers", type=int, default=12)
    ap.add_argument("--num-heads", type=int, default=12)
    ap.add_argument("--embed-size", type=int, default=768)
    ap.add_argument("--vocab-size", type=int, default=50272)
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="fp16")
    ap.add_argument("--int8-mode", type=int, default=0)
    ap.add_argument("--batch-size", type=int, default=1, help="copies of the prompt decoded together")
    ap.add_argument("--output-length", type=int, default=256)
    ap.add_argument("--beam-width", type=int, default=1)
    ap.add_argument("--top-k", type=int, default=20)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--len-penalty", type=float, default=0.0)
    ap.add_argument("--diversity-rate", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.2)
    ap.add_argument("--time", action="store_true", help="print the device time of every generation")
    return ap


def build_tokenizer(args):
    if args.tokenizer_file is not None:
        from tokenizers import Tokenizer

        return Tokenizer.from_file(args.tokenizer_file)
    if not (args.vocab_file and args.merges_file):
        raise SystemExit("pass --tokenizer-file, or --vocab-file and --merges-file")
    from tokenizers import ByteLevelBPETokenizer

    return ByteLevelBPETokenizer.from_file(args.vocab_file, args.merges_file)


def sampling_kwargs(args):
    return dict(output_length=args.output_length, beam_width=args.beam_width, top_k=args.top_k, top_p=args.top_p,
                diversity_rate=args.diversity_rate, temperature=args.temperature, len_penalty=args.len_penalty,
                repetition_penalty=args.repetition_penalty, random_seed=0)


def main(argv=None):
    args = get_parser().parse_args(argv)
    ft = load_ft()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    if world > 1:
        torch.distributed.init_process_group("nccl")
    tok = build_tokenizer(args)
    model = build_model(ft, args.weight_path.format(i=rank), args.num_layers, args.num_heads, args.embed_size,
                        args.vocab_size, world, dtype=DTYPES[args.dtype], int8_mode=args.int8_mode)
    while True:
        obj = [None]
        if rank == 0:
            try:
                prompt = input("Prompt: ").rstrip()
            except EOFError:
                prompt = None
            obj = [None if prompt is None else tok.encode(prompt).ids]
        if world > 1:
            torch.distributed.broadcast_object_list(obj, src=0)
        if obj[0] is None:
            break
        if len(obj[0]) == 0:
            continue
        batch = [list(obj[0])] * args.batch_size
        if args.time:
            ms = measure_time(generate, model, batch, **sampling_kwargs(args))
            if rank == 0:
                print(f"{ms:.1f} ms for {args.batch_size} x {args.output_length} tokens")
        out = generate(model, batch, **sampling_kwargs(args))
        if rank == 0:
            print(f"Output: {tok.decode(out[0])}")


if __name__ == "__main__":
    try:
        main()
    except ImportError as e:
        sys.exit(str(e))
