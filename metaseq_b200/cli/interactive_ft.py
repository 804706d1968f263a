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


def build_model(ft, weights_path: str, num_layers: int, num_heads: int, embed_size: int, vocab_size: int,
                tensor_para_size: int, dtype=torch.float16):
    state = torch.load(weights_path, map_location="cuda", weights_only=False)
    weights = state["weights"] if isinstance(state, dict) else state
    int8_w = state.get("int8_weights", []) if isinstance(state, dict) else []
    int8_s = state.get("int8_scales", []) if isinstance(state, dict) else []
    head_dim = embed_size // num_heads
    return ft.ParallelGptOp(num_heads, head_dim, 4 * embed_size, num_layers, 0, vocab_size, 2, 2, tensor_para_size, 1,
                            1 if int8_w else 0, 1e-5, "pre_layernorm", "relu", False, 0, weights, int8_w, int8_s)


def generate(model, token_ids, output_length: int, top_k=0, top_p=0.9, temperature=1.0):
    lengths = torch.tensor([len(t) for t in token_ids], dtype=torch.int32)
    width = int(lengths.max())
    batch = torch.zeros(len(token_ids), width, dtype=torch.int32)
    for i, t in enumerate(token_ids):
        batch[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
    n = len(token_ids)
    return model.forward(batch.cuda(), lengths.cuda(), output_length, 1, torch.full((n,), top_k, dtype=torch.int32),
                         torch.full((n,), top_p), torch.ones(n), torch.full((n,), temperature), torch.ones(n),
                         torch.ones(n), torch.zeros(n, dtype=torch.int64), 0)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--weight-path", required=True, help="pattern with {i} for the tensor-parallel rank")
    ap.add_argument("--vocab-file", required=True)
    ap.add_argument("--merges-file", required=True)
    ap.add_argument("--num-layers", type=int, default=96)
    ap.add_argument("--num-heads", type=int, default=96)
    ap.add_argument("--embed-size", type=int, default=12288)
    ap.add_argument("--vocab-size", type=int, default=50272)
    ap.add_argument("--output-length", type=int, default=256)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--temperature", type=float, default=1.0)
    args = ap.parse_args(argv)
    ft = load_ft()
    from tokenizers import ByteLevelBPETokenizer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    if world > 1:
        torch.distributed.init_process_group("nccl")
    tok = ByteLevelBPETokenizer(args.vocab_file, args.merges_file)
    model = build_model(ft, args.weight_path.format(i=rank), args.num_layers, args.num_heads, args.embed_size,
                        args.vocab_size, world)
    while True:
        obj = [None]
        if rank == 0:
            try:
                obj = [tok.encode(input("Prompt: ")).ids]
            except EOFError:
                obj = [None]
        if world > 1:
            torch.distributed.broadcast_object_list(obj, src=0)
        if obj[0] is None:
            break
        out = generate(model, [[2] + list(obj[0])], args.output_length, top_p=args.top_p, temperature=args.temperature)
        if rank == 0:
            print(tok.decode(out[0][0].tolist()))


if __name__ == "__main__":
    try:
        main()
    except ImportError as e:
        sys.exit(str(e))
