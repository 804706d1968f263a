"""One-token decode step of a ``TransformerDecoder`` replayed from a CUDA graph.

The reference decodes through the module tree, one Python call per op and per layer, with the key/value
cache grown by ``torch.cat`` every step (metaseq/sequence_generator.py:246-330,
metaseq/modules/multihead_attention.py:428-476).  At one token per sequence the device work of a step is a
few hundred short kernels, so a step costs what the host needs to launch them.  Here the whole step —
embedding, every layer, the final norm and the vocabulary projection — is captured once per batch size and
replayed with one launch:

* the key/value caches are preallocated and owned by the step object, so their addresses are constants of
  the graph; they are handed to the prefill through the usual ``incremental_state`` dictionary;
* everything that changes from step to step lives in device memory: the token ids, the running count of
  non-padding tokens (learned positions), and the number of cached positions, which the attention kernel reads
  and which the graph itself increments;
* the append of the new key/value rows happens inside the attention kernel.

With tensor parallelism the graph holds the layers: the row-parallel products (attention output, second
feed-forward matrix) run as one kernel each that also sums over the ranks (``parallel/symm.py:DecodeReduce``),
while the vocabulary-parallel embedding and projection, one collective each per step, stay outside the graph
on the library's collectives.

Restrictions (the caller falls back to the module path otherwise): 16-bit weights on a GPU, pre-norm layers with
ReLU or GELU, head size 64 or 128, no document-separator attention; with tensor parallelism at most 8 ranks and
64 sequences.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from metaseq_b200.modules.multihead_attention import KVCache
from metaseq_b200.modules.transformer_decoder_layer import ModelParallelTransformerDecoderLayer as TransformerDecoderLayer
from metaseq_b200.ops import functional as F
from metaseq_b200.parallel import mpu

_MAX_CACHED_STEPS = 3
_CACHE_MEMORY_FRACTION = 0.35  # of the device memory, for the key/value caches of all cached buckets together


def bucket_rows(rows: int) -> int:
    """Batch sizes share graphs and caches in buckets (powers of two up to 64, then multiples of 64), so that a
    service whose batches vary in size does not capture a graph and allocate caches for every size it meets.
    The rows beyond the live ones carry padding tokens."""
    b = 1
    while b < rows and b < 64:
        b *= 2
    return b if rows <= 64 else -(-rows // 64) * 64


def _tp_world() -> int:
    try:
        return mpu.get_tensor_model_parallel_world_size()
    except Exception:
        return 1


class GraphedDecodeStep:
    """Static buffers, caches and the captured graph for ``rows`` sequences decoded together."""

    @staticmethod
    def supported(decoder, rows: int = 1) -> bool:
        from metaseq_b200.models.transformer_decoder import UNSPECIFIED_DOC_SEP, ModelParallelTransformerDecoder as TransformerDecoder

        if not isinstance(decoder, TransformerDecoder):
            return False
        w = decoder.embed_tokens.weight
        if not (w.is_cuda and w.dtype in (torch.float16, torch.bfloat16) and F.use_kernels(w)):
            return False
        if decoder.training or decoder.sequence_parallel:
            return False
        if _tp_world() > 1 and (_tp_world() > 8 or bucket_rows(rows) > 64 or w.shape[1] % 128 != 0):
            return False
        if decoder.self_attn_doc_sep != UNSPECIFIED_DOC_SEP or w.shape[1] % 8 != 0:
            return False
        if getattr(decoder, "alibi_slopes", None) is not None:
            return False  # the decode-attention kernel carries no position bias
        if decoder.embed_positions is not None and not hasattr(decoder.embed_positions, "weight"):
            return False
        if decoder.layer_norm is None or decoder.layer_norm.weight is None \
                or decoder.output_projection.weight.dtype != w.dtype:
            return False
        for layer in decoder.layers:
            if not isinstance(layer, TransformerDecoderLayer):
                return False
            a = layer.self_attn
            if layer.activation_name not in ("relu", "gelu") or not F.decode_head_dim_ok(a.head_dim):
                return False
            for lin in (a.qkv_proj, a.out_proj, layer.fc1, layer.fc2):
                if lin.weight.dtype != w.dtype or lin.weight.shape[0] % 8 or lin.weight.shape[1] % 8:
                    return False
            if layer.self_attn_layer_norm.weight is None or layer.self_attn_layer_norm.weight.dtype != w.dtype:
                return False
        return True

    @classmethod
    def for_decoder(cls, decoder, rows: int, min_capacity: int) -> "GraphedDecodeStep":
        """The step object serving ``rows`` sequences (it is built for the bucket ``rows`` falls into) with room
        for ``min_capacity`` positions, kept on the decoder (the newest few buckets only: each holds a full set of
        caches)."""
        table: Dict[int, GraphedDecodeStep] = decoder.__dict__.setdefault("_graphed_decode_steps", {})
        width = bucket_rows(rows)
        step = table.pop(width, None)
        if step is not None and (step.capacity < min_capacity or step.signature != cls._signature(decoder)):
            step = None  # too short, or the model's parameters were replaced since the graph was captured
        if step is None:
            limit = int(decoder.max_positions()) + 2
            capacity = min(limit, max(min_capacity, -(-min_capacity // 256) * 256))
            need = cls._cache_bytes(decoder, width, capacity)
            budget = cls._cache_budget(decoder)
            # least recently used buckets go first: by count, and so that all caches together stay within a
            # fraction of the device memory (a 64-row bucket of a large model is tens of GB)
            while table and (len(table) >= _MAX_CACHED_STEPS or
                             need + sum(st.cache_bytes for st in table.values()) > budget):
                table.pop(next(iter(table)))
            try:
                step = cls(decoder, width, capacity)
            except torch.cuda.OutOfMemoryError:
                table.clear()
                torch.cuda.empty_cache()
                step = cls(decoder, width, capacity)
        table[width] = step  # most recently used last
        step.live = rows
        return step

    @staticmethod
    def _cache_bytes(decoder, rows: int, capacity: int) -> int:
        w = decoder.embed_tokens.weight
        per_layer = sum(2 * rows * capacity * layer.self_attn.num_heads_partition * layer.self_attn.head_dim
                        for layer in decoder.layers)
        return per_layer * w.element_size()

    @staticmethod
    def _cache_budget(decoder) -> int:
        w = decoder.embed_tokens.weight
        total = torch.cuda.get_device_properties(w.device).total_memory if w.is_cuda else 1 << 40
        return int(_CACHE_MEMORY_FRACTION * total)

    @staticmethod
    def _signature(decoder):
        """Addresses of the parameters the graph reads: a captured graph is valid only while they stay put
        (``load_state_dict`` copies in place and keeps it valid; ``.half()`` or ``.to(device)`` do not)."""
        return tuple(p.data_ptr() for p in decoder.parameters())

    def __init__(self, decoder, rows: int, capacity: int):
        self.decoder = decoder
        self.signature = self._signature(decoder)
        self.cache_bytes = self._cache_bytes(decoder, rows, capacity)
        self.rows = rows  # rows of the graph and the caches
        self.live = rows  # rows in use (set by for_decoder); the others carry padding
        self.views: List[KVCache] = []
        w = decoder.embed_tokens.weight
        self.device, self.dtype = w.device, w.dtype
        self.capacity = int(capacity)
        self.pad = int(decoder.padding_idx)
        self.caches: List[KVCache] = []
        for layer in decoder.layers:
            width = layer.self_attn.num_heads_partition * layer.self_attn.head_dim
            self.caches.append(KVCache(rows, self.capacity, width, self.dtype, self.device))
        self.tok = torch.zeros(rows, dtype=torch.long, device=self.device)
        self.count = torch.zeros(rows, dtype=torch.long, device=self.device)  # non-padding tokens so far
        self.length = torch.zeros(1, dtype=torch.int32, device=self.device)  # cached positions
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._length_hint = 1
        self.tp = _tp_world()
        self.reduce = None
        if self.tp > 1:
            from metaseq_b200.ops import _lib
            from metaseq_b200.parallel.symm import DecodeReduce

            D = w.shape[1]
            self.reduce = decoder.__dict__.get("_decode_reduce")
            if self.reduce is None:  # created by all ranks together; shared by the step objects of this decoder
                self.reduce = DecodeReduce(mpu.get_tensor_model_parallel_group(), self.device, 64, D, self.dtype)
                decoder.__dict__["_decode_reduce"] = self.reduce
            lib = _lib.kernels()
            first = decoder.layers[0]
            # one grid for every row-parallel product of the step (they share flags and epoch counters)
            self._split = min(lib.msq_gemm_skinny_split(D, first.self_attn.out_proj.weight.shape[1]),
                              lib.msq_gemm_skinny_split(D, first.fc2.weight.shape[1]))
            # the embedding sum and the next-token records travel through one small exchange kernel inside the graph
            from metaseq_b200.parallel.symm import WordsExchange

            self.exchange = decoder.__dict__.get("_decode_exchange")
            if self.exchange is None or self.exchange.cap < 64 * D // 2:
                self.exchange = WordsExchange(mpu.get_tensor_model_parallel_group(), self.device, 64 * D // 2)
                decoder.__dict__["_decode_exchange"] = self.exchange
            self.vocab_start = int(decoder.embed_tokens.vocab_start_index)
            self.local_logits: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ state
    def new_state(self) -> Dict:
        """An ``incremental_state`` whose caches are the first ``live`` rows of the ones the graph addresses,
        emptied."""
        state: Dict = {}
        self.views = []
        for layer, cache in zip(self.decoder.layers, self.caches):
            cache.length = 0
            view = cache
            if self.live != self.rows:
                view = KVCache.__new__(KVCache)
                view.k, view.v, view.length = cache.k[: self.live], cache.v[: self.live], 0
            self.views.append(view)
            state[layer.self_attn._cache_key] = view
        return state

    def begin(self, prefix_tokens: torch.Tensor) -> None:
        """Call after the prefill over ``prefix_tokens`` ``[live, T]`` went through the caches."""
        assert prefix_tokens.shape[0] == self.live and self.views
        self.count.zero_()
        self.count[: self.live] = prefix_tokens.ne(self.pad).sum(dim=1)
        filled = self.views[0].length
        assert filled == prefix_tokens.shape[1] and all(c.length == filled for c in self.views)
        assert all(v.k.data_ptr() == c.k.data_ptr() for v, c in zip(self.views, self.caches)), \
            "a cache was reallocated during the prefill"
        for cache in self.caches:
            cache.length = filled
        self.length.fill_(filled)
        self._length_hint = max(1, filled)

    # ------------------------------------------------------------------- step
    def _embed(self) -> torch.Tensor:
        """Embedding of ``self.tok`` at the next position of every row; advances the position counters."""
        dec = self.decoder
        tok = self.tok
        nonpad = tok.ne(self.pad)
        self.count.add_(nonpad)
        pos_w = dec.embed_positions.weight if dec.embed_positions is not None else None
        positions = torch.where(nonpad, self.count + self.pad, torch.full_like(self.count, self.pad)) \
            if pos_w is not None else None
        w = dec.embed_tokens.weight
        if self.tp == 1:
            return F.embed_fwd(tok, positions, w, pos_w, dec.embed_scale)
        # each token's row lives on one rank (zeros elsewhere): the sum over ranks is the embedding
        start = dec.embed_tokens.vocab_start_index
        x = F.embed_fwd(tok, None, w, None, dec.embed_scale, start, start + w.shape[0], add_positions=False)
        x = self.exchange.sum(x)
        if pos_w is not None:
            x = x + torch.nn.functional.embedding(positions, pos_w)
        return x

    def _row_parallel(self, x, lin, residual):
        if self.tp == 1:
            return F.gemm(x, lin.weight, bias=lin.bias, residual=residual)
        return self.reduce.gemm_all_reduce(x, lin.weight, bias=lin.bias, residual=residual, split=self._split)

    def _layers(self, x: torch.Tensor) -> torch.Tensor:
        dec = self.decoder
        for layer, cache in zip(dec.layers, self.caches):
            a = layer.self_attn
            ln1, ln2 = layer.self_attn_layer_norm, layer.final_layer_norm
            h, _, _ = F.layer_norm_fwd(x, ln1.weight, ln1.bias, ln1.eps)
            qkv = F.gemm(h, a.qkv_proj.weight, bias=a.qkv_proj.bias)  # (k | v | q) per row, this rank's heads
            dp = qkv.shape[1] // 3
            ctx = F.decode_attn_step(qkv[:, 2 * dp:], qkv[:, 0:dp], qkv[:, dp:2 * dp], cache.k, cache.v, self.length,
                                     a.num_heads_partition, a.scaling, self._length_hint)
            x = self._row_parallel(ctx, a.out_proj, x)
            h, _, _ = F.layer_norm_fwd(x, ln2.weight, ln2.bias, ln2.eps)
            relu = layer.activation_name == "relu"
            f = F.gemm(h, layer.fc1.weight, bias=layer.fc1.bias, relu=relu, gelu=not relu)
            x = self._row_parallel(f, layer.fc2, x)
        fl = dec.layer_norm
        x, _, _ = F.layer_norm_fwd(x, fl.weight, fl.bias, fl.eps)
        self.length.add_(1)
        return x

    def _logits(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's columns of the logits (all of them without tensor parallelism)."""
        return F.gemm(x, self.decoder.output_projection.weight)

    def _run(self) -> torch.Tensor:
        """What the graph holds: the whole step, embedding to (this rank's slice of the) logits.  Under tensor
        parallelism the sums over ranks inside it are the fused GEMM + all-reduce of the row-parallel products and
        the small exchange kernel of the embedding; no library collective is part of a step."""
        with F.dependent_launch():  # every GEMM operand ``b`` in the chain is a model weight
            return self._logits(self._layers(self._embed()))

    def _capture(self) -> None:
        # Warm up on a side stream (lazy initialisation of libraries must not happen under capture), then
        # restore the device-side state that the warm-up advanced.
        assert self.reduce is None or self.reduce.calls % 2 == 0
        saved = (self.count.clone(), self.length.clone())
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._run()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.count.copy_(saved[0])
        self.length.copy_(saved[1])
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self._run()
        if self.tp == 1:
            self.logits = out
        else:
            self.local_logits = out
            assert self.reduce.calls % 2 == 0  # replays keep the alternation of the staging buffers
        # the capture itself executes nothing, so the state is still the restored one
        self.graph = graph

    @torch.no_grad()
    def step(self, new_tokens: torch.Tensor, gather: bool = True) -> torch.Tensor:
        """Feeds one token per row; returns the ``[rows, V]`` logits (a buffer reused by the next step).  Under
        tensor parallelism ``gather=False`` returns this rank's ``[rows, V / p]`` columns instead (global column =
        ``vocab_start`` + local column), for callers that pick the token from the shards (``pick_greedy``)."""
        filled = self.caches[0].length
        if filled + 1 > self.capacity:
            raise RuntimeError(f"decode step beyond the cache capacity of {self.capacity} positions")
        if self.live == self.rows:
            self.tok.copy_(new_tokens)
        else:
            self.tok.fill_(self.pad)
            self.tok[: self.live] = new_tokens
        if self.graph is None:
            self._capture()
        self.graph.replay()
        for cache in self.caches:
            cache.length = filled + 1
        for view in self.views:
            view.length = filled + 1
        if self.tp == 1:
            logits = self.logits
        elif gather:
            logits = self._gather_logits(self.local_logits)
        else:
            logits = self.local_logits
        return logits if self.live == self.rows else logits[: self.live]

    def _gather_logits(self, local: torch.Tensor) -> torch.Tensor:
        """``[rows, V]`` from every rank's ``[rows, V / p]`` columns through the peer-memory exchange kernel (the
        reference gathers them with a library all-gather per token: metaseq/modules/megatron/mpu/mappings.py:97);
        the library collective remains only for slices with an odd number of 16-bit columns."""
        rows, vp = local.shape
        if local.element_size() != 2 or vp % 2 or not local.is_contiguous():
            from metaseq_b200.parallel import mappings

            return mappings.gather_from_tensor_model_parallel_region(local)
        words = rows * vp // 2
        ex = self.decoder.__dict__.get("_decode_logits_exchange")
        if ex is None or ex.cap < words:
            from metaseq_b200.parallel.symm import WordsExchange

            if ex is not None:
                ex.close()
            ex = WordsExchange(mpu.get_tensor_model_parallel_group(), self.device, self.rows * vp // 2)
            self.decoder.__dict__["_decode_logits_exchange"] = ex
        every = ex.gather(local.view(torch.int32)).view(local.dtype)  # [p, rows, V / p]
        return every.permute(1, 0, 2).reshape(rows, self.tp * vp)

    @torch.no_grad()
    def pick_greedy(self, local_logits: torch.Tensor, banned=(), only: Optional[int] = None):
        """Arg-max token and its log-probability per row from vocabulary-parallel logits, without gathering them.
        Every rank reduces its own columns to (max, sum-exp, best allowed value, its global index), the records of
        all ranks are exchanged by one small kernel, and every rank merges them the same way.  ``banned``: global
        token ids that must not be chosen; ``only``: the one token that may be.  Ties go to the lowest index, as
        ``torch.max`` does on gathered logits."""
        lo, width = self.vocab_start, local_logits.shape[1]
        lf = local_logits.float()
        lf = torch.where(torch.isnan(lf), torch.full_like(lf, float("-inf")), lf)
        m = lf.max(dim=-1).values
        s = torch.exp(lf - m[:, None]).sum(dim=-1)
        cand = lf.clone()
        if only is not None:
            keep = cand[:, only - lo].clone() if lo <= only < lo + width else None
            cand.fill_(float("-inf"))
            if keep is not None:
                cand[:, only - lo] = keep
        for t in banned:
            if lo <= t < lo + width:
                cand[:, t - lo] = float("-inf")
        bv, bi = cand.max(dim=-1)
        rec = torch.stack([m, s, bv, (bi + lo).float()], dim=-1).contiguous()  # indices < 2^24 are exact in fp32
        if rec.shape[0] != self.rows:  # the exchange has one shape per step object: pad to the graph's rows
            pad = torch.zeros(self.rows - rec.shape[0], 4, dtype=rec.dtype, device=rec.device)
            rec = torch.cat([rec, pad], dim=0)
        every = self.exchange.gather(rec)[:, : local_logits.shape[0]]  # [world, rows, 4]
        gm = every[..., 0].max(dim=0).values
        lse = gm + torch.log((every[..., 1] * torch.exp(every[..., 0] - gm)).sum(dim=0))
        winner = every[..., 2].argmax(dim=0, keepdim=True)  # first maximum = lowest rank = lowest token id
        tok = every[..., 3].gather(0, winner).squeeze(0).long()
        score = every[..., 2].gather(0, winner).squeeze(0) - lse
        return score, tok
