"""The reference's ``metaseq.distributed`` import path.

The distributed runtime of this package lives in ``metaseq_b200.parallel``; this package only makes
``from metaseq_b200.distributed import utils as distributed_utils`` (the most common import in code written against
the reference), ``metaseq_b200.distributed.fully_sharded_data_parallel``, ``.rendezvous``, ``.module_proxy_wrapper``
and ``.stitch_fsdp_ckpt`` resolve to the modules that implement them.  Nothing is defined here.
"""
import sys
import types

from metaseq_b200.checkpoint import consolidate_fsdp_shards as _consolidate
from metaseq_b200.checkpoint import reshard_mp as _reshard_mp
from metaseq_b200.parallel import fsdp as fully_sharded_data_parallel
from metaseq_b200.parallel import module_proxy_wrapper, rendezvous, utils
from metaseq_b200.parallel.fsdp import FullyShardedDataParallel, fsdp_enable_wrap, fsdp_wrap  # noqa: F401
from metaseq_b200.parallel.module_proxy_wrapper import ModuleProxyWrapper  # noqa: F401

# the reference keeps the shard-stitching helpers in one module; here they sit beside the tools that use them
stitch_fsdp_ckpt = types.ModuleType(__name__ + ".stitch_fsdp_ckpt", "Alias module: see checkpoint/consolidate_fsdp_shards.py "
                                    "and checkpoint/reshard_mp.py.")
for _source, _names in ((_consolidate, ("consolidate_fsdp_shards", "consolidate_model_parallel", "handle_qkv_proj")),
                        (_reshard_mp, ("reshard_megatron_parts", "get_n_layers", "find_num_parts"))):
    for _name in _names:
        setattr(stitch_fsdp_ckpt, _name, getattr(_source, _name))

for _alias, _module in (("utils", utils), ("rendezvous", rendezvous), ("module_proxy_wrapper", module_proxy_wrapper),
                        ("fully_sharded_data_parallel", fully_sharded_data_parallel),
                        ("stitch_fsdp_ckpt", stitch_fsdp_ckpt)):
    sys.modules[__name__ + "." + _alias] = _module
