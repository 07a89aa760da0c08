"""B200-native (sm_100a) KV-cache attention path of simple-llm, behind the reference's API.

``from llm_experiments_b200 import gpu`` gives the reference's operator names for this path
(``kv_cache_create/reset/update``, ``attention_with_kv_cache``, ``flash_attention``,
``batch_begin/commit`` and the buffer helpers).  All compute runs in ``libb2kv.so``, a C-ABI
CUDA library declared in ``include/b2kv.h``; importing this package fails if it is not built.
The directory name carries a hyphen, so import it through ``__graft_entry__.import_package``
(or any importlib loader) under the module name ``llm_experiments_b200``.
"""
from . import _native, gpu  # noqa: F401

__all__ = ["gpu"]
