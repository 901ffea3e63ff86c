"""B200 (sm_100a) FP8 GEMM library -- Python host layer over the C ABI.

The directory name is not an identifier; import it through ``load_package()`` in
``__graft_entry__.py`` (it registers the package as ``tcfp8_b200``).

    from tcfp8_b200 import gemm        # GEMM / GEMM4: the reference's operator surface
    from tcfp8_b200 import shard       # N-sharded multi-GPU plan
"""
from . import _cabi  # noqa: F401
from . import gemm, shard  # noqa: F401

__all__ = ["gemm", "shard", "_cabi"]
