"""B200-native drop-in for the certified decode-attention modules of DotCache.

Only the certified path is provided: `dotcache.kernels.*` and
`dotcache.backends.{certified_blackwell,cuda_pagein}` with the reference's
names and argument meaning, implemented over libcqa_b200.so (sm_100a CUDA).
"""
__all__ = ["kernels", "backends"]
