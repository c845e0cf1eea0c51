"""skywalker_b200: B200-native alias-method graph sampling and random walks.

The compute path is the CUDA library libskywalker_b200.so (C ABI in include/skywalker_b200.h);
this package is the Python host mirror of the reference's operator interface.  There is no CPU
path: importing `skywalker_b200.api` without the built library raises ImportError.
"""
from ._capi import (APP_DEEPWALK, APP_NODE2VEC, APP_PPR, INVALID_VERTEX, KHOP_TAKE_ALL, MODE_OFFLINE,
                    MODE_ONLINE, WALK_CACHE_TABLES, WALK_UNBIASED, WALK_BUILD_TABLES, WALK_DIRECT_SLOTS,
                    KHOP_UNBIASED, KHOP_DISTINCT)

__all__ = ["APP_DEEPWALK", "APP_NODE2VEC", "APP_PPR", "INVALID_VERTEX", "KHOP_TAKE_ALL", "MODE_OFFLINE",
           "MODE_ONLINE", "WALK_CACHE_TABLES", "WALK_UNBIASED", "WALK_BUILD_TABLES", "WALK_DIRECT_SLOTS", "KHOP_UNBIASED", "KHOP_DISTINCT"]
