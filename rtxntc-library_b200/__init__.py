"""B200-native decoder for NTC (neural texture compression) texture sets.

The directory name is not a Python identifier; load it with `__graft_entry__.load_package()` (or
importlib) under the module name `rtxntc_library_b200`.
"""
from . import container, geometry, sharding, synthetic  # noqa: F401
