"""twilight_b200: B200-native (sm_100a) Select-then-Prune decode attention.

Sub-packages: ``kernel`` (operator API over the C ABI), ``pyimpl`` (the reference's selector /
pruner interface), plus ``cache`` (paged KV layout), ``step`` (fused decode step), ``gen``
(synthetic inputs) and ``dist`` (sharding over the GPUs of one node).
"""
__version__ = "0.1.0"
