"""B200-native (sm_100a) FP8 block-scaled routed-MoE layer behind the Netra engine contract."""
__version__ = "0.1.0"
