"""B200-native (sm_100a) implementation of the MoE m-grouped FP8 block-scaled GEMM hot path."""
__version__ = "0.1"
